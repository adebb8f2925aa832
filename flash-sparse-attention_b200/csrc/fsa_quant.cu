// Per-tensor FP8 quantisation (bandwidth-bound): absolute maximum, scaled cast, and the widening cast
// back to 16 bits. Restates flash_sparse_attn/ops/triton/quant.py:6-64: scale = FP8_MAX / amax,
// x_fp8 = round_to_nearest_even(x * scale), returned scale = amax / FP8_MAX in the input's type
// (e5m2: FP8_MAX = 57344, e4m3fn: 448). Nothing here synchronises with the host: the second kernel
// reads the maximum the first one left in device memory.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fsa_b200.h"
#include "fsa_params.h"

namespace fsa {

namespace {

constexpr int QT = 256;  // threads per block

template <typename T>
__device__ __forceinline__ float to_f32(T v) {
  return float(v);
}

template <int FP8>
__device__ __forceinline__ float fp8_max() {
  return FP8 == FSA_DT_E5M2 ? 57344.0f : 448.0f;
}
template <int FP8>
__device__ __forceinline__ uint8_t f32_to_fp8(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, FP8 == FSA_DT_E5M2 ? __NV_E5M2 : __NV_E4M3);
}
template <int FP8>
__device__ __forceinline__ float fp8_to_f32(uint8_t v) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)v, FP8 == FSA_DT_E5M2 ? __NV_E5M2 : __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

// 16 bytes of input per thread and iteration; the tail is handled element-wise by the last threads.
template <typename T>
__global__ void __launch_bounds__(QT) amax_kernel(const T* __restrict__ x, long long n, unsigned* amax_bits) {
  constexpr int V = 16 / sizeof(T);
  const long long nvec = n / V;
  float m = 0.f;
  for (long long i = (long long)blockIdx.x * QT + threadIdx.x; i < nvec; i += (long long)gridDim.x * QT) {
    const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(x) + i);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int j = 0; j < V; ++j) m = fmaxf(m, fabsf(to_f32(e[j])));
  }
  if (blockIdx.x == 0)
    for (long long i = nvec * V + threadIdx.x; i < n; i += QT) m = fmaxf(m, fabsf(to_f32(x[i])));
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, s));
  __shared__ float wmax[QT / 32];
  if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int w = 0; w < QT / 32; ++w) m = fmaxf(m, wmax[w]);
    // non-negative floats order like their bit patterns
    atomicMax(amax_bits, __float_as_uint(m));
  }
}

template <typename T, int FP8>
__global__ void __launch_bounds__(QT) quantize_kernel(const T* __restrict__ x, uint8_t* __restrict__ out,
                                                     const float* amax, T* scale_out, long long n) {
  constexpr int V = 16 / sizeof(T);
  const float a = *amax;
  const float scale = __fdiv_rn(fp8_max<FP8>(), a);
  if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = T(__fdiv_rn(a, fp8_max<FP8>()));
  const long long nvec = n / V;
  for (long long i = (long long)blockIdx.x * QT + threadIdx.x; i < nvec; i += (long long)gridDim.x * QT) {
    const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(x) + i);
    const T* e = reinterpret_cast<const T*>(&raw);
    alignas(8) uint8_t q[V];
#pragma unroll
    for (int j = 0; j < V; ++j) q[j] = f32_to_fp8<FP8>(to_f32(e[j]) * scale);
    if (V == 8)
      *reinterpret_cast<uint2*>(out + i * V) = *reinterpret_cast<const uint2*>(q);
    else
      *reinterpret_cast<uint32_t*>(out + i * V) = *reinterpret_cast<const uint32_t*>(q);
  }
  if (blockIdx.x == 0)
    for (long long i = nvec * V + threadIdx.x; i < n; i += QT) out[i] = f32_to_fp8<FP8>(to_f32(x[i]) * scale);
}

// out = T(float(x_fp8) * scale) (scale optional, one element of type T): the widening itself is exact
// for both FP8 formats in bf16 and fp16.
template <typename T, int FP8>
__global__ void __launch_bounds__(QT) widen_kernel(const uint8_t* __restrict__ x, T* __restrict__ out,
                                                  const T* scale, long long n) {
  const float s = scale ? float(*scale) : 1.0f;
  const long long nvec = n / 16;
  for (long long i = (long long)blockIdx.x * QT + threadIdx.x; i < nvec; i += (long long)gridDim.x * QT) {
    const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(x) + i);
    const uint8_t* e = reinterpret_cast<const uint8_t*>(&raw);
    alignas(16) T o[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) o[j] = T(fp8_to_f32<FP8>(e[j]) * s);
    uint4* dst = reinterpret_cast<uint4*>(out + i * 16);
    dst[0] = reinterpret_cast<const uint4*>(o)[0];
    dst[1] = reinterpret_cast<const uint4*>(o)[1];
  }
  if (blockIdx.x == 0)
    for (long long i = nvec * 16 + threadIdx.x; i < n; i += QT) out[i] = T(fp8_to_f32<FP8>(x[i]) * s);
}

unsigned grid_for(long long n_items) {
  const int sms = fsa::device_sm_count();
  const long long want = (n_items + QT - 1) / QT;
  const long long cap = (long long)sms * 8;  // 8 resident blocks of 256 threads per SM
  return (unsigned)(want < 1 ? 1 : (want < cap ? want : cap));
}

template <typename T>
int quantize_typed(const void* x, void* out, void* scale_out, float* amax_ws, long long n, int fp8, cudaStream_t s) {
  constexpr int V = 16 / sizeof(T);
  const unsigned grid = grid_for(n / V);
  amax_kernel<T><<<grid, QT, 0, s>>>(reinterpret_cast<const T*>(x), n, reinterpret_cast<unsigned*>(amax_ws));
  if (fp8 == FSA_DT_E5M2)
    quantize_kernel<T, FSA_DT_E5M2><<<grid, QT, 0, s>>>(reinterpret_cast<const T*>(x), reinterpret_cast<uint8_t*>(out),
                                                         amax_ws, reinterpret_cast<T*>(scale_out), n);
  else
    quantize_kernel<T, FSA_DT_E4M3><<<grid, QT, 0, s>>>(reinterpret_cast<const T*>(x), reinterpret_cast<uint8_t*>(out),
                                                         amax_ws, reinterpret_cast<T*>(scale_out), n);
  return cudaGetLastError() == cudaSuccess ? FSA_OK : FSA_ERR_LAUNCH;
}

template <typename T>
int widen_typed(const void* x, void* out, const void* scale, long long n, int fp8, cudaStream_t s) {
  const unsigned grid = grid_for(n / 16);
  if (fp8 == FSA_DT_E5M2)
    widen_kernel<T, FSA_DT_E5M2><<<grid, QT, 0, s>>>(reinterpret_cast<const uint8_t*>(x), reinterpret_cast<T*>(out),
                                                      reinterpret_cast<const T*>(scale), n);
  else
    widen_kernel<T, FSA_DT_E4M3><<<grid, QT, 0, s>>>(reinterpret_cast<const uint8_t*>(x), reinterpret_cast<T*>(out),
                                                      reinterpret_cast<const T*>(scale), n);
  return cudaGetLastError() == cudaSuccess ? FSA_OK : FSA_ERR_LAUNCH;
}

}  // namespace

}  // namespace fsa

extern "C" {

int fsa_quantize_fp8(const void* x, void* x_fp8, void* scale_out, float* amax_ws, int64_t n, int x_dtype,
                     int fp8_dtype, void* stream_) {
  if (!x || !x_fp8 || !scale_out || !amax_ws || n < 0) return FSA_ERR_INVALID_ARG;
  if (fp8_dtype != FSA_DT_E5M2 && fp8_dtype != FSA_DT_E4M3) return FSA_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(x_fp8) & 7)) return FSA_ERR_INVALID_ARG;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  if (cudaMemsetAsync(amax_ws, 0, sizeof(float), s) != cudaSuccess) return FSA_ERR_LAUNCH;
  switch (x_dtype) {
    case FSA_DT_BF16:
      return fsa::quantize_typed<__nv_bfloat16>(x, x_fp8, scale_out, amax_ws, n, fp8_dtype, s);
    case FSA_DT_FP16:
      return fsa::quantize_typed<__half>(x, x_fp8, scale_out, amax_ws, n, fp8_dtype, s);
    case FSA_DT_F32:
      return fsa::quantize_typed<float>(x, x_fp8, scale_out, amax_ws, n, fp8_dtype, s);
    default:
      return FSA_ERR_UNSUPPORTED;
  }
}

int fsa_fp8_widen(const void* x_fp8, void* out, const void* scale, int64_t n, int fp8_dtype, int out_dtype,
                  void* stream_) {
  if (!x_fp8 || !out || n < 0) return FSA_ERR_INVALID_ARG;
  if (fp8_dtype != FSA_DT_E5M2 && fp8_dtype != FSA_DT_E4M3) return FSA_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(x_fp8) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return FSA_ERR_INVALID_ARG;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  if (out_dtype == FSA_DT_BF16) return fsa::widen_typed<__nv_bfloat16>(x_fp8, out, scale, n, fp8_dtype, s);
  if (out_dtype == FSA_DT_FP16) return fsa::widen_typed<__half>(x_fp8, out, scale, n, fp8_dtype, s);
  return FSA_ERR_UNSUPPORTED;
}

}  // extern "C"
