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

// Block-scaled quantisation: one block of 128 threads per (sequence, head, 128-position block), one thread per
// position (its head_dim elements in registers): absolute maximum over the block -> scale = amax / FP8_MAX
// (0 for an all-zero block, so that it never sets the largest scale of a head) -> scaled cast. Positions past the sequence end count as zeros and are not written.
// With `x` null only the de-quantisation is run the other way round: out16 = fp8 * scale (dequant = true).
template <typename T, int FP8>
__global__ void __launch_bounds__(128) quantize_block_kernel(const T* __restrict__ x, uint8_t* __restrict__ x8,
                                                            float* __restrict__ scales, const int* cu, int seqlen,
                                                            int heads, int head_dim, int nblk, long long sb,
                                                            long long ss, long long sh, long long qb, long long qs,
                                                            long long qh) {
  const int blk = blockIdx.x % nblk;
  const int h = (blockIdx.x / nblk) % heads;
  const int b = blockIdx.x / (nblk * heads);
  const int off = cu ? cu[b] : 0;
  const int len = cu ? cu[b + 1] - off : seqlen;
  const int r = blk * 128 + threadIdx.x;
  const bool live = r < len;
  const T* src = x + (cu ? 0 : (long long)b * sb) + (long long)(off + r) * ss + (long long)h * sh;
  uint4 v[16];  // up to 128 16-bit elements
  const int chunks = head_dim / 8;
  float m = 0.f;
#pragma unroll
  for (int c = 0; c < 16; ++c) {
    v[c] = make_uint4(0, 0, 0, 0);
    if (live && c < chunks) {
      v[c] = __ldcg(reinterpret_cast<const uint4*>(src) + c);
      const T* e = reinterpret_cast<const T*>(&v[c]);
#pragma unroll
      for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(to_f32(e[j])));
    }
  }
#pragma unroll
  for (int sft = 16; sft > 0; sft >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, sft));
  __shared__ float wmax[4];
  if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = m;
  __syncthreads();
  m = fmaxf(fmaxf(wmax[0], wmax[1]), fmaxf(wmax[2], wmax[3]));
  const float scale = m > 0.f ? __fdiv_rn(m, fp8_max<FP8>()) : 0.0f;
  const float inv = m > 0.f ? __fdiv_rn(fp8_max<FP8>(), m) : 0.0f;
  if (threadIdx.x == 0) scales[((long long)b * heads + h) * nblk + blk] = scale;
  if (!live) return;
  uint8_t* dst = x8 + (cu ? 0 : (long long)b * qb) + (long long)(off + r) * qs + (long long)h * qh;
#pragma unroll
  for (int c = 0; c < 16; ++c) {
    if (c < chunks) {
      const T* e = reinterpret_cast<const T*>(&v[c]);
      alignas(8) uint8_t q[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) q[j] = f32_to_fp8<FP8>(to_f32(e[j]) * inv);
      *reinterpret_cast<uint2*>(dst + c * 8) = *reinterpret_cast<const uint2*>(q);
    }
  }
}

// out[b, r, h, :] = T(float(x8[b, r, h, :]) * scales[b, h, r / 128]): what the backward runs on.
template <typename T, int FP8>
__global__ void __launch_bounds__(128) dequantize_block_kernel(const uint8_t* __restrict__ x8, T* __restrict__ out,
                                                              const float* __restrict__ scales, const int* cu,
                                                              int seqlen, int heads, int head_dim, int nblk,
                                                              long long qb, long long qs, long long qh, long long ob,
                                                              long long os, long long oh) {
  const int blk = blockIdx.x % nblk;
  const int h = (blockIdx.x / nblk) % heads;
  const int b = blockIdx.x / (nblk * heads);
  const int off = cu ? cu[b] : 0;
  const int len = cu ? cu[b + 1] - off : seqlen;
  const int r = blk * 128 + threadIdx.x;
  if (r >= len) return;
  const float sc = scales[((long long)b * heads + h) * nblk + blk];
  const uint8_t* src = x8 + (cu ? 0 : (long long)b * qb) + (long long)(off + r) * qs + (long long)h * qh;
  T* dst = out + (cu ? 0 : (long long)b * ob) + (long long)(off + r) * os + (long long)h * oh;
  for (int c = 0; c < head_dim / 8; ++c) {
    const uint2 raw = *reinterpret_cast<const uint2*>(src + c * 8);
    const uint8_t* e = reinterpret_cast<const uint8_t*>(&raw);
    alignas(16) T o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = T(fp8_to_f32<FP8>(e[j]) * sc);
    *reinterpret_cast<uint4*>(dst + c * 8) = *reinterpret_cast<const uint4*>(o);
  }
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

int fsa_quantize_fp8_blockwise(const FsaBlockQuantArgs* a, void* stream_) {
  if (!a || !a->x16 || !a->x8 || !a->scales) return FSA_ERR_INVALID_ARG;
  if (a->batch <= 0 || a->heads <= 0 || a->seqlen <= 0 || a->head_dim <= 0 || a->head_dim > 128 || a->head_dim % 8)
    return FSA_ERR_UNSUPPORTED;
  if (a->fp8_dtype != FSA_DT_E5M2 && a->fp8_dtype != FSA_DT_E4M3) return FSA_ERR_UNSUPPORTED;
  if (a->x_dtype != FSA_DT_BF16 && a->x_dtype != FSA_DT_FP16) return FSA_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(a->x16) & 15) || (reinterpret_cast<uintptr_t>(a->x8) & 7) || (a->x_stride_s % 8) ||
      (a->x_stride_h % 8) || (a->x_stride_b % 8) || (a->q_stride_s % 8) || (a->q_stride_h % 8) || (a->q_stride_b % 8))
    return FSA_ERR_INVALID_ARG;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  const int nblk = (a->seqlen + 127) / 128;
  const unsigned grid = (unsigned)((long long)a->batch * a->heads * nblk);
#define FSA_BQ(T_, F_)                                                                                                   \
  if (a->dequantize)                                                                                                     \
    fsa::dequantize_block_kernel<T_, F_><<<grid, 128, 0, s>>>(                                                          \
        reinterpret_cast<const uint8_t*>(a->x8), reinterpret_cast<T_*>(a->x16), a->scales, a->cu_seqlens, a->seqlen,     \
        a->heads, a->head_dim, nblk, a->q_stride_b, a->q_stride_s, a->q_stride_h, a->x_stride_b, a->x_stride_s,          \
        a->x_stride_h);                                                                                                  \
  else                                                                                                                   \
    fsa::quantize_block_kernel<T_, F_><<<grid, 128, 0, s>>>(                                                            \
        reinterpret_cast<const T_*>(a->x16), reinterpret_cast<uint8_t*>(a->x8), a->scales, a->cu_seqlens, a->seqlen,     \
        a->heads, a->head_dim, nblk, a->x_stride_b, a->x_stride_s, a->x_stride_h, a->q_stride_b, a->q_stride_s,          \
        a->q_stride_h);
  if (a->x_dtype == FSA_DT_BF16) {
    if (a->fp8_dtype == FSA_DT_E4M3) {
      FSA_BQ(__nv_bfloat16, FSA_DT_E4M3)
    } else {
      FSA_BQ(__nv_bfloat16, FSA_DT_E5M2)
    }
  } else {
    if (a->fp8_dtype == FSA_DT_E4M3) {
      FSA_BQ(__half, FSA_DT_E4M3)
    } else {
      FSA_BQ(__half, FSA_DT_E5M2)
    }
  }
#undef FSA_BQ
  return cudaGetLastError() == cudaSuccess ? FSA_OK : FSA_ERR_LAUNCH;
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
