// Bandwidth-bound helper kernels around the attention main loops: split-KV combine.
#include "fsa_ptx.cuh"
#include "fsa_params.h"
#include "fsa_aux.h"

namespace fsa {

namespace {

// One warp merges the partial results of one (row, head): running max / sum over the splits in the
// base-2 domain, partials with lse = -inf contribute nothing, final lse is converted to natural log.
// Restates _fwd_combine_kernel (flash_sparse_attn/ops/triton/flash_fwd_combine.py:118-161) and
// _dec_combine_kernel (flash_dec_combine.py:15-153).
template <typename T, int VEC>
__global__ void __launch_bounds__(256) combine_kernel(CombineParams p) {
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long long)p.rows * p.heads) return;
  const int h = (int)(item % p.heads);
  const long long row = item / p.heads;
  const int b = (int)(row / p.rows_per_batch);
  const long long s = row - (long long)b * p.rows_per_batch;

  const float* lp = p.lse_partial + (long long)h * p.lp_sh + row;
  const float* op = p.out_partial + (row * p.heads + h) * p.head_dim;
  float e_max = -INFINITY, e_sum = 0.f;
  float acc[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
  const int d0 = lane * VEC;
  const bool active = d0 < p.head_dim;
  for (int sp = 0; sp < p.num_splits; ++sp) {
    const float lse_s = lp[(long long)sp * p.lp_ss];
    const float new_max = fmaxf(lse_s, e_max);
    const float old_scale = (e_max == -INFINITY) ? 0.f : exp2f(e_max - new_max);
    const float w = (lse_s == -INFINITY) ? 0.f : exp2f(lse_s - new_max);
    if (active) {
      const float* src = op + (long long)sp * p.op_ss + d0;
#pragma unroll
      for (int i = 0; i < VEC; i += 4) {
        const float4 v = *reinterpret_cast<const float4*>(src + i);
        acc[i] = acc[i] * old_scale + w * v.x;
        acc[i + 1] = acc[i + 1] * old_scale + w * v.y;
        acc[i + 2] = acc[i + 2] * old_scale + w * v.z;
        acc[i + 3] = acc[i + 3] * old_scale + w * v.w;
      }
    }
    e_sum = e_sum * old_scale + w;
    e_max = new_max;
  }
  const float inv = (e_sum == 0.f || e_sum != e_sum) ? 0.f : 1.0f / e_sum;
  if (active) {
    T* dst = reinterpret_cast<T*>(p.out) + (long long)b * p.o_sb + s * p.o_sm + (long long)h * p.o_sh + d0;
#pragma unroll
    for (int i = 0; i < VEC; i += 2) {
      *reinterpret_cast<uint32_t*>(dst + i) = pack2<T>(acc[i] * inv, acc[i + 1] * inv);
    }
  }
  if (lane == 0) {
    const float lse = (e_sum > 0.f) ? (e_max + log2f(e_sum)) * 0.6931471805599453f : -INFINITY;
    p.lse[(long long)b * p.l_sb + (long long)h * p.l_sh + s] = lse;
  }
}

}  // namespace

cudaError_t launch_combine(const CombineParams& p, int dtype, cudaStream_t stream) {
  const long long items = (long long)p.rows * p.heads;
  if (items <= 0) return cudaSuccess;
  const int warps = 8;
  const unsigned grid = (unsigned)((items + warps - 1) / warps);
  if (p.head_dim % 4 != 0 || p.head_dim > 256) return cudaErrorInvalidValue;
  // VEC floats per lane, 32 lanes: head_dim <= 128 -> 4, <= 256 -> 8
  if (p.head_dim <= 128) {
    if (dtype == DT_BF16)
      combine_kernel<__nv_bfloat16, 4><<<grid, warps * 32, 0, stream>>>(p);
    else
      combine_kernel<__half, 4><<<grid, warps * 32, 0, stream>>>(p);
  } else {
    if (dtype == DT_BF16)
      combine_kernel<__nv_bfloat16, 8><<<grid, warps * 32, 0, stream>>>(p);
    else
      combine_kernel<__half, 8><<<grid, warps * 32, 0, stream>>>(p);
  }
  return cudaGetLastError();
}

}  // namespace fsa
