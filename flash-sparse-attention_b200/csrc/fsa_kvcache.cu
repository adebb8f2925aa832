// The two small steps in front of a top-k decode, as device work with no host round trip:
//
//  * kv append: the new key / value rows of every sequence go to positions seqused_k[b] .. + new_tokens of the
//    cache (contiguous, or paged through the page table; a sequence that grows into a page-table slot without a
//    page takes one from a device-side stack of free pages), and seqused_k advances. The reference leaves this to
//    the caller (its README lists a KV-cache manager as future work); its decode reads exactly this layout
//    (flash_sparse_attn/ops/triton/paged_kv.py:10-30).
//  * index localisation for a sharded cache: from global top-k positions keep the ones inside this shard's
//    [lo, hi) of each sequence, shift them to shard-local positions and move them to the front of the row (order
//    kept); the count per row lets the decode kernel visit only the tiles that hold indices.
//
// Both are HBM-bound copies / integer passes: 16-byte chunks, one warp per cache row, one CTA per row of indices.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fsa_b200.h"
#include "fsa_params.h"

namespace fsa {

namespace {

// One thread per sequence: remember where the new rows start, make sure the pages they fall into exist, advance
// the length. A drained free stack sets the status word (value 3) and leaves the slot unallocated: the copy
// kernel then skips those rows instead of writing through a negative page number.
__global__ void kv_reserve_kernel(const FsaKvAppendArgs a) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= a.batch) return;
  const int pos = a.seqused_k[b];
  a.pos_ws[b] = pos;
  if (a.page_table) {
    const int first = pos / a.page_size, last = (pos + a.new_tokens - 1) / a.page_size;
    for (int pi = first; pi <= last && pi < a.page_table_stride; ++pi) {
      int32_t* slot = a.page_table + (long long)b * a.page_table_stride + pi;
      if (*slot >= 0) continue;
      if (!a.free_pages || !a.free_count) {
        atomicExch(a.status, 3);
        continue;
      }
      const int idx = atomicSub(a.free_count, 1) - 1;
      if (idx < 0) {
        atomicAdd(a.free_count, 1);
        atomicExch(a.status, 3);
        continue;
      }
      *slot = a.free_pages[idx];
    }
  }
  a.seqused_k[b] = pos + a.new_tokens;
}

// One warp per (sequence, new token, KV head) row of K and of V: 16-byte chunks.
__global__ void __launch_bounds__(256) kv_copy_kernel(const FsaKvAppendArgs a, int elem_bytes) {
  const int lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long n_items = (long long)a.batch * a.new_tokens * a.heads_kv;
  if (item >= n_items) return;
  const int h = (int)(item % a.heads_kv);
  const int t = (int)((item / a.heads_kv) % a.new_tokens);
  const int b = (int)(item / ((long long)a.heads_kv * a.new_tokens));
  const int pos = a.pos_ws[b] + t;
  long long dst_row;
  if (a.page_table) {
    const int pi = pos / a.page_size;
    if (pi >= a.page_table_stride) return;
    const int page = a.page_table[(long long)b * a.page_table_stride + pi];
    if (page < 0) return;
    dst_row = (long long)page * a.cache_stride_b + (long long)(pos % a.page_size) * a.cache_stride_s;
  } else {
    if (pos >= a.capacity) return;
    dst_row = (long long)b * a.cache_stride_b + (long long)pos * a.cache_stride_s;
  }
  dst_row += (long long)h * a.cache_stride_h;
  const long long src_row = (long long)b * a.new_stride_b + (long long)t * a.new_stride_s + (long long)h * a.new_stride_h;
  const int chunks = a.head_dim * elem_bytes / 16;
  const char* ks = reinterpret_cast<const char*>(a.k_new) + src_row * elem_bytes;
  const char* vs = reinterpret_cast<const char*>(a.v_new) + src_row * elem_bytes;
  char* kd = reinterpret_cast<char*>(a.k_cache) + dst_row * elem_bytes;
  char* vd = reinterpret_cast<char*>(a.v_cache) + dst_row * elem_bytes;
  for (int c = lane; c < chunks; c += 32) {
    reinterpret_cast<uint4*>(kd)[c] = __ldg(reinterpret_cast<const uint4*>(ks) + c);
    reinterpret_cast<uint4*>(vd)[c] = __ldg(reinterpret_cast<const uint4*>(vs) + c);
  }
}

// One CTA of 256 threads per row of indices: stable compaction of the positions inside [lo, hi), shifted by -lo.
// Every thread takes eight consecutive entries of a 2048-entry chunk (two 16-byte loads), the CTA scans the
// per-thread counts (warp shuffles, then the eight warp totals), and the kept entries go out in their original order.
__global__ void __launch_bounds__(256) localize_kernel(const int32_t* idx, long long idx_stride, const int32_t* bounds,
                                                       int32_t* out, long long out_stride, int32_t* count, int topk) {
  __shared__ int warp_tot[8];
  __shared__ int carry_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int row = blockIdx.x;
  const int lo = bounds[2 * row], hi = bounds[2 * row + 1];
  const int32_t* src = idx + (long long)row * idx_stride;
  int32_t* dst = out + (long long)row * out_stride;
  const bool vec = ((reinterpret_cast<uintptr_t>(src) & 15) == 0) && ((topk & 7) == 0);
  int carry = 0;
  for (int c0 = 0; c0 < topk; c0 += 2048) {
    const int i0 = c0 + tid * 8;
    int v[8];
    if (vec && i0 + 8 <= topk) {
      const int4 a = __ldg(reinterpret_cast<const int4*>(src + i0)), b = __ldg(reinterpret_cast<const int4*>(src + i0 + 4));
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
      v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = (i0 + j < topk) ? __ldg(src + i0 + j) : -1;
    }
    int n = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) n += (v[j] >= lo && v[j] < hi) ? 1 : 0;
    int incl = n;  // inclusive scan over the warp
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, s);
      if (lane >= s) incl += t;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    int base = carry;
#pragma unroll
    for (int w = 0; w < 8; ++w) base += (w < warp) ? warp_tot[w] : 0;
    int at = base + incl - n;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (v[j] >= lo && v[j] < hi) dst[at++] = v[j] - lo;
    if (tid == 255) carry_s = base + incl;
    __syncthreads();
    carry = carry_s;
  }
  for (int i = carry + tid; i < topk; i += 256) dst[i] = -1;
  if (tid == 0) count[row] = carry;
}

}  // namespace

}  // namespace fsa

extern "C" int fsa_kv_append(const FsaKvAppendArgs* a, void* stream_) {
  if (!a || !a->k_new || !a->v_new || !a->k_cache || !a->v_cache || !a->seqused_k || !a->pos_ws || !a->status)
    return FSA_ERR_INVALID_ARG;
  if (a->batch <= 0 || a->new_tokens <= 0 || a->heads_kv <= 0 || a->head_dim <= 0) return FSA_ERR_INVALID_ARG;
  const int es = (a->dtype == FSA_DT_BF16 || a->dtype == FSA_DT_FP16) ? 2 : ((a->dtype == FSA_DT_E4M3 || a->dtype == FSA_DT_E5M2) ? 1 : 0);
  if (!es) return FSA_ERR_UNSUPPORTED;
  if ((a->head_dim * es) % 16) return FSA_ERR_UNSUPPORTED;  // rows move in 16-byte chunks
  const int64_t strides[6] = {a->cache_stride_b, a->cache_stride_s, a->cache_stride_h, a->new_stride_b, a->new_stride_s, a->new_stride_h};
  for (int64_t s : strides)
    if ((s * es) % 16) return FSA_ERR_INVALID_ARG;
  const uintptr_t ptrs[4] = {(uintptr_t)a->k_new, (uintptr_t)a->v_new, (uintptr_t)a->k_cache, (uintptr_t)a->v_cache};
  for (uintptr_t q : ptrs)
    if (q & 15) return FSA_ERR_INVALID_ARG;
  if (a->page_table && (a->page_size <= 0 || a->page_table_stride <= 0)) return FSA_ERR_INVALID_ARG;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  fsa::kv_reserve_kernel<<<(a->batch + 127) / 128, 128, 0, stream>>>(*a);
  if (cudaGetLastError() != cudaSuccess) return FSA_ERR_LAUNCH;
  const long long items = (long long)a->batch * a->new_tokens * a->heads_kv;
  fsa::kv_copy_kernel<<<(unsigned)((items + 7) / 8), 256, 0, stream>>>(*a, es);
  return cudaGetLastError() == cudaSuccess ? FSA_OK : FSA_ERR_LAUNCH;
}

extern "C" int fsa_localize_indices(const int32_t* indices, int64_t indices_stride, const int32_t* key_bounds,
                                    int32_t* out, int64_t out_stride, int32_t* count, int rows, int topk,
                                    void* stream_) {
  if (!indices || !key_bounds || !out || !count || rows < 0 || topk <= 0) return FSA_ERR_INVALID_ARG;
  if (rows == 0) return FSA_OK;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  fsa::localize_kernel<<<rows, 256, 0, stream>>>(indices, indices_stride, key_bounds, out, out_stride, count, topk);
  return cudaGetLastError() == cudaSuccess ? FSA_OK : FSA_ERR_LAUNCH;
}
