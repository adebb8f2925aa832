// Top-k position selection for the decode path: per row of scores the k largest entries, returned as
// ascending positions - what `gather_kv_indices` of the decode operators expects. Restates
// flash_sparse_attn/utils/mask.py:20-44 (torch.topk(..., sorted=False) followed by a sort of the indices)
// as one kernel without a sort: a radix select (8 bits per pass) finds the k-th largest key exactly, then one
// ordered compaction pass writes the selected positions in index order. Among equal scores at the
// threshold the lowest positions win (torch leaves that choice unspecified). NaN orders above +inf, as
// in torch.topk. Integer work on L2-resident rows: a cluster of 1 to 8 CTAs of 1024 threads per row (as many as
// keep the grid within the SM count), three (16-bit scores) or five (fp32) passes over the row with 16-byte loads,
// plus a counting pass when the row is shared.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fsa_b200.h"
#include "fsa_params.h"

namespace fsa {

namespace {

constexpr int TK_THREADS = 1024;
constexpr int TK_V = 8;  // consecutive entries per thread and step (one or two 16-byte loads)

// Monotone map to an unsigned key: larger value, larger key (-0 < +0 is harmless for a selection). 16-bit
// inputs keep 16-bit keys (two radix passes instead of four).
template <typename T>
struct KeyOf {
  static constexpr int kBits = 16;
  __device__ static uint32_t key(T v) {
    const uint32_t b = *reinterpret_cast<const unsigned short*>(&v);
    return (b & 0x8000u) ? (~b & 0xffffu) : (b | 0x8000u);
  }
};
template <>
struct KeyOf<float> {
  static constexpr int kBits = 32;
  __device__ static uint32_t key(float v) {
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
  }
};

// Keys of entries [i0, i0 + TK_V) of a row; entries past n get `fill`.
template <typename T>
__device__ __forceinline__ void load_keys(const T* row, bool vec_ok, int i0, int n, uint32_t fill, uint32_t* keys) {
  if (vec_ok && i0 + TK_V <= n) {
    constexpr int NV = TK_V * sizeof(T) / 16;
    uint4 raw[NV];
#pragma unroll
    for (int v = 0; v < NV; ++v) raw[v] = __ldg(reinterpret_cast<const uint4*>(row + i0) + v);
    const T* e = reinterpret_cast<const T*>(raw);
#pragma unroll
    for (int j = 0; j < TK_V; ++j) keys[j] = KeyOf<T>::key(e[j]);
  } else {
#pragma unroll
    for (int j = 0; j < TK_V; ++j) keys[j] = (i0 + j < n) ? KeyOf<T>::key(row[i0 + j]) : fill;
  }
}

// Inclusive scan of `v` over the block; returns the inclusive prefix of this thread and the block total.
__device__ __forceinline__ uint32_t block_scan(uint32_t v, uint32_t* warp_tot, uint32_t* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t x = v;
#pragma unroll
  for (int s = 1; s < 32; s <<= 1) {
    const uint32_t y = __shfl_up_sync(0xffffffffu, x, s);
    if (lane >= s) x += y;
  }
  if (lane == 31) warp_tot[warp] = x;
  __syncthreads();
  if (warp == 0) {
    uint32_t w = warp_tot[lane];  // TK_THREADS / 32 == 32 warps
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
      const uint32_t y = __shfl_up_sync(0xffffffffu, w, s);
      if (lane >= s) w += y;
    }
    warp_tot[lane] = w;  // inclusive totals of the warps
  }
  __syncthreads();
  const uint32_t before = warp == 0 ? 0u : warp_tot[warp - 1];
  *total = warp_tot[TK_THREADS / 32 - 1];
  __syncthreads();  // warp_tot is reused by the next call
  return x + before;
}

// One thread-block cluster per row: CTA `rank` of `csize` owns the slice [rank * chunk, (rank + 1) * chunk) of the
// row. The histograms of a radix pass are summed over the cluster through distributed shared memory (every CTA
// reads all of them and walks the bins itself, so all agree without a broadcast); for the compaction every CTA
// first counts the greater / equal entries of its slice and takes the counts of the slices before it as its base.
// With 64 rows one CTA per row would leave more than half of a B200's 148 SMs idle.
template <typename T, typename I>
__global__ void __launch_bounds__(TK_THREADS) topk_kernel(const T* __restrict__ scores, long long row_stride, int n, int k,
                                                          I* __restrict__ out, int csize, int chunk) {
  static_assert(TK_THREADS == 1024, "block_scan assumes 32 warps");
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ uint32_t hist[256];
  __shared__ uint32_t warp_tot[TK_THREADS / 32];
  __shared__ uint32_t sel_prefix, sel_remaining;
  __shared__ uint32_t slice_cnt[2];  // greater / equal entries of this CTA's slice
  const int rank = (int)cluster.block_rank();
  const int row_idx = blockIdx.x / csize;
  const T* row = scores + (long long)row_idx * row_stride;
  I* dst = out + (long long)row_idx * k;
  const int tid = threadIdx.x;
  const bool vec_ok = (reinterpret_cast<uintptr_t>(row) & 15) == 0;
  constexpr int PASSES = KeyOf<T>::kBits / 8;
  constexpr int STEP = TK_THREADS * TK_V;
  const int lo = rank * chunk < n ? rank * chunk : n;
  const int hi = lo + chunk < n ? lo + chunk : n;  // this CTA's slice [lo, hi); chunk is a multiple of TK_V

  // ---- radix select: after pass d the top 8(d+1) bits of the k-th largest key are known ----------------
  uint32_t prefix = 0, remaining = (uint32_t)k;  // keys above the prefix range so far: k - remaining
  for (int pass = 0; pass < PASSES; ++pass) {
    const int shift = KeyOf<T>::kBits - 8 - 8 * pass;
    const uint32_t mask_hi = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = tid; i < 256; i += TK_THREADS) hist[i] = 0;
    __syncthreads();
    for (int start = lo; start < hi; start += STEP) {
      const int i0 = start + tid * TK_V;
      if (i0 < hi) {
        uint32_t keys[TK_V];
        load_keys(row, vec_ok, i0, hi, 0u, keys);
#pragma unroll
        for (int j = 0; j < TK_V; ++j)
          if (i0 + j < hi && (keys[j] & mask_hi) == prefix) atomicAdd(&hist[(keys[j] >> shift) & 255u], 1u);
      }
    }
    cluster.sync();  // every CTA's histogram is complete
    uint32_t total_bin = 0;
    if (tid < 256)
      for (int r = 0; r < csize; ++r) total_bin += *cluster.map_shared_rank(&hist[tid], r);
    cluster.sync();  // all remote reads done: the histograms may be cleared again
    if (tid < 256) hist[tid] = total_bin;
    __syncthreads();
    if (tid == 0) {
      // walk the bins from the top until `remaining` keys are covered
      uint32_t rem = remaining;
      int bin = 255;
      for (; bin > 0; --bin) {
        if (hist[bin] >= rem) break;
        rem -= hist[bin];
      }
      sel_prefix = prefix | ((uint32_t)bin << shift);
      sel_remaining = rem;  // how many keys of this bin (with this prefix) are still needed
    }
    __syncthreads();
    prefix = sel_prefix;
    remaining = sel_remaining;
    __syncthreads();
  }
  const uint32_t thr = prefix;         // key of the k-th largest entry
  const uint32_t need_eq = remaining;  // entries equal to it that belong to the selection (lowest positions)

  // ---- counts of this slice, bases from the slices before it ------------------------------------------
  uint32_t base_gt = 0, base_eq = 0;  // greater / equal entries before the current step of this CTA
  if (csize > 1) {
    uint32_t c_gt = 0, c_eq = 0;
    for (int start = lo; start < hi; start += STEP) {
      const int i0 = start + tid * TK_V;
      if (i0 < hi) {
        uint32_t keys[TK_V];
        load_keys(row, vec_ok, i0, hi, 0u, keys);
#pragma unroll
        for (int j = 0; j < TK_V; ++j)
          if (i0 + j < hi) {
            c_gt += keys[j] > thr ? 1u : 0u;
            c_eq += keys[j] == thr ? 1u : 0u;
          }
      }
    }
    uint32_t tot;
    block_scan(c_gt, warp_tot, &tot);
    if (tid == 0) slice_cnt[0] = tot;
    block_scan(c_eq, warp_tot, &tot);
    if (tid == 0) slice_cnt[1] = tot;
    cluster.sync();
    for (int r = 0; r < rank; ++r) {
      base_gt += *cluster.map_shared_rank(&slice_cnt[0], r);
      base_eq += *cluster.map_shared_rank(&slice_cnt[1], r);
    }
  }

  // ---- ordered compaction: every thread owns TK_V consecutive entries, positions come out ascending ----------
  for (int start = lo; start < hi; start += STEP) {
    const int i0 = start + tid * TK_V;
    uint32_t keys[TK_V];
    uint32_t cnt = 0;  // greater in the low half, equal in the high half (a step has <= 8192 entries)
    if (i0 < hi) {
      load_keys(row, vec_ok, i0, hi, 0u, keys);
#pragma unroll
      for (int j = 0; j < TK_V; ++j)
        if (i0 + j < hi) cnt += (keys[j] > thr ? 1u : 0u) | (keys[j] == thr ? 0x10000u : 0u);
    }
    uint32_t total;
    const uint32_t inc = block_scan(cnt, warp_tot, &total);
    uint32_t gt_before = base_gt + (inc & 0xffffu) - (cnt & 0xffffu);
    uint32_t eq_before = base_eq + (inc >> 16) - (cnt >> 16);
    if (i0 < hi && cnt != 0u) {
#pragma unroll
      for (int j = 0; j < TK_V; ++j) {
        if (i0 + j >= hi) break;
        const bool gt = keys[j] > thr, eq = keys[j] == thr;
        if (gt || (eq && eq_before < need_eq)) dst[gt_before + (eq_before < need_eq ? eq_before : need_eq)] = (I)(i0 + j);
        gt_before += gt ? 1u : 0u;
        eq_before += eq ? 1u : 0u;
      }
    }
    base_gt += total & 0xffffu;
    base_eq += total >> 16;
  }
  cluster.sync();  // nobody leaves while another CTA may still read its shared memory
}

// Cluster size: the largest power of two up to 8 that keeps rows * size within the SM count, and leaves a slice
// of at least one step per CTA.
inline int topk_cluster_size(int rows, int n) {
  int c = 1;
  const int sms = device_sm_count();
  while (c < 8 && rows * (c * 2) <= sms && n / (c * 2) >= TK_THREADS * TK_V) c *= 2;
  return c;
}

template <typename T, typename I>
cudaError_t launch_topk_t(const void* scores, long long row_stride, int rows, int n, int k, void* out, cudaStream_t stream) {
  const int csize = topk_cluster_size(rows, n);
  int chunk = (n + csize - 1) / csize;
  chunk = (chunk + TK_V - 1) / TK_V * TK_V;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(rows * csize), 1, 1);
  cfg.blockDim = dim3(TK_THREADS, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)csize;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, topk_kernel<T, I>, reinterpret_cast<const T*>(scores), row_stride, n, k,
                            reinterpret_cast<I*>(out), csize, chunk);
}

template <typename T>
cudaError_t launch_topk(const void* scores, long long row_stride, int rows, int n, int k, void* out, int out64,
                        cudaStream_t stream) {
  if (out64) return launch_topk_t<T, long long>(scores, row_stride, rows, n, k, out, stream);
  return launch_topk_t<T, int>(scores, row_stride, rows, n, k, out, stream);
}

}  // namespace

}  // namespace fsa

extern "C" int fsa_topk_indices(const void* scores, int dtype, int rows, int n, int64_t row_stride, int k, void* out,
                                int out_is_int64, void* stream_) {
  if (!scores || !out || rows < 0 || n <= 0 || k <= 0 || k > n || row_stride < n) return FSA_ERR_INVALID_ARG;
  if (rows == 0) return FSA_OK;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  cudaError_t e;
  switch (dtype) {
    case FSA_DT_BF16:
      e = fsa::launch_topk<__nv_bfloat16>(scores, row_stride, rows, n, k, out, out_is_int64, stream);
      break;
    case FSA_DT_FP16:
      e = fsa::launch_topk<__half>(scores, row_stride, rows, n, k, out, out_is_int64, stream);
      break;
    case FSA_DT_F32:
      e = fsa::launch_topk<float>(scores, row_stride, rows, n, k, out, out_is_int64, stream);
      break;
    default:
      return FSA_ERR_UNSUPPORTED;
  }
  return e == cudaSuccess ? FSA_OK : FSA_ERR_LAUNCH;
}
