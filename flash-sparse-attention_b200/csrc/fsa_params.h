// Kernel-side parameter blocks (internal; the C ABI structs in include/fsa_b200.h are translated
// into these by fsa_api.cu).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

namespace fsa {

enum : unsigned {
  F_CAUSAL = 1u << 0,
  F_LOCAL = 1u << 1,
  F_SPLIT = 1u << 2,     // split-KV (forward/decode) or split-QO (backward)
  F_VARLEN_Q = 1u << 3,  // rows of Q/O addressed through cu_seqlens_q
  F_VARLEN_K = 1u << 4,
  F_PAGED = 1u << 5,
  F_PACK_GQA = 1u << 6,
  F_USED_Q = 1u << 7,  // seqused_q present
  F_USED_K = 1u << 8,
  F_LOGSIGMOID = 1u << 9,
  F_ADAPT_GATE = 1u << 10,
  F_GATHER = 1u << 11,
  F_LSE_LOG2 = 1u << 12,   // store lse in base 2 (split partials), else natural log
  F_KV_RAGGED = 1u << 13,  // rows past the key length may hold foreign data: zero V tails in smem
  F_DETERMINISTIC = 1u << 14,  // backward: dQ contributions of the key tiles are added in a fixed order
};

enum { KIND_DENSE = 0, KIND_SPARSE = 1, KIND_GATED = 2 };
enum { DT_BF16 = 0, DT_FP16 = 1, DT_E4M3 = 2, DT_E5M2 = 3, DT_F32 = 4 };

struct alignas(64) FwdKernelParams {
  CUtensorMap map_q, map_k, map_v;
  void* out;         // T* [rows, Hq, D] or float* partial when F_SPLIT
  float* lse;        // final or partial
  const int* cu_q;   // [B+1] or null
  const int* cu_k;
  const int* used_q;  // [B] or null
  const int* used_k;
  const int* page_table;  // [B, pt_stride]
  const int* windows;     // [Hkv, win_stride] = sink, left, right, near
  const void* alpha;      // gated: [B, Hq, Sq] (row-contiguous), element type T
  const void* delta;      // gated: [B, Hkv, Sk]
  int* status;            // device word: 0 ok, non-zero = a bounded wait expired
  uint8_t* tile_map;      // optional [B, Hgrid, num_m_blocks, num_splits, n_tiles_k]: 1 computed, 2 skipped
  long long o_sb, o_sm, o_sh, o_ss;
  long long l_sb, l_sh, l_ss;
  long long a_sb, a_sh, d_sb, d_sh;
  int B, Hq, Hkv, G, gpack;
  int D;       // real head size (<= the kernel's HD; the tail loads as zeros and is not written)
  int sq, sk;  // static lengths (max lengths for varlen)
  int num_splits, num_m_blocks, num_pairs, hgrid;
  int page_size, pt_stride, win_stride, n_tiles_k;
  float scale_log2, softmax_thr, gate_thr, v_scale;
  const float* qkv_scale;  // optional device fp32 [3]: de-quantisation scales of q, k, v
  const float* gate_ws;    // gated: per-tile extremes, see GateWsLayout
  const float* q_bscale;   // block-scaled FP8: [B, Hq, num_m_blocks], [B, Hkv, n_tiles_k] x 2; or all null
  const float* k_bscale;
  const float* v_bscale;
  unsigned flags;
};

struct alignas(64) BwdKernelParams {
  CUtensorMap map_q, map_k, map_v, map_do, map_dq;
  const float* lse2_ws;   // [Hq, ws_sh] minus the base-2 log-sum-exp, tile-padded rows
  const float* dpsum_ws;  // [Hq, ws_sh] minus rowsum(O * dO); zero at padding rows
  void* dk_out;           // T* [rows_k, Hkv, D] (strided) or float partial [splits, ...] when F_SPLIT
  void* dv_out;
  const int* cu_q;
  const int* cu_k;
  const int* used_q;
  const int* used_k;
  const int* windows;
  int* status;
  uint8_t* tile_map;  // optional [B, Hq, n_tiles_k, num_splits, num_m_blocks]
  const void* alpha_ws;  // gated: T [Hq, ws_sh], tile-padded rows, zero outside the sequences
  const void* delta;     // gated: T [B, Hkv, Sk] | [Hkv, Tk]
  float* da_accum;       // gated: [Hq, ws_sh] fp32, zeroed; receives atomic adds
  const float* gate_ws;  // gated: per-tile extremes of alpha / delta (gate_ws_bytes), or null
  const unsigned short* dq_order;  // deterministic: [B, Hkv, n_tiles_k, num_m_blocks] rank of a key tile among
                                   // the key tiles that add into a query tile (descending key index)
  int* dq_turn;                    // deterministic: [B, Hq, num_m_blocks] zeroed; one tick per finished key tile
  void* dd_out;          // gated: T* laid out like delta, or float partial [splits, ...] when F_SPLIT
  long long d_sb, d_sh, dd_ss;
  long long dkv_sb, dkv_sn, dkv_sh, dkv_ss;
  long long ws_sh;
  int D;  // real head size (<= the kernel's HD)
  int B, Hq, Hkv, G;
  int sq, sk;
  int num_splits, n_tiles_k, num_m_blocks, win_stride;
  float scale_log2, softmax_scale, softmax_thr, gate_thr;
  unsigned flags;
};

struct DecKernelParams {
  const void* q;  // [B, Hq, D]
  const void* k;  // [B, Sk, Hkv, D] | packed [Tk, Hkv, D] | paged [pages, page, Hkv, D]
  const void* v;
  void* out;           // [B, Hq, D]
  float* lse;          // [B, Hq]
  float* out_partial;  // [splits, B, Hq, D]
  float* lse_partial;  // [splits, Hq, B] base-2
  const int* cu_k;
  const int* used_k;
  const int* page_table;
  const int* gather_idx;
  const int* windows;
  const void* alpha;  // gated: [B, Hq]
  const void* delta;  // gated: [B, Hkv, Sk] | [Hkv, Tk] | paged [pages, Hkv, page]
  uint8_t* tile_map;  // optional [B, Hkv, n_tiles] over 16-key tiles
  long long q_sb, q_sh, k_sb, k_sn, k_sh, o_sb, o_sh, l_sb, l_sh, a_sb, a_sh, d_sb, d_sh;
  int B, Hq, Hkv, G;
  int sk, sk_capacity, topk;
  int num_splits, page_size, pt_stride, gi_stride, win_stride, n_tiles;
  float scale_log2, softmax_thr, gate_thr;
  const float* qkv_scale;  // optional device fp32 [3]
  const int* thr_sk;       // optional [B]: key count that normalises the softmax threshold (a shard passes the whole length)
  long long op_ss, lp_ss;  // elements between the partials of consecutive splits
  float* gate_ws;          // gated, optional: float2 (max, min) of delta per (sequence, KV head, 16-key tile)
  const int* gather_count; // optional [B]: leading entries of a row of gather_idx that can be valid
  const int* key_bounds;   // optional [B, 2]: gathered positions outside [lo, hi) are masked, others shifted by -lo
  // peer exchange (optional): partials go to the receive buffer of every rank, arrivals are counted there
  unsigned char* peer_base[16];
  long long peer_block_floats;
  int peer_world, peer_rank;
  int D;  // real head size (<= the kernel's HD)
  unsigned flags;
};

// Gated forward workspace: float2 (max, min) of alpha per (batch, grid head, 128-row query tile), then float2
// (max, min) of delta per (batch, KV head, 128-key tile). Rows / keys past a sequence count as 0, like the
// reference's masked loads (scheduler.py:1658-1691).
inline size_t gate_ws_alpha_floats(int B, int hgrid, int num_m_blocks) { return 2 * (size_t)B * hgrid * num_m_blocks; }
inline size_t gate_ws_bytes(int B, int hgrid, int num_m_blocks, int Hkv, int n_tiles_k) {
  return sizeof(float) * (gate_ws_alpha_floats(B, hgrid, num_m_blocks) + 2 * (size_t)B * Hkv * n_tiles_k);
}

// Opt a kernel in to `smem` bytes of dynamic shared memory on the CURRENT device. The attribute is per device, so
// the caller keeps one bit per device ordinal (`done`, one word per kernel instantiation); setting it twice is
// harmless, which makes a race between host threads benign. Devices beyond 63 set it on every launch.
template <typename Kernel>
inline cudaError_t smem_opt_in(Kernel kern, int smem, std::atomic<unsigned long long>& done) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const unsigned long long bit = dev < 64 ? (1ull << dev) : 0ull;
  if (bit && (done.load(std::memory_order_acquire) & bit)) return cudaSuccess;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e == cudaSuccess && bit) done.fetch_or(bit, std::memory_order_release);
  return e;
}

// Multiprocessor count of the current device (148 on B200), cached per device ordinal.
inline int device_sm_count() {
  static std::atomic<int> cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev < 64) {
    const int c = cache[dev].load(std::memory_order_relaxed);
    if (c > 0) return c;
  }
  int sms = 148;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms = 148;
  if (dev < 64) cache[dev].store(sms, std::memory_order_relaxed);
  return sms;
}

}  // namespace fsa
