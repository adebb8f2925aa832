// Parameter blocks and launchers of the helper kernels (internal).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "fsa_params.h"

namespace fsa {

// out_partial [num_splits, rows, heads, head_dim] fp32 (contiguous), lse_partial addressed as
// split*lp_ss + head*lp_sh + row (base-2 log-sum-exp). `rows` = batch*seqlen (or packed total);
// rows_per_batch splits a row index into (batch, position) for the strided final tensors.
struct CombineParams {
  const float* out_partial;
  const float* lse_partial;
  void* out;
  float* lse;
  long long op_ss, lp_ss, lp_sh;
  long long o_sb, o_sm, o_sh;
  long long l_sb, l_sh;
  int rows, rows_per_batch, heads, head_dim, num_splits;
  // Peer exchange (context-parallel decode): when `peer_flags` is set the partials were stored by other GPUs. Every
  // CTA first waits (bounded) until flag r of every rank r has reached step * arrivals_per_step, `step` being the
  // count of exchanges this rank has sent; the partials are read from buffer (step - 1) & 1, `buf_stride` floats apart.
  const unsigned long long* peer_flags;
  const unsigned long long* peer_step;
  int* status;
  long long buf_stride;
  int peer_world, arrivals_per_step;
};

// Backward pre-pass over every (query row, head): dpsum = sum_d O*dO, lse2 = lse * log2(e) (NaN -> 1e6,
// clamped at -1e6), both written NEGATED at tile-padded row positions.
struct BwdPreParams {
  const void* out;
  const void* dout;
  const float* lse;
  float* lse2_ws;
  float* dpsum_ws;
  const int* cu_q;
  float* dq_accum;    // optional: [heads, ws_sh, head_dim_pad] fp32, the rows of real queries are cleared here
  const void* alpha;  // optional (gated): T [B, heads, sq] | [heads, total_q]
  void* alpha_ws;     // optional (gated): T [heads, ws_sh], pre-zeroed; receives alpha at the padded rows
  long long a_sb, a_sh;
  long long o_sb, o_sm, o_sh, do_sb, do_sm, do_sh, l_sb, l_sh, ws_sh;
  int B, sq, total_q, heads, head_dim, varlen;
  int head_dim_pad;  // 64 or 128: lanes per row = head_dim_pad / 8
};
// Backward post-pass: dq = dq_accum * scale in the 16-bit type (and dalpha = da_accum * scale when given,
// flash_sparse_attn/ops/triton/flash_bwd_postprocess.py:106-148).
struct BwdPostParams {
  const float* dq_accum;  // [Hq, ws_sh, D]
  void* dq;
  const int* cu_q;
  const float* da_accum;  // optional [Hq, ws_sh]
  void* da;               // optional T, laid out like alpha
  long long da_sb, da_sh;
  long long dq_sb, dq_sm, dq_sh, ws_sh;
  int B, sq, total_q, heads, head_dim, varlen;
  int head_dim_pad;  // row pitch of dq_accum (64 or 128)
  float scale;
};
// Sum of per-split fp32 partials [splits, n] into a strided 16-bit tensor of rows x heads x head_dim.
struct SplitSumParams {
  const float* partial;
  void* out;
  long long part_ss;  // elements between splits
  long long o_sb, o_sn, o_sh;
  int rows, rows_per_batch, heads, head_dim, num_splits;
};

// out[i] = sum over splits of partial[split * part_ss + i] for i < n, in split order (16-bit out).
struct FlatSumParams {
  const float* partial;
  void* out;
  long long part_ss, n;
  int num_splits;
};

// Deterministic dQ: for every (batch, KV head, query tile) number the key tiles that visit it, highest
// key tile first; the main kernel adds its dQ tiles in that order.
struct DqOrderParams {
  unsigned short* order;  // [B, Hkv, n_tiles_k, num_m_blocks]
  const int* cu_q;
  const int* cu_k;
  const int* used_q;
  const int* used_k;
  const int* windows;
  int B, Hkv, sq, sk, num_splits, n_tiles_k, num_m_blocks, win_stride;
  unsigned flags;  // F_CAUSAL | F_LOCAL | F_SPLIT | F_VARLEN_* | F_USED_*
};
// Gated forward: per-tile extremes of alpha and delta (layout: gate_ws_bytes in fsa_params.h). The kernels derive
// every gate-skip decision from these, before a key tile is loaded (activations.py:265-299 needs nothing else).
struct GateExtParams {
  const void* alpha;  // T [B, Hq, Sq] | [Hq, Tq], position-contiguous
  const void* delta;  // T [B, Hkv, Sk] | [Hkv, Tk] | paged [pages, Hkv, page]
  float* gate_ws;
  const int* cu_q;
  const int* cu_k;
  const int* used_q;
  const int* used_k;
  const int* page_table;
  long long a_sb, a_sh, d_sb, d_sh;
  int B, Hq, Hkv, G, gpack, hgrid, sq, sk, num_m_blocks, n_tiles_k, page_size, pt_stride;
  unsigned flags;  // F_VARLEN_* | F_USED_* | F_PAGED
};
cudaError_t launch_gate_ext(const GateExtParams& p, int dtype, cudaStream_t stream);
cudaError_t launch_dq_order(const DqOrderParams& p, cudaStream_t stream);
cudaError_t launch_flat_sum(const FlatSumParams& p, int dtype, cudaStream_t stream);
cudaError_t launch_bwd_pre(const BwdPreParams& p, int dtype, cudaStream_t stream);
cudaError_t launch_bwd_post(const BwdPostParams& p, int dtype, cudaStream_t stream);
cudaError_t launch_split_sum(const SplitSumParams& p, int dtype, cudaStream_t stream);
cudaError_t launch_bwd(const BwdKernelParams& p, int kind, int dtype, int head_dim, cudaStream_t stream);
cudaError_t launch_dec(const DecKernelParams& p, int kind, int dtype, int head_dim, cudaStream_t stream);
cudaError_t launch_combine(const CombineParams& p, int dtype, cudaStream_t stream);
cudaError_t launch_fwd(const FwdKernelParams& p, int kind, int dtype, int head_dim, cudaStream_t stream);

}  // namespace fsa
