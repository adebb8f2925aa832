/*
 * C ABI of libfsa_b200.so - sm_100a attention kernels behind the flash-sparse-attention operator API.
 *
 * Every entry point takes plain device pointers, sizes and element strides; it never allocates,
 * frees or keeps a pointer past its return, never synchronises the host with the device and launches
 * on the CUDA stream handed in (a cudaStream_t passed as void*), so a call sequence can be captured
 * into a CUDA graph by the caller. All workspaces are caller-owned; the fsa_*_workspace_bytes functions
 * say how large each has to be. The library keeps no per-call state: the only process-wide data are caches of
 * per-device facts (multiprocessor count, which kernels were opted in to large shared memory, the driver entry
 * point for tensor maps), all safe to race on. Return value: 0 on success, a negative FSA_ERR_* code otherwise
 * (fsa_status_string() names it); nothing throws or aborts.
 *
 * Device-side trouble: every kernel wait is bounded; a kernel that gives up sets the caller's `status` word
 * (non-zero) and drains. The word is STICKY: kernels launched while it is non-zero return at once without
 * writing their outputs, so a caller must read it (after synchronising) before trusting results, and zero it to
 * go on.
 *
 * ev_before / ev_after (optional, may be null): cudaEvent_t handles recorded on the launch stream right before
 * and right after the call's MAIN kernel, so that a benchmark can time that kernel inside a full step without a
 * profiler (the reference's benchmarks time whole operator calls, tests/benchmark_forward.py:114).
 *
 * Each function states which host launcher of the reference Python package it stands in for
 * (paths relative to the reference repository root).
 */
#ifndef FSA_B200_H_
#define FSA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FSA_ABI_VERSION 2

enum {
  FSA_OK = 0,
  FSA_ERR_INVALID_ARG = -1, /* null pointer, bad size, misaligned stride */
  FSA_ERR_UNSUPPORTED = -2, /* valid request outside what the kernels implement */
  FSA_ERR_LAUNCH = -3,      /* CUDA reported an error at launch / descriptor creation */
  FSA_ERR_NO_DRIVER = -4,   /* cuTensorMapEncodeTiled could not be resolved (no CUDA driver) */
  FSA_ERR_SCRATCH_TOO_SMALL = -5, /* fsa_decode_static_scratch: the partials exceed the built-in workspace */
  FSA_ERR_SCRATCH_UNAVAILABLE = -6 /* fsa_decode_static_scratch: the built-in workspace could not be set up on this
                                      device (its first use loads it; a device with no free memory refuses) */
};

enum { FSA_KIND_DENSE = 0, FSA_KIND_SPARSE = 1, FSA_KIND_GATED = 2 };
enum { FSA_DT_BF16 = 0, FSA_DT_FP16 = 1, FSA_DT_E4M3 = 2, FSA_DT_E5M2 = 3, FSA_DT_F32 = 4 };

/* flags shared by the argument blocks */
enum {
  FSA_F_CAUSAL = 1u << 0,
  FSA_F_LOCAL = 1u << 1,
  FSA_F_SPLIT = 1u << 2,      /* split-KV (forward, decode) / split-QO (backward) */
  FSA_F_PACK_GQA = 1u << 3,   /* rows of one query tile interleave the G heads of a KV head */
  FSA_F_LOGSIGMOID = 1u << 4, /* gated: gate = logsigmoid(alpha*delta), else alpha*delta */
  FSA_F_ADAPT_GATE = 1u << 5,
  FSA_F_DETERMINISTIC = 1u << 6 /* backward: add the dQ tiles of the key tiles in a fixed order */
};

/*
 * Forward pass. Stands in for _flash_{dense,sparse,gated}_attn_forward and their varlen twins
 * (flash_sparse_attn/ops/triton/flash_sparse_fwd.py:520-758 and :761-988, flash_dense_fwd.py,
 * flash_gated_fwd.py) including the split-KV combine (flash_fwd_combine.py:164-232).
 *
 * Layouts (element strides, innermost head_dim stride must be 1):
 *   q   [batch, seqlen_q, heads_q, head_dim]            or packed [total_q, heads_q, head_dim]
 *   k,v [batch, seqlen_k, heads_kv, head_dim]           or packed [total_k, heads_kv, head_dim]
 *                                                       or paged  [num_pages, page_size, heads_kv, head_dim]
 *   out like q; lse [batch, heads_q, seqlen_q] fp32     or packed [heads_q, total_q]
 *   out_partial [num_splits, rows, heads_q, head_dim] fp32, lse_partial [num_splits, heads_q, rows] fp32
 *     with rows = batch*seqlen_q (or total_q); only read/written when FSA_F_SPLIT is set.
 *   window_sizes int32 [heads_kv, 4] = (sink, left, right, near) as in
 *     flash_sparse_attn/ops/triton/scheduler.py:56-61.
 * Packed (varlen) mode is selected by cu_seqlens_q / cu_seqlens_k being non-null; paged mode by
 * page_table being non-null.
 */
typedef struct FsaFwdArgs {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  float* lse;
  float* out_partial;
  float* lse_partial;
  const void* alpha; /* gated: [batch, heads_q, seqlen_q] (or [heads_q, total_q]), dtype of q */
  const void* delta; /* gated: [batch, heads_kv, seqlen_k] (or [heads_kv, total_k]) */
  const int32_t* cu_seqlens_q; /* [batch + 1] */
  const int32_t* cu_seqlens_k;
  const int32_t* seqused_q; /* [batch] */
  const int32_t* seqused_k;
  const int32_t* page_table;   /* [batch, page_table_stride] */
  const int32_t* window_sizes; /* [heads_kv, window_stride] */
  int32_t* status;             /* device word, zeroed by the caller once; set non-zero when a kernel gave up */
  uint8_t* tile_map;           /* optional debug output, see fsa_fwd_tile_map_bytes(); may be null */
  int64_t q_stride_b, q_stride_s, q_stride_h;
  int64_t k_stride_b, k_stride_s, k_stride_h; /* paged: _b = page stride */
  int64_t v_stride_b, v_stride_s, v_stride_h;
  int64_t o_stride_b, o_stride_s, o_stride_h;
  int64_t lse_stride_b, lse_stride_h;
  int64_t alpha_stride_b, alpha_stride_h; /* gated: alpha[b, h, position] (position stride 1) */
  int64_t delta_stride_b, delta_stride_h; /* gated: delta[b, h_kv, position]; paged: delta[page, h_kv, row] */
  int32_t batch, seqlen_q, seqlen_k; /* varlen: max_seqlen_q / max_seqlen_k */
  int32_t total_q, total_k;          /* varlen: rows of the packed tensors */
  int32_t heads_q, heads_kv, head_dim;
  int32_t num_pages, page_size, page_table_stride, window_stride;
  int32_t num_splits;
  int32_t tile_m, tile_n; /* 0 = default (128, 128) */
  int32_t kind, dtype;
  uint32_t flags;
  float softmax_scale, softmax_threshold, gate_threshold;
  /* optional: three fp32 values on the device, the per-tensor de-quantisation scales of q, k, v
   * (scheduler.py:298-307: logits scale *= q_scale * k_scale; out *= v_scale). Null = all 1.
   * With dtype FSA_DT_E4M3 / FSA_DT_E5M2 (head_dim 128) q, k, v are FP8, both GEMMs run as
   * tcgen05 kind::f8f6f4 with P rounded to the same FP8 format, out / alpha / delta are bf16. */
  const float* qkv_scale;
  /* gated kind: workspace of fsa_fwd_workspace_bytes().gate_ws bytes (written by this call): per-tile extremes
   * of alpha and delta, from which every role of the kernel derives the gate-skip decisions before a key tile
   * is loaded. */
  float* gate_ws;
  /* Block-scaled FP8 inputs (dtype FSA_DT_E4M3 / FSA_DT_E5M2, head_dim 128, dense and sparse kinds, no packed
   * GQA): fp32 scales per 128-position block, as fsa_quantize_fp8_blockwise writes them -
   * q_block_scale [batch, heads_q, ceil(seqlen_q / 128)], k_block_scale / v_block_scale [batch, heads_kv,
   * ceil(seqlen_k / 128)] (blocks counted from the start of each sequence, i.e. the kernel's own tiles). All
   * three or none; with them qkv_scale must be null. logits = (Q8 K8^T) * q_scale[m] * k_scale[n] *
   * softmax_scale per tile; P is multiplied by v_scale[n] / v_run before it is rounded to FP8, v_run being the
   * largest value scale the query tile has met so far (the accumulator is rescaled when it grows), and the
   * output by the final v_run. Not in the reference, whose quantisation is per tensor
   * (flash_sparse_attn/ops/triton/quant.py:42-64). */
  const float* q_block_scale;
  const float* k_block_scale;
  const float* v_block_scale;
  void* ev_before;
  void* ev_after;
} FsaFwdArgs;

int fsa_fwd(const FsaFwdArgs* args, void* stream);

/* Bytes of the optional per-tile debug map for these arguments: one byte per
 * (batch, grid head, 128-row query tile, split, 128-key tile): 0 = not visited, 1 = computed,
 * 2 = skipped by the softmax threshold, 3 = skipped by the gate bound. */
size_t fsa_fwd_tile_map_bytes(const FsaFwdArgs* args);

/*
 * Backward pass. Stands in for _flash_{dense,sparse}_attn_backward and the varlen twins
 * (flash_sparse_attn/ops/triton/flash_sparse_bwd.py:491-748 and :751-1026) including the pre-process
 * (flash_bwd_preprocess.py:198-266), the post-process (flash_bwd_postprocess.py:151-213) and the
 * reduction over QO splits (flash_sparse_bwd.py:741-746).
 *
 * q/k/v/out/dout/dq/dk/dv use the forward layouts (dout, dq like q; dk, dv like k). lse is the forward
 * output (natural log). Caller-owned fp32 workspaces, all sized with R = fsa_bwd_padded_rows():
 *   lse2_ws  [heads_q, R]            dpsum_ws [heads_q, R]
 *   dq_accum [heads_q, R, head_dim rounded up to 64 or 128]  (zeroed by this call)
 *   dk_partial, dv_partial [num_splits, rows_k, heads_kv, head_dim] only when FSA_F_SPLIT and
 *   num_splits > 1 (rows_k = batch*seqlen_k or total_k); otherwise null.
 * dq is accumulated with TMA reduce-adds in fp32 (summation order across key tiles is not fixed,
 * like the reference's atomics); dk and dv are reduced inside one CTA per key tile in a fixed order.
 * FSA_KIND_GATED additionally returns dalpha (fp32 atomics into da_accum, then scaled and rounded) and
 * ddelta (reduced inside the CTA over the query heads of the group, fixed order); flags
 * FSA_F_LOGSIGMOID / FSA_F_ADAPT_GATE as in the forward.
 */
typedef struct FsaBwdArgs {
  const void* q;
  const void* k;
  const void* v;
  const void* out;
  const void* dout;
  const float* lse;
  void* dq;
  void* dk;
  void* dv;
  float* lse2_ws;
  float* dpsum_ws;
  float* dq_accum;
  float* dk_partial;
  float* dv_partial;
  const int32_t* cu_seqlens_q;
  const int32_t* cu_seqlens_k;
  const int32_t* seqused_q;
  const int32_t* seqused_k;
  const int32_t* window_sizes;
  int32_t* status;
  uint8_t* tile_map; /* optional [batch, heads_q, key tiles, splits, query tiles]; may be null */
  int64_t q_stride_b, q_stride_s, q_stride_h;
  int64_t k_stride_b, k_stride_s, k_stride_h;
  int64_t v_stride_b, v_stride_s, v_stride_h;
  int64_t o_stride_b, o_stride_s, o_stride_h;
  int64_t do_stride_b, do_stride_s, do_stride_h;
  int64_t dq_stride_b, dq_stride_s, dq_stride_h;
  int64_t dk_stride_b, dk_stride_s, dk_stride_h; /* dv must share dk's strides */
  int64_t lse_stride_b, lse_stride_h;
  int32_t batch, seqlen_q, seqlen_k;
  int32_t total_q, total_k;
  int32_t heads_q, heads_kv, head_dim;
  int32_t window_stride;
  int32_t num_splits;
  int32_t tile_m, tile_n; /* 0 = default (128, 128) */
  int32_t kind, dtype;
  uint32_t flags;
  float softmax_scale, softmax_threshold, gate_threshold;
  /* gated kind only (flash_sparse_attn/ops/triton/flash_gated_bwd.py:682-981); null otherwise */
  const void* alpha;  /* [batch, heads_q, seqlen_q] | packed [heads_q, total_q]; 16-bit like q */
  const void* delta;  /* [batch, heads_kv, seqlen_k] | packed [heads_kv, total_k]; position stride 1 */
  void* dalpha;       /* laid out like alpha */
  void* ddelta;       /* laid out like delta */
  void* alpha_ws;     /* workspace, 16-bit [heads_q, R] (zeroed by this call) */
  float* da_accum;    /* workspace, fp32 [heads_q, R] (zeroed by this call) */
  float* dd_partial;  /* [num_splits, numel(delta)] fp32, only when FSA_F_SPLIT and num_splits > 1 */
  int64_t alpha_stride_b, alpha_stride_h;
  int64_t delta_stride_b, delta_stride_h;
  int64_t delta_numel; /* elements of delta / ddelta (contiguous) */
  /* FSA_F_DETERMINISTIC only: workspaces (both written by this call)
   *   dq_order uint16 [batch, heads_kv, ceil(seqlen_k/128), ceil(seqlen_q/128)]
   *   dq_turn  int32  [batch, heads_q, ceil(seqlen_q/128)]
   * dQ then no longer depends on the order in which CTAs happen to run: every key tile waits (bounded) for
   * the key tiles above it before its reduce-add into a query tile; results are bitwise reproducible. */
  uint16_t* dq_order;
  int32_t* dq_turn;
  /* gated kind: workspace of fsa_bwd_workspace_bytes().gate_ws bytes (written by this call): per-tile extremes of
   * alpha and delta, from which every role of the kernel takes the gate-skip decisions before a query tile is
   * loaded. */
  float* gate_ws;
  void* ev_before;
  void* ev_after;
} FsaBwdArgs;

int fsa_bwd(const FsaBwdArgs* args, void* stream);

/* Rows of the tile-padded backward workspaces: every sequence starts on a multiple of 128 rows
 * (batch*ceil128(seqlen_q), or ceil128(total_q + 128*batch) for packed input). Host arithmetic. */
int64_t fsa_bwd_padded_rows(int batch, int seqlen_q, int total_q, int is_varlen);

/*
 * Decode: one query position per sequence against a KV cache. Stands in for
 * _flash_{dense,sparse}_attn_decode and the varlen twins
 * (flash_sparse_attn/ops/triton/flash_sparse_dec.py:519-744, :747-952) including the split combine
 * (flash_dec_combine.py:156-222).
 *   q [batch, heads_q, head_dim]; out like q; lse [batch, heads_q] fp32
 *   k, v: [batch, seqlen_k, heads_kv, head_dim] | packed [total_k, heads_kv, head_dim] + cu_seqlens_k |
 *         paged [num_pages, page_size, heads_kv, head_dim] + page_table [batch, page_table_stride]
 *   gather_kv_indices int32 [batch, topk]: logical key positions to attend to, negative = masked; then
 *     neither windows nor sequence lengths apply (flash_sparse_dec.py:321-357). May be combined with a
 *     page table: the position is translated through it (not available in the reference,
 *     assert_inputs.py:303-305).
 *   out_partial [num_splits, batch, heads_q, head_dim], lse_partial [num_splits, heads_q, batch] fp32
 *     (base-2 lse): written when num_splits > 1 or when partial_only is set. With partial_only the
 *     call stops after the partials (no combine), for callers that merge partials of several
 *     devices themselves with fsa_combine.
 *   head_dim: a multiple of 8 up to 256 with 16-bit inputs (sizes above 128 run eight query heads of a KV head per
 *     pass over the keys), 128 with FP8 inputs. fsa_fwd takes the same sizes, fsa_bwd stops at 128.
 */
typedef struct FsaDecArgs {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  float* lse;
  float* out_partial;
  float* lse_partial;
  const int32_t* cu_seqlens_k;
  const int32_t* seqused_k;
  const int32_t* page_table;
  const int32_t* gather_kv_indices;
  const int32_t* window_sizes;
  const void* alpha; /* gated: [batch, heads_q], dtype of q */
  const void* delta; /* gated: [batch, heads_kv, seqlen_k] | [heads_kv, total_k] | paged [num_pages, heads_kv, page_size] */
  int32_t* status;
  uint8_t* tile_map; /* optional [batch, heads_kv, 16-key tiles]; may be null */
  int64_t q_stride_b, q_stride_h;
  int64_t k_stride_b, k_stride_s, k_stride_h; /* v must share k's strides */
  int64_t o_stride_b, o_stride_h;
  int64_t lse_stride_b, lse_stride_h;
  int64_t alpha_stride_b, alpha_stride_h;
  int64_t delta_stride_b, delta_stride_h;
  int32_t batch, seqlen_k, total_k;
  int32_t heads_q, heads_kv, head_dim;
  int32_t topk, gather_stride;
  int32_t num_pages, page_size, page_table_stride, window_stride;
  int32_t num_splits;
  int32_t partial_only;
  int32_t kind, dtype;
  uint32_t flags;
  float softmax_scale, softmax_threshold, gate_threshold;
  const float* qkv_scale; /* optional, as in FsaFwdArgs */
  /* Decoding one shard of a longer key sequence (KV-sequence context parallelism); all optional.
   *   thr_seqlen_k [batch]: key count that normalises the softmax threshold (threshold / count,
   *     seqlen_info.py:141-149) and the default gate threshold; null = the count this call sees. A shard passes
   *     the length of the whole sequence so that its skip decisions use the same bound as an unsharded call.
   *   key_bounds [batch, 2] = (lo, hi) per sequence: with gather_kv_indices, positions outside [lo, hi) are
   *     treated as masked (-1) and the others address the cache at position - lo; null switches this off. */
  const int32_t* thr_seqlen_k;
  const int32_t* key_bounds;
  /* gather_count [batch] (optional): only the first gather_count[b] entries of row b of gather_kv_indices can be
   * valid (the rest are -1), so the kernel visits only the 16-key tiles that hold them: what
   * fsa_localize_indices produces for one shard of a sharded cache. */
  const int32_t* gather_count;
  /* Elements between the partials of consecutive splits in out_partial / lse_partial; 0 = dense
   * (batch*heads_q*head_dim and heads_q*batch). A caller that wants partial outputs and log-sum-exps of one
   * split side by side in ONE buffer (to ship them with a single all-gather) sets both to
   * batch*heads_q*(head_dim + 1) and points lse_partial at out_partial + batch*heads_q*head_dim. */
  int64_t out_partial_stride, lse_partial_stride;
  /* gated kind, optional: workspace of fsa_decode_workspace_bytes().gate_ws bytes (written by this call) with the
   * extremes of delta per 16-key tile; with it the gate-skip decision of a tile is taken before its rows are
   * requested, without it when the tile is consumed. */
  float* gate_ws;
  void* ev_before;
  void* ev_after;
  /* Optional, with partial_only and the packed partial layout (both strides = batch*heads_q*(head_dim + 1)): the
   * peer regions of a context-parallel group (struct FsaPeerArgs below). The kernel then stores its partials
   * straight into the receive buffer of EVERY rank instead of out_partial and counts its CTAs' arrivals there, so
   * the step is fsa_decode -> fsa_peer_combine with arrivals_per_step = batch * heads_kv * num_splits and no
   * fsa_peer_push. block_floats must equal num_splits * batch*heads_q*(head_dim + 1). */
  const struct FsaPeerArgs_* peers;
} FsaDecArgs;

int fsa_decode(const FsaDecArgs* args, void* stream);

/*
 * Merge `num_partials` partial attention results (base-2 log-sum-exp weights) into the final output:
 * the combine step of flash_sparse_attn/ops/triton/flash_dec_combine.py:15-153 /
 * flash_fwd_combine.py:15-161, exposed so that partials gathered from several devices (KV-sequence
 * context parallelism) can be merged with the same arithmetic.
 *   out_partial [num_partials, rows, heads, head_dim] fp32, lse_partial [num_partials, heads, rows] fp32
 *   out [rows, heads, head_dim] (contiguous, dtype), lse [rows, heads] fp32 natural log
 *   out_partial_stride / lse_partial_stride: elements between consecutive partials, 0 = dense (see FsaDecArgs)
 */
int fsa_combine(const float* out_partial, const float* lse_partial, void* out, float* lse, int num_partials,
                int rows, int heads, int head_dim, int dtype, int64_t out_partial_stride,
                int64_t lse_partial_stride, void* stream);

/*
 * Split-KV decode without any caller-provided (or freshly allocated) workspace. This entry point has
 * no counterpart in the reference, whose launcher allocates its partial buffers with torch.empty on
 * every call (flash_sparse_attn/ops/triton/flash_sparse_dec.py:637-646).
 *
 * It is fsa_decode with the split workspace taken from a fixed array of FSA_STATIC_SCRATCH_BYTES that
 * is part of the library image: meant for callers that cannot obtain device memory at
 * call time (all memory already owned by a serving pool, a frozen memory plan, no tolerance for the
 * implicit synchronisation of cudaMalloc / cudaFree). args->out_partial / lse_partial are ignored and
 * partial_only must be 0; everything else means what it means for fsa_decode.
 *   - num_splits * batch * heads_q * (head_dim + 1) floats must fit in the array, otherwise the call
 *     returns FSA_ERR_SCRATCH_TOO_SMALL and launches nothing.
 *   - The array is shared by all calls and keeps the previous call's contents; the kernels overwrite
 *     every slot they later read, so nothing has to be cleared. Calls that may run concurrently on
 *     one GPU race on it: order them.
 *   - The first call on each device resolves the array's address with cudaGetSymbolAddress. Under CUDA's lazy
 *     module loading that look-up is also what makes the array resident on the device: it takes the 16 MiB
 *     from the device's free memory and synchronises implicitly (FSA_ERR_SCRATCH_UNAVAILABLE if the device
 *     cannot provide them). Make that first call at start-up, before a memory pool claims the rest of the GPU
 *     and before starting any stream capture. From then on a GPU holds the array until the process exits.
 * It calls no cudaMalloc, cudaFree or other allocating routine; after the first call per device it changes
 * neither the device's free memory nor the host-device synchronisation state.
 */
#define FSA_STATIC_SCRATCH_BYTES (16u * 1024u * 1024u)
int fsa_decode_static_scratch(const FsaDecArgs* args, void* stream);
size_t fsa_static_scratch_bytes(void);

/* Integer schedule of one forward query tile, for checking against the reference's
 * AttnFwdBlockScheduler.create (flash_sparse_attn/ops/triton/scheduler.py:836-948). out9 receives
 * n_min, n_max, n_max_no_mask, win_min, win_max, win_min_no_mask, win_max_no_mask, sink_min, sink_max.
 * is_split: bit 0 = split-KV; bit 1 = the decode kernel's variant, which for a single query position rounds
 * the start of the near-diagonal range down instead of up (the reference's rounding,
 * block_info.py:60-64, leaves the first partial tile of the near band unvisited).
 * Pure host arithmetic: callable without a GPU. */
void fsa_debug_fwd_schedule(int seqlen_q, int seqlen_k, int m_block, int split_idx, const int32_t window[4],
                            int num_splits, int tile_n, int tile_m, int is_causal, int is_local, int is_split,
                            int qhead_per_kvhead_packgqa, int32_t out9[9]);
/* Same for one backward key tile (AttnBwdBlockScheduler.create, scheduler.py:994-1101): m_min, m_max,
 * m_min_no_mask, win_min, win_max, win_min_no_mask, win_max_no_mask, sink_min, sink_max. */
void fsa_debug_bwd_schedule(int seqlen_q, int seqlen_k, int n_block, int split_idx, const int32_t window[4],
                            int num_splits, int tile_n, int tile_m, int is_causal, int is_local, int is_split,
                            int32_t out9[9]);

/*
 * Sizes in bytes of the caller-owned workspaces of one call (0 = not needed), from the dimensions, kind, dtype,
 * flags and num_splits of the argument block; pointers in it are not read. The reference's launchers derive the
 * same sizes inline (flash_sparse_fwd.py:637-660, flash_sparse_bwd.py:610-668, flash_sparse_dec.py:637-646).
 * Host arithmetic only.
 */
typedef struct FsaFwdWorkspace {
  size_t out_partial, lse_partial; /* split-KV partials */
  size_t gate_ws;                  /* gated kind */
} FsaFwdWorkspace;
typedef struct FsaBwdWorkspace {
  size_t lse2_ws, dpsum_ws, dq_accum;
  size_t dk_partial, dv_partial; /* split-QO */
  size_t alpha_ws, da_accum, dd_partial, gate_ws; /* gated kind */
  size_t dq_order, dq_turn;      /* FSA_F_DETERMINISTIC */
} FsaBwdWorkspace;
typedef struct FsaDecWorkspace {
  size_t out_partial, lse_partial;
  size_t gate_ws; /* gated kind */
} FsaDecWorkspace;
int fsa_fwd_workspace_bytes(const FsaFwdArgs* args, FsaFwdWorkspace* sizes);
int fsa_bwd_workspace_bytes(const FsaBwdArgs* args, FsaBwdWorkspace* sizes);
int fsa_decode_workspace_bytes(const FsaDecArgs* args, FsaDecWorkspace* sizes);

const char* fsa_status_string(int code);
/*
 * Per-tensor FP8 quantisation, the contract of flash_sparse_attn/ops/triton/quant.py:42-64:
 * scale = FP8_MAX / max|x|, x_fp8 = rne(x * scale), *scale_out = max|x| / FP8_MAX in x's type
 * (FSA_DT_E5M2: 57344, FSA_DT_E4M3: 448). x: n contiguous elements of x_dtype (bf16 / fp16 / fp32,
 * 16-byte aligned); amax_ws: caller-owned 4-byte device workspace (zeroed by this call). Two kernels,
 * no host synchronisation.
 */
int fsa_quantize_fp8(const void* x, void* x_fp8, void* scale_out, float* amax_ws, int64_t n, int x_dtype,
                     int fp8_dtype, void* stream);

/*
 * Block-scaled FP8 quantisation of a [batch, seqlen, heads, head_dim] tensor (or packed [total, heads, head_dim] with
 * cu_seqlens; seqlen is then the longest sequence): for every (sequence, head, block of 128 consecutive positions
 * counted from the start of the sequence) scale = max|x| / FP8_MAX (0 for an all-zero block), x8 = rne(x / scale),
 * scales[batch, heads, ceil(seqlen / 128)] fp32. With `dequantize` set the call runs the other way round:
 * x16 = x8 * scale (what the backward pass runs on). head_dim a multiple of 8 up to 128; strides in elements.
 * Not in the reference (per-tensor scales only, quant.py:42-64): an internal format with its own error bound.
 */
typedef struct FsaBlockQuantArgs {
  void* x16;      /* bf16 / fp16: input of the quantisation, output of the de-quantisation */
  void* x8;       /* FP8: output / input */
  float* scales;  /* [batch, heads, ceil(seqlen / 128)] */
  const int32_t* cu_seqlens; /* [batch + 1] or null */
  int64_t x_stride_b, x_stride_s, x_stride_h;
  int64_t q_stride_b, q_stride_s, q_stride_h;
  int32_t batch, seqlen, heads, head_dim;
  int32_t x_dtype, fp8_dtype;
  int32_t dequantize;
} FsaBlockQuantArgs;
int fsa_quantize_fp8_blockwise(const FsaBlockQuantArgs* args, void* stream);

/*
 * out[i] = (out_dtype)(float(x_fp8[i]) * *scale), scale optional (one element of out_dtype on the
 * device; null = 1). The load-time de-quantisation of scheduler.py:2133-2148 as one pass; with a null
 * scale the widening is exact. Both pointers 16-byte aligned.
 */
int fsa_fp8_widen(const void* x_fp8, void* out, const void* scale, int64_t n, int fp8_dtype, int out_dtype,
                  void* stream);

/*
 * Top-k position selection in front of the gathered decode: for every row of `scores`
 * [rows, n] (bf16 / fp16 / fp32, `row_stride` elements between rows) the positions of the k largest
 * entries in ascending order, int32 or int64 [rows, k]. Same contract as
 * flash_sparse_attn/utils/mask.py:20-44 (torch.topk + sort of the indices); among equal scores at the
 * threshold the lowest positions are taken, NaN orders above +inf. One CTA per row: four-pass radix
 * select, then an ordered compaction (no sort).
 */
int fsa_topk_indices(const void* scores, int dtype, int rows, int n, int64_t row_stride, int k, void* out,
                     int out_is_int64, void* stream);

/*
 * KV-cache append: k_new / v_new [batch, new_tokens, heads_kv, head_dim] go to positions seqused_k[b] ..
 * seqused_k[b] + new_tokens of the cache, then seqused_k[b] advances by new_tokens; no host round trip, two
 * small kernels. The cache is contiguous [batch, capacity, heads_kv, head_dim] or, with page_table, paged
 * [num_pages, page_size, heads_kv, head_dim] - the layouts the decode entry points read. Paged: a page-table slot
 * that holds a negative number has no page yet; the call pops one from `free_pages` (a stack of free page
 * numbers whose height is the device counter *free_count). Rows that find no room (capacity exceeded, page table
 * full, free stack empty) are dropped and the status word is set to 3.
 * No counterpart in the reference, which leaves cache management to the caller (its README lists a KV-cache
 * manager as future work); the layout is the one its decode reads (flash_sparse_attn/ops/triton/paged_kv.py:10-30).
 * All strides in elements; rows move in 16-byte chunks (head_dim * element size and all strides multiples of 16
 * bytes). pos_ws: caller-owned int32 [batch] workspace.
 */
typedef struct FsaKvAppendArgs {
  const void* k_new;
  const void* v_new;
  void* k_cache;
  void* v_cache;
  int32_t* seqused_k;  /* [batch] */
  int32_t* page_table; /* [batch, page_table_stride] or null */
  int32_t* free_pages; /* optional */
  int32_t* free_count; /* optional */
  int32_t* pos_ws;
  int32_t* status;
  int64_t new_stride_b, new_stride_s, new_stride_h;
  int64_t cache_stride_b, cache_stride_s, cache_stride_h; /* paged: _b = page stride; v_cache shares them */
  int32_t batch, new_tokens, heads_kv, head_dim;
  int32_t capacity; /* contiguous cache: positions per sequence */
  int32_t page_size, page_table_stride;
  int32_t dtype;
} FsaKvAppendArgs;
int fsa_kv_append(const FsaKvAppendArgs* args, void* stream);

/* ---- Peer exchange of decode partials (context-parallel decode over the GPUs of one node) -------------------
 * No counterpart in the reference (it has no multi-GPU code). Every rank owns one region (fsa_peer_alloc: cudaMalloc,
 * so that it can be exported), opens the regions of the others (fsa_peer_open on their handles) and then, per step:
 * fsa_decode with partial_only writes this rank's partials in the packed form (out_partial_stride /
 * lse_partial_stride), fsa_peer_push stores that block into the receive buffer of EVERY rank (plain peer stores, no
 * multicast) and counts an arrival there, fsa_peer_combine waits until every rank's arrivals of the step are in and
 * merges world * partials_per_rank partials. The wait is bounded (about two seconds): on expiry the status word is
 * set to 4 and the kernel finishes with what it has. The step counter lives on the device, so a captured CUDA graph
 * of the three calls can be replayed. All ranks must run the same number of steps; the two receive buffers alternate. */
#define FSA_PEER_MAX_RANKS 16
typedef struct {
  unsigned char bytes[64];
} FsaIpcHandle;
typedef struct FsaPeerArgs_ {
  void* region[FSA_PEER_MAX_RANKS]; /* region of rank r as mapped in THIS process (own: from fsa_peer_alloc) */
  int world;
  int rank;
  int64_t block_floats; /* floats one rank sends per step: partials_per_rank * rows * heads * (head_dim + 1) */
} FsaPeerArgs;
int fsa_peer_region_bytes(int world, int64_t block_floats, int64_t* bytes);
int fsa_peer_alloc(int64_t bytes, void** region, FsaIpcHandle* handle); /* synchronises; call at set-up time */
int fsa_peer_open(const FsaIpcHandle* handle, void** region);           /* FSA_ERR_UNSUPPORTED if it cannot be mapped */
int fsa_peer_close(void* region);
int fsa_peer_free(void* region);
int fsa_peer_push(const FsaPeerArgs* args, const float* block, void* stream);
/* arrivals_per_step: how many arrivals a rank counts per step - 0 for fsa_peer_push (its own grid), the number of
 * decode CTAs (batch * heads_kv * num_splits) when fsa_decode stored the partials itself (FsaDecArgs.peers). */
int fsa_peer_combine(const FsaPeerArgs* args, void* out, float* lse, int partials_per_rank, int rows, int heads,
                     int head_dim, int dtype, int arrivals_per_step, int* status, void* stream);

/*
 * One shard's view of global top-k positions: for every row keep the positions inside [lo, hi) (key_bounds
 * [rows, 2]), shift them by -lo, move them to the front of the output row in their original order, fill the rest
 * with -1 and write how many were kept to count[row]. Feeds FsaDecArgs.gather_kv_indices / gather_count of a rank
 * that holds positions [lo, hi) of every sequence. No counterpart in the reference (it has no multi-GPU code).
 */
int fsa_localize_indices(const int32_t* indices, int64_t indices_stride, const int32_t* key_bounds, int32_t* out,
                         int64_t out_stride, int32_t* count, int rows, int topk, void* stream);

int fsa_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FSA_B200_H_ */
