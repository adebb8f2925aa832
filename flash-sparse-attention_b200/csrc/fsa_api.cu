// extern "C" boundary of libfsa_b200.so: argument validation, TMA descriptor construction, kernel
// selection. No torch types, no allocation, no host<->device synchronisation.
#include <cuda.h>
#include <cuda_runtime.h>
#include <string.h>
#include "../../include/fsa_b200.h"
#include "fsa_aux.h"
#include "fsa_params.h"
#include "fsa_schedule.h"

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
    (void)cudaGetLastError();
  }
  return fn;
}

CUtensorMapDataType tma_dtype(int dt) {
  switch (dt) {
    case FSA_DT_BF16: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    case FSA_DT_FP16: return CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    default: return CU_TENSOR_MAP_DATA_TYPE_UINT8;
  }
}
int dtype_bytes(int dt) { return (dt == FSA_DT_BF16 || dt == FSA_DT_FP16) ? 2 : (dt == FSA_DT_F32 ? 4 : 1); }

// 3-D map over the fp32 dQ accumulator [heads, rows, head_dim] with 32 x 32 boxes (one warp's share).
int make_map_dq(CUtensorMap* map, const float* base, uint64_t head_dim, uint64_t rows, uint64_t heads) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return FSA_ERR_NO_DRIVER;
  if (reinterpret_cast<uintptr_t>(base) & 15) return FSA_ERR_INVALID_ARG;
  cuuint64_t dims[3] = {head_dim, rows, heads};
  cuuint64_t strides[2] = {head_dim * 4, rows * head_dim * 4};
  cuuint32_t box[3] = {32, 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FSA_OK : FSA_ERR_LAUNCH;
}

// 4-D map over a [d3, d2, d1, head_dim] tensor (head_dim contiguous); strides in elements.
int make_map4(CUtensorMap* map, int dt, const void* base, uint64_t head_dim, uint64_t d1, int64_t s1, uint64_t d2,
              int64_t s2, uint64_t d3, int64_t s3, uint32_t box0, uint32_t box1, uint32_t box2) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return FSA_ERR_NO_DRIVER;
  const uint64_t es = dtype_bytes(dt);
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((s1 * es) & 15) || ((s2 * es) & 15) || ((s3 * es) & 15))
    return FSA_ERR_INVALID_ARG;
  if (d1 == 0 || d2 == 0 || d3 == 0) return FSA_ERR_INVALID_ARG;
  cuuint64_t dims[4] = {head_dim, d1, d2, d3};
  cuuint64_t strides[3] = {(cuuint64_t)s1 * es, (cuuint64_t)s2 * es, (cuuint64_t)s3 * es};
  cuuint32_t box[4] = {box0, box1, box2, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, tma_dtype(dt), 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FSA_OK : FSA_ERR_LAUNCH;
}

int cdiv(int a, int b) { return (a + b - 1) / b; }

// Head sizes that are a multiple of 8 up to 128 run on the 64- or 128-wide kernels: TMA fills the missing
// columns of every row with zeros (they add nothing to any dot product) and the epilogues do not write them.
bool head_dim_ok(int d) { return d >= 8 && d <= 128 && d % 8 == 0; }
int head_dim_kernel(int d) { return d <= 64 ? 64 : 128; }
// the forward and decode kernels also come 256 columns wide (16-bit inputs); the backward stops at 128
bool head_dim_ok_wide(int d) { return d >= 8 && d <= 256 && d % 8 == 0; }
int head_dim_kernel_wide(int d) { return d <= 64 ? 64 : (d <= 128 ? 128 : 256); }
// the forward also exists 192 columns wide (two stages of K fit there)
int head_dim_kernel_fwd(int d) { return d <= 128 ? head_dim_kernel_wide(d) : (d <= 192 ? 192 : 256); }

// optional per-call timing events around the main kernel
void mark(void* ev, cudaStream_t s) {
  if (ev) cudaEventRecord(reinterpret_cast<cudaEvent_t>(ev), s);
}

}  // namespace

extern "C" {

int fsa_abi_version(void) { return FSA_ABI_VERSION; }

const char* fsa_status_string(int code) {
  switch (code) {
    case FSA_OK: return "ok";
    case FSA_ERR_INVALID_ARG: return "invalid argument (null pointer, bad size, or stride/base not 16-byte aligned)";
    case FSA_ERR_UNSUPPORTED: return "unsupported combination (head_dim must be a multiple of 8 up to 128 - forward and decode with 16-bit inputs: up to 256 -, dtype bf16/fp16/fp8, ...)";
    case FSA_ERR_LAUNCH: return "CUDA error at launch or tensor-map creation";
    case FSA_ERR_NO_DRIVER: return "CUDA driver entry point cuTensorMapEncodeTiled unavailable";
    case FSA_ERR_SCRATCH_UNAVAILABLE:
      return "the built-in workspace could not be set up on this device (cudaGetSymbolAddress failed: its first "
             "use loads the array, which needs 16 MiB of free device memory)";
    case FSA_ERR_SCRATCH_TOO_SMALL:
      return "request does not fit the built-in workspace: num_splits * batch * heads_q * (head_dim + 1) floats "
             "must be at most 16 MiB";
    default: return "unknown status";
  }
}

void fsa_debug_fwd_schedule(int seqlen_q, int seqlen_k, int m_block, int split_idx, const int32_t window[4],
                            int num_splits, int tile_n, int tile_m, int is_causal, int is_local, int is_split,
                            int gpack, int32_t out9[9]) {
  FsaWindow w = {window[0], window[1], window[2], window[3]};
  // bit 1 of is_split selects the exact-cover variant used by the decode kernel
  FsaFwdSched s = fsa_fwd_schedule(seqlen_q, seqlen_k, m_block, split_idx, w, num_splits, tile_n, tile_m,
                                   is_causal != 0, is_local != 0, (is_split & 1) != 0, gpack, (is_split & 2) != 0);
  out9[0] = s.n_min;
  out9[1] = s.n_max;
  out9[2] = s.n_max_no_mask;
  out9[3] = s.win_min;
  out9[4] = s.win_max;
  out9[5] = s.win_min_no_mask;
  out9[6] = s.win_max_no_mask;
  out9[7] = s.sink_min;
  out9[8] = s.sink_max;
}

void fsa_debug_bwd_schedule(int seqlen_q, int seqlen_k, int n_block, int split_idx, const int32_t window[4],
                            int num_splits, int tile_n, int tile_m, int is_causal, int is_local, int is_split,
                            int32_t out9[9]) {
  FsaWindow w = {window[0], window[1], window[2], window[3]};
  FsaBwdSched s = fsa_bwd_schedule(seqlen_q, seqlen_k, n_block, split_idx, w, num_splits, tile_n, tile_m,
                                   is_causal != 0, is_local != 0, is_split != 0);
  out9[0] = s.m_min;
  out9[1] = s.m_max;
  out9[2] = s.m_min_no_mask;
  out9[3] = s.win_min;
  out9[4] = s.win_max;
  out9[5] = s.win_min_no_mask;
  out9[6] = s.win_max_no_mask;
  out9[7] = s.sink_min;
  out9[8] = s.sink_max;
}

static int fwd_geometry(const FsaFwdArgs* a, int* gpack, int* num_m_blocks, int* hgrid, int* sk_static,
                        int* n_tiles_k) {
  if (a->heads_kv <= 0 || a->heads_q % a->heads_kv != 0) return FSA_ERR_INVALID_ARG;
  const int G = a->heads_q / a->heads_kv;
  const bool pack = (a->flags & FSA_F_PACK_GQA) && G > 1;
  *gpack = pack ? G : 1;
  if (pack && (128 % G) != 0) return FSA_ERR_UNSUPPORTED;
  *num_m_blocks = cdiv(a->seqlen_q * *gpack, 128);
  *hgrid = pack ? a->heads_kv : a->heads_q;
  *sk_static = a->page_table ? a->page_table_stride * a->page_size : a->seqlen_k;
  *n_tiles_k = cdiv(*sk_static, 128);
  return FSA_OK;
}

int fsa_fwd_workspace_bytes(const FsaFwdArgs* a, FsaFwdWorkspace* w) {
  if (!a || !w) return FSA_ERR_INVALID_ARG;
  memset(w, 0, sizeof(*w));
  int gpack, nmb, hgrid, sk, ntk;
  const int rc = fwd_geometry(a, &gpack, &nmb, &hgrid, &sk, &ntk);
  if (rc != FSA_OK) return rc;
  if ((a->flags & FSA_F_SPLIT) && a->num_splits > 0) {
    const size_t rows = a->cu_seqlens_q ? (size_t)a->total_q : (size_t)a->batch * a->seqlen_q;
    w->out_partial = sizeof(float) * (size_t)a->num_splits * rows * a->heads_q * a->head_dim;
    w->lse_partial = sizeof(float) * (size_t)a->num_splits * rows * a->heads_q;
  }
  if (a->kind == FSA_KIND_GATED) w->gate_ws = fsa::gate_ws_bytes(a->batch, hgrid, nmb, a->heads_kv, ntk);
  return FSA_OK;
}

int fsa_bwd_workspace_bytes(const FsaBwdArgs* a, FsaBwdWorkspace* w) {
  if (!a || !w) return FSA_ERR_INVALID_ARG;
  memset(w, 0, sizeof(*w));
  if (a->batch <= 0 || a->heads_q <= 0 || a->heads_kv <= 0 || !head_dim_ok(a->head_dim)) return FSA_ERR_INVALID_ARG;
  const bool varlen_q = a->cu_seqlens_q != nullptr, varlen_k = a->cu_seqlens_k != nullptr;
  const size_t R = (size_t)fsa_bwd_padded_rows(a->batch, a->seqlen_q, a->total_q, varlen_q);
  const size_t es = dtype_bytes(a->dtype);
  w->lse2_ws = w->dpsum_ws = sizeof(float) * (size_t)a->heads_q * R;
  w->dq_accum = sizeof(float) * (size_t)a->heads_q * R * head_dim_kernel(a->head_dim);
  const int ns = (a->flags & FSA_F_SPLIT) ? a->num_splits : 1;
  const size_t rows_k = varlen_k ? (size_t)a->total_k : (size_t)a->batch * a->seqlen_k;
  if (ns > 1) w->dk_partial = w->dv_partial = sizeof(float) * (size_t)ns * rows_k * a->heads_kv * a->head_dim;
  if (a->kind == FSA_KIND_GATED) {
    w->alpha_ws = es * (size_t)a->heads_q * R;
    w->da_accum = sizeof(float) * (size_t)a->heads_q * R;
    if (ns > 1) w->dd_partial = sizeof(float) * (size_t)ns * (size_t)a->delta_numel;
    w->gate_ws = fsa::gate_ws_bytes(a->batch, a->heads_q, cdiv(a->seqlen_q, 128), a->heads_kv, cdiv(a->seqlen_k, 128));
  }
  if (a->flags & FSA_F_DETERMINISTIC) {
    const size_t ntk = cdiv(a->seqlen_k, 128), ntq = cdiv(a->seqlen_q, 128);
    w->dq_order = sizeof(uint16_t) * (size_t)a->batch * a->heads_kv * ntk * ntq;
    w->dq_turn = sizeof(int32_t) * (size_t)a->batch * a->heads_q * ntq;
  }
  return FSA_OK;
}

int fsa_decode_workspace_bytes(const FsaDecArgs* a, FsaDecWorkspace* w) {
  if (!a || !w) return FSA_ERR_INVALID_ARG;
  memset(w, 0, sizeof(*w));
  if (a->batch <= 0 || a->heads_q <= 0 || a->head_dim <= 0) return FSA_ERR_INVALID_ARG;
  const int ns = a->num_splits > 0 ? a->num_splits : 1;
  if (ns > 1 || a->partial_only) {
    w->out_partial = sizeof(float) * (size_t)ns * a->batch * a->heads_q * a->head_dim;
    w->lse_partial = sizeof(float) * (size_t)ns * a->batch * a->heads_q;
  }
  if (a->kind == FSA_KIND_GATED && a->heads_kv > 0) {
    const int keys = a->gather_kv_indices ? a->topk : (a->page_table ? a->page_table_stride * a->page_size : a->seqlen_k);
    w->gate_ws = sizeof(float) * 2 * (size_t)a->batch * a->heads_kv * cdiv(keys, 16);
  }
  return FSA_OK;
}

size_t fsa_fwd_tile_map_bytes(const FsaFwdArgs* a) {
  int gpack, nmb, hgrid, sk, ntk;
  if (!a || fwd_geometry(a, &gpack, &nmb, &hgrid, &sk, &ntk) != FSA_OK) return 0;
  const int ns = (a->flags & FSA_F_SPLIT) ? a->num_splits : 1;
  return (size_t)a->batch * hgrid * nmb * ns * ntk;
}

int fsa_fwd(const FsaFwdArgs* a, void* stream_) {
  if (!a || !a->q || !a->k || !a->v || !a->out || !a->lse || !a->status) return FSA_ERR_INVALID_ARG;
  if (a->batch <= 0 || a->heads_q <= 0 || a->head_dim <= 0) return FSA_ERR_INVALID_ARG;
  if (!head_dim_ok_wide(a->head_dim)) return FSA_ERR_UNSUPPORTED;
  const bool fp8 = a->dtype == FSA_DT_E4M3 || a->dtype == FSA_DT_E5M2;
  if (a->dtype != FSA_DT_BF16 && a->dtype != FSA_DT_FP16 && !fp8) return FSA_ERR_UNSUPPORTED;
  if (fp8 && a->head_dim != 128) return FSA_ERR_UNSUPPORTED;  // FP8 tiles: one 128-byte swizzle row per head row
  const int out_dtype = fp8 ? FSA_DT_BF16 : a->dtype;        // flash_sparse_fwd.py:634
  const uint32_t box0 = fp8 ? 128 : 64;                       // elements in a 128-byte row
  if (a->kind != FSA_KIND_DENSE && a->kind != FSA_KIND_SPARSE && a->kind != FSA_KIND_GATED) return FSA_ERR_UNSUPPORTED;
  if (a->kind == FSA_KIND_GATED && (!a->alpha || !a->delta)) return FSA_ERR_INVALID_ARG;
  if ((a->tile_m && a->tile_m != 128) || (a->tile_n && a->tile_n != 128)) return FSA_ERR_UNSUPPORTED;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const bool varlen_q = a->cu_seqlens_q != nullptr, varlen_k = a->cu_seqlens_k != nullptr;
  const bool paged = a->page_table != nullptr;
  const bool split = (a->flags & FSA_F_SPLIT) != 0;
  const int ns = split ? a->num_splits : 1;
  if (ns <= 0) return FSA_ERR_INVALID_ARG;
  if (split && (!a->out_partial || !a->lse_partial)) return FSA_ERR_INVALID_ARG;
  if ((a->flags & FSA_F_LOCAL) && !a->window_sizes) return FSA_ERR_INVALID_ARG;
  if (paged && (varlen_k || (a->page_size != 32 && a->page_size != 64 && a->page_size != 128 && a->page_size != 256)))
    return FSA_ERR_UNSUPPORTED;
  if (a->seqlen_q <= 0) return FSA_OK;  // nothing to do

  int gpack, num_m_blocks, hgrid, sk_static, n_tiles_k;
  int rc = fwd_geometry(a, &gpack, &num_m_blocks, &hgrid, &sk_static, &n_tiles_k);
  if (rc != FSA_OK) return rc;
  const int G = a->heads_q / a->heads_kv;

  fsa::FwdKernelParams p;
  memset(&p, 0, sizeof(p));
  const long long rows_q = varlen_q ? a->total_q : (long long)a->batch * a->seqlen_q;
  // Q: [B, Sq, Hq, D] or [total_q, Hq, D]
  {
    const uint64_t d_rows = varlen_q ? (uint64_t)a->total_q : (uint64_t)a->seqlen_q;
    const uint64_t d_b = varlen_q ? 1 : (uint64_t)a->batch;
    const int64_t s_b = varlen_q ? a->q_stride_s * (int64_t)a->total_q : a->q_stride_b;
    rc = make_map4(&p.map_q, a->dtype, a->q, a->head_dim, a->heads_q, a->q_stride_h, d_rows, a->q_stride_s, d_b, s_b,
                   box0, gpack, 128 / gpack);
    if (rc != FSA_OK) return rc;
  }
  {
    uint64_t d_rows, d_b;
    int64_t ks_b, vs_b;
    uint32_t box_rows = 128;
    if (paged) {
      d_rows = a->page_size;
      d_b = a->num_pages;
      ks_b = a->k_stride_b;
      vs_b = a->v_stride_b;
      box_rows = a->page_size < 128 ? a->page_size : 128;
    } else if (varlen_k) {
      d_rows = a->total_k;
      d_b = 1;
      ks_b = a->k_stride_s * (int64_t)a->total_k;
      vs_b = a->v_stride_s * (int64_t)a->total_k;
    } else {
      d_rows = a->seqlen_k;
      d_b = a->batch;
      ks_b = a->k_stride_b;
      vs_b = a->v_stride_b;
    }
    if (d_rows == 0) return FSA_ERR_INVALID_ARG;
    rc = make_map4(&p.map_k, a->dtype, a->k, a->head_dim, a->heads_kv, a->k_stride_h, d_rows, a->k_stride_s, d_b, ks_b,
                   box0, 1, box_rows);
    if (rc != FSA_OK) return rc;
    rc = make_map4(&p.map_v, a->dtype, a->v, a->head_dim, a->heads_kv, a->v_stride_h, d_rows, a->v_stride_s, d_b, vs_b,
                   box0, 1, box_rows);
    if (rc != FSA_OK) return rc;
  }
  p.cu_q = a->cu_seqlens_q;
  p.cu_k = a->cu_seqlens_k;
  p.used_q = a->seqused_q;
  p.used_k = a->seqused_k;
  p.page_table = a->page_table;
  p.windows = a->window_sizes;
  p.alpha = a->alpha;
  p.delta = a->delta;
  p.a_sb = a->alpha_stride_b;
  p.a_sh = a->alpha_stride_h;
  p.d_sb = a->delta_stride_b;
  p.d_sh = a->delta_stride_h;
  p.status = a->status;
  p.tile_map = a->tile_map;
  if (split) {
    p.out = a->out_partial;
    p.lse = a->lse_partial;
    p.o_sb = (long long)a->seqlen_q * a->heads_q * a->head_dim;
    p.o_sm = (long long)a->heads_q * a->head_dim;
    p.o_sh = a->head_dim;
    p.o_ss = rows_q * a->heads_q * a->head_dim;
    p.l_sb = a->seqlen_q;
    p.l_sh = rows_q;
    p.l_ss = rows_q * a->heads_q;
  } else {
    p.out = a->out;
    p.lse = a->lse;
    p.o_sb = a->o_stride_b;
    p.o_sm = a->o_stride_s;
    p.o_sh = a->o_stride_h;
    p.o_ss = 0;
    p.l_sb = a->lse_stride_b;
    p.l_sh = a->lse_stride_h;
    p.l_ss = 0;
  }
  if ((p.o_sm % 8) || (p.o_sh % 8) || (p.o_sb % 8)) return FSA_ERR_INVALID_ARG;  // 16-byte row stores
  p.B = a->batch;
  p.Hq = a->heads_q;
  p.Hkv = a->heads_kv;
  p.G = G;
  p.gpack = gpack;
  p.sq = a->seqlen_q;
  p.sk = sk_static;
  p.num_splits = ns;
  p.num_m_blocks = num_m_blocks;
  // head sizes above 128: one query tile per CTA (the 256-wide kernel), otherwise two
  p.num_pairs = head_dim_kernel_wide(a->head_dim) > 128 ? num_m_blocks : cdiv(num_m_blocks, 2);
  p.hgrid = hgrid;
  p.page_size = a->page_size;
  p.pt_stride = a->page_table_stride;
  p.win_stride = a->window_stride;
  p.n_tiles_k = n_tiles_k;
  p.scale_log2 = a->softmax_scale * 1.44269504089f;
  p.softmax_thr = a->softmax_threshold;
  p.gate_thr = a->gate_threshold;
  p.v_scale = 1.0f;
  p.qkv_scale = a->qkv_scale;
  unsigned f = 0;
  if (a->flags & FSA_F_CAUSAL) f |= fsa::F_CAUSAL;
  if (a->flags & FSA_F_LOCAL) f |= fsa::F_LOCAL;
  if (split) f |= fsa::F_SPLIT | fsa::F_LSE_LOG2;
  if (varlen_q) f |= fsa::F_VARLEN_Q;
  if (varlen_k) f |= fsa::F_VARLEN_K;
  if (paged) f |= fsa::F_PAGED;
  if (gpack > 1) f |= fsa::F_PACK_GQA;
  if (a->seqused_q) f |= fsa::F_USED_Q;
  if (a->seqused_k) f |= fsa::F_USED_K;
  if (varlen_k || paged || a->seqused_k) f |= fsa::F_KV_RAGGED;
  if (a->flags & FSA_F_LOGSIGMOID) f |= fsa::F_LOGSIGMOID;
  if (a->flags & FSA_F_ADAPT_GATE) f |= fsa::F_ADAPT_GATE;
  p.flags = f;

  if (a->q_block_scale || a->k_block_scale || a->v_block_scale) {
    if (!a->q_block_scale || !a->k_block_scale || !a->v_block_scale || a->qkv_scale)
      return FSA_ERR_INVALID_ARG;
    if (!fp8 || a->kind == FSA_KIND_GATED || gpack > 1 || paged) return FSA_ERR_UNSUPPORTED;
    p.q_bscale = a->q_block_scale;
    p.k_bscale = a->k_block_scale;
    p.v_bscale = a->v_block_scale;
  }
  if (a->kind == FSA_KIND_GATED) {
    if (!a->gate_ws) return FSA_ERR_INVALID_ARG;
    fsa::GateExtParams ge;
    memset(&ge, 0, sizeof(ge));
    ge.alpha = a->alpha;
    ge.delta = a->delta;
    ge.gate_ws = a->gate_ws;
    ge.cu_q = a->cu_seqlens_q;
    ge.cu_k = a->cu_seqlens_k;
    ge.used_q = a->seqused_q;
    ge.used_k = a->seqused_k;
    ge.page_table = a->page_table;
    ge.a_sb = a->alpha_stride_b;
    ge.a_sh = a->alpha_stride_h;
    ge.d_sb = a->delta_stride_b;
    ge.d_sh = a->delta_stride_h;
    ge.B = a->batch;
    ge.Hq = a->heads_q;
    ge.Hkv = a->heads_kv;
    ge.G = G;
    ge.gpack = gpack;
    ge.hgrid = hgrid;
    ge.sq = a->seqlen_q;
    ge.sk = sk_static;
    ge.num_m_blocks = num_m_blocks;
    ge.n_tiles_k = n_tiles_k;
    ge.page_size = a->page_size;
    ge.pt_stride = a->page_table_stride;
    ge.flags = f & (fsa::F_VARLEN_Q | fsa::F_VARLEN_K | fsa::F_USED_Q | fsa::F_USED_K | fsa::F_PAGED);
    if (fsa::launch_gate_ext(ge, out_dtype, stream) != cudaSuccess) return FSA_ERR_LAUNCH;
    p.gate_ws = a->gate_ws;
  }
  mark(a->ev_before, stream);
  p.D = a->head_dim;
  cudaError_t e = fsa::launch_fwd(p, a->kind, a->dtype, head_dim_kernel_fwd(a->head_dim), stream);
  mark(a->ev_after, stream);
  if (e == cudaErrorInvalidValue) return FSA_ERR_UNSUPPORTED;
  if (e != cudaSuccess) return FSA_ERR_LAUNCH;

  if (split) {
    fsa::CombineParams c;
    memset(&c, 0, sizeof(c));
    c.out_partial = a->out_partial;
    c.lse_partial = a->lse_partial;
    c.out = a->out;
    c.lse = a->lse;
    c.op_ss = p.o_ss;
    c.lp_ss = p.l_ss;
    c.lp_sh = p.l_sh;
    c.o_sb = varlen_q ? 0 : a->o_stride_b;
    c.o_sm = a->o_stride_s;
    c.o_sh = a->o_stride_h;
    c.l_sb = varlen_q ? 0 : a->lse_stride_b;
    c.l_sh = a->lse_stride_h;
    c.rows = (int)rows_q;
    c.rows_per_batch = varlen_q ? a->total_q : a->seqlen_q;
    c.heads = a->heads_q;
    c.head_dim = a->head_dim;
    c.num_splits = ns;
    e = fsa::launch_combine(c, out_dtype, stream);
    if (e != cudaSuccess) return FSA_ERR_LAUNCH;
  }
  return FSA_OK;
}

int64_t fsa_bwd_padded_rows(int batch, int seqlen_q, int total_q, int is_varlen) {
  if (is_varlen) return ((int64_t)total_q + 128ll * batch + 127) / 128 * 128;
  return (int64_t)batch * (((int64_t)seqlen_q + 127) / 128 * 128);
}

int fsa_bwd(const FsaBwdArgs* a, void* stream_) {
  if (!a || !a->q || !a->k || !a->v || !a->out || !a->dout || !a->lse || !a->dq || !a->dk || !a->dv || !a->status)
    return FSA_ERR_INVALID_ARG;
  if (!a->lse2_ws || !a->dpsum_ws || !a->dq_accum) return FSA_ERR_INVALID_ARG;
  if (a->batch <= 0 || a->heads_q <= 0 || a->heads_kv <= 0 || a->heads_q % a->heads_kv) return FSA_ERR_INVALID_ARG;
  if (!head_dim_ok(a->head_dim)) return FSA_ERR_UNSUPPORTED;
  const int hdk = head_dim_kernel(a->head_dim);  // also the row pitch of dq_accum
  if (a->dtype != FSA_DT_BF16 && a->dtype != FSA_DT_FP16) return FSA_ERR_UNSUPPORTED;
  if (a->kind != FSA_KIND_DENSE && a->kind != FSA_KIND_SPARSE && a->kind != FSA_KIND_GATED)
    return FSA_ERR_UNSUPPORTED;
  const bool gated = a->kind == FSA_KIND_GATED;
  if (gated && (!a->alpha || !a->delta || !a->dalpha || !a->ddelta || !a->alpha_ws || !a->da_accum))
    return FSA_ERR_INVALID_ARG;
  if ((a->tile_m && a->tile_m != 128) || (a->tile_n && a->tile_n != 128)) return FSA_ERR_UNSUPPORTED;
  if ((a->flags & FSA_F_LOCAL) && !a->window_sizes) return FSA_ERR_INVALID_ARG;
  if (a->dk_stride_b % 8 || a->dk_stride_s % 8 || a->dk_stride_h % 8) return FSA_ERR_INVALID_ARG;
  if (a->o_stride_b % 8 || a->o_stride_s % 8 || a->o_stride_h % 8 || a->do_stride_b % 8 || a->do_stride_s % 8 ||
      a->do_stride_h % 8 || a->dq_stride_b % 8 || a->dq_stride_s % 8 || a->dq_stride_h % 8)
    return FSA_ERR_INVALID_ARG;  // rows are moved in 16-byte pieces
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const bool varlen_q = a->cu_seqlens_q != nullptr, varlen_k = a->cu_seqlens_k != nullptr;
  const int ns = (a->flags & FSA_F_SPLIT) ? a->num_splits : 1;
  if (ns <= 0) return FSA_ERR_INVALID_ARG;
  const bool split = ns > 1;
  if (split && (!a->dk_partial || !a->dv_partial)) return FSA_ERR_INVALID_ARG;
  if (split && gated && (!a->dd_partial || a->delta_numel <= 0)) return FSA_ERR_INVALID_ARG;
  const bool det = a->flags & FSA_F_DETERMINISTIC;
  if (det && (!a->dq_order || !a->dq_turn)) return FSA_ERR_INVALID_ARG;
  if (a->seqlen_q <= 0 || a->seqlen_k <= 0) return FSA_OK;
  const int64_t R = fsa_bwd_padded_rows(a->batch, a->seqlen_q, a->total_q, varlen_q);
  const long long rows_k = varlen_k ? a->total_k : (long long)a->batch * a->seqlen_k;

  // pre-pass + accumulator reset
  fsa::BwdPreParams pre;
  memset(&pre, 0, sizeof(pre));
  pre.out = a->out;
  pre.dout = a->dout;
  pre.lse = a->lse;
  pre.lse2_ws = a->lse2_ws;
  pre.dpsum_ws = a->dpsum_ws;
  pre.cu_q = a->cu_seqlens_q;
  pre.o_sb = a->o_stride_b;
  pre.o_sm = a->o_stride_s;
  pre.o_sh = a->o_stride_h;
  pre.do_sb = a->do_stride_b;
  pre.do_sm = a->do_stride_s;
  pre.do_sh = a->do_stride_h;
  pre.l_sb = a->lse_stride_b;
  pre.l_sh = a->lse_stride_h;
  pre.ws_sh = R;
  pre.B = a->batch;
  pre.sq = a->seqlen_q;
  pre.total_q = a->total_q;
  pre.heads = a->heads_q;
  pre.head_dim = a->head_dim;
  pre.head_dim_pad = hdk;
  pre.varlen = varlen_q;
  if (gated) {
    if (cudaMemsetAsync(a->alpha_ws, 0, 2 * (size_t)a->heads_q * R, stream) != cudaSuccess) return FSA_ERR_LAUNCH;
    if (cudaMemsetAsync(a->da_accum, 0, sizeof(float) * (size_t)a->heads_q * R, stream) != cudaSuccess)
      return FSA_ERR_LAUNCH;
    pre.alpha = a->alpha;
    pre.alpha_ws = a->alpha_ws;
    pre.a_sb = a->alpha_stride_b;
    pre.a_sh = a->alpha_stride_h;
  }
  // padding rows of dpsum must hold finite values (they meet zero probabilities in a packed product)
  if (cudaMemsetAsync(a->dpsum_ws, 0, sizeof(float) * (size_t)a->heads_q * R, stream) != cudaSuccess)
    return FSA_ERR_LAUNCH;
  // the pre-pass clears the accumulator rows it visits (padding rows are never read); a cudaMemsetAsync of the
  // whole accumulator in front of a pre-pass that only reads measured slower (0.795 vs 0.778 ms per bench step)
  pre.dq_accum = a->dq_accum;
  if (fsa::launch_bwd_pre(pre, a->dtype, stream) != cudaSuccess) return FSA_ERR_LAUNCH;

  fsa::BwdKernelParams p;
  memset(&p, 0, sizeof(p));
  int rc;
  {
    const uint64_t d_rows = varlen_q ? (uint64_t)a->total_q : (uint64_t)a->seqlen_q;
    const uint64_t d_b = varlen_q ? 1 : (uint64_t)a->batch;
    rc = make_map4(&p.map_q, a->dtype, a->q, a->head_dim, a->heads_q, a->q_stride_h, d_rows, a->q_stride_s, d_b,
                   varlen_q ? a->q_stride_s * (int64_t)a->total_q : a->q_stride_b, 64, 1, 128);
    if (rc != FSA_OK) return rc;
    rc = make_map4(&p.map_do, a->dtype, a->dout, a->head_dim, a->heads_q, a->do_stride_h, d_rows, a->do_stride_s, d_b,
                   varlen_q ? a->do_stride_s * (int64_t)a->total_q : a->do_stride_b, 64, 1, 128);
    if (rc != FSA_OK) return rc;
  }
  {
    const uint64_t d_rows = varlen_k ? (uint64_t)a->total_k : (uint64_t)a->seqlen_k;
    const uint64_t d_b = varlen_k ? 1 : (uint64_t)a->batch;
    rc = make_map4(&p.map_k, a->dtype, a->k, a->head_dim, a->heads_kv, a->k_stride_h, d_rows, a->k_stride_s, d_b,
                   varlen_k ? a->k_stride_s * (int64_t)a->total_k : a->k_stride_b, 64, 1, 128);
    if (rc != FSA_OK) return rc;
    rc = make_map4(&p.map_v, a->dtype, a->v, a->head_dim, a->heads_kv, a->v_stride_h, d_rows, a->v_stride_s, d_b,
                   varlen_k ? a->v_stride_s * (int64_t)a->total_k : a->v_stride_b, 64, 1, 128);
    if (rc != FSA_OK) return rc;
  }
  rc = make_map_dq(&p.map_dq, a->dq_accum, hdk, R, a->heads_q);
  if (rc != FSA_OK) return rc;
  p.lse2_ws = a->lse2_ws;
  p.dpsum_ws = a->dpsum_ws;
  p.cu_q = a->cu_seqlens_q;
  p.cu_k = a->cu_seqlens_k;
  p.used_q = a->seqused_q;
  p.used_k = a->seqused_k;
  p.windows = a->window_sizes;
  p.status = a->status;
  p.tile_map = a->tile_map;
  if (split) {
    p.dk_out = a->dk_partial;
    p.dv_out = a->dv_partial;
    p.dkv_sb = (long long)a->seqlen_k * a->heads_kv * a->head_dim;
    p.dkv_sn = (long long)a->heads_kv * a->head_dim;
    p.dkv_sh = a->head_dim;
    p.dkv_ss = rows_k * a->heads_kv * a->head_dim;
  } else {
    p.dk_out = a->dk;
    p.dv_out = a->dv;
    p.dkv_sb = a->dk_stride_b;
    p.dkv_sn = a->dk_stride_s;
    p.dkv_sh = a->dk_stride_h;
    p.dkv_ss = 0;
  }
  p.ws_sh = R;
  p.B = a->batch;
  p.Hq = a->heads_q;
  p.Hkv = a->heads_kv;
  p.G = a->heads_q / a->heads_kv;
  p.sq = a->seqlen_q;
  p.sk = a->seqlen_k;
  p.num_splits = ns;
  p.n_tiles_k = cdiv(a->seqlen_k, 128);
  p.num_m_blocks = cdiv(a->seqlen_q, 128);
  p.win_stride = a->window_stride;
  p.scale_log2 = a->softmax_scale * 1.44269504089f;
  p.softmax_scale = a->softmax_scale;
  p.softmax_thr = a->softmax_threshold;
  unsigned f = 0;
  if (gated) {
    p.alpha_ws = a->alpha_ws;
    p.delta = a->delta;
    p.da_accum = a->da_accum;
    p.dd_out = split ? (void*)a->dd_partial : a->ddelta;
    p.d_sb = a->delta_stride_b;
    p.d_sh = a->delta_stride_h;
    p.dd_ss = a->delta_numel;
    p.gate_thr = a->gate_threshold;
    if (a->flags & FSA_F_LOGSIGMOID) f |= fsa::F_LOGSIGMOID;
    if (a->flags & FSA_F_ADAPT_GATE) f |= fsa::F_ADAPT_GATE;
  }
  if (a->flags & FSA_F_CAUSAL) f |= fsa::F_CAUSAL;
  if (a->flags & FSA_F_LOCAL) f |= fsa::F_LOCAL;
  if (split) f |= fsa::F_SPLIT;
  if (varlen_q) f |= fsa::F_VARLEN_Q;
  if (varlen_k) f |= fsa::F_VARLEN_K;
  if (a->seqused_q) f |= fsa::F_USED_Q;
  if (a->seqused_k) f |= fsa::F_USED_K;
  p.flags = f;
  if (det) {
    fsa::DqOrderParams op;
    memset(&op, 0, sizeof(op));
    op.order = a->dq_order;
    op.cu_q = a->cu_seqlens_q;
    op.cu_k = a->cu_seqlens_k;
    op.used_q = a->seqused_q;
    op.used_k = a->seqused_k;
    op.windows = a->window_sizes;
    op.B = a->batch;
    op.Hkv = a->heads_kv;
    op.sq = a->seqlen_q;
    op.sk = a->seqlen_k;
    op.num_splits = ns;
    op.n_tiles_k = p.n_tiles_k;
    op.num_m_blocks = p.num_m_blocks;
    op.win_stride = a->window_stride;
    op.flags = f;
    if (fsa::launch_dq_order(op, stream) != cudaSuccess) return FSA_ERR_LAUNCH;
    if (cudaMemsetAsync(a->dq_turn, 0, sizeof(int32_t) * (size_t)a->batch * a->heads_q * p.num_m_blocks, stream) !=
        cudaSuccess)
      return FSA_ERR_LAUNCH;
    p.dq_order = a->dq_order;
    p.dq_turn = a->dq_turn;
    p.flags |= fsa::F_DETERMINISTIC;
  }
  if (gated && a->gate_ws) {
    fsa::GateExtParams ge;
    memset(&ge, 0, sizeof(ge));
    ge.alpha = a->alpha;
    ge.delta = a->delta;
    ge.gate_ws = a->gate_ws;
    ge.cu_q = a->cu_seqlens_q;
    ge.cu_k = a->cu_seqlens_k;
    ge.used_q = a->seqused_q;
    ge.used_k = a->seqused_k;
    ge.a_sb = a->alpha_stride_b;
    ge.a_sh = a->alpha_stride_h;
    ge.d_sb = a->delta_stride_b;
    ge.d_sh = a->delta_stride_h;
    ge.B = a->batch;
    ge.Hq = a->heads_q;
    ge.Hkv = a->heads_kv;
    ge.G = p.G;
    ge.gpack = 1;
    ge.hgrid = a->heads_q;
    ge.sq = a->seqlen_q;
    ge.sk = a->seqlen_k;
    ge.num_m_blocks = p.num_m_blocks;
    ge.n_tiles_k = p.n_tiles_k;
    ge.flags = f & (fsa::F_VARLEN_Q | fsa::F_VARLEN_K | fsa::F_USED_Q | fsa::F_USED_K);
    if (fsa::launch_gate_ext(ge, a->dtype, stream) != cudaSuccess) return FSA_ERR_LAUNCH;
    p.gate_ws = a->gate_ws;
  }
  mark(a->ev_before, stream);
  p.D = a->head_dim;
  cudaError_t e = fsa::launch_bwd(p, a->kind, a->dtype, hdk, stream);
  mark(a->ev_after, stream);
  if (e == cudaErrorInvalidValue) return FSA_ERR_UNSUPPORTED;
  if (e != cudaSuccess) return FSA_ERR_LAUNCH;

  fsa::BwdPostParams post;
  memset(&post, 0, sizeof(post));
  post.dq_accum = a->dq_accum;
  post.dq = a->dq;
  post.cu_q = a->cu_seqlens_q;
  post.dq_sb = a->dq_stride_b;
  post.dq_sm = a->dq_stride_s;
  post.dq_sh = a->dq_stride_h;
  post.ws_sh = R;
  post.B = a->batch;
  post.sq = a->seqlen_q;
  post.total_q = a->total_q;
  post.heads = a->heads_q;
  post.head_dim = a->head_dim;
  post.head_dim_pad = hdk;
  post.varlen = varlen_q;
  post.scale = a->softmax_scale;
  if (gated) {
    post.da_accum = a->da_accum;
    post.da = a->dalpha;
    post.da_sb = a->alpha_stride_b;
    post.da_sh = a->alpha_stride_h;
  }
  if (fsa::launch_bwd_post(post, a->dtype, stream) != cudaSuccess) return FSA_ERR_LAUNCH;
  if (split && gated) {
    fsa::FlatSumParams fs;
    memset(&fs, 0, sizeof(fs));
    fs.partial = a->dd_partial;
    fs.out = a->ddelta;
    fs.part_ss = a->delta_numel;
    fs.n = a->delta_numel;
    fs.num_splits = ns;
    if (fsa::launch_flat_sum(fs, a->dtype, stream) != cudaSuccess) return FSA_ERR_LAUNCH;
  }

  if (split) {
    for (int which = 0; which < 2; ++which) {
      fsa::SplitSumParams sp;
      memset(&sp, 0, sizeof(sp));
      sp.partial = which == 0 ? a->dk_partial : a->dv_partial;
      sp.out = which == 0 ? a->dk : a->dv;
      sp.part_ss = p.dkv_ss;
      sp.o_sb = varlen_k ? 0 : a->dk_stride_b;
      sp.o_sn = a->dk_stride_s;
      sp.o_sh = a->dk_stride_h;
      sp.rows = (int)rows_k;
      sp.rows_per_batch = varlen_k ? a->total_k : a->seqlen_k;
      sp.heads = a->heads_kv;
      sp.head_dim = a->head_dim;
      sp.num_splits = ns;
      if (fsa::launch_split_sum(sp, a->dtype, stream) != cudaSuccess) return FSA_ERR_LAUNCH;
    }
  }
  return FSA_OK;
}

int fsa_combine(const float* out_partial, const float* lse_partial, void* out, float* lse, int num_partials,
                int rows, int heads, int head_dim, int dtype, int64_t out_partial_stride,
                int64_t lse_partial_stride, void* stream_) {
  if (!out_partial || !lse_partial || !out || !lse || num_partials <= 0 || rows < 0 || heads <= 0)
    return FSA_ERR_INVALID_ARG;
  if (dtype != FSA_DT_BF16 && dtype != FSA_DT_FP16) return FSA_ERR_UNSUPPORTED;
  fsa::CombineParams c;
  memset(&c, 0, sizeof(c));
  c.out_partial = out_partial;
  c.lse_partial = lse_partial;
  c.out = out;
  c.lse = lse;
  c.op_ss = out_partial_stride > 0 ? out_partial_stride : (long long)rows * heads * head_dim;
  c.lp_ss = lse_partial_stride > 0 ? lse_partial_stride : (long long)rows * heads;
  c.lp_sh = rows;
  c.o_sb = (long long)heads * head_dim;
  c.o_sm = 0;
  c.o_sh = head_dim;
  c.l_sb = heads;
  c.l_sh = 1;
  c.rows = rows;
  c.rows_per_batch = 1;
  c.heads = heads;
  c.head_dim = head_dim;
  c.num_splits = num_partials;
  cudaError_t e = fsa::launch_combine(c, dtype, reinterpret_cast<cudaStream_t>(stream_));
  if (e == cudaErrorInvalidValue) return FSA_ERR_UNSUPPORTED;
  return e == cudaSuccess ? FSA_OK : FSA_ERR_LAUNCH;
}

int fsa_decode(const FsaDecArgs* a, void* stream_) {
  if (!a || !a->q || !a->k || !a->v || !a->status) return FSA_ERR_INVALID_ARG;
  if (a->batch <= 0 || a->heads_q <= 0 || a->heads_kv <= 0 || a->heads_q % a->heads_kv) return FSA_ERR_INVALID_ARG;
  if (!head_dim_ok_wide(a->head_dim)) return FSA_ERR_UNSUPPORTED;
  const bool fp8 = a->dtype == FSA_DT_E4M3 || a->dtype == FSA_DT_E5M2;  // q, k, v in FP8; out / alpha / delta bf16
  if (a->dtype != FSA_DT_BF16 && a->dtype != FSA_DT_FP16 && !fp8) return FSA_ERR_UNSUPPORTED;
  if (fp8 && a->head_dim != 128) return FSA_ERR_UNSUPPORTED;
  if (a->kind != FSA_KIND_DENSE && a->kind != FSA_KIND_SPARSE && a->kind != FSA_KIND_GATED) return FSA_ERR_UNSUPPORTED;
  if (a->kind == FSA_KIND_GATED && (!a->alpha || !a->delta)) return FSA_ERR_INVALID_ARG;
  if ((a->flags & FSA_F_LOCAL) && !a->window_sizes) return FSA_ERR_INVALID_ARG;
  const bool paged = a->page_table != nullptr, gather = a->gather_kv_indices != nullptr;
  const bool varlen_k = a->cu_seqlens_k != nullptr;
  if (paged && varlen_k) return FSA_ERR_UNSUPPORTED;
  if (paged && (a->page_size <= 0 || (a->page_size & (a->page_size - 1)))) return FSA_ERR_INVALID_ARG;  // power of two
  const int ns = a->num_splits > 0 ? a->num_splits : 1;
  const bool partial = ns > 1 || a->partial_only;
  if (partial && (!a->out_partial || !a->lse_partial)) return FSA_ERR_INVALID_ARG;
  if (!a->partial_only && (!a->out || !a->lse)) return FSA_ERR_INVALID_ARG;
  if ((a->k_stride_s % 8) || (a->k_stride_h % 8) || (a->k_stride_b % 8) ||
      (reinterpret_cast<uintptr_t>(a->k) & 15) || (reinterpret_cast<uintptr_t>(a->v) & 15))
    return FSA_ERR_INVALID_ARG;  // 16-byte row copies
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);

  fsa::DecKernelParams p;
  memset(&p, 0, sizeof(p));
  p.q = a->q;
  p.k = a->k;
  p.v = a->v;
  p.out = a->out;
  p.lse = a->lse;
  p.out_partial = a->out_partial;
  p.lse_partial = a->lse_partial;
  p.cu_k = a->cu_seqlens_k;
  p.used_k = a->seqused_k;
  p.page_table = a->page_table;
  p.gather_idx = a->gather_kv_indices;
  p.windows = a->window_sizes;
  p.alpha = a->alpha;
  p.delta = a->delta;
  p.a_sb = a->alpha_stride_b;
  p.a_sh = a->alpha_stride_h;
  p.d_sb = a->delta_stride_b;
  p.d_sh = a->delta_stride_h;
  p.gate_thr = a->gate_threshold;
  p.qkv_scale = a->qkv_scale;
  p.tile_map = a->tile_map;
  p.q_sb = a->q_stride_b;
  p.q_sh = a->q_stride_h;
  p.k_sb = a->k_stride_b;
  p.k_sn = a->k_stride_s;
  p.k_sh = a->k_stride_h;
  p.o_sb = a->o_stride_b;
  p.o_sh = a->o_stride_h;
  p.l_sb = a->lse_stride_b;
  p.l_sh = a->lse_stride_h;
  p.B = a->batch;
  p.Hq = a->heads_q;
  p.Hkv = a->heads_kv;
  p.G = a->heads_q / a->heads_kv;
  p.sk = paged ? a->page_table_stride * a->page_size : a->seqlen_k;
  p.sk_capacity = a->seqlen_k;
  p.topk = a->topk;
  p.num_splits = ns;
  p.page_size = a->page_size;
  p.pt_stride = a->page_table_stride;
  p.gi_stride = a->gather_stride;
  p.win_stride = a->window_stride;
  p.n_tiles = cdiv(gather ? a->topk : p.sk, 16);
  p.scale_log2 = a->softmax_scale * 1.44269504089f;
  p.softmax_thr = a->softmax_threshold;
  unsigned f = 0;
  if ((a->flags & FSA_F_LOCAL) && !gather) f |= fsa::F_LOCAL;
  if (partial) f |= fsa::F_SPLIT;
  if (varlen_k) f |= fsa::F_VARLEN_K;
  if (paged) f |= fsa::F_PAGED;
  if (gather) f |= fsa::F_GATHER;
  if (a->seqused_k) f |= fsa::F_USED_K;
  if (a->flags & FSA_F_LOGSIGMOID) f |= fsa::F_LOGSIGMOID;
  p.flags = f;
  p.op_ss = a->out_partial_stride > 0 ? a->out_partial_stride : (long long)a->batch * a->heads_q * a->head_dim;
  p.lp_ss = a->lse_partial_stride > 0 ? a->lse_partial_stride : (long long)a->batch * a->heads_q;
  p.thr_sk = a->thr_seqlen_k;
  p.key_bounds = gather ? a->key_bounds : nullptr;
  p.gather_count = gather ? a->gather_count : nullptr;
  p.gate_ws = a->gate_ws;
  if (a->peers) {
    // partials straight into the receive buffers of a context-parallel group: packed layout only
    const FsaPeerArgs* pe = a->peers;
    const long long per = (long long)a->batch * a->heads_q * (a->head_dim + 1);
    if (!a->partial_only || !a->out_partial || pe->world <= 0 || pe->world > FSA_PEER_MAX_RANKS || pe->rank < 0 ||
        pe->rank >= pe->world || p.op_ss != per || p.lp_ss != per || pe->block_floats != per * ns ||
        a->lse_partial != a->out_partial + (long long)a->batch * a->heads_q * a->head_dim)
      return FSA_ERR_INVALID_ARG;
    for (int r = 0; r < pe->world; ++r) {
      if (!pe->region[r] || (reinterpret_cast<uintptr_t>(pe->region[r]) & 255)) return FSA_ERR_INVALID_ARG;
      p.peer_base[r] = reinterpret_cast<unsigned char*>(pe->region[r]);
    }
    p.peer_world = pe->world;
    p.peer_rank = pe->rank;
    p.peer_block_floats = pe->block_floats;
  }
  mark(a->ev_before, stream);
  p.D = a->head_dim;
  cudaError_t e = fsa::launch_dec(p, a->kind, a->dtype, head_dim_kernel_wide(a->head_dim), stream);
  mark(a->ev_after, stream);
  if (e == cudaErrorInvalidValue) return FSA_ERR_UNSUPPORTED;
  if (e != cudaSuccess) return FSA_ERR_LAUNCH;
  if (partial && !a->partial_only) {
    fsa::CombineParams c;
    memset(&c, 0, sizeof(c));
    c.out_partial = a->out_partial;
    c.lse_partial = a->lse_partial;
    c.out = a->out;
    c.lse = a->lse;
    c.op_ss = p.op_ss;
    c.lp_ss = p.lp_ss;
    c.lp_sh = a->batch;
    c.o_sb = a->o_stride_b;
    c.o_sm = 0;
    c.o_sh = a->o_stride_h;
    c.l_sb = a->lse_stride_b;
    c.l_sh = a->lse_stride_h;
    c.rows = a->batch;
    c.rows_per_batch = 1;
    c.heads = a->heads_q;
    c.head_dim = a->head_dim;
    c.num_splits = ns;
    e = fsa::launch_combine(c, fp8 ? FSA_DT_BF16 : a->dtype, stream);
    if (e != cudaSuccess) return FSA_ERR_LAUNCH;
  }
  return FSA_OK;
}

}  // extern "C"
