// Forward attention for sm_100a: tcgen05 MMAs with TMEM accumulators, TMA-fed K/V rings,
// warp-specialised roles.
//
// One CTA owns TWO consecutive 128-row query tiles of one head (so every K/V tile it pulls from
// L2 is used by 256 query rows) and walks the key tiles both tiles visit, in descending order.
// Replaces, per CTA, two programs of the reference's `_fwd_{dense,sparse}_kernel`
// (flash_sparse_attn/ops/triton/flash_sparse_fwd.py:91-502, flash_dense_fwd.py:89-498) at
// TILE_M = TILE_N = 128: same tile schedule, same masks, same online-softmax recurrences and the
// same per-tile skip rule (activations.py:103-166), evaluated independently for each 128-row tile.
//
// Roles (384 threads = 3 warpgroups, registers rebalanced with setmaxnreg):
//   warps 0-3  : softmax group 0 (query tile 0), one thread per query row / TMEM lane
//   warps 4-7  : softmax group 1 (query tile 1)
//   warp  8    : producer - TMA loads of Q, K ring, V ring; allocates / frees TMEM
//   warp  9    : MMA issuer - S = Q K^T and O_tile = P V on the tensor cores
//   warps 10-11: idle
//
// TMEM columns: S0 | S1 | O0 | O1, 128 each (O uses HD columns). P (16-bit) is written back over the
// first 64 columns of its own S block and consumed from TMEM as the A operand of P V.
// The output accumulates in TMEM across key tiles. A softmax thread keeps a reference maximum per
// row that is only moved (and O rescaled in TMEM) when the true running maximum has drifted by
// more than 2^8 from it: sums and outputs stay exact up to rounding because every term carries the
// same reference, and the skip rule reads the same in terms of the reference pair (m, l).
#include "fsa_ptx.cuh"
#include "fsa_params.h"
#include "fsa_schedule.h"


namespace fsa {

namespace {

constexpr int TM = 128;  // query rows per softmax group
constexpr int TN = 128;  // keys per tile
constexpr int NTHREADS = 384;  // three warpgroups: softmax 0, softmax 1, {producer, MMA, 2 idle}
// Two K and two V stages. V(t) and K(t + 1) are consumed by the same loop step of the MMA issuer, so they
// arrive on one barrier and one "consumed" barrier per step releases both: every barrier the issuer touches
// costs it 130-250 cycles even when it is already complete. (A third V stage, loaded a whole step earlier, did
// not shorten the issuer's wait: it is not load latency.)
// Head sizes above 128 (the 192- and 256-wide instantiations): a tile is 48 / 64 KB, so a CTA holds ONE query tile
// (the second softmax group idles; its TMEM columns belong to the wider output accumulator of the first) and one
// stage of V - the load of V(t) then starts when P V(t - 1) has completed and runs under the softmax of tile t. K
// keeps two stages where they fit (192 wide).
template <int HD>
struct FwdShape {
  static constexpr int QT = HD > 128 ? 1 : 2;       // query tiles (softmax groups at work) per CTA
  static constexpr int KSTAGES = HD > 192 ? 1 : 2;
  static constexpr int VSTAGES = HD > 128 ? 1 : 2;
};

template <int HD, int ES = 2>
struct FwdSmem {
  static constexpr int kTileBytes = TM * HD * ES;  // one Q / K / V tile of ES-byte elements
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + FwdShape<HD>::QT * kTileBytes;
  static constexpr int kV = kK + FwdShape<HD>::KSTAGES * kTileBytes;
  static constexpr int kBar = kV + FwdShape<HD>::VSTAGES * kTileBytes;
  static constexpr int kTotal = kBar + 2048 + 1024;  // barriers/flags/delta ring + alignment slack
};

// Output / gate element type that goes with an input element type.
template <typename T>
struct OutType {
  using type = T;
};
template <>
struct OutType<__nv_fp8_e4m3> {
  using type = __nv_bfloat16;
};
template <>
struct OutType<__nv_fp8_e5m2> {
  using type = __nv_bfloat16;
};

struct FwdBars {
  uint64_t q_full;
  uint64_t k0_full;     // first K tile
  uint64_t kv_full[2];  // step t (slot t & 1): V(t) and K(t + 1) have landed (two producer arrivals)
  uint64_t kv_empty[2];  // signal c (slot c & 1): K(c) and V(c - 1) have been consumed; c = 0 comes from the prologue
  uint64_t s_full[2], p_full[2], o_final[2], wg_sync[2];
  uint64_t d_full[2], d_empty[2];  // gated: delta ring (stager warp -> softmax warps)
  uint32_t tmem_base;
  int abort_flag;
  int skip_flag[2][2];   // [group][parity of the group's tile counter]
  int vote_any[2][2][4]; // [group][parity][warp]: bit0 = some row wants the tile, bit1 = some row votes skip
  alignas(16) float dl[2][TN + 4];  // gated: delta of the key tile as fp32 (read as float4), then its max and min
};

static_assert(offsetof(FwdBars, dl) % 16 == 0 && sizeof(FwdBars) <= 2048, "FwdBars layout");

struct SeqInfo {
  int b, split, head, hkv;  // head = query head, or kv head when packing GQA rows
  int off_q, off_k, sq, sk;
  FsaWindow w;
};

// Row-local view of the masks in flash_sparse_attn/ops/triton/mask.py:60-102: for one query row
// the visible key columns form up to three intervals (near band, distant band, sink prefix).
struct RowMask {
  int diag;            // last causally visible column: q_idx + (sk - sq)
  int near_lo;         // near band    = (near_lo, diag]
  int far_lo, far_hi;  // distant band = (far_lo, far_hi]
  int sink_hi;         // sink         = [0, sink_hi) intersected with [0, diag]
  int sk;
  bool row_ok;
};

// Visible columns of one row inside key tile [k0, k0 + TN), as three half-open intervals of the
// tile-local index, already clipped to the key length. Unused intervals are empty (len 0).
struct TileMask {
  int lo[3];
  unsigned len[3];
};

__device__ __forceinline__ TileMask make_tile_mask(const RowMask& rm, int mode, int k0) {
  TileMask tm;
  const int seq_hi = rm.row_ok ? min(rm.sk - k0, TN) : 0;
  auto clip = [&](int idx, int a, int b) {  // [a, b) in key coordinates -> tile-local, clipped
    a = max(a - k0, 0);
    b = min(b - k0, seq_hi);
    tm.lo[idx] = a;
    tm.len[idx] = b > a ? unsigned(b - a) : 0u;
  };
  if (mode == FSA_MASK_SEQLEN) {
    clip(0, 0, rm.sk);
    clip(1, 0, 0);
    clip(2, 0, 0);
  } else if (mode == FSA_MASK_CAUSAL) {
    clip(0, 0, rm.diag + 1);
    clip(1, 0, 0);
    clip(2, 0, 0);
  } else {
    clip(0, rm.near_lo + 1, rm.diag + 1);
    clip(1, rm.far_lo + 1, rm.far_hi + 1);
    if (mode == FSA_MASK_LOCAL_SINK)
      clip(2, 0, min(rm.sink_hi, rm.diag + 1));
    else
      clip(2, 0, 0);
  }
  return tm;
}
__device__ __forceinline__ bool tile_col_visible(const TileMask& tm, int i) {
  return (unsigned(i - tm.lo[0]) < tm.len[0]) | (unsigned(i - tm.lo[1]) < tm.len[1]) |
         (unsigned(i - tm.lo[2]) < tm.len[2]);
}

// BSCALE: FP8 inputs with one scale per 128-position block (a separate instantiation: as a run-time switch it cost
// the per-tensor FP8 forward 10 %).
template <int HD, typename T, int KIND, bool BSCALE = false>
__global__ void __launch_bounds__(NTHREADS, 1) fwd_kernel(const __grid_constant__ FwdKernelParams p) {
  // T is the element type of Q, K, V and of P: bf16 / fp16 (kind::f16) or FP8 e4m3 / e5m2 (kind::f8f6f4,
  // flash_sparse_attn/ops/triton/flash_sparse_fwd.py:49, :84-86 under IS_QUANT). Outputs and the gate
  // vectors are 16-bit (bf16 for FP8 inputs, flash_sparse_fwd.py:634).
  constexpr int ES = sizeof(T);
  constexpr bool F8 = ES == 1;
  constexpr int SLAB = 128 / ES;      // elements per 128-byte swizzle row
  using TO = typename OutType<T>::type;
  using SM = FwdSmem<HD, ES>;
  constexpr int KK_QK = HD * ES / 32;  // MMAs per S tile: every MMA consumes 32 bytes of the head dimension
  constexpr int KK_PV = TN * ES / 32;  // MMAs per P V tile: 32 bytes of the key dimension each
  constexpr int OCH = HD / 32;        // 32-column chunks of an O tile
  constexpr int QT = FwdShape<HD>::QT, KSTAGES = FwdShape<HD>::KSTAGES, VSTAGES = FwdShape<HD>::VSTAGES;
  constexpr bool IS_BF16 = (sizeof(T) == 2) && !__is_same(T, __half);
  static_assert(!F8 || HD == 128, "FP8 tiles are one 128-byte swizzle row wide");
  constexpr uint32_t TMEM_S0 = 0, TMEM_O0 = 256;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  FwdBars* bars = reinterpret_cast<FwdBars*>(smem + SM::kBar);
  volatile int* abort_flag = &bars->abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool causal = p.flags & F_CAUSAL, local = p.flags & F_LOCAL, split_kv = p.flags & F_SPLIT;

  // ---- work decode: heads fastest (K/V reuse in L2), heavy query tiles first --------------------
  SeqInfo si;
  int pair;
  {
    int idx = blockIdx.x;
    si.head = idx % p.hgrid;
    idx /= p.hgrid;
    const int bs = idx % (p.B * p.num_splits);
    pair = p.num_pairs - 1 - idx / (p.B * p.num_splits);
    si.b = bs / p.num_splits;
    si.split = bs - si.b * p.num_splits;
    si.hkv = (p.flags & F_PACK_GQA) ? si.head : si.head / p.G;
    si.off_q = (p.flags & F_VARLEN_Q) ? p.cu_q[si.b] : 0;
    si.off_k = (p.flags & F_VARLEN_K) ? p.cu_k[si.b] : 0;
    si.sq = (p.flags & F_USED_Q) ? p.used_q[si.b]
                                 : ((p.flags & F_VARLEN_Q) ? p.cu_q[si.b + 1] - si.off_q : p.sq);
    si.sk = (p.flags & F_USED_K) ? p.used_k[si.b]
                                 : ((p.flags & F_VARLEN_K) ? p.cu_k[si.b + 1] - si.off_k : p.sk);
    if (local) {
      const int* wp = p.windows + (long long)si.hkv * p.win_stride;
      si.w.sink = wp[0];
      si.w.left = wp[1];
      si.w.right = wp[2];
      si.w.near_ = wp[3];
    } else {
      si.w.sink = si.w.left = si.w.right = si.w.near_ = 0;
    }
  }
  const int gpack = p.gpack;
  const int m_blocks_here = fsa_cdiv(si.sq * gpack, TM);  // query tiles this sequence really has

  // Both groups' schedules are needed by every role.
  FsaFwdSched sched[2];
  bool q_valid[2];
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    const int mb = pair * QT + q;
    q_valid[q] = q < QT && mb < m_blocks_here;
    // One query position with windows and split-KV: the reference's rounding drops the first, partial tile of
    // the near band (block_info.py:60-64) although its eager ground truth sees those keys; like the decode
    // kernel, this one visits them (the flag only matters for that combination).
    sched[q] = fsa_fwd_schedule(si.sq, si.sk, mb, si.split, si.w, p.num_splits, TN, TM, causal, local, split_kv,
                                gpack, /*cover_single_query=*/true);
    if (!q_valid[q] || fsa_fwd_sched_empty(sched[q])) {
      sched[q].n_min = sched[q].n_max = sched[q].n_max_no_mask = 0;
      sched[q].win_min = sched[q].win_max = sched[q].win_min_no_mask = sched[q].win_max_no_mask = 0;
      sched[q].sink_min = sched[q].sink_max = 0;
    }
  }
  auto first_tile = [&]() {
    const int a = fsa_fwd_next_tile_below(sched[0], 1 << 28, local);
    const int b = fsa_fwd_next_tile_below(sched[1], 1 << 28, local);
    return fsa_imax(a, b);
  };
  auto next_tile = [&](int n) {
    // common case first: the tile just below is visited by one of the two groups
    const int c = n - 1;
    if (!local && ((c >= sched[0].n_min && c < sched[0].n_max) || (c >= sched[1].n_min && c < sched[1].n_max))) return c;
    const int a = fsa_fwd_next_tile_below(sched[0], n, local);
    const int b = fsa_fwd_next_tile_below(sched[1], n, local);
    return fsa_imax(a, b);
  };

  // ---- gated: which tiles each group really computes ---------------------------------------------
  // The gate bound of a tile (flash_sparse_attn/ops/triton/activations.py:265-299) needs only the extremes of alpha
  // over the query tile and of delta over the key tile - both computed beforehand by gate_ext_kernel - and one
  // running scalar per query tile. So every role (producer, MMA issuer, delta stager, softmax warps) walks the
  // tiles with its own copy of that scalar and reaches the same decisions without talking to the others: a tile
  // that both groups skip is never loaded, multiplied or staged (flash_gated_fwd.py:54-56 runs nothing for it).
  // The first tile of a group is never skipped: its running bound starts at -inf, the difference is +inf.
  float gw_amax[2] = {0.f, 0.f}, gw_amin[2] = {0.f, 0.f}, gw_thr[2] = {0.f, 0.f}, gw_run[2] = {-INFINITY, -INFINITY};
  float gw_c = 0.f;
  const float2* gw_dext = nullptr;
  if (KIND == KIND_GATED) {
    gw_c = p.qkv_scale ? p.scale_log2 * p.qkv_scale[0] * p.qkv_scale[1] : p.scale_log2;
    const float2* aext = reinterpret_cast<const float2*>(p.gate_ws);
    gw_dext = aext + (long long)p.B * p.hgrid * p.num_m_blocks + ((long long)si.b * p.Hkv + si.hkv) * p.n_tiles_k;
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const int mb = pair * QT + q;
      if (mb < p.num_m_blocks) {
        const float2 e = __ldg(aext + ((long long)si.b * p.hgrid + si.head) * p.num_m_blocks + mb);
        gw_amax[q] = e.x;
        gw_amin[q] = e.y;
      }
      // flash_sparse_attn/ops/triton/seqlen_info.py:156-191: the adaptive bound is smallest at the tile's first row
      float g_thr = p.gate_thr;
      if (causal && (p.flags & F_ADAPT_GATE))
        g_thr = p.gate_thr * (float((mb * TM) / gpack + (si.sk - si.sq)) + 1.0f) / float(si.sk);
      gw_thr[q] = log2f(g_thr);
    }
  }
  // Next tile below n_prev that at least one group computes; keep[q] says which. mark_q >= 0: this thread records
  // the gate-skipped tiles of group mark_q in the tile map (value 3).
  auto walk_next = [&](int n_prev, bool* keep, int mark_q) -> int {
    int n = next_tile(n_prev);
    if constexpr (KIND != KIND_GATED) {
      keep[0] = n >= 0 && fsa_fwd_tile_mode(sched[0], n, causal, local) >= 0;
      keep[1] = n >= 0 && fsa_fwd_tile_mode(sched[1], n, causal, local) >= 0;
      return n;
    } else {
    while (n >= 0) {
      const float2 de = __ldg(gw_dext + n);  // (max, min) of delta over the key tile
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        keep[q] = fsa_fwd_tile_mode(sched[q], n, causal, local) >= 0;
        if (keep[q]) {
          const float gmc = fmaxf(fmaxf(gw_amax[q] * de.x, gw_amax[q] * de.y), fmaxf(gw_amin[q] * de.x, gw_amin[q] * de.y));
          const bool skip = (gmc - gw_run[q]) * gw_c < gw_thr[q];
          if (!skip) gw_run[q] = fmaxf(gmc, gw_run[q]);
          keep[q] = !skip;
          if (skip && mark_q == q && p.tile_map) {
            const int mb = pair * QT + q;
            p.tile_map[((((long long)si.b * p.hgrid + si.head) * p.num_m_blocks + mb) * p.num_splits + si.split) *
                           p.n_tiles_k + n] = 3;
          }
        }
      }
      if (keep[0] || keep[1]) return n;
      n = next_tile(n);
    }
    keep[0] = keep[1] = false;
    return -1;
    }
  };
  constexpr int WALK_START = 1 << 28;

  // ---- setup ---------------------------------------------------------------------------------
  if (tid == 0) {
    mbar_init(&bars->q_full, 1);
    mbar_init(&bars->k0_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->kv_full[s], 2);
      mbar_init(&bars->kv_empty[s], 1);
    }
    for (int q = 0; q < 2; ++q) {
      mbar_init(&bars->s_full[q], 1);
      mbar_init(&bars->p_full[q], 4);  // one arrival per warp of the group
      mbar_init(&bars->o_final[q], 1);
      mbar_init(&bars->wg_sync[q], 4);
      mbar_init(&bars->d_full[q], 1);
      mbar_init(&bars->d_empty[q], 8);
    }
    bars->abort_flag = (*reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    mbar_fence_init();
  }
  if (warp == 8) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  const int kv_row_coord_b = (p.flags & (F_VARLEN_K | F_PAGED)) ? 0 : si.b;

  // Register budget: the two softmax groups hold a 128-wide fp32 output row per thread and take
  // the registers the third warpgroup does not need.
  if (warp >= 8) {
    // third warpgroup: all four warps release registers at the same instruction
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
  if (warp == 8) {
    // =============================== producer ================================================
    if (lane == 0 && !*abort_flag) {
      tma_prefetch_desc(&p.map_q);
      tma_prefetch_desc(&p.map_k);
      tma_prefetch_desc(&p.map_v);
      // Q tiles
      {
        uint32_t bytes = 0;
        for (int q = 0; q < 2; ++q)
          if (q_valid[q]) bytes += SM::kTileBytes;
        if (bytes) {
          mbar_arrive_expect_tx(&bars->q_full, bytes);
          for (int q = 0; q < 2; ++q) {
            if (!q_valid[q]) continue;
            const int mb = pair * QT + q;
            uint8_t* dst = smem + SM::kQ + q * SM::kTileBytes;
            const int row0 = (mb * TM) / gpack;  // token index of the tile's first row
            const int head0 = (p.flags & F_PACK_GQA) ? si.hkv * p.G : si.head;
            const int bq = (p.flags & F_VARLEN_Q) ? 0 : si.b;
            for (int d = 0; d < HD; d += SLAB)
              tma_load_4d(dst + (d / SLAB) * (TM * 128), &p.map_q, &bars->q_full, d, head0, si.off_q + row0, bq);
          }
        }
      }
      auto load_kv = [&](const CUtensorMap* map, uint8_t* dst, uint64_t* bar, int n) {
        // one 128-key tile = HD/64 column slabs x (paged: several pages | one box)
        if (p.flags & F_PAGED) {
          const int rows_per_box = p.page_size < TN ? p.page_size : TN;
          const int nbox = TN / rows_per_box;
          uint32_t bytes = 0;
          int pages[4];
          for (int i = 0; i < nbox; ++i) {
            const int r0 = n * TN + i * rows_per_box;
            pages[i] = (r0 < si.sk) ? p.page_table[(long long)si.b * p.pt_stride + r0 / p.page_size] : -1;
            if (pages[i] >= 0) bytes += rows_per_box * HD * ES;
          }
          mbar_arrive_expect_tx(bar, bytes);
          for (int i = 0; i < nbox; ++i) {
            if (pages[i] < 0) continue;
            const int r0 = n * TN + i * rows_per_box;
            for (int d = 0; d < HD; d += SLAB)
              tma_load_4d(dst + (d / SLAB) * (TN * 128) + i * rows_per_box * 128, map, bar, d, si.hkv,
                          r0 % p.page_size, pages[i]);
          }
        } else {
          mbar_arrive_expect_tx(bar, SM::kTileBytes);
          for (int d = 0; d < HD; d += SLAB)
            tma_load_4d(dst + (d / SLAB) * (TN * 128), map, bar, d, si.hkv, si.off_k + n * TN, kv_row_coord_b);
        }
      };
      int t = 0, seen = 0;
      bool ok = true;
      bool keep_unused[2];
      int n = (KIND == KIND_GATED) ? walk_next(WALK_START, keep_unused, -1) : first_tile();
      if (n >= 0) {
        load_kv(&p.map_k, smem + SM::kK, &bars->k0_full, n);
      }
      while (n >= 0 && ok) {
        const int n_next = (KIND == KIND_GATED) ? walk_next(n, keep_unused, -1) : next_tile(n);
        // Release signals arrive in order (signal c: K(c) and V(c - 1) consumed). V(t) goes into the slot of
        // V(t - 2) and K(t + 1) into the slot of K(t - 1): both free after signal t - 1.
        auto need_signal = [&](int c) {
          while (ok && seen <= c) {
            ok = mbar_wait(&bars->kv_empty[seen & 1], (seen >> 1) & 1, abort_flag);
            ++seen;
          }
        };
        // V(t) replaces V(t - VSTAGES), K(t + 1) replaces K(t + 1 - KSTAGES): both are free after this signal
        need_signal(t - (KSTAGES < VSTAGES ? KSTAGES : VSTAGES) + 1);
        if (!ok) break;
        // V is prefetched like K, before the softmax groups have voted on the tile: waiting for the vote
        // would put a full load latency between every S tile and its P V product, and in this
        // tensor-bound kernel a V tile that ends up unused only costs an L2 read: on inputs where 82 % of the
        // tiles are skipped, leaving ALL V loads out changed the kernel time by 1 % (1.476 -> 1.462 ms at
        // S = 16384), so L2 traffic is not what a skipped tile costs. (The reference skips the load,
        // flash_sparse_fwd.py:60-88; it matters there because its tiles are loaded by the same warps that
        // compute.) A skipped tile still skips the softmax work and the P V product.
        load_kv(&p.map_v, smem + SM::kV + (t % VSTAGES) * SM::kTileBytes, &bars->kv_full[t & 1], n);
        if (n_next >= 0)
          load_kv(&p.map_k, smem + SM::kK + ((t + 1) % KSTAGES) * SM::kTileBytes, &bars->kv_full[t & 1], n_next);
        else
          mbar_arrive(&bars->kv_full[t & 1]);  // the barrier counts two arrivals per step
        n = n_next;
        ++t;
      }
    }
    __syncwarp();
  } else if (warp == 10) {
    // =============================== delta stager (gated only) ================================
    // delta of every visited key tile as fp32 in a 2-slot ring, with the tile's max / min for the
    // gate bound (flash_sparse_attn/ops/triton/flash_gated_fwd.py:100-115). Keys past the sequence
    // read as 0, like the reference's masked load (scheduler.py:1674-1691).
    if (KIND == KIND_GATED) {
      bool ok = !*abort_flag;
      const TO* dbase = reinterpret_cast<const TO*>(p.delta);
      int t = 0;
      bool keep_unused[2];
      for (int n = walk_next(WALK_START, keep_unused, -1); n >= 0 && ok; n = walk_next(n, keep_unused, -1), ++t) {
        const int s = t & 1, use = t >> 1;
        if (use > 0) ok = mbar_wait(&bars->d_empty[s], (use - 1) & 1, abort_flag);
        if (!ok) break;
        float dv[4];
        float dmax = -INFINITY, dmin = INFINITY;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int k = n * TN + lane * 4 + j;
          float v = 0.f;
          if (k < si.sk) {
            long long e;
            if (p.flags & F_PAGED) {
              const int page = p.page_table[(long long)si.b * p.pt_stride + k / p.page_size];
              e = (long long)page * p.d_sb + (long long)si.hkv * p.d_sh + (k % p.page_size);
            } else {
              e = (long long)((p.flags & F_VARLEN_K) ? 0 : si.b) * p.d_sb + (long long)si.hkv * p.d_sh + si.off_k + k;
            }
            v = float(dbase[e]);
          }
          dv[j] = v;
          dmax = fmaxf(dmax, v);
          dmin = fminf(dmin, v);
        }
#pragma unroll
        for (int sft = 16; sft > 0; sft >>= 1) {
          dmax = fmaxf(dmax, __shfl_xor_sync(0xffffffffu, dmax, sft));
          dmin = fminf(dmin, __shfl_xor_sync(0xffffffffu, dmin, sft));
        }
        *reinterpret_cast<float4*>(&bars->dl[s][lane * 4]) = make_float4(dv[0], dv[1], dv[2], dv[3]);
        if (lane == 0) {
          bars->dl[s][TN] = dmax;
          bars->dl[s][TN + 1] = dmin;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->d_full[s]);
      }
    }
  } else if (warp == 9) {
    // =============================== MMA issuer ==============================================
    constexpr int F8_FMT = __is_same(T, __nv_fp8_e5m2) ? 1 : 0;
    constexpr uint32_t idesc_s = F8 ? umma_idesc_f8(TM, TN, F8_FMT, F8_FMT, false, false)
                                    : umma_idesc_f16(TM, TN, IS_BF16, false, false);
    constexpr uint32_t idesc_o = F8 ? umma_idesc_f8(TM, HD, F8_FMT, F8_FMT, false, true)
                                    : umma_idesc_f16(TM, HD, IS_BF16, false, true);
    const uint32_t sQ = smem_u32(smem + SM::kQ), sK = smem_u32(smem + SM::kK), sV = smem_u32(smem + SM::kV);
    bool ok = !*abort_flag;
    int cnt[2] = {0, 0};
    bool o_started[2] = {false, false};
    bool act[2], last[2];
    int n = (KIND == KIND_GATED) ? walk_next(WALK_START, act, -1) : first_tile();
    // Every lane runs the same (warp-uniform) descriptor arithmetic; the MMA and commit instructions carry the
    // one-lane predicate themselves.
    const uint32_t lead = lane == 0 ? 1u : 0u;
    const uint32_t dq_lo = umma_desc_lo(sQ, 16), dk_lo = umma_desc_lo(sK, 16), dv_lo = umma_desc_lo(sV, TN * 128);
    // The MMA loops are unrolled where this warp is the critical resource (dense and sparse kinds: rolled they cost
    // 9-14 %) and stay rolled for the gated kind, whose softmax warps carry the gate arithmetic (5 % faster rolled).
    constexpr int ISSUE_UNROLL = (KIND == KIND_GATED) ? 1 : 8;
    auto issue_s = [&](int q, int ks) {
      const uint32_t aq = dq_lo + ((q * SM::kTileBytes) >> 4), bk = dk_lo + ((ks * SM::kTileBytes) >> 4);
#pragma unroll ISSUE_UNROLL
      for (int kk = 0; kk < KK_QK; ++kk) {
        const uint32_t koff = (kk >> 2) * (TM * 128) + (kk & 3) * 32;
        if (F8)
          umma_f8_ss_lead(lead, tmem_base + TMEM_S0 + q * 128, umma_desc_at(aq, koff), umma_desc_at(bk, koff), idesc_s,
                          kk > 0);
        else
          umma_ss_lead(lead, tmem_base + TMEM_S0 + q * 128, umma_desc_at(aq, koff), umma_desc_at(bk, koff), idesc_s,
                       kk > 0);
      }
      umma_commit_lead(lead, &bars->s_full[q]);
    };
    if (n >= 0 && ok) {
      ok = mbar_wait(&bars->q_full, 0, abort_flag);
      ok = ok && mbar_wait(&bars->k0_full, 0, abort_flag);
      tc_fence_after();
      if (ok) {
        for (int q = 0; q < 2; ++q)
          if ((KIND == KIND_GATED) ? act[q] : (fsa_fwd_tile_mode(sched[q], n, causal, local) >= 0)) issue_s(q, 0);
        umma_commit_lead(lead, &bars->kv_empty[0]);
      }
    }
    int t = 0;
    // The tensor pipe takes an MMA from a thread about as fast as it executes one: while its MMAs run this warp
    // is blocked in their issue, and whatever it does between a group publishing P and the next MMA is time the
    // pipe idles. So everything that does not depend on P (the walk over the tiles, who takes part in the next
    // tile, the K / V arrivals) happens before the wait for P. (One issuer per group was tried: the second
    // polling warp slows the softmax warps of its scheduler more than the overlap gains.)
    if (KIND != KIND_GATED) {
#pragma unroll
      for (int q = 0; q < 2; ++q) act[q] = n >= 0 && fsa_fwd_tile_mode(sched[q], n, causal, local) >= 0;
    }
    while (n >= 0 && ok) {
      bool act_next[2];
      const int n_next = (KIND == KIND_GATED) ? walk_next(n, act_next, -1) : next_tile(n);
      const int vs = t % VSTAGES;
      const int ks_next = (t + 1) % KSTAGES;
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        if (KIND == KIND_GATED) {
          // whether a later tile of this group survives the gate is not known yet: the output barriers are
          // committed after the loop instead
          last[q] = false;
        } else if (!local) {  // one contiguous range of tiles per group
          act_next[q] = n_next >= sched[q].n_min && n_next < sched[q].n_max;
          last[q] = act[q] && n == sched[q].n_min;
        } else {
          act_next[q] = n_next >= 0 && fsa_fwd_tile_mode(sched[q], n_next, causal, local) >= 0;
          last[q] = act[q] && fsa_fwd_next_tile_below(sched[q], n, local) < 0;
        }
      }
      ok = mbar_wait(&bars->kv_full[t & 1], (t >> 1) & 1, abort_flag);  // V(t) and K(t + 1)
      if (!ok) break;
      if ((p.flags & F_KV_RAGGED) && (n + 1) * TN > si.sk) {
        // keys past the sequence end carry probability 0 but their V rows may hold
        // anything: clear them so that 0 * garbage cannot produce NaN
        const int r0 = si.sk - n * TN;
        uint8_t* vt = smem + SM::kV + vs * SM::kTileBytes;
        constexpr int CPR = HD * ES / 16;  // 16-byte chunks per row
        for (int i = lane; i < (TN - r0) * CPR; i += 32) {
          const int r = r0 + i / CPR, c = i % CPR;
          *reinterpret_cast<uint4*>(vt + (c >> 3) * (TN * 128) + sw128_offset(r, c & 7)) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async_smem();
        __syncwarp();
      }
      const uint32_t bv = dv_lo + ((vs * SM::kTileBytes) >> 4);
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        if (act[q]) {
          ok = ok && mbar_wait(&bars->p_full[q], cnt[q] & 1, abort_flag);
          if (!ok) break;
          const bool skip = (KIND != KIND_DENSE) && bars->skip_flag[q][cnt[q] & 1];
          cnt[q]++;
          tc_fence_after();
          if (!skip) {
#pragma unroll ISSUE_UNROLL
            for (int kk = 0; kk < KK_PV; ++kk) {
              if (F8)
                umma_f8_ts_lead(lead, tmem_base + TMEM_O0 + q * 128, tmem_base + TMEM_S0 + q * 128 + kk * 8,
                                umma_desc_at(bv, kk * 4096), idesc_o, (kk > 0 || o_started[q]) ? 1u : 0u);
              else
                umma_ts_lead(lead, tmem_base + TMEM_O0 + q * 128, tmem_base + TMEM_S0 + q * 128 + kk * 8,
                             umma_desc_at(bv, kk * 2048), idesc_o, (kk > 0 || o_started[q]) ? 1u : 0u);
            }
            o_started[q] = true;
          }
          // last key tile of this group: tell it when its output is complete
          if (last[q]) umma_commit_lead(lead, &bars->o_final[q]);
        }
        if (act_next[q]) {
          if (!act[q]) tc_fence_after();
          issue_s(q, ks_next);
        }
      }
      if (!ok) break;
      // signal t + 1: V(t) and K(t + 1) are free once the MMAs issued so far have completed
      umma_commit_lead(lead, &bars->kv_empty[(t + 1) & 1]);
      n = n_next;
      act[0] = act_next[0];
      act[1] = act_next[1];
      ++t;
    }
    if (KIND == KIND_GATED && ok) {
      // completion of everything issued so far = both outputs are final
      for (int q = 0; q < 2; ++q)
        if (o_started[q]) umma_commit_lead(lead, &bars->o_final[q]);
    }
  }
  } else {
    // =============================== softmax groups ==========================================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    const int q = warp >> 2;        // group / query tile
    const int wq = warp & 3;        // warp within group == TMEM lane quadrant
    const int row = wq * 32 + lane; // row within the tile
    const int mb = pair * QT + q;
    const uint32_t lane_addr = uint32_t(wq * 32) << 16;
    const uint32_t tS = tmem_base + lane_addr + TMEM_S0 + q * 128;
    const uint32_t tO = tmem_base + lane_addr + TMEM_O0 + q * 128;

    const int offs_m = mb * TM + row;
    const int q_idx = offs_m / gpack;
    const int q_head = (p.flags & F_PACK_GQA) ? si.hkv * p.G + (offs_m - q_idx * gpack) : si.head;
    RowMask rm;
    rm.row_ok = q_idx < si.sq;
    rm.sk = si.sk;
    rm.diag = q_idx + (si.sk - si.sq);
    rm.near_lo = rm.diag - si.w.near_;
    rm.far_hi = rm.diag - si.w.near_ - si.w.right;
    rm.far_lo = rm.far_hi - si.w.left;
    rm.sink_hi = si.w.sink;
    const FsaFwdSched my = sched[q];  // registers, not the indexed copy

    float thr_log2 = 0.f;
    if (KIND != KIND_DENSE) {
      // flash_sparse_attn/ops/triton/seqlen_info.py:118-153
      const float visible = causal ? float(q_idx + (si.sk - si.sq) + 1) : float(si.sk);
      thr_log2 = log2f(fmaxf(fminf(p.softmax_thr / visible, 1.0f), 0.0f));
    }
    // Block-scaled FP8: the scale of the logits changes from key tile to key tile, so the scores are multiplied by it
    // right after they leave TMEM and everything below works on scaled logits (cc = 1). The value block's scale is
    // folded into P relative to a running reference v_run - the largest value scale this row has met so far - and
    // the output accumulator is rescaled when that reference grows (like the running maximum); the output is
    // multiplied by the final reference. Blocks more than 2^9 below the running reference underflow in FP8 P, i.e.
    // contributions that small relative to the largest block a row has seen are dropped.
    constexpr bool bscaled = F8 && BSCALE;
    const float* kbs = bscaled ? p.k_bscale + ((long long)si.b * p.Hkv + si.hkv) * p.n_tiles_k : nullptr;
    const float* vbs = bscaled ? p.v_bscale + ((long long)si.b * p.Hkv + si.hkv) * p.n_tiles_k : nullptr;
    const float c = bscaled ? p.scale_log2 * p.q_bscale[((long long)si.b * p.Hq + q_head) * p.num_m_blocks +
                                                        (mb < p.num_m_blocks ? mb : 0)]
                            : (p.qkv_scale ? p.scale_log2 * p.qkv_scale[0] * p.qkv_scale[1] : p.scale_log2);
    const float cc = bscaled ? 1.0f : c;  // factor between the values held in sr[] and base-2 logits
    float v_run = 0.f;  // block-scaled: running reference of the value scale (uniform over the tile's rows)
    const float v_scale = p.qkv_scale ? p.qkv_scale[2] : p.v_scale;
    float m_ref = -INFINITY;  // reference maximum all stored exponentials are relative to
    float l_ref = 0.f;        // sum of exp2((s - m_ref) * c)
    float lg_l = -INFINITY;   // log2(l_ref) for the skip test, refreshed at the end of a tile (off the S -> P path)
    bool have_o = false;      // some P V has been issued for this tile
    int cnt_s = 0;
    bool ok = !*abort_flag;
    const bool has_work = q_valid[q] && !fsa_fwd_sched_empty(my);

    // ---- gated: alpha of this row ----------------------------------------------------------------------
    float alpha = 0.f;
    if (KIND == KIND_GATED) {
      if (rm.row_ok && q_valid[q]) {
        const TO* ab = reinterpret_cast<const TO*>(p.alpha);
        alpha = float(ab[(long long)((p.flags & F_VARLEN_Q) ? 0 : si.b) * p.a_sb + (long long)q_head * p.a_sh +
                         si.off_q + q_idx]);
      }
    }

    int t_merged = -1;
    bool keep[2] = {false, false};
    const int mark_q = (wq == 0 && lane == 0) ? q : -1;  // one thread per group records its gate-skipped tiles
    int n = -1;
    if (KIND == KIND_GATED)
      n = walk_next(WALK_START, keep, mark_q);
    else if (has_work)
      n = first_tile();
    for (; n >= 0 && ok; n = (KIND == KIND_GATED) ? walk_next(n, keep, mark_q) : next_tile(n)) {
      ++t_merged;
      const int mode = has_work ? fsa_fwd_tile_mode(my, n, causal, local) : -1;
      const int ds = t_merged & 1;
      if (KIND == KIND_GATED) {
        // every tile that reaches this loop was staged by the delta warp (one of the groups computes it)
        ok = mbar_wait(&bars->d_full[ds], (t_merged >> 1) & 1, abort_flag);
        if (!ok) break;
        if (!keep[q]) {  // not in this group's schedule, or skipped by its gate: nothing was issued for it
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars->d_empty[ds]);
          continue;
        }
      } else if (mode < 0) {
        continue;
      }
      ok = mbar_wait(&bars->s_full[q], cnt_s & 1, abort_flag);
      if (!ok) break;
      tc_fence_after();
      const int par = cnt_s & 1;
      cnt_s++;
      const int k0 = n * TN;

      // ---- scores of this row: TMEM -> registers (warp-collective loads, one wait) ---------------
      uint32_t sr[TN];
#pragma unroll
      for (int ch = 0; ch < TN / 32; ++ch) tmem_ld32(tS + ch * 32, &sr[ch * 32]);
      tmem_ld_wait();
      float p_mul = 1.0f, o_mul = 1.0f;
      if constexpr (F8) {
        if (bscaled) {
          const float ct = c * kbs[n];
#pragma unroll
          for (int i = 0; i < TN; ++i) sr[i] = __float_as_uint(__uint_as_float(sr[i]) * ct);
        }
      }
      if (KIND == KIND_GATED) {
        // logits = (q.k + g(alpha * delta_j)) * scale, g = logsigmoid or identity
        // (flash_sparse_attn/ops/triton/flash_gated_fwd.py:104-122, activations.py:245-262)
        const float4* d4 = reinterpret_cast<const float4*>(&bars->dl[ds][0]);
        const bool logsig = p.flags & F_LOGSIGMOID;
#pragma unroll
        for (int i = 0; i < TN; i += 4) {
          const float4 dd = d4[i >> 2];
          const float dv[4] = {dd.x, dd.y, dd.z, dd.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float x = alpha * dv[j];
            float gte = x;
            if (logsig)
              gte = log_sigmoid_fast(x);
            sr[i + j] = __float_as_uint(__uint_as_float(sr[i + j]) + gte);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->d_empty[ds]);
      }
      if (mode != FSA_MASK_NONE) {
        const TileMask tm = make_tile_mask(rm, mode, k0);
        // most masked tiles leave every row one interval (causal diagonal, one window band, key tail):
        // one compare per entry instead of three
        const int n_iv = (tm.len[0] != 0u) + (tm.len[1] != 0u) + (tm.len[2] != 0u);
        if (__all_sync(0xffffffffu, n_iv <= 1)) {
          const int which = tm.len[1] != 0u ? 1 : (tm.len[2] != 0u ? 2 : 0);
          const int nlo = -(which == 1 ? tm.lo[1] : (which == 2 ? tm.lo[2] : tm.lo[0]));
          const unsigned len = which == 1 ? tm.len[1] : (which == 2 ? tm.len[2] : tm.len[0]);
#pragma unroll
          for (int i = 0; i < TN; ++i)
            if (unsigned(i + nlo) >= len) sr[i] = 0xff800000u;  // -inf
        } else {
#pragma unroll
          for (int i = 0; i < TN; ++i)
            if (!tile_col_visible(tm, i)) sr[i] = 0xff800000u;  // -inf
        }
      } else if (!rm.row_ok) {
        // rows past the query length read as zero scores in fully visible tiles
#pragma unroll
        for (int i = 0; i < TN; ++i) sr[i] = 0u;
      }

      // ---- row maximum ------------------------------------------------------------------------------
      float mx[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        mx[j] = fmaxf(__uint_as_float(sr[j * 32]), __uint_as_float(sr[j * 32 + 1]));
#pragma unroll
        for (int i = 2; i < 32; i += 2)
          mx[j] = max3(mx[j], __uint_as_float(sr[j * 32 + i]), __uint_as_float(sr[j * 32 + i + 1]));
      }
      const float m_cur = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));

      // ---- tile skip vote (flash_sparse_attn/ops/triton/activations.py:129-138) -----------------
      bool skip = false;
      if (KIND != KIND_DENSE) {
        const float d = (m_cur - m_ref) * cc - lg_l;
        const float val = d - thr_log2;
        const unsigned want = __ballot_sync(0xffffffffu, val >= 0.0f);
        const unsigned drop = __ballot_sync(0xffffffffu, val < 0.0f);
        // group-wide exchange through a (bounded) mbarrier rather than bar.sync, so that an
        // aborting pipeline can never leave part of the group parked on a hardware barrier
        if (lane == 0) {
          bars->vote_any[q][par][wq] = (want ? 1 : 0) | (drop ? 2 : 0);
          mbar_arrive(&bars->wg_sync[q]);
        }
        // a warp holding a row that wants the tile already knows the outcome ("keep") and moves on;
        // only warps whose rows all vote "skip" have to hear from the others. Every warp still
        // arrives once per tile, and none can reach the next tile's vote before all have arrived
        // here (the next S tile is only issued after all four warps published P or the skip).
        if (!want) {
          ok = mbar_wait(&bars->wg_sync[q], par, abort_flag);
          if (!ok) break;
          const int v = bars->vote_any[q][par][0] | bars->vote_any[q][par][1] | bars->vote_any[q][par][2] |
                        bars->vote_any[q][par][3];
          // max over rows ignores NaN rows; a tile is skipped iff that max is < 0
          skip = !(v & 1) && (v & 2);
        }
      }
      // The verdict goes to the MMA issuer (and to the tile map) right before this thread's arrival on p_full,
      // whose release orders it: for a kept tile that is after the exponentials, not in front of them.
      auto publish_verdict = [&](bool skipped) {
        if (KIND != KIND_DENSE && wq == 0 && lane == 0) {
          bars->skip_flag[q][par] = skipped ? 1 : 0;
          if (p.tile_map) {
            const long long idx =
                ((((long long)si.b * p.hgrid + si.head) * p.num_m_blocks + mb) * p.num_splits + si.split) *
                    p.n_tiles_k + n;
            p.tile_map[idx] = skipped ? 2 : 1;
          }
        }
      };
      if (skip) {
        publish_verdict(true);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->p_full[q]);
        continue;
      }

      // ---- move the reference maximum only when it lags by more than 2^8 -------------------------
      float m_cand = fmaxf(m_cur, m_ref);
      if (mode != FSA_MASK_NONE) m_cand = fmaxf(m_cand, -1e6f);
      const bool need = !((m_cand - m_ref) * cc <= 8.0f);  // also true on the first tile (m_ref = -inf)
      float scale = 1.0f;
      if (need) {
        scale = ex2_approx((m_ref - m_cand) * cc);
        m_ref = m_cand;
        l_ref *= scale;
      }
      if constexpr (F8) {
        if (bscaled) {  // only for a tile that is kept: a skipped tile must not move the reference
          const float svn = vbs[n];
          if (svn > v_run) {  // the accumulator moves to the larger unit (nothing to move before the first P V)
            o_mul = v_run > 0.f ? __fdividef(v_run, svn) : 1.0f;
            v_run = svn;
          }
          p_mul = v_run > 0.f ? __fdividef(svn, v_run) : 0.0f;
        }
      }
      // s_full for this tile was committed after the previous P V of this group, so O is at rest
      if (have_o && (__any_sync(0xffffffffu, need) || o_mul != 1.0f)) {
        const float o_scale = scale * o_mul;
#pragma unroll
        for (int ch = 0; ch < OCH; ++ch) {
          uint32_t r[32];
          tmem_ld32(tO + ch * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * o_scale);
          tmem_st32(tO + ch * 32, r);
        }
      }

      // ---- P = exp2(S*c - m*c), row sum, publish P (16-bit pairs) over the S columns -----------------
      const float2 c2 = make_float2(cc, cc);
      const float neg_mc = -(m_ref * cc);
      const float2 nm2 = make_float2(neg_mc, neg_mc);
      float2 sum2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
      for (int ch = 0; ch < TN / 32; ++ch) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float2 ta = fma2(make_float2(__uint_as_float(sr[ch * 32 + i]), __uint_as_float(sr[ch * 32 + i + 1])),
                                 c2, nm2);
          const float2 tb =
              fma2(make_float2(__uint_as_float(sr[ch * 32 + i + 2]), __uint_as_float(sr[ch * 32 + i + 3])), c2, nm2);
          float2 ea, eb;
          ea.x = ex2_approx(ta.x);
          ea.y = ex2_approx(ta.y);
          eb.x = ex2_approx(tb.x);
          eb.y = ex2_approx(tb.y);
          sum2[0] = add2(sum2[0], ea);
          sum2[1] = add2(sum2[1], eb);
          if constexpr (F8) {
            pk[i >> 2] = bscaled ? pack4_fp8<T>(ea.x * p_mul, ea.y * p_mul, eb.x * p_mul, eb.y * p_mul)
                                 : pack4_fp8<T>(ea.x, ea.y, eb.x, eb.y);
          } else {
            pk[i >> 1] = pack2<T>(ea.x, ea.y);
            pk[(i >> 1) + 1] = pack2<T>(eb.x, eb.y);
          }
        }
        if constexpr (F8)
          tmem_st8(tS + ch * 8, pk);
        else
          tmem_st16(tS + ch * 16, pk);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      publish_verdict(false);
      if (lane == 0) mbar_arrive(&bars->p_full[q]);
      l_ref += (sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y);
      if (KIND != KIND_DENSE) lg_l = lg2_approx(l_ref);
      have_o = true;
    }

    // ---- epilogue (flash_sparse_attn/ops/triton/activations.py:169-203) ---------------------------
    if (ok && have_o) {
      ok = mbar_wait(&bars->o_final[q], 0, abort_flag);
      tc_fence_after();
    }
    if (ok && q_valid[q]) {
      const bool dead = (l_ref == 0.0f) || (l_ref != l_ref);
      const float inv = dead ? 1.0f : (bscaled ? v_run : v_scale) / l_ref;
      float lse = dead ? -INFINITY : m_ref * cc + log2f(l_ref);
      if (!(p.flags & F_LSE_LOG2)) lse *= 0.6931471805599453f;
      const long long tok = si.off_q + q_idx;
      if (rm.row_ok)
        p.lse[(long long)((p.flags & F_VARLEN_Q) ? 0 : si.b) * p.l_sb + (long long)q_head * p.l_sh +
              (long long)si.split * p.l_ss + ((p.flags & F_VARLEN_Q) ? tok : q_idx)] = lse;
      const long long obase = (long long)((p.flags & F_VARLEN_Q) ? 0 : si.b) * p.o_sb + tok * p.o_sm +
                              (long long)q_head * p.o_sh + (long long)si.split * p.o_ss;
#pragma unroll
      for (int ch = 0; ch < OCH; ++ch) {
        uint32_t r[32];
        if (have_o) {
          tmem_ld32(tO + ch * 32, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        if (rm.row_ok) {
          if (p.flags & F_SPLIT) {
            float* dst = reinterpret_cast<float*>(p.out) + obase + ch * 32;
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              if (ch * 32 + i < p.D)
                *reinterpret_cast<float4*>(dst + i) =
                    make_float4(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv,
                                __uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
          } else {
            TO* dst = reinterpret_cast<TO*>(p.out) + obase + ch * 32;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 v;
              v.x = pack2<TO>(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
              v.y = pack2<TO>(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
              v.z = pack2<TO>(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv);
              v.w = pack2<TO>(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv);
              if (ch * 32 + i < p.D) *reinterpret_cast<uint4*>(dst + i) = v;
            }
          }
        }
      }
    }
  }

  // ---- teardown ------------------------------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *abort_flag) atomicExch(p.status, 1);
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int HD, typename T, int KIND, bool BSCALE = false>
cudaError_t launch_one(const FwdKernelParams& p, cudaStream_t stream) {
  auto kern = fwd_kernel<HD, T, KIND, BSCALE>;
  constexpr int smem = FwdSmem<HD, sizeof(T)>::kTotal;
  static std::atomic<unsigned long long> opted_in{0};  // one bit per device: the attribute is per device
  if (cudaError_t e = smem_opt_in(kern, smem, opted_in); e != cudaSuccess) return e;
  const long long grid = (long long)p.num_pairs * p.hgrid * p.B * p.num_splits;
  if (grid <= 0) return cudaSuccess;
  kern<<<(unsigned)grid, NTHREADS, smem, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace

// kind: KIND_*, dtype: DT_BF16 / DT_FP16, head_dim: 64 or 128. Returns cudaErrorInvalidValue for
// unsupported combinations.

cudaError_t launch_fwd(const FwdKernelParams& p, int kind, int dtype, int head_dim, cudaStream_t stream) {
  if (p.k_bscale) {  // block-scaled FP8: dense and sparse kinds at head_dim 128
    if (head_dim != 128 || kind == KIND_GATED) return cudaErrorInvalidValue;
    if (dtype == DT_E4M3)
      return kind == KIND_DENSE ? launch_one<128, __nv_fp8_e4m3, KIND_DENSE, true>(p, stream)
                                : launch_one<128, __nv_fp8_e4m3, KIND_SPARSE, true>(p, stream);
    if (dtype == DT_E5M2)
      return kind == KIND_DENSE ? launch_one<128, __nv_fp8_e5m2, KIND_DENSE, true>(p, stream)
                                : launch_one<128, __nv_fp8_e5m2, KIND_SPARSE, true>(p, stream);
    return cudaErrorInvalidValue;
  }
#define FSA_FWD_CASE(HD_, T_, DT_)                                                  \
  if (head_dim == HD_ && dtype == DT_) {                                            \
    if (kind == KIND_DENSE) return launch_one<HD_, T_, KIND_DENSE>(p, stream);      \
    if (kind == KIND_SPARSE) return launch_one<HD_, T_, KIND_SPARSE>(p, stream);    \
    if (kind == KIND_GATED) return launch_one<HD_, T_, KIND_GATED>(p, stream);      \
  }
  FSA_FWD_CASE(128, __nv_bfloat16, DT_BF16)
  FSA_FWD_CASE(128, __half, DT_FP16)
  FSA_FWD_CASE(64, __nv_bfloat16, DT_BF16)
  FSA_FWD_CASE(64, __half, DT_FP16)
  FSA_FWD_CASE(192, __nv_bfloat16, DT_BF16)
  FSA_FWD_CASE(192, __half, DT_FP16)
  FSA_FWD_CASE(256, __nv_bfloat16, DT_BF16)
  FSA_FWD_CASE(256, __half, DT_FP16)
  FSA_FWD_CASE(128, __nv_fp8_e4m3, DT_E4M3)
  FSA_FWD_CASE(128, __nv_fp8_e5m2, DT_E5M2)
#undef FSA_FWD_CASE
  return cudaErrorInvalidValue;
}

}  // namespace fsa
