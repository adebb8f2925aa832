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
// The running output lives in registers: every P V lands in a fresh O tile that the owning
// softmax thread adds to its row accumulator before it publishes the next P.
#include "fsa_ptx.cuh"
#include "fsa_params.h"
#include "fsa_schedule.h"

namespace fsa {

namespace {

constexpr int TM = 128;  // query rows per softmax group
constexpr int TN = 128;  // keys per tile
constexpr int NTHREADS = 384;  // three warpgroups: softmax 0, softmax 1, {producer, MMA, 2 idle}
constexpr int KSTAGES = 2;
constexpr int VSTAGES = 2;

template <int HD>
struct FwdSmem {
  static constexpr int kTileBytes = TM * HD * 2;  // one Q / K / V tile of 16-bit elements
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + 2 * kTileBytes;
  static constexpr int kV = kK + KSTAGES * kTileBytes;
  static constexpr int kBar = kV + VSTAGES * kTileBytes;
  static constexpr int kTotal = kBar + 512 + 1024;  // barriers/flags + alignment slack
};

struct FwdBars {
  uint64_t q_full;
  uint64_t k_full[KSTAGES], k_empty[KSTAGES];
  uint64_t v_full[VSTAGES], v_empty[VSTAGES];
  uint64_t s_full[2], p_full[2], o_full[2], vote[2], wg_sync[2];
  uint32_t tmem_base;
  int abort_flag;
  int skip_flag[2][2];   // [group][parity of the group's tile counter]
  int vote_any[2][2][4]; // [group][parity][warp]: bit0 = some row wants the tile, bit1 = some row votes skip
};

struct SeqInfo {
  int b, split, head, hkv;  // head = query head, or kv head when packing GQA rows
  int off_q, off_k, sq, sk;
  FsaWindow w;
};

// Row-local view of the masks in flash_sparse_attn/ops/triton/mask.py:60-102: for one query row
// the visible key columns form up to three intervals.
struct RowMask {
  int diag;     // last causally visible column: q_idx + (sk - sq)
  int near_lo;  // near band  = (near_lo, diag]
  int far_lo, far_hi;  // distant band = (far_lo, far_hi]
  int sink_hi;  // sink = [0, sink_hi)
  int sk;
  bool row_ok;
};

__device__ __forceinline__ bool col_visible(const RowMask& rm, int mode, int k) {
  if (!(rm.row_ok && k < rm.sk)) return false;
  if (mode == FSA_MASK_SEQLEN) return true;
  if (mode == FSA_MASK_CAUSAL) return k <= rm.diag;
  bool ok = (k <= rm.diag && k > rm.near_lo) || (k <= rm.far_hi && k > rm.far_lo);
  if (mode == FSA_MASK_LOCAL_SINK) ok = ok || (k < rm.sink_hi && k <= rm.diag);
  return ok;
}

template <int HD, typename T, int KIND>
__global__ void __launch_bounds__(NTHREADS, 1) fwd_kernel(const __grid_constant__ FwdKernelParams p) {
  using SM = FwdSmem<HD>;
  constexpr int KK_QK = HD / 16;      // MMAs (K = 16) per S tile
  constexpr int KK_PV = TN / 16;      // MMAs per P V tile
  constexpr int OCH = HD / 32;        // 32-column chunks of an O tile
  constexpr bool IS_BF16 = (sizeof(T) == 2) && !__is_same(T, __half);
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
    const int mb = pair * 2 + q;
    q_valid[q] = mb < m_blocks_here;
    sched[q] = fsa_fwd_schedule(si.sq, si.sk, mb, si.split, si.w, p.num_splits, TN, TM, causal, local, split_kv,
                                gpack);
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
    const int a = fsa_fwd_next_tile_below(sched[0], n, local);
    const int b = fsa_fwd_next_tile_below(sched[1], n, local);
    return fsa_imax(a, b);
  };

  // ---- setup ---------------------------------------------------------------------------------
  if (tid == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < KSTAGES; ++s) {
      mbar_init(&bars->k_full[s], 1);
      mbar_init(&bars->k_empty[s], 1);
    }
    for (int s = 0; s < VSTAGES; ++s) {
      mbar_init(&bars->v_full[s], 1);
      mbar_init(&bars->v_empty[s], 1);
    }
    for (int q = 0; q < 2; ++q) {
      mbar_init(&bars->s_full[q], 1);
      mbar_init(&bars->p_full[q], 4);  // one arrival per warp of the group
      mbar_init(&bars->o_full[q], 1);
      mbar_init(&bars->vote[q], 1);
      mbar_init(&bars->wg_sync[q], 4);
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
            const int mb = pair * 2 + q;
            uint8_t* dst = smem + SM::kQ + q * SM::kTileBytes;
            const int row0 = (mb * TM) / gpack;  // token index of the tile's first row
            const int head0 = (p.flags & F_PACK_GQA) ? si.hkv * p.G : si.head;
            const int bq = (p.flags & F_VARLEN_Q) ? 0 : si.b;
            for (int d = 0; d < HD; d += 64)
              tma_load_4d(dst + (d / 64) * (TM * 128), &p.map_q, &bars->q_full, d, head0, si.off_q + row0, bq);
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
            if (pages[i] >= 0) bytes += rows_per_box * HD * 2;
          }
          mbar_arrive_expect_tx(bar, bytes);
          for (int i = 0; i < nbox; ++i) {
            if (pages[i] < 0) continue;
            const int r0 = n * TN + i * rows_per_box;
            for (int d = 0; d < HD; d += 64)
              tma_load_4d(dst + (d / 64) * (TN * 128) + i * rows_per_box * 128, map, bar, d, si.hkv,
                          r0 % p.page_size, pages[i]);
          }
        } else {
          mbar_arrive_expect_tx(bar, SM::kTileBytes);
          for (int d = 0; d < HD; d += 64)
            tma_load_4d(dst + (d / 64) * (TN * 128), map, bar, d, si.hkv, si.off_k + n * TN, kv_row_coord_b);
        }
      };
      int t = 0;
      int cnt[2] = {0, 0};
      bool ok = true;
      int n = first_tile();
      if (n >= 0) {
        load_kv(&p.map_k, smem + SM::kK, &bars->k_full[0], n);
      }
      while (n >= 0 && ok) {
        const int n_next = next_tile(n);
        if (n_next >= 0) {
          const int s = (t + 1) % KSTAGES;
          const int use = (t + 1) / KSTAGES;
          if (use > 0) ok = mbar_wait(&bars->k_empty[s], (use - 1) & 1, abort_flag);
          if (!ok) break;
          load_kv(&p.map_k, smem + SM::kK + s * SM::kTileBytes, &bars->k_full[s], n_next);
        }
        bool need_v = false;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          if (fsa_fwd_tile_mode(sched[q], n, causal, local) < 0) continue;
          if (KIND != KIND_DENSE) {
            ok = ok && mbar_wait(&bars->vote[q], cnt[q] & 1, abort_flag);
            if (ok && !bars->skip_flag[q][cnt[q] & 1]) need_v = true;
          } else {
            need_v = true;
          }
          cnt[q]++;
        }
        if (!ok) break;
        {
          const int s = t % VSTAGES;
          const int use = t / VSTAGES;
          if (use > 0) ok = mbar_wait(&bars->v_empty[s], (use - 1) & 1, abort_flag);
          if (!ok) break;
          if (need_v)
            load_kv(&p.map_v, smem + SM::kV + s * SM::kTileBytes, &bars->v_full[s], n);
          else
            mbar_arrive(&bars->v_full[s]);
        }
        n = n_next;
        ++t;
      }
    }
    __syncwarp();
  } else if (warp == 9) {
    // =============================== MMA issuer ==============================================
    constexpr uint32_t idesc_s = umma_idesc_f16(TM, TN, IS_BF16, false, false);
    constexpr uint32_t idesc_o = umma_idesc_f16(TM, HD, IS_BF16, false, true);
    const uint32_t sQ = smem_u32(smem + SM::kQ), sK = smem_u32(smem + SM::kK), sV = smem_u32(smem + SM::kV);
    bool ok = !*abort_flag;
    int cnt[2] = {0, 0};
    int n = first_tile();
    auto issue_s = [&](int q, int ks) {
      if (lane == 0) {
#pragma unroll
        for (int kk = 0; kk < KK_QK; ++kk) {
          const uint32_t koff = (kk >> 2) * (TM * 128) + (kk & 3) * 32;
          umma_ss(tmem_base + TMEM_S0 + q * 128, umma_smem_desc(sQ + q * SM::kTileBytes + koff, 16, 1024),
                  umma_smem_desc(sK + ks * SM::kTileBytes + koff, 16, 1024), idesc_s, kk > 0);
        }
        umma_commit(&bars->s_full[q]);
      }
      __syncwarp();
    };
    if (n >= 0 && ok) {
      ok = mbar_wait(&bars->q_full, 0, abort_flag);
      ok = ok && mbar_wait(&bars->k_full[0], 0, abort_flag);
      tc_fence_after();
      if (ok) {
        for (int q = 0; q < 2; ++q)
          if (fsa_fwd_tile_mode(sched[q], n, causal, local) >= 0) issue_s(q, 0);
        if (lane == 0) umma_commit(&bars->k_empty[0]);
        __syncwarp();
      }
    }
    int t = 0;
    while (n >= 0 && ok) {
      const int n_next = next_tile(n);
      const int vs = t % VSTAGES;
      bool v_ready = false, k_ready = false, any_pv = false;
      const int ks_next = (t + 1) % KSTAGES;
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        if (fsa_fwd_tile_mode(sched[q], n, causal, local) >= 0) {
          ok = ok && mbar_wait(&bars->p_full[q], cnt[q] & 1, abort_flag);
          if (!ok) break;
          const bool skip = (KIND != KIND_DENSE) && bars->skip_flag[q][cnt[q] & 1];
          cnt[q]++;
          if (!v_ready) {
            ok = mbar_wait(&bars->v_full[vs], (t / VSTAGES) & 1, abort_flag);
            if (!ok) break;
            v_ready = true;
            if ((p.flags & F_KV_RAGGED) && (n + 1) * TN > si.sk) {
              // keys past the sequence end carry probability 0 but their V rows may hold
              // anything: clear them so that 0 * garbage cannot produce NaN
              const int r0 = si.sk - n * TN;
              uint8_t* vt = smem + SM::kV + vs * SM::kTileBytes;
              for (int i = lane; i < (TN - r0) * (HD / 8); i += 32) {
                const int r = r0 + i / (HD / 8), c = i % (HD / 8);
                *reinterpret_cast<uint4*>(vt + (c >> 3) * (TN * 128) + sw128_offset(r, c & 7)) =
                    make_uint4(0, 0, 0, 0);
              }
              fence_proxy_async_smem();
              __syncwarp();
            }
          }
          tc_fence_after();
          if (!skip) {
            if (lane == 0) {
#pragma unroll
              for (int kk = 0; kk < KK_PV; ++kk) {
                umma_ts(tmem_base + TMEM_O0 + q * 128, tmem_base + TMEM_S0 + q * 128 + kk * 8,
                        umma_smem_desc(sV + vs * SM::kTileBytes + kk * 2048, TN * 128, 1024), idesc_o, kk > 0);
              }
              umma_commit(&bars->o_full[q]);
            }
            __syncwarp();
            any_pv = true;
          }
        }
        if (n_next >= 0 && fsa_fwd_tile_mode(sched[q], n_next, causal, local) >= 0) {
          if (!k_ready) {
            ok = mbar_wait(&bars->k_full[ks_next], ((t + 1) / KSTAGES) & 1, abort_flag);
            if (!ok) break;
            k_ready = true;
            tc_fence_after();
          }
          issue_s(q, ks_next);
        }
      }
      if (!ok) break;
      if (!v_ready) {
        // nobody consumed this V slot (cannot happen: every visited tile has an active group),
        // still keep the ring in step
        ok = mbar_wait(&bars->v_full[vs], (t / VSTAGES) & 1, abort_flag);
      }
      if (lane == 0) {
        if (any_pv)
          umma_commit(&bars->v_empty[vs]);
        else
          mbar_arrive(&bars->v_empty[vs]);
        if (n_next >= 0) umma_commit(&bars->k_empty[ks_next]);
      }
      __syncwarp();
      n = n_next;
      ++t;
    }
  }
  } else {
    // =============================== softmax groups ==========================================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    const int q = warp >> 2;        // group / query tile
    const int wq = warp & 3;        // warp within group == TMEM lane quadrant
    const int row = wq * 32 + lane; // row within the tile
    const int mb = pair * 2 + q;
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

    float thr_log2 = 0.f;
    if (KIND != KIND_DENSE) {
      // flash_sparse_attn/ops/triton/seqlen_info.py:118-153
      const float visible = causal ? float(q_idx + (si.sk - si.sq) + 1) : float(si.sk);
      thr_log2 = log2f(fmaxf(fminf(p.softmax_thr / visible, 1.0f), 0.0f));
    }
    const float c = p.scale_log2;
    float row_max = -INFINITY, row_sum = 0.f;
    float o_acc[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) o_acc[i] = 0.f;
    bool pending_o = false;
    int cnt_s = 0, cnt_o = 0;
    bool ok = !*abort_flag;
    const bool has_work = q_valid[q] && !fsa_fwd_sched_empty(sched[q]);

    auto add_o_tile = [&](float scale) {
      // o_acc = (o_acc + O_tile) * scale
#pragma unroll
      for (int ch = 0; ch < OCH; ++ch) {
        uint32_t r[32];
        tmem_ld32(tO + ch * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o_acc[ch * 32 + i] = (o_acc[ch * 32 + i] + __uint_as_float(r[i])) * scale;
      }
    };

    for (int n = fsa_fwd_next_tile_below(sched[q], 1 << 28, local); n >= 0 && ok && has_work;
         n = fsa_fwd_next_tile_below(sched[q], n, local)) {
      const int mode = fsa_fwd_tile_mode(sched[q], n, causal, local);
      ok = mbar_wait(&bars->s_full[q], cnt_s & 1, abort_flag);
      if (!ok) break;
      tc_fence_after();
      const int par = cnt_s & 1;
      cnt_s++;
      const int k0 = n * TN;

      // ---- pass 1: masked row maximum ----------------------------------------------------------
      // (TMEM loads are warp-collective: every lane takes the same path, per-row special cases
      // are applied to the values afterwards)
      float m_cur = -INFINITY;
#pragma unroll
      for (int ch = 0; ch < TN / 32; ++ch) {
        uint32_t r[32];
        tmem_ld32(tS + ch * 32, r);
        tmem_ld_wait();
        if (mode == FSA_MASK_NONE) {
#pragma unroll
          for (int i = 0; i < 32; ++i) m_cur = fmaxf(m_cur, __uint_as_float(r[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (col_visible(rm, mode, k0 + ch * 32 + i)) m_cur = fmaxf(m_cur, __uint_as_float(r[i]));
        }
      }
      // rows past the query length read as zero scores in fully visible tiles
      if (mode == FSA_MASK_NONE && !rm.row_ok) m_cur = 0.f;

      // ---- tile skip vote (flash_sparse_attn/ops/triton/activations.py:129-138) -----------------
      bool skip = false;
      if (KIND != KIND_DENSE) {
        const float d = (m_cur - row_max) * c - log2f(row_sum);
        const float val = d - thr_log2;
        const unsigned want = __ballot_sync(0xffffffffu, val >= 0.0f);
        const unsigned drop = __ballot_sync(0xffffffffu, val < 0.0f);
        // group-wide exchange through a (bounded) mbarrier rather than bar.sync, so that an
        // aborting pipeline can never leave part of the group parked on a hardware barrier
        if (lane == 0) {
          bars->vote_any[q][par][wq] = (want ? 1 : 0) | (drop ? 2 : 0);
          mbar_arrive(&bars->wg_sync[q]);
        }
        ok = mbar_wait(&bars->wg_sync[q], par, abort_flag);
        if (!ok) break;
        const int v = bars->vote_any[q][par][0] | bars->vote_any[q][par][1] | bars->vote_any[q][par][2] |
                      bars->vote_any[q][par][3];
        // max over rows ignores NaN rows; a tile is skipped iff that max is < 0
        skip = !(v & 1) && (v & 2);
        if (wq == 0 && lane == 0) {
          bars->skip_flag[q][par] = skip ? 1 : 0;
          if (p.tile_map) {
            const long long idx =
                ((((long long)si.b * p.hgrid + si.head) * p.num_m_blocks + mb) * p.num_splits + si.split) *
                    p.n_tiles_k + n;
            p.tile_map[idx] = skip ? 2 : 1;
          }
          __threadfence_block();
          mbar_arrive(&bars->vote[q]);
        }
      }
      if (skip) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->p_full[q]);
        continue;
      }

      // ---- online softmax update ------------------------------------------------------------------
      float m_new = fmaxf(m_cur, row_max);
      if (mode != FSA_MASK_NONE) m_new = fmaxf(m_new, -1e6f);
      const float scale = ex2_approx((row_max - m_new) * c);
      row_max = m_new;
      const float m_c = m_new * c;

      // the previous P V result must be folded in before its TMEM tile is overwritten
      if (pending_o) {
        ok = mbar_wait(&bars->o_full[q], cnt_o & 1, abort_flag);
        if (!ok) break;
        cnt_o++;
        tc_fence_after();
        add_o_tile(scale);
        pending_o = false;
      } else {
#pragma unroll
        for (int i = 0; i < HD; ++i) o_acc[i] *= scale;
      }

      // ---- pass 2: P = exp2(S*c - m*c), row sum, publish P in TMEM ----------------------------------
      float sum = 0.f;
#pragma unroll
      for (int ch = 0; ch < TN / 32; ++ch) {
        uint32_t r[32];
        tmem_ld32(tS + ch * 32, r);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float s0 = __uint_as_float(r[i]), s1 = __uint_as_float(r[i + 1]);
          if (mode == FSA_MASK_NONE) {
            if (!rm.row_ok) s0 = s1 = 0.f;
          } else {
            if (!col_visible(rm, mode, k0 + ch * 32 + i)) s0 = -INFINITY;
            if (!col_visible(rm, mode, k0 + ch * 32 + i + 1)) s1 = -INFINITY;
          }
          const float p0 = ex2_approx(fmaf(s0, c, -m_c));
          const float p1 = ex2_approx(fmaf(s1, c, -m_c));
          sum += p0;
          sum += p1;
          pk[i >> 1] = pack2<T>(p0, p1);
        }
        tmem_st16(tS + ch * 16, pk);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_full[q]);
      row_sum = row_sum * scale + sum;
      pending_o = true;
    }

    if (ok && pending_o) {
      ok = mbar_wait(&bars->o_full[q], cnt_o & 1, abort_flag);
      if (ok) {
        tc_fence_after();
        add_o_tile(1.0f);
      }
    }

    // ---- epilogue (flash_sparse_attn/ops/triton/activations.py:169-203) ---------------------------
    if (ok && q_valid[q] && rm.row_ok) {
      const bool dead = (row_sum == 0.0f) || (row_sum != row_sum);
      const float inv = dead ? 1.0f : p.v_scale / row_sum;
      float lse = dead ? -INFINITY : row_max * c + log2f(row_sum);
      if (!(p.flags & F_LSE_LOG2)) lse *= 0.6931471805599453f;
      const long long tok = si.off_q + q_idx;
      p.lse[(long long)((p.flags & F_VARLEN_Q) ? 0 : si.b) * p.l_sb + (long long)q_head * p.l_sh +
            (long long)si.split * p.l_ss + ((p.flags & F_VARLEN_Q) ? tok : q_idx)] = lse;
      const long long obase = (long long)((p.flags & F_VARLEN_Q) ? 0 : si.b) * p.o_sb + tok * p.o_sm +
                              (long long)q_head * p.o_sh + (long long)si.split * p.o_ss;
      if (p.flags & F_SPLIT) {
        float* dst = reinterpret_cast<float*>(p.out) + obase;
#pragma unroll
        for (int i = 0; i < HD; i += 4) {
          *reinterpret_cast<float4*>(dst + i) =
              make_float4(o_acc[i] * inv, o_acc[i + 1] * inv, o_acc[i + 2] * inv, o_acc[i + 3] * inv);
        }
      } else {
        T* dst = reinterpret_cast<T*>(p.out) + obase;
#pragma unroll
        for (int i = 0; i < HD; i += 8) {
          uint4 v;
          v.x = pack2<T>(o_acc[i] * inv, o_acc[i + 1] * inv);
          v.y = pack2<T>(o_acc[i + 2] * inv, o_acc[i + 3] * inv);
          v.z = pack2<T>(o_acc[i + 4] * inv, o_acc[i + 5] * inv);
          v.w = pack2<T>(o_acc[i + 6] * inv, o_acc[i + 7] * inv);
          *reinterpret_cast<uint4*>(dst + i) = v;
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

template <int HD, typename T, int KIND>
cudaError_t launch_one(const FwdKernelParams& p, cudaStream_t stream) {
  auto kern = fwd_kernel<HD, T, KIND>;
  constexpr int smem = FwdSmem<HD>::kTotal;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  const long long grid = (long long)p.num_pairs * p.hgrid * p.B * p.num_splits;
  if (grid <= 0) return cudaSuccess;
  kern<<<(unsigned)grid, NTHREADS, smem, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace

// kind: KIND_*, dtype: DT_BF16 / DT_FP16, head_dim: 64 or 128. Returns cudaErrorInvalidValue for
// unsupported combinations.
cudaError_t launch_fwd(const FwdKernelParams& p, int kind, int dtype, int head_dim, cudaStream_t stream) {
#define FSA_FWD_CASE(HD_, T_, DT_)                                                  \
  if (head_dim == HD_ && dtype == DT_) {                                            \
    if (kind == KIND_DENSE) return launch_one<HD_, T_, KIND_DENSE>(p, stream);      \
    if (kind == KIND_SPARSE) return launch_one<HD_, T_, KIND_SPARSE>(p, stream);    \
  }
  FSA_FWD_CASE(128, __nv_bfloat16, DT_BF16)
  FSA_FWD_CASE(128, __half, DT_FP16)
  FSA_FWD_CASE(64, __nv_bfloat16, DT_BF16)
  FSA_FWD_CASE(64, __half, DT_FP16)
#undef FSA_FWD_CASE
  return cudaErrorInvalidValue;
}

}  // namespace fsa
