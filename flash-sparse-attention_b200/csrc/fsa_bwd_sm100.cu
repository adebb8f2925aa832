// Backward attention for sm_100a: five tcgen05 GEMMs per (key tile, query tile) pair with TMEM
// accumulators, TMA-fed Q / dO ring, warp-specialised roles.
//
// One CTA owns one 128-key tile of one KV head and walks every 128-row query tile that attends to
// it, for each of the G query heads of the group in turn. dK and dV therefore accumulate inside the
// CTA (TMEM) across tiles AND across the group's heads - no atomics and a fixed summation order -
// while each dQ tile is added into an fp32 accumulator with a TMA reduce-add.
// It stands in for `_bwd_{dense,sparse}_kernel`
// (flash_sparse_attn/ops/triton/flash_sparse_bwd.py:29-473, flash_dense_bwd.py) at TILE_M = TILE_N =
// 128: same tile schedule (scheduler.py:994-1101), same masks, the same stateless skip rule on the
// true probabilities (flash_sparse_bwd.py:61-79). Unlike the reference's grid over query heads, the
// G heads of a KV head are looped inside the CTA, which is what removes the fp32 atomics on dK/dV
// (scheduler.py:2194-2206).
//
// Everything is computed transposed so that one thread owns one KEY row (TMEM lane):
//   S^T  = K Q^T              [keys x queries]      P^T = exp2(S^T * c - lse2[q])
//   dP^T = V dO^T
//   dS^T = P^T o (dP^T - dpsum[q])
//   dV  += P^T dO      (A = P^T from TMEM)
//   dK  += dS^T Q      (A = dS^T from shared memory, K-major)
//   dQ   = dS K        (A = dS^T from shared memory, read MN-major)
//
// Roles (512 threads, four warpgroups): warps 0-7 compute P^T and dS^T (warps 0-3 own query columns 0-63 of the
// tile, warps 4-7 columns 64-127; both cover all 128 key lanes), warp 8 producer (TMA), warp 9 MMA issuer, warp 10
// dQ drain (deterministic mode only: takes the turns and issues the TMA reduce-adds of the staged dQ tiles), warp
// 11 idle (register budgets are set per warpgroup), warps 12-15 dQ read-out: TMEM -> registers -> staging ->
// TMA reduce-add, so that the accumulator block shared by dP^T and dQ is free again a few hundred cycles after
// the dQ MMAs finish and the compute warps never touch dQ.
// TMEM columns: [0,128) S^T, then P^T packed into [0,32) and [96,128) | [128,256) dP^T, later dQ |
// [256,384) dV | [384,512) dK.
#include "fsa_ptx.cuh"
#include "fsa_params.h"
#include "fsa_schedule.h"
#include "fsa_aux.h"


namespace fsa {

namespace {

constexpr int TM = 128;  // query rows per step
constexpr int TN = 128;  // keys per CTA
constexpr int NTHREADS = 512;

template <int HD>
struct BwdSmem {
  static constexpr int kTile = 128 * HD * 2;
  static constexpr int kK = 0;
  static constexpr int kV = kK + kTile;
  static constexpr int kQ = kV + kTile;        // 2 stages
  static constexpr int kDO = kQ + 2 * kTile;   // 1 stage: dO lives only from dP^T to dV of its step
  static constexpr int kDS = kDO + kTile;      // dS^T (16-bit, 128 x 128)
  static constexpr int kStage = kDS + 32768;   // dQ staging for the TMA reduce-add: 8 warps x 4 KB
  static constexpr int kAux = kStage + 32768;  // lse2[2][128], dpsum[2][128] fp32, alpha[2][128] 16-bit (gated)
  static constexpr int kBar = kAux + 2560;
  static constexpr int kTotal = kBar + 256;
};

struct BwdBars {
  uint64_t kv_full, q_full[2], q_empty[2], do_full, do_empty;
  uint64_t s_full, p_full, dp_full, ds_full, dq_full, dq_empty, vote_sync, acc_full;
  uint64_t dd_sync;  // gated: second column group -> first, partial ddelta handed over in shared memory
  uint64_t stg_full, stg_free;  // dQ staging: compute warps -> drain warp (job posted) and back (buffers read)
  int job[2][4];                // job descriptors {first row, head, query tile, code}, slot = job index & 1
  int dqjob[2][4];              // MMA issuer -> dQ warps: {first row, head, query tile, code} of the dQ tile in TMEM
  uint32_t tmem_base;
  int abort_flag;
  unsigned char vote_any[2][8];
};
static_assert(sizeof(BwdBars) <= 256, "barrier block too large");

// Visible query columns of one key row inside query tile [q0, q0 + TM), as up to three half-open
// intervals of the tile-local index (mask.py:52-102 read along the query axis).
struct ColMask {
  int lo[3];
  unsigned len[3];
};

struct SegList {
  int beg[6], end[6], mode[6];
  int n;
  int total;
};

// Query tiles visited by one key tile, in the reference's phase order
// (flash_sparse_bwd.py:315-464): every phase ascending.
__device__ __forceinline__ SegList make_segments(const FsaBwdSched& s, bool causal, bool local) {
  SegList l;
  l.n = 0;
  l.total = 0;
  auto add = [&](int b, int e, int mode) {
    if (e > b) {
      l.beg[l.n] = b;
      l.end[l.n] = e;
      l.mode[l.n] = mode;
      l.n++;
      l.total += e - b;
    }
  };
  // The reference clamps m_min_no_mask to m_max only under split-QO (scheduler.py:1041-1043); without the
  // clamp its masked loop can run past the last query tile (a short query against a long key sequence), where
  // every load is masked off. Here such a tile would read workspace rows that do not exist: clip it.
  const int m_nm = fsa_imin(s.m_min_no_mask, s.m_max);
  if (causal || local) add(s.m_min, m_nm, local ? FSA_MASK_LOCAL : FSA_MASK_CAUSAL);
  if (!local) add((causal || local) ? m_nm : s.m_min, s.m_max, FSA_MASK_NONE);
  if (local) {
    add(s.win_min, s.win_min_no_mask, FSA_MASK_LOCAL);
    add(s.win_min_no_mask, s.win_max_no_mask, FSA_MASK_NONE);
    add(s.win_max_no_mask, s.win_max, FSA_MASK_LOCAL);
    add(s.sink_min, s.sink_max, FSA_MASK_LOCAL_SINK);
  }
  return l;
}
// Walks the query tiles of a SegList in order without searching: (m, mode) of the current step. The common case
// (the next tile of the same segment) is an increment and a compare; the segment table is only touched when a
// segment ends.
struct SegIter {
  int seg, m, end, mode;
};
__device__ __forceinline__ SegIter seg_begin(const SegList& l) {
  SegIter s;
  s.seg = 0;
  s.m = l.n > 0 ? l.beg[0] : 0;
  s.end = l.n > 0 ? l.end[0] : 0;
  s.mode = l.n > 0 ? l.mode[0] : FSA_MASK_NONE;
  return s;
}
__device__ __forceinline__ void seg_next(const SegList& l, SegIter& s) {
  s.m++;
  if (s.m >= s.end) {
    s.seg++;
#pragma unroll
    for (int i = 1; i < 6; ++i)
      if (i == s.seg && i < l.n) {
        s.m = l.beg[i];
        s.end = l.end[i];
        s.mode = l.mode[i];
      }
  }
}

__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* map, const void* src, int c0, int c1, int c2) {
  asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

template <int HD, typename T, int KIND>
__global__ void __launch_bounds__(NTHREADS, 1) bwd_kernel(const __grid_constant__ BwdKernelParams p) {
  using SM = BwdSmem<HD>;
  constexpr int KK_D = HD / 16;   // MMAs over the head dimension (S^T, dP^T)
  constexpr int KK_M = TM / 16;   // MMAs over the query rows (dV, dK)
  constexpr int KK_N = TN / 16;   // MMAs over the keys (dQ)
  constexpr int HALF = HD / 2;    // output columns per compute group
  constexpr bool IS_BF16 = !__is_same(T, __half);
  constexpr uint32_t TMEM_S = 0, TMEM_DP = 128, TMEM_DV = 256, TMEM_DK = 384;

  extern __shared__ __align__(1024) uint8_t smem[];
  BwdBars* bars = reinterpret_cast<BwdBars*>(smem + SM::kBar);
  volatile int* abort_flag = &bars->abort_flag;
  float* s_lse = reinterpret_cast<float*>(smem + SM::kAux);          // [2][128]
  float* s_dps = reinterpret_cast<float*>(smem + SM::kAux + 1024);   // [2][128]
  T* s_alpha = reinterpret_cast<T*>(smem + SM::kAux + 2048);         // [2][128] (gated)

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool causal = p.flags & F_CAUSAL, local = p.flags & F_LOCAL, split_qo = p.flags & F_SPLIT;

  // ---- work decode ------------------------------------------------------------------------------
  int idx = blockIdx.x;
  int n_block;
  if (p.flags & F_DETERMINISTIC) {
    // key tiles in descending order, slowest index: a CTA only ever waits for CTAs launched before it
    const int per_tile = p.Hkv * p.B * p.num_splits;
    n_block = p.n_tiles_k - 1 - idx / per_tile;
    idx %= per_tile;
  } else {
    // Key tiles in ascending order, slowest index: under a causal / window mask the first key tiles meet the most
    // query tiles, so the longest CTAs start first and the short ones fill the tail (512 CTAs on 148 SMs are 3.5
    // rounds: with the key tile as the fastest index the last round began with the longest CTAs). CTAs that run
    // side by side still share their Q / dO tiles through L2: neighbouring key tiles of one head are per_tile apart.
    const int per_tile = p.Hkv * p.B * p.num_splits;
    n_block = idx / per_tile;
    idx %= per_tile;
  }
  const int hkv = idx % p.Hkv;
  idx /= p.Hkv;
  const int b = idx / p.num_splits;
  const int split = idx - b * p.num_splits;
  const int off_q = (p.flags & F_VARLEN_Q) ? p.cu_q[b] : 0;
  const int off_k = (p.flags & F_VARLEN_K) ? p.cu_k[b] : 0;
  const int sq = (p.flags & F_USED_Q) ? p.used_q[b] : ((p.flags & F_VARLEN_Q) ? p.cu_q[b + 1] - off_q : p.sq);
  const int sk = (p.flags & F_USED_K) ? p.used_k[b] : ((p.flags & F_VARLEN_K) ? p.cu_k[b + 1] - off_k : p.sk);
  if (n_block * TN >= sk) return;  // nothing of this key tile exists (before any allocation)
  if (smem_u32(smem) & 1023u) {    // the tile buffers need a 1024-byte aligned base
    if (tid == 0) atomicExch(p.status, 2);
    return;
  }
  const long long pad_off = (p.flags & F_VARLEN_Q) ? (long long)((off_q + b * 128) / 128) * 128
                                                   : (long long)b * ((p.sq + 127) / 128) * 128;
  FsaWindow w = {0, 0, 0, 0};
  if (local) {
    const int* wp = p.windows + (long long)hkv * p.win_stride;
    w.sink = wp[0];
    w.left = wp[1];
    w.right = wp[2];
    w.near_ = wp[3];
  }
  const FsaBwdSched sched = fsa_bwd_schedule(sq, sk, n_block, split, w, p.num_splits, TN, TM, causal, local, split_qo);
  const SegList segs = make_segments(sched, causal, local);
  const int NT = segs.total;       // query tiles per head
  const int N_IT = NT * p.G;       // steps of this CTA (before gate-skipped ones are dropped)

  // ---- the steps of this CTA, in order: (head of the group, query tile) ------------------------------------
  // Gated kind: the gate bound of a step (flash_sparse_attn/ops/triton/flash_gated_bwd.py:61-79,
  // activations.py:265-299) needs only the extremes of delta over this key tile, the extremes of alpha over the
  // query tile (both precomputed by gate_ext_kernel) and a running scalar that restarts with every head, so every
  // role walks the steps with its own copy of that scalar and drops the same ones: for a gate-skipped step no
  // Q / dO tile is loaded and no MMA is issued (the reference runs nothing for it either). The deterministic
  // mode keeps every step in the stream (a skipped one still has to pass its turn on) and takes the decision in
  // the compute warps, after S^T, as before.
  const bool preskip = (KIND == KIND_GATED) && !(p.flags & F_DETERMINISTIC) && p.gate_ws != nullptr;
  float gw_dmax = 0.f, gw_dmin = 0.f;
  const float2* gw_aext = nullptr;
  if (preskip) {
    const float2* ext = reinterpret_cast<const float2*>(p.gate_ws);
    const float2 de = __ldg(ext + (long long)p.B * p.Hq * p.num_m_blocks + ((long long)b * p.Hkv + hkv) * p.n_tiles_k + n_block);
    gw_dmax = de.x;
    gw_dmin = de.y;
    gw_aext = ext + ((long long)b * p.Hq + (long long)hkv * p.G) * p.num_m_blocks;
  }
  struct StepWalk {
    int g, idx;
    SegIter si;
    float run;
  };
  auto walk_begin = [&]() {
    StepWalk w;
    w.g = 0;
    w.idx = 0;
    w.si = seg_begin(segs);
    w.run = -INFINITY;
    return w;
  };
  // Next step that is computed: head g of the group, query tile m, mask mode, first step of its head. `mark`: this
  // thread records the dropped steps in the tile map (value 3). Returns false at the end.
  auto walk_next = [&](StepWalk& w, int& g, int& m, int& mode, bool& first, bool mark) -> bool {
    for (;;) {
      if (NT == 0 || w.g >= p.G) return false;
      if (w.idx == NT) {
        w.g++;
        w.idx = 0;
        w.si = seg_begin(segs);
        w.run = -INFINITY;
        continue;
      }
      g = w.g;
      m = w.si.m;
      mode = w.si.mode;
      first = w.idx == 0;
      seg_next(segs, w.si);
      w.idx++;
      if (preskip) {
        const float2 ae = __ldg(gw_aext + (long long)g * p.num_m_blocks + m);
        float g_thr = p.gate_thr;
        if (causal && (p.flags & F_ADAPT_GATE)) g_thr = p.gate_thr * (float(m * TM + (sk - sq)) + 1.0f) / float(sk);
        const float gmc = fmaxf(fmaxf(ae.x * gw_dmax, ae.x * gw_dmin), fmaxf(ae.y * gw_dmax, ae.y * gw_dmin));
        const bool skip = (gmc - w.run) * p.scale_log2 < log2f(g_thr);
        if (!skip) {
          w.run = fmaxf(gmc, w.run);
        } else {
          if (mark && p.tile_map)
            p.tile_map[((((long long)b * p.Hq + hkv * p.G + g) * p.n_tiles_k + n_block) * p.num_splits + split) *
                           p.num_m_blocks + m] = 3;
          continue;
        }
      }
      return true;
    }
  };

  // ---- setup ---------------------------------------------------------------------------------
  if (tid == 0) {
    mbar_init(&bars->kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->q_full[s], 1);
      mbar_init(&bars->q_empty[s], 1);
    }
    mbar_init(&bars->s_full, 1);
    mbar_init(&bars->p_full, 8);
    mbar_init(&bars->dp_full, 1);
    mbar_init(&bars->ds_full, 8);
    mbar_init(&bars->dq_full, 1);
    mbar_init(&bars->dq_empty, 4);
    mbar_init(&bars->do_full, 1);
    mbar_init(&bars->do_empty, 1);
    mbar_init(&bars->vote_sync, 8);
    mbar_init(&bars->acc_full, 1);
    mbar_init(&bars->dd_sync, 4);
    mbar_init(&bars->stg_full, 4);
    mbar_init(&bars->stg_free, 1);
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
  const int bq = (p.flags & F_VARLEN_Q) ? 0 : b;
  const int bk = (p.flags & F_VARLEN_K) ? 0 : b;

  if (warp >= 12) {
    // =============================== dQ read-out ================================================
    // One warp per TMEM lane quadrant (32 query rows). Per dQ tile: 64 columns at a time leave TMEM for registers
    // and go through this warp's two 4 KB staging buffers into TMA reduce-adds; the TMEM block is handed back
    // as soon as the last columns are in registers. The path from an SM to L2 moves about 21 bytes per clock, so
    // the 64 KB of a tile take about as long as the MMAs of a step: these warps pace themselves on the reads of
    // the staging buffers and nobody else waits for them.
    asm volatile("setmaxnreg.dec.sync.aligned.u32 96;");
    const int wq = warp & 3;
    const uint32_t lane_addr = uint32_t(wq * 32) << 16;
    uint8_t* stage = smem + SM::kStage + wq * 8192;
    const bool det = p.flags & F_DETERMINISTIC;
    constexpr int NP = HD / 64;  // 64-column pairs of 32-column chunks per dQ tile
    constexpr uint32_t TMEM_DQ = 128;
    bool ok = !*abort_flag;
    int jobs = 0;  // staging jobs handed to the drain warp so far (deterministic mode; same count in all four warps)
    // wait until the drain warp's TMA reads of the previous job have left the staging buffers
    auto stage_wait_free = [&]() {
      if (jobs > 0 && !mbar_wait(&bars->stg_free, (jobs - 1) & 1, abort_flag)) ok = false;
    };
    // hand a job to the drain warp: {first row of the tile, head, query tile, code}
    // code = kind (0 chunk pair, 1 pass, 2 exit) | pair << 4 | last pair of the tile << 8
    auto stage_post = [&](int row0, int head, int m, int code) {
      if (wq == 0 && lane == 0) {
        volatile int* jd = bars->job[jobs & 1];
        jd[0] = row0;
        jd[1] = head;
        jd[2] = m;
        jd[3] = code;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->stg_full);
      jobs++;
    };
    auto stage_store = [&](uint8_t* buf, const uint32_t* r) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        *reinterpret_cast<uint4*>(buf + lane * 128 + ((j ^ (lane & 7)) << 4)) =
            make_uint4(r[j * 4], r[j * 4 + 1], r[j * 4 + 2], r[j * 4 + 3]);
    };
    for (int j = 0; ok; ++j) {
      ok = mbar_wait(&bars->dq_full, j & 1, abort_flag);
      if (!ok) break;
      const volatile int* jd = bars->dqjob[j & 1];
      const int row0 = jd[0], head = jd[1], m = jd[2], code = jd[3];
      if (code == 2) break;
      if (code == 1) {  // deterministic mode: a skipped tile adds nothing but still takes (and passes on) its turn
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->dq_empty);
        stage_wait_free();
        if (!ok) break;
        stage_post(0, head, m, 1);
        continue;
      }
      tc_fence_after();
#pragma unroll
      for (int cp = 0; cp < NP; ++cp) {
        uint32_t r[64];
        tmem_ld32(tmem_base + lane_addr + TMEM_DQ + cp * 64, &r[0]);
        tmem_ld32(tmem_base + lane_addr + TMEM_DQ + cp * 64 + 32, &r[32]);
        tmem_ld_wait();
        if (cp == NP - 1) {  // all of this warp's dQ values are in registers: the TMEM block may be overwritten
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars->dq_empty);
        }
        if (det) {
          stage_wait_free();
          if (!ok) break;
        } else {
          if (lane == 0) bulk_wait_read0();  // the engine has read the previous contents of both buffers
          __syncwarp();
        }
        stage_store(stage, &r[0]);
        stage_store(stage + 4096, &r[32]);
        fence_proxy_async_smem();
        __syncwarp();
        if (det) {
          stage_post(row0, head, m, 0 | (cp << 4) | ((cp == NP - 1 ? 1 : 0) << 8));
        } else if (lane == 0) {
          tma_reduce_add_3d(&p.map_dq, stage, cp * 64, row0 + wq * 32, head);
          tma_reduce_add_3d(&p.map_dq, stage + 4096, cp * 64 + 32, row0 + wq * 32, head);
          bulk_commit();
        }
      }
    }
    if (det) {
      stage_wait_free();
      stage_post(0, 0, 0, 2);  // the drain warp leaves (also when this warp is bailing out: it must not be left waiting)
    }
    if (lane == 0) bulk_wait0();
    __syncwarp();
  } else if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
    if (warp == 8) {
      // =============================== producer ==============================================
      if (lane == 0 && !*abort_flag) {
        tma_prefetch_desc(&p.map_q);
        tma_prefetch_desc(&p.map_do);
        tma_prefetch_desc(&p.map_k);
        tma_prefetch_desc(&p.map_v);
        mbar_arrive_expect_tx(&bars->kv_full, 2 * SM::kTile);
        for (int d = 0; d < HD; d += 64) {
          tma_load_4d(smem + SM::kK + (d / 64) * (TN * 128), &p.map_k, &bars->kv_full, d, hkv, off_k + n_block * TN, bk);
          tma_load_4d(smem + SM::kV + (d / 64) * (TN * 128), &p.map_v, &bars->kv_full, d, hkv, off_k + n_block * TN, bk);
        }
        // Q (with the row statistics of its tile) runs two steps ahead in a 2-stage ring; dO has one
        // buffer and is reloaded as soon as dV of the previous step has consumed it.
        bool ok = true;
        StepWalk wk = walk_begin();
        int g = 0, m = 0, mode_unused = 0;
        bool first_unused = false;
        for (int it = 0; ok && walk_next(wk, g, m, mode_unused, first_unused, false); ++it) {
          const int st = it & 1, use = it >> 1;
          const int head = hkv * p.G + g;
          if (use > 0) ok = mbar_wait(&bars->q_empty[st], (use - 1) & 1, abort_flag);
          if (!ok) break;
          mbar_arrive_expect_tx(&bars->q_full[st], SM::kTile + 1024 + (KIND == KIND_GATED ? 256 : 0));
          for (int d = 0; d < HD; d += 64)
            tma_load_4d(smem + SM::kQ + st * SM::kTile + (d / 64) * (TM * 128), &p.map_q, &bars->q_full[st], d, head,
                        off_q + m * TM, bq);
          const long long wrow = (long long)head * p.ws_sh + pad_off + (long long)m * TM;
          bulk_load_1d(s_lse + st * 128, p.lse2_ws + wrow, 512, &bars->q_full[st]);
          bulk_load_1d(s_dps + st * 128, p.dpsum_ws + wrow, 512, &bars->q_full[st]);
          if (KIND == KIND_GATED)
            bulk_load_1d(s_alpha + st * 128, reinterpret_cast<const T*>(p.alpha_ws) + wrow, 256, &bars->q_full[st]);
          if (it > 0) ok = mbar_wait(&bars->do_empty, (it - 1) & 1, abort_flag);
          if (!ok) break;
          mbar_arrive_expect_tx(&bars->do_full, SM::kTile);
          for (int d = 0; d < HD; d += 64)
            tma_load_4d(smem + SM::kDO + (d / 64) * (TM * 128), &p.map_do, &bars->do_full, d, head, off_q + m * TM, bq);
        }
      }
      __syncwarp();
    } else if (warp == 9) {
      // =============================== MMA issuer ==============================================
      constexpr uint32_t idesc_s = umma_idesc_f16(TN, TM, IS_BF16, false, false);   // S^T, dP^T: [keys x queries]
      constexpr uint32_t idesc_dv = umma_idesc_f16(TN, HD, IS_BF16, false, true);   // dV: A from TMEM, B = dO MN-major
      constexpr uint32_t idesc_dk = umma_idesc_f16(TN, HD, IS_BF16, false, true);   // dK: A = dS^T K-major, B = Q MN-major
      constexpr uint32_t idesc_dq = umma_idesc_f16(TM, HD, IS_BF16, true, true);    // dQ: A = dS^T MN-major, B = K MN-major
      const uint32_t sK = smem_u32(smem + SM::kK), sV = smem_u32(smem + SM::kV), sQ = smem_u32(smem + SM::kQ),
                     sDO = smem_u32(smem + SM::kDO), sDS = smem_u32(smem + SM::kDS);
      bool ok = !*abort_flag && N_IT > 0;
      (void)N_IT;
      // The MMA loops stay rolled where the compute warps carry the skip vote and the masks (their code is what the
      // schedulers fetch most; measured 2-3 % faster on the windowed sparse workload) and are unrolled for the dense
      // kind (rolled: 4 % slower there).
      constexpr int ISSUE_UNROLL = (KIND == KIND_DENSE) ? 8 : 1;
      // The whole warp runs the (uniform) descriptor arithmetic and every MMA carries the single-lane predicate: a
      // divergent branch around the MMAs would cost more issue time per MMA than the MMA takes to execute. A
      // descriptor is (low word, constant high word); moving inside a tile is an add on the low word.
      const uint32_t lead = lane == 0 ? 1u : 0u;
      const uint32_t k_lo = umma_desc_lo(sK, 16), v_lo = umma_desc_lo(sV, 16), do_lo = umma_desc_lo(sDO, 16),
                     ds_lo = umma_desc_lo(sDS, 16);                                  // K-major operands
      const uint32_t do_mn = umma_desc_lo(sDO, TM * 128), ds_mn = umma_desc_lo(sDS, 128 * 128),
                     k_mn = umma_desc_lo(sK, TN * 128);                              // MN-major operands
      const uint32_t q_lo0 = umma_desc_lo(sQ, 16), q_mn0 = umma_desc_lo(sQ, TM * 128);
      constexpr uint32_t Q_STAGE = SM::kTile >> 4;  // low-word distance between the two Q stages
      auto issue_st = [&](int st) {
        const uint32_t q_lo = q_lo0 + st * Q_STAGE;
#pragma unroll ISSUE_UNROLL
        for (int kk = 0; kk < KK_D; ++kk) {
          const uint32_t koff = (kk >> 2) * (128 * 128) + (kk & 3) * 32;
          umma_ss_lead(lead, tmem_base + TMEM_S, umma_desc_at(k_lo, koff), umma_desc_at(q_lo, koff), idesc_s, kk > 0);
        }
        umma_commit_lead(lead, &bars->s_full);
      };
      StepWalk wk = walk_begin();
      int g_nxt = 0, m_nxt = 0, mode_unused = 0;
      bool first_unused = false;
      bool has_cur = ok && walk_next(wk, g_nxt, m_nxt, mode_unused, first_unused, false);
      const bool det = p.flags & F_DETERMINISTIC;
      int n_jobs = 0;  // dQ tiles (and, deterministic mode, passes) handed to the dQ warps so far
      // descriptor of the dQ tile the next commit on dq_full announces; written well before the MMAs it follows
      auto post_dq_job = [&](int g, int m, int code) {
        if (lane == 0) {
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(smem_u32(bars->dqjob[n_jobs & 1])),
                       "r"((int)(pad_off + (long long)m * TM)), "r"(hkv * p.G + g), "r"(m), "r"(code)
                       : "memory");
          __threadfence_block();
        }
      };
      if (has_cur) {
        ok = mbar_wait(&bars->kv_full, 0, abort_flag);
        ok = ok && mbar_wait(&bars->q_full[0], 0, abort_flag);
        tc_fence_after();
        if (ok) issue_st(0);
      }
      int n_live = 0;  // steps that were not skipped so far
      bool acc_started = false;
      for (int it = 0; has_cur && ok; ++it) {
        const int st = it & 1;
        const int g_cur = g_nxt, m_cur = m_nxt;
        const bool has_next = walk_next(wk, g_nxt, m_nxt, mode_unused, first_unused, false);
        // The verdict of the skip vote is read straight from the votes (the compute warps publish them well before
        // the exponentials), so that dP^T is under way while P^T is still being computed.
        bool skip = false;
        if (KIND != KIND_DENSE) {
          ok = mbar_wait(&bars->vote_sync, it & 1, abort_flag);
          if (!ok) break;
          const unsigned long long vv = *reinterpret_cast<const volatile unsigned long long*>(&bars->vote_any[it & 1][0]);
          const bool any_want = (vv & 0x0101010101010101ull) != 0ull, any_drop = (vv & 0x0202020202020202ull) != 0ull;
          skip = !any_want && any_drop;
        }
        ok = mbar_wait(&bars->do_full, it & 1, abort_flag);  // every phase is observed, skipped step or not
        if (!ok) break;
        tc_fence_after();
        if (!skip || det) {
          // the dQ warps have read the previous tile out of the block that dP^T is about to overwrite (and both
          // descriptor slots are free again)
          if (n_jobs > 0) ok = mbar_wait(&bars->dq_empty, (n_jobs - 1) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
        }
        if (skip && det) {  // a skipped tile still takes its turn in the order of the dQ adds
          post_dq_job(g_cur, m_cur, 1);
          umma_commit_lead(lead, &bars->dq_full);
          n_jobs++;
        }
        if (!skip) {
          post_dq_job(g_cur, m_cur, 0);
#pragma unroll ISSUE_UNROLL
          for (int kk = 0; kk < KK_D; ++kk) {
            const uint32_t koff = (kk >> 2) * (128 * 128) + (kk & 3) * 32;
            umma_ss_lead(lead, tmem_base + TMEM_DP, umma_desc_at(v_lo, koff), umma_desc_at(do_lo, koff), idesc_s, kk > 0);
          }
          umma_commit_lead(lead, &bars->dp_full);
        }
        ok = mbar_wait(&bars->p_full, it & 1, abort_flag);  // P^T is in TMEM (every phase is observed)
        if (!ok) break;
        tc_fence_after();
        if (!skip) {
#pragma unroll ISSUE_UNROLL
          for (int kk = 0; kk < KK_M; ++kk) {
            const uint32_t a_col = (kk < 4) ? kk * 8 : 96 + (kk - 4) * 8;
            umma_ts_lead(lead, tmem_base + TMEM_DV, tmem_base + TMEM_S + a_col, umma_desc_at(do_mn, kk * 2048), idesc_dv,
                         (kk > 0 || acc_started) ? 1u : 0u);
          }
        }
        umma_commit_lead(lead, &bars->do_empty);  // dO may be overwritten once dV has read it
        if (has_next) {
          ok = mbar_wait(&bars->q_full[(it + 1) & 1], ((it + 1) >> 1) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          issue_st((it + 1) & 1);
        }
        if (!skip) {
          ok = mbar_wait(&bars->ds_full, n_live & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          // dQ first: its tile has to leave TMEM before dP^T of the next step can be issued
#pragma unroll ISSUE_UNROLL
          for (int kk = 0; kk < KK_N; ++kk)
            umma_ss_lead(lead, tmem_base + TMEM_DP, umma_desc_at(ds_mn, kk * 2048), umma_desc_at(k_mn, kk * 2048), idesc_dq,
                         kk > 0);
          umma_commit_lead(lead, &bars->dq_full);
          const uint32_t q_mn = q_mn0 + st * Q_STAGE;
#pragma unroll ISSUE_UNROLL
          for (int kk = 0; kk < KK_M; ++kk)
            umma_ss_lead(lead, tmem_base + TMEM_DK, umma_desc_at(ds_lo, (kk >> 2) * (128 * 128) + (kk & 3) * 32),
                         umma_desc_at(q_mn, kk * 2048), idesc_dk, (kk > 0 || acc_started) ? 1u : 0u);
          acc_started = true;
          n_live++;
          n_jobs++;
        }
        umma_commit_lead(lead, &bars->q_empty[st]);
        has_cur = has_next;
      }
      umma_commit_lead(lead, &bars->acc_full);
      // The dQ warps leave. Every one of them must have seen the phase of the last tile before dq_full moves on
      // again (two arrivals in a row would carry the barrier past a waiter's parity).
      if (n_jobs > 0 && ok) ok = mbar_wait(&bars->dq_empty, (n_jobs - 1) & 1, abort_flag);
      if (!*abort_flag) {
        post_dq_job(0, 0, 2);
        umma_commit_lead(lead, &bars->dq_full);
      }
    } else if (warp == 10) {
      // =============================== dQ drain =================================================
      // Deterministic mode only (otherwise every dQ warp issues the reduce-adds of its own buffers, which
      // measured 3 % faster). Jobs arrive in order: a 64-column pair of chunks of a dQ tile staged by the four
      // dQ warps (lane i issues the reduce-add of the 4 KB buffer i), "pass" for a skipped tile and
      // "exit". This warp waits for the tile's turn before the first chunk and passes it on when the adds
      // of the last chunk have completed (one tick of the per-(head, query tile) counter per key tile), so
      // the dQ warps never wait for a turn or for the completion of an add.
      const bool det = p.flags & F_DETERMINISTIC;
      bool ok = det && !*abort_flag;  // without deterministic mode the compute warps issue their own reduce-adds
      // one counter per (head, query tile); a link of the chain costs the issue-to-completion latency of the
      // tile's reduce-adds (per-chunk chains were tried: the drain warp then blocks on every completion
      // and the whole pipeline slows down)
      auto turn_ptr = [&](int head, int m) { return p.dq_turn + ((long long)b * p.Hq + head) * p.num_m_blocks + m; };
      auto turn_wait = [&](int head, int m) {
        if (lane == 0) {
          const int target =
              (int)p.dq_order[(((long long)b * p.Hkv + hkv) * p.n_tiles_k + n_block) * p.num_m_blocks + m];
          const int* tp = turn_ptr(head, m);
          const long long t_end = clock64() + FSA_WAIT_CYCLES;
          int seen;
          for (;;) {
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(tp) : "memory");
            if (seen == target || *abort_flag) break;
            if (clock64() > t_end) {
              *abort_flag = 1;
              break;
            }
            __nanosleep(64);
          }
        }
        __syncwarp();
      };
      auto turn_pass = [&](int head, int m) {
        if (lane == 0) {
          __threadfence();
          atomicAdd(turn_ptr(head, m), 1);
        }
      };
      for (int j = 0; ok; ++j) {
        ok = mbar_wait(&bars->stg_full, j & 1, abort_flag);
        if (!ok) break;
        const volatile int* jd = bars->job[j & 1];
        const int row0 = jd[0], head = jd[1], m = jd[2], code = jd[3];
        const int kind = code & 3, chunk = (code >> 4) & 1;
        const bool last = (code >> 8) & 1;
        if (kind == 2) break;
        if (det && (kind == 1 || chunk == 0)) {
          turn_wait(head, m);
          if (*abort_flag) break;
        }
        if (kind == 0 && lane < 8) {
          tma_reduce_add_3d(&p.map_dq, smem + SM::kStage + lane * 4096, chunk * 64 + (lane & 1) * 32,
                            row0 + (lane >> 1) * 32, head);
          bulk_commit();
          bulk_wait_read0();
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->stg_free);
        if (det && (kind == 1 || last)) {
          if (kind == 0 && lane < 8) bulk_wait0();  // the adds have landed: the next key tile may add
          __syncwarp();
          turn_pass(head, m);
        }
      }
      if (lane < 8) bulk_wait0();
      __syncwarp();
    }
  } else {
    // =============================== compute warps ===========================================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 176;");
    const int cw = warp;            // 0..7
    const int wg = cw >> 2;         // which half of the query columns / output columns
    const int wq = cw & 3;          // TMEM lane quadrant
    const int row = wq * 32 + lane; // key row (S^T, dP^T, dV, dK)
    const uint32_t lane_addr = uint32_t(wq * 32) << 16;
    const int k_idx = n_block * TN + row;
    const bool row_ok = k_idx < sk;
    const int off = sk - sq;
    const float c = p.scale_log2;
    uint8_t* ds_buf = smem + SM::kDS;

    bool ok = !*abort_flag;
    uint32_t pk[32];  // P^T of the step in flight, packed pairs (this thread's 64 query columns)
    int n_live = 0;
    bool skip_cur = false;
    int m_cur = 0, g_cur = 0;  // query tile / head of the step whose dS is being handled

    // ---- gated: delta of this key row, its extremes over the key tile, running gate bound --------
    // (flash_sparse_attn/ops/triton/flash_gated_bwd.py:406-421; keys past the sequence read as zero)
    float dlt = 0.f, d_max = 0.f, d_min = 0.f, dd_acc = 0.f, gate_max = -INFINITY;
    const bool logsig = p.flags & F_LOGSIGMOID;
    const float lg_thr = p.softmax_thr > 0.f ? log2f(p.softmax_thr) : -INFINITY;  // for the skip thresholds
    if (KIND == KIND_GATED) {
      const T* dp = reinterpret_cast<const T*>(p.delta) + (long long)bk * p.d_sb + (long long)hkv * p.d_sh + off_k;
      float mx = -INFINITY, mn = INFINITY;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int kj = n_block * TN + j * 32 + lane;
        const float v = kj < sk ? float(dp[kj]) : 0.f;
        if (j == wq) dlt = v;
        mx = fmaxf(mx, v);
        mn = fminf(mn, v);
      }
#pragma unroll
      for (int sft = 16; sft > 0; sft >>= 1) {
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, sft));
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, sft));
      }
      d_max = mx;
      d_min = mn;
    }
    auto unpack16 = [&](uint32_t v, float& lo, float& hi) {
      if (IS_BF16) {
        lo = __uint_as_float(v << 16);
        hi = __uint_as_float(v & 0xffff0000u);
      } else {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&v));
        lo = f.x;
        hi = f.y;
      }
    };

    auto col_mask = [&](int mode, int m) {
      ColMask cm;
      const int q0 = m * TM;
      const int seq_hi = row_ok ? min(sq - q0, TM) : 0;
      auto clip = [&](int i, long long a, long long bnd) {
        long long lo = a - q0, hi = bnd - q0;
        if (lo < 0) lo = 0;
        if (hi > seq_hi) hi = seq_hi;
        cm.lo[i] = (int)lo;
        cm.len[i] = hi > lo ? unsigned(hi - lo) : 0u;
      };
      const long long base = (long long)k_idx - off;  // first causally visible query
      if (mode == FSA_MASK_NONE || mode == FSA_MASK_SEQLEN) {
        clip(0, 0, sq);
        clip(1, 0, 0);
        clip(2, 0, 0);
      } else if (mode == FSA_MASK_CAUSAL) {
        clip(0, base, (long long)sq);
        clip(1, 0, 0);
        clip(2, 0, 0);
      } else {
        clip(0, base, base + w.near_);
        clip(1, base + w.near_ + w.right, base + w.near_ + w.right + w.left);
        if (mode == FSA_MASK_LOCAL_SINK && k_idx < w.sink)
          clip(2, base, (long long)sq);
        else
          clip(2, 0, 0);
      }
      return cm;
    };
    auto visible = [&](const ColMask& cm, int i) {
      return (unsigned(i - cm.lo[0]) < cm.len[0]) | (unsigned(i - cm.lo[1]) < cm.len[1]) |
             (unsigned(i - cm.lo[2]) < cm.len[2]);
    };

    // ---- P step: scores -> probabilities (and the skip vote) ------------------------------------
    StepWalk wk = walk_begin();
    const bool mark_steps = cw == 0 && lane == 0;  // one thread records the dropped steps in the tile map
    int m_p = 0, g_p = 0;  // query tile and head (within the group) of the step p_step just handled
    // returns the skip decision; steps are visited in order: (g, m, mode, first step of its head) from the walk
    auto p_step = [&](int it, int g, int m, int mode, bool first_of_head) -> bool {
      const int st = it & 1, par = it & 1;
      g_p = g;
      m_p = m;
      // skip thresholds of the group's first and last query column: worked out before S is waited for
      // (log2(clamp(threshold / visible, 0, 1)) = min(log2 threshold - log2 visible, 0); threshold <= 0 gives -inf)
      const int q_first = m * TM + wg * 64;
      const float vis_first = causal ? float(q_first + off + 1) : float(sk);
      const float vis_last = causal ? float(q_first + 63 + off + 1) : float(sk);
      float thr_hi = 0.f, thr_lo = 0.f;
      if (KIND != KIND_DENSE) {
        thr_hi = fminf(lg_thr - lg2_approx(vis_first), 0.0f);
        thr_lo = fminf(lg_thr - lg2_approx(vis_last), 0.0f);
      }
      if (!mbar_wait(&bars->s_full, par, abort_flag)) {
        ok = false;
        return true;
      }
      // lse2 / dpsum arrived with the Q tile; observing the barrier makes them visible here
      if (!mbar_wait(&bars->q_full[st], (it >> 1) & 1, abort_flag)) {
        ok = false;
        return true;
      }
      tc_fence_after();
      bool gate_skip = false;
      if (KIND == KIND_GATED && !preskip) {
        // bound of the gate over the tile against a running maximum that restarts with every query head
        // (flash_gated_bwd.py:61-79, activations.py:265-299, seqlen_info.py:156-191)
        if (first_of_head) gate_max = -INFINITY;
        const uint2 av = *reinterpret_cast<const uint2*>(s_alpha + st * 128 + lane * 4);
        float a4[4];
        unpack16(av.x, a4[0], a4[1]);
        unpack16(av.y, a4[2], a4[3]);
        float mx = -INFINITY, mn = INFINITY;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float v = (m * TM + lane * 4 + j < sq) ? a4[j] : 0.f;
          mx = fmaxf(mx, v);
          mn = fminf(mn, v);
        }
#pragma unroll
        for (int sft = 16; sft > 0; sft >>= 1) {
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, sft));
          mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, sft));
        }
        float g_thr = p.gate_thr;
        if (causal && (p.flags & F_ADAPT_GATE)) g_thr = p.gate_thr * (float(m * TM + off) + 1.0f) / float(sk);
        const float gmc = fmaxf(fmaxf(mx * d_max, mx * d_min), fmaxf(mn * d_max, mn * d_min));
        gate_skip = (gmc - gate_max) * c < log2f(g_thr);
        if (!gate_skip) gate_max = fmaxf(gmc, gate_max);
      }
      uint32_t sr[64];
      tmem_ld32(tmem_base + lane_addr + TMEM_S + wg * 64, &sr[0]);
      tmem_ld32(tmem_base + lane_addr + TMEM_S + wg * 64 + 32, &sr[32]);
      tmem_ld_wait();
      const bool ragged = ((m + 1) * TM > sq) || ((n_block + 1) * TN > sk);
      const bool masked = (mode != FSA_MASK_NONE) || ragged;
      ColMask cm = {{0, 0, 0}, {0u, 0u, 0u}};
      if (masked) cm = col_mask(mode, m);  // 64-bit interval arithmetic: only for the tiles that need it
      const float4* lse4 = reinterpret_cast<const float4*>(s_lse + st * 128 + wg * 64);
      float x[64];  // log2 of the probabilities
      if (KIND == KIND_GATED) {
        // logits = (q.k + g(alpha_q * delta_k)) * scale, g = logsigmoid or identity (flash_gated_bwd.py:81-98)
        const uint4* al4 = reinterpret_cast<const uint4*>(s_alpha + st * 128 + wg * 64);
#pragma unroll
        for (int i = 0; i < 64; i += 8) {
          const uint4 av = al4[i >> 3];
          float a8[8];
          unpack16(av.x, a8[0], a8[1]);
          unpack16(av.y, a8[2], a8[3]);
          unpack16(av.z, a8[4], a8[5]);
          unpack16(av.w, a8[6], a8[7]);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float gx = a8[j] * dlt;
            float gte = gx;
            if (logsig)
              gte = log_sigmoid_fast(gx);
            sr[i + j] = __float_as_uint(__uint_as_float(sr[i + j]) + gte);
          }
        }
      }
      const float2 c2 = make_float2(c, c);
#pragma unroll
      for (int i = 0; i < 64; i += 4) {
        const float4 l = lse4[i >> 2];  // minus lse2
        const float2 xa = fma2(make_float2(__uint_as_float(sr[i]), __uint_as_float(sr[i + 1])), c2, make_float2(l.x, l.y));
        const float2 xb =
            fma2(make_float2(__uint_as_float(sr[i + 2]), __uint_as_float(sr[i + 3])), c2, make_float2(l.z, l.w));
        x[i] = xa.x;
        x[i + 1] = xa.y;
        x[i + 2] = xb.x;
        x[i + 3] = xb.y;
      }
      // A tile that the reference runs WITHOUT a mask (flash_sparse_bwd.py:339-359) takes part in its skip vote with
      // whatever lies past the sequence ends: a query column past sq reads S = 0 (plus the gate of alpha = 0) and
      // lse2 = 0 (masked loads, scheduler.py:2173-2179), so its log2 p - threshold is >= 0 unless the threshold is
      // 0, and the tile is kept; a key row past sk reads S = gate only and votes with g c - lse2[q]. Those entries
      // are masked out of P below, but their vote is reproduced here.
      bool oor_want = false;
      if (KIND != KIND_DENSE && mode == FSA_MASK_NONE && ragged) {
        if ((m + 1) * TM > sq) {
          const float x_oor = (KIND == KIND_GATED && logsig) ? -0.6931472f * c : 0.f;
          const float vis_oor = causal ? float(m * TM + TM - 1 + off + 1) : float(sk);
          oor_want = x_oor - fminf(lg_thr - lg2_approx(vis_oor), 0.0f) >= 0.0f;
        } else if (!row_ok) {
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            const float vis_i = causal ? float(q_first + i + off + 1) : float(sk);
            oor_want |= (x[i] - fminf(lg_thr - lg2_approx(vis_i), 0.0f) >= 0.0f);
          }
        }
      }
      if (masked) {
        const int n_iv = (cm.len[0] != 0u) + (cm.len[1] != 0u) + (cm.len[2] != 0u);
        if (__all_sync(0xffffffffu, n_iv <= 1)) {  // at most one interval per key row: one compare per entry
          const int which = cm.len[1] != 0u ? 1 : (cm.len[2] != 0u ? 2 : 0);
          const int nlo = wg * 64 - (which == 1 ? cm.lo[1] : (which == 2 ? cm.lo[2] : cm.lo[0]));
          const unsigned len = which == 1 ? cm.len[1] : (which == 2 ? cm.len[2] : cm.len[0]);
#pragma unroll
          for (int i = 0; i < 64; ++i)
            if (unsigned(i + nlo) >= len) x[i] = -INFINITY;
        } else {
#pragma unroll
          for (int i = 0; i < 64; ++i)
            if (!visible(cm, wg * 64 + i)) x[i] = -INFINITY;
        }
      }
      bool skip = false;
      if (KIND != KIND_DENSE) {
        // skip iff max over the tile of (log2 p - thr_log2[q]) < 0 (flash_sparse_bwd.py:61-79);
        // thresholds of this group's 64 query columns live two per lane and travel by shuffle
        // The threshold falls as the query index grows (causal) or is one number (otherwise): the row
        // maximum against the thresholds of the group's first and last column settles most votes at
        // once; only a warp with a lane in between compares entry by entry.
        // The verdict is one bit for the whole tile ("does any entry want it"), so the common case is settled by the
        // first sixteen columns: if the maximum of those reaches the largest threshold of the group in any lane,
        // the tile is kept and the rest of the vote is not computed.
        const bool exact_only = vis_first < 1.0f;  // warp-uniform
        auto chain16 = [&](int j) {
          float v = fmaxf(x[j * 16], x[j * 16 + 1]);
#pragma unroll
          for (int i = 2; i < 16; i += 2) v = max3(v, x[j * 16 + i], x[j * 16 + i + 1]);
          return v;
        };
        const float mx_first = chain16(0);
        bool want = mx_first >= thr_hi, drop = false;
        if (exact_only || !__any_sync(0xffffffffu, want)) {
          const float mx = fmaxf(fmaxf(mx_first, chain16(1)), fmaxf(chain16(2), chain16(3)));
          want = mx >= thr_hi;
          drop = mx < thr_lo;
          const bool unsure = exact_only || (!want && !drop);
          // once a lane of this warp is sure that it wants the tile, the lanes in between do not matter any more
          const bool settled = !exact_only && __any_sync(0xffffffffu, want);
          if (!settled && __any_sync(0xffffffffu, unsure)) {
            const int q_a = q_first + lane, q_b = q_a + 32;
            const float vis_a = causal ? float(q_a + off + 1) : float(sk);
            const float vis_b = causal ? float(q_b + off + 1) : float(sk);
            const float thr_a = fminf(lg_thr - lg2_approx(vis_a), 0.0f);
            const float thr_b = fminf(lg_thr - lg2_approx(vis_b), 0.0f);
            want = false;
            drop = false;
#pragma unroll
            for (int i = 0; i < 64; ++i) {
              const float t = __shfl_sync(0xffffffffu, i < 32 ? thr_a : thr_b, i & 31);
              const float v = x[i] - t;
              want |= (v >= 0.0f);
              drop |= (v < 0.0f);
            }
          }
        }
        want |= oor_want;
        if (KIND == KIND_GATED && gate_skip) {
          want = false;
          drop = true;
        }
        const unsigned w_any = __ballot_sync(0xffffffffu, want);
        const unsigned d_any = __ballot_sync(0xffffffffu, drop);
        if (lane == 0) {
          bars->vote_any[par][cw] = (w_any ? 1 : 0) | (d_any ? 2 : 0);
          mbar_arrive(&bars->vote_sync);
        }
        // A warp with an entry that wants the tile knows the outcome ("keep") and moves on; only warps whose
        // entries all vote "skip" wait for the others. Every warp arrives once per step, and none reaches the vote
        // of the step after next (same slot) before all have arrived here: S of the next step is only issued
        // after all eight warps published P or the skip.
        if (!w_any) {
          if (!mbar_wait(&bars->vote_sync, par, abort_flag)) {
            ok = false;
            return true;
          }
          int v = 0;
#pragma unroll
          for (int i = 0; i < 8; ++i) v |= bars->vote_any[par][i];
          skip = !(v & 1) && (v & 2);
        }
        if (cw == 0 && lane == 0) {
          if (p.tile_map) {
            const int head = hkv * p.G + g;
            p.tile_map[((((long long)b * p.Hq + head) * p.n_tiles_k + n_block) * p.num_splits + split) *
                           p.num_m_blocks + m] = skip ? (gate_skip ? 3 : 2) : 1;
          }
        }
      }
      if (!skip) {
#pragma unroll
        for (int i = 0; i < 64; i += 2) pk[i >> 1] = pack2<T>(ex2_approx(x[i]), ex2_approx(x[i + 1]));
        const uint32_t pcol = (wg == 0) ? 0u : 96u;
        tmem_st16(tmem_base + lane_addr + TMEM_S + pcol, &pk[0]);
        tmem_st16(tmem_base + lane_addr + TMEM_S + pcol + 16, &pk[16]);
        tmem_st_wait();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_full);
      return skip;
    };

    // ---- dS step: dS^T = P^T o (dP^T - dpsum) into shared memory ------------------------------------
    auto ds_step = [&](int it) {
      const int st = it & 1;
      if (!mbar_wait(&bars->dp_full, n_live & 1, abort_flag)) {
        ok = false;
        return;
      }
      tc_fence_after();
      uint32_t dr[64];
      tmem_ld32(tmem_base + lane_addr + TMEM_DP + wg * 64, &dr[0]);
      tmem_ld32(tmem_base + lane_addr + TMEM_DP + wg * 64 + 32, &dr[32]);
      tmem_ld_wait();
      const float4* dps4 = reinterpret_cast<const float4*>(s_dps + st * 128 + wg * 64);
      const uint4* al4 = reinterpret_cast<const uint4*>(s_alpha + st * 128 + wg * 64);
      uint8_t* slab = ds_buf + wg * (128 * 128);
      float da_r[8];  // gated: per chunk, one column's dalpha summed over 8 lanes
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        const float4 d0 = dps4[ch * 2], d1 = dps4[ch * 2 + 1];  // minus dpsum
        const float nd[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          // both factors are rounded to the 16-bit type and so is their product, like the reference
          // (flash_sparse_bwd.py:93-96). Masked entries carry p = 0 and the other factor is always finite
          // (out-of-range rows of V and dO load as zeros, padding rows of dpsum are zero), so they stay 0.
          const float2 t = add2(make_float2(__uint_as_float(dr[ch * 8 + j]), __uint_as_float(dr[ch * 8 + j + 1])),
                                make_float2(nd[j], nd[j + 1]));
          o[j >> 1] = hmul2<T>(pk[(ch * 8 + j) >> 1], pack2_sat<T>(t.x, t.y));
        }
        *reinterpret_cast<uint4*>(slab + sw128_offset(row, ch)) = make_uint4(o[0], o[1], o[2], o[3]);
        if (KIND == KIND_GATED) {
          // dalpha[q] += sum_k dS g'(alpha_q delta_k) delta_k, ddelta[k] += sum_q dS g'(alpha_q delta_k) alpha_q,
          // g' = sigmoid(-x) for the logsigmoid gate, 1 for the identity (flash_gated_bwd.py:84-88, :152-160)
          const uint4 av = al4[ch];
          float a8[8], v[8];
          unpack16(av.x, a8[0], a8[1]);
          unpack16(av.y, a8[2], a8[3]);
          unpack16(av.z, a8[4], a8[5]);
          unpack16(av.w, a8[6], a8[7]);
#pragma unroll
          for (int j = 0; j < 8; j += 2) {
            float e0, e1;
            unpack16(o[j >> 1], e0, e1);
            if (logsig) {
              e0 *= __fdividef(1.0f, 1.0f + ex2_approx(a8[j] * dlt * 1.4426950408889634f));
              e1 *= __fdividef(1.0f, 1.0f + ex2_approx(a8[j + 1] * dlt * 1.4426950408889634f));
            }
            dd_acc = fmaf(e0, a8[j], dd_acc);
            dd_acc = fmaf(e1, a8[j + 1], dd_acc);
            v[j] = e0 * dlt;
            v[j + 1] = e1 * dlt;
          }
          // three butterfly steps fold the 8 columns onto lane bits 4, 3, 2: one column per lane, summed over 8 lanes
          const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4;
          float u[4], t2[2];
#pragma unroll
          for (int j = 0; j < 4; ++j)
            u[j] = (b4 ? v[j + 4] : v[j]) + __shfl_xor_sync(0xffffffffu, b4 ? v[j] : v[j + 4], 16);
#pragma unroll
          for (int j = 0; j < 2; ++j)
            t2[j] = (b3 ? u[j + 2] : u[j]) + __shfl_xor_sync(0xffffffffu, b3 ? u[j] : u[j + 2], 8);
          da_r[ch] = (b2 ? t2[1] : t2[0]) + __shfl_xor_sync(0xffffffffu, b2 ? t2[0] : t2[1], 4);
        }
      }
      if (KIND == KIND_GATED) {
        // two more steps fold the 8 chunks onto lane bits 1, 0: each lane ends with two complete column sums
        const bool b1 = lane & 2, b0 = lane & 1;
        float u[4], z[2];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          u[j] = (b1 ? da_r[j + 4] : da_r[j]) + __shfl_xor_sync(0xffffffffu, b1 ? da_r[j] : da_r[j + 4], 2);
#pragma unroll
        for (int j = 0; j < 2; ++j)
          z[j] = (b0 ? u[j + 2] : u[j]) + __shfl_xor_sync(0xffffffffu, b0 ? u[j] : u[j + 2], 1);
        const int g = g_cur, m = m_cur;
        const int chunk0 = (b1 ? 4 : 0) + (b0 ? 2 : 0);
        const int cin = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
        float* dst = p.da_accum + (long long)(hkv * p.G + g) * p.ws_sh + pad_off + (long long)m * TM + wg * 64 + cin;
        atomicAdd(dst + chunk0 * 8, z[0]);
        atomicAdd(dst + (chunk0 + 1) * 8, z[1]);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->ds_full);
    };

    int w_g = 0, w_m = 0, w_mode = 0;
    bool w_first = false;
    bool has_cur = ok && walk_next(wk, w_g, w_m, w_mode, w_first, mark_steps);
    const bool any_step = has_cur;
    if (has_cur) {
      skip_cur = p_step(0, w_g, w_m, w_mode, w_first);
      m_cur = m_p;
      g_cur = g_p;
    }
    for (int it = 0; has_cur && ok; ++it) {
      if (!skip_cur) {
        ds_step(it);
        n_live++;
      }
      bool skip_next = false;
      const bool has_next = walk_next(wk, w_g, w_m, w_mode, w_first, mark_steps);
      if (ok && has_next) skip_next = p_step(it + 1, w_g, w_m, w_mode, w_first);
      skip_cur = skip_next;
      m_cur = m_p;
      g_cur = g_p;
      has_cur = has_next;
    }

    // ---- epilogue: dK (scaled) and dV of this key tile ------------------------------------------------
    if (ok) {
      bool have = false;
      if (any_step) {
        ok = mbar_wait(&bars->acc_full, 0, abort_flag);
        tc_fence_after();
        have = n_live > 0;
      }
      if (ok) {
        const long long rowk = off_k + k_idx;
#pragma unroll
        for (int which = 0; which < 2; ++which) {
          const uint32_t tcol = which == 0 ? TMEM_DV : TMEM_DK;
          const float mul = which == 0 ? 1.0f : p.softmax_scale;
          void* outp = which == 0 ? p.dv_out : p.dk_out;
          const long long base = (long long)((p.flags & F_VARLEN_K) ? 0 : b) * p.dkv_sb + rowk * p.dkv_sn +
                                 (long long)hkv * p.dkv_sh + (long long)split * p.dkv_ss + wg * HALF;
#pragma unroll
          for (int ch = 0; ch < HALF / 32; ++ch) {
            uint32_t r[32];
            if (have) {
              tmem_ld32(tmem_base + lane_addr + tcol + wg * HALF + ch * 32, r);
              tmem_ld_wait();
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = 0u;
            }
            if (row_ok) {
              if (p.flags & F_SPLIT) {
                float* dst = reinterpret_cast<float*>(outp) + base + ch * 32;
#pragma unroll
                for (int i = 0; i < 32; i += 4)
                  if (wg * HALF + ch * 32 + i < p.D)
                    *reinterpret_cast<float4*>(dst + i) =
                        make_float4(__uint_as_float(r[i]) * mul, __uint_as_float(r[i + 1]) * mul,
                                    __uint_as_float(r[i + 2]) * mul, __uint_as_float(r[i + 3]) * mul);
              } else {
                T* dst = reinterpret_cast<T*>(outp) + base + ch * 32;
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                  uint4 v;
                  v.x = pack2<T>(__uint_as_float(r[i]) * mul, __uint_as_float(r[i + 1]) * mul);
                  v.y = pack2<T>(__uint_as_float(r[i + 2]) * mul, __uint_as_float(r[i + 3]) * mul);
                  v.z = pack2<T>(__uint_as_float(r[i + 4]) * mul, __uint_as_float(r[i + 5]) * mul);
                  v.w = pack2<T>(__uint_as_float(r[i + 6]) * mul, __uint_as_float(r[i + 7]) * mul);
                  if (wg * HALF + ch * 32 + i < p.D) *reinterpret_cast<uint4*>(dst + i) = v;
                }
              }
            }
          }
        }
      }
    }
    // ---- gated epilogue: ddelta of this key row = (columns 0-63) + (columns 64-127), scaled -------------
    if (KIND == KIND_GATED && ok) {
      float* tmp = s_lse;  // every load of the ring has been consumed by now
      if (wg == 1) {
        tmp[row] = dd_acc;
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->dd_sync);
      } else {
        ok = mbar_wait(&bars->dd_sync, 0, abort_flag);
        if (ok && row_ok) {
          const float val = (dd_acc + tmp[row]) * p.softmax_scale;
          const long long at = (long long)bk * p.d_sb + (long long)hkv * p.d_sh + off_k + k_idx;
          if (p.flags & F_SPLIT)
            reinterpret_cast<float*>(p.dd_out)[(long long)split * p.dd_ss + at] = val;
          else
            reinterpret_cast<T*>(p.dd_out)[at] = T(val);
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
cudaError_t launch_one(const BwdKernelParams& p, cudaStream_t stream) {
  auto kern = bwd_kernel<HD, T, KIND>;
  constexpr int smem = BwdSmem<HD>::kTotal;
  static std::atomic<unsigned long long> opted_in{0};  // one bit per device: the attribute is per device
  if (cudaError_t e = smem_opt_in(kern, smem, opted_in); e != cudaSuccess) return e;
  const long long grid = (long long)p.n_tiles_k * p.Hkv * p.B * p.num_splits;
  if (grid <= 0) return cudaSuccess;
  kern<<<(unsigned)grid, NTHREADS, smem, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace


cudaError_t launch_bwd(const BwdKernelParams& p, int kind, int dtype, int head_dim, cudaStream_t stream) {
#define FSA_BWD_CASE(HD_, T_, DT_)                                               \
  if (head_dim == HD_ && dtype == DT_) {                                         \
    if (kind == KIND_DENSE) return launch_one<HD_, T_, KIND_DENSE>(p, stream);   \
    if (kind == KIND_SPARSE) return launch_one<HD_, T_, KIND_SPARSE>(p, stream); \
    if (kind == KIND_GATED) return launch_one<HD_, T_, KIND_GATED>(p, stream);   \
  }
  FSA_BWD_CASE(128, __nv_bfloat16, DT_BF16)
  FSA_BWD_CASE(128, __half, DT_FP16)
  FSA_BWD_CASE(64, __nv_bfloat16, DT_BF16)
  FSA_BWD_CASE(64, __half, DT_FP16)
#undef FSA_BWD_CASE
  return cudaErrorInvalidValue;
}

}  // namespace fsa
