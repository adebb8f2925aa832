// Decode attention (one query position per sequence) for sm_100a: a bandwidth kernel.
//
// One CTA serves one KV head of one sequence (and one KV split). The G query heads of that KV head
// are the rows of a 16-row tile (packed GQA, like the reference's decode: scheduler.py:2455-2461).
// The CTA's key range is cut into four contiguous sub-ranges, one per warp; each warp streams its
// keys in 16-key tiles through a private 2-stage cp.async ring (16-byte copies, zero-fill for
// masked / out-of-range rows), runs a complete flash-decoding recurrence on them with mma.sync
// m16n8k16 (the arithmetic is ~8 FLOP/byte, far below the tensor roofline, so the legacy MMA path
// is enough and keeps the kernel free to run several CTAs per SM), and the four partial states are
// merged in shared memory at the end. In terms of the reference's schedule every warp is one KV
// split: the tile ranges come from the same functions with 4 x num_splits splits
// (block_info.py:5-123 for contiguous / paged caches, :321-349 for gathered top-k lists).
// With 16-bit inputs and at most 8 query heads per KV head - and always at head sizes above 128 - the two
// products run transposed (keys on the M side of the MMA, query rows on N = 8; see dec_kernel), eight query
// rows per pass over the keys.
//
// Key addressing covers the reference's three modes and their combination:
//   contiguous  row = key position                               (flash_sparse_dec.py:673-678)
//   paged       row = page_table[b, pos / page] * page + pos % page   (paged_kv.py:10-30)
//   gathered    pos = gather_kv_indices[b, i], negative = masked     (topk_gather_kv.py:5-77)
//   gathered + paged: the gathered logical position goes through the page table (the reference
//   rejects this combination, assert_inputs.py:303-305; here it is defined as the composition).
#include <mma.h>
#include "fsa_aux.h"
#include <type_traits>

#include "fsa_params.h"
#include "fsa_ptx.cuh"
#include "fsa_schedule.h"

namespace fsa {

namespace {

constexpr int DTN = 16;      // keys per warp tile
// cp.async ring depth per warp: 2 tiles of 16-bit rows, 4 of FP8 rows (same shared memory, twice as many row
// fetches in flight). Measured on the paged top-k configuration: depth 2 / 3 = 100.6 / 101.9 us in bf16, 103.4 /
// 106.1 us in FP8; three CTAs per SM (168 registers, depth 2) 120 us.
#ifndef FSA_DEC_STAGES16
#define FSA_DEC_STAGES16 2
#endif
#ifndef FSA_DEC_MINBLOCKS
#define FSA_DEC_MINBLOCKS 2
#endif
template <int ES>
struct DecStages {
  static constexpr int value = ES == 1 ? 2 * FSA_DEC_STAGES16 : FSA_DEC_STAGES16;
};
constexpr int DWARPS = 4;

template <int HD, int ES = 2>
struct DecSmem {
  static constexpr int kRow = HD * ES;                // bytes per key row
  static constexpr int kTile = DTN * kRow;            // one K or V tile
  static constexpr int kWarp = DecStages<ES>::value * 2 * kTile;   // ring of one warp
  static constexpr int kMerge = DWARPS * (16 * HD * 4 + 16 * 8);  // O, m, l of every warp
  static constexpr int kTotal = (DWARPS * kWarp > kMerge ? DWARPS * kWarp : kMerge);
};

// 16-byte asynchronous copy global -> shared: shared address as a register + compile-time offset, run-time source size
// (0: the 16 bytes are zero-filled, nothing is read)
template <int DOFF>
__device__ __forceinline__ void cp_async16_at(uint32_t dst, const void* src, int sz) {
  asm volatile("cp.async.cg.shared.global [%0 + %3], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz), "n"(DOFF) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// compile-time loop: f(std::integral_constant<int, I>) for I = BEGIN .. END - 1
template <int BEGIN, int END, typename F>
__device__ __forceinline__ void unroll_copy(F&& f) {
  if constexpr (BEGIN < END) {
    f(std::integral_constant<int, BEGIN>{});
    unroll_copy<BEGIN + 1, END>(f);
  }
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
// FP8 -> fp16 pairs (exact). `w` holds four FP8 bytes b0..b3; SEL picks two of them:
// 0 -> (b0, b1), 1 -> (b2, b3), 2 -> (b0, b2), 3 -> (b1, b3).
template <typename T, int SEL>
__device__ __forceinline__ uint32_t fp8x2_to_f16x2(uint32_t w) {
  constexpr int first = SEL == 0 ? 0 : (SEL == 1 ? 2 : (SEL == 2 ? 0 : 1));
  constexpr int second = SEL == 0 ? 1 : (SEL == 1 ? 3 : (SEL == 2 ? 2 : 3));
  uint32_t r;
  if (__is_same(T, __nv_fp8_e5m2)) {
    // e5m2 is the upper byte of an fp16: place the bytes at positions 1 and 3
    asm("prmt.b32 %0, %1, 0, %2;" : "=r"(r) : "r"(w), "n"(0x0404 | (first << 4) | (second << 12)));
  } else {
    uint32_t pair;
    asm("prmt.b32 %0, %1, 0, %2;" : "=r"(pair) : "r"(w), "n"(0x4400 | first | (second << 4)));
    asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, lo;\n\t}" : "=r"(r) : "r"(pair));
  }
  return r;
}

// Input element type -> type of the mma.sync operands / of the outputs and gate vectors.
template <typename T>
struct DecTypes {
  using mma = T;
  using out = T;
};
template <>
struct DecTypes<__nv_fp8_e4m3> {
  using mma = __half;
  using out = __nv_bfloat16;
};
template <>
struct DecTypes<__nv_fp8_e5m2> {
  using mma = __half;
  using out = __nv_bfloat16;
};

template <typename T>
__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__half>(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 8 x 8 matrix of 16-bit values held by a warp (lane (g, t): row g, columns 2t, 2t+1) -> its transpose
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}

// TR (16-bit inputs, at most 8 query heads per KV head): the products run transposed, S^T = K Q^T and
// O^T = V^T P^T, so that the 16 keys of a tile fill the M = 16 side of mma.m16n8k16 and the (up to) 8 query rows the
// N = 8 side. With the rows on M, half of every fragment is padding when a KV head serves 8 query heads: transposed, the
// accumulator takes 32 registers instead of 64, the Q fragments 16 instead of 32, a tile needs 8 + 8 MMAs instead of
// 16 + 16, and three CTAs fit an SM instead of two. P^T reaches its B-operand layout through movmatrix.
// OCC: CTAs per SM the kernel is compiled for (the transposed variant exists for 2 and for 3).
template <int HD, typename T, int KIND, bool TR, int OCC>
__global__ void __launch_bounds__(DWARPS * 32, OCC) dec_kernel(const DecKernelParams p) {
  // T: element type of q, k, v. FP8 (e4m3 / e5m2, head size 128) tiles are copied as bytes and widened
  // exactly to fp16 in registers in front of the fp16 mma.sync; a 16-byte chunk of a key row then holds
  // 16 head columns, used in the order the fragments deliver them (q follows the same order).
  constexpr int ES = sizeof(T);
  constexpr bool F8 = ES == 1;
  using TM = typename DecTypes<T>::mma;   // mma.sync operand type
  using TO = typename DecTypes<T>::out;   // outputs, alpha, delta
  using SM = DecSmem<HD, ES>;
  constexpr int CH = HD * ES / 16;  // 16-byte chunks per key row
  constexpr int DSTAGES = DecStages<ES>::value;
  static_assert(!F8 || HD == 128, "FP8 rows are 128 bytes: eight chunks, as the swizzle assumes");
  static_assert(!(TR && F8), "the transposed products take 16-bit tiles");
  extern __shared__ __align__(128) uint8_t dsm[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;

  int idx = blockIdx.x;
  const int hkv = idx % p.Hkv;
  idx /= p.Hkv;
  const int b = idx / p.num_splits;
  const int split = idx - b * p.num_splits;
  const bool gather = p.flags & F_GATHER, paged = p.flags & F_PAGED, local = p.flags & F_LOCAL;
  // peer exchange: which of the two receive buffers this step uses (the count of exchanges sent so far lives in this
  // rank's region; the last CTA of the grid advances it)
  unsigned long long peer_step = 0;
  long long peer_slot = 0;
  if (p.peer_world > 0) {
    peer_step = *reinterpret_cast<const volatile unsigned long long*>(p.peer_base[p.peer_rank] + 128);
    peer_slot = ((long long)(peer_step & 1ull) * p.peer_world + p.peer_rank) * p.peer_block_floats;
  }
  const int off_k = (p.flags & F_VARLEN_K) ? p.cu_k[b] : 0;
  const int sk = (p.flags & F_USED_K) ? p.used_k[b] : ((p.flags & F_VARLEN_K) ? p.cu_k[b + 1] - off_k : p.sk);
  const int bk = (p.flags & F_VARLEN_K) ? 0 : b;
  FsaWindow w = {0, 0, 0, 0};
  if (local) {
    const int* wp = p.windows + (long long)hkv * p.win_stride;
    w.sink = wp[0];
    w.left = wp[1];
    w.right = wp[2];
    w.near_ = wp[3];
  }
  const int nsub = p.num_splits * DWARPS;
  const int sub = split * DWARPS + warp;
  // gathered rows: only the leading `topk` entries can be valid (all of them unless the caller says fewer)
  const int topk = (gather && p.gather_count) ? min(p.topk, p.gather_count[b]) : p.topk;
  const FsaFwdSched sched = gather ? fsa_topk_schedule(topk, sub, nsub, DTN)
                                   : fsa_fwd_schedule(1, sk, 0, sub, w, nsub, DTN, 16, false, local, true, p.G,
                                                      /*cover_single_query=*/true);
  const bool loc_sched = local && !gather;
  const float c = p.qkv_scale ? p.scale_log2 * p.qkv_scale[0] * p.qkv_scale[1] : p.scale_log2;
  const float v_scale = p.qkv_scale ? p.qkv_scale[2] : 1.0f;
  // threshold / visible keys (seqlen_info.py:141-149); a shard of a longer sequence is told the whole length
  const float thr_keys = float(p.thr_sk ? p.thr_sk[b] : sk);
  const float thr_log2 = (KIND != KIND_DENSE) ? log2f(fmaxf(fminf(p.softmax_thr / thr_keys, 1.0f), 0.0f)) : 0.f;
  const int* gidx = gather ? p.gather_idx + (long long)b * p.gi_stride : nullptr;
  const int key_lo = p.key_bounds ? p.key_bounds[2 * b] : 0, key_hi = p.key_bounds ? p.key_bounds[2 * b + 1] : 0;
  const int* ptab = paged ? p.page_table + (long long)b * p.pt_stride : nullptr;
  const int capacity = paged ? p.pt_stride * p.page_size
                             : ((p.flags & F_VARLEN_K) ? p.cu_k[b + 1] - off_k : p.sk_capacity);

  // page sizes are powers of two (checked on the host): positions split into page / row by shift and mask
  const int page_shift = paged ? (31 - __clz(p.page_size)) : 0;
  const int page_mask = paged ? (p.page_size - 1) : 0;
  uint8_t* ring = dsm + warp * SM::kWarp;
  const char* kbase = reinterpret_cast<const char*>(p.k);
  const char* vbase = reinterpret_cast<const char*>(p.v);

  // lane constants of the tile copies (see issue_tile)
  constexpr int RPI = 32 / CH;  // rows per warp instruction
  static_assert(RPI >= 1 && RPI <= 8 && (RPI & (RPI - 1)) == 0 && DTN % RPI == 0, "copy layout");
  const int lane_h = lane / CH, lane_ch = lane % CH;
  const bool lane_col_ok = lane_ch * (16 / ES) < p.D;  // columns past the real head size read as zeros
  const int lane_sz = lane_col_ok ? 16 : 0;
  const char* lane_k = kbase + (lane_col_ok ? lane_ch * 16 : 0);
  const char* lane_v = vbase + (lane_col_ok ? lane_ch * 16 : 0);
  const uint32_t lane_x4 = uint32_t((lane_ch ^ lane_h) << 4);
  const uint32_t ring_u32 = smem_u32(ring);

  // Address translation of a tile runs two tiles ahead of its copies, one dependent load per loop iteration, so that
  // neither the read of the gathered position nor the page-table look-up behind it stalls the warp in front of the
  // copies: stage A reads the position of key `lane` of a tile (gathered: from the index row), stage B - one
  // iteration later, when that load has landed - maps it into this shard and reads its page, and the iteration
  // after that turns (position, page) into the row address and issues the copies.
  auto xlat_a = [&](int n) -> int {
    int raw = -1;
    if (n >= 0 && lane < DTN) {
      const int i = n * DTN + lane;
      if (gather)
        raw = (i < topk) ? gidx[i] : -1;
      else
        raw = (i < sk) ? i : -1;
    }
    return raw;
  };
  auto xlat_b = [&](int raw, int* pos_out) -> int {
    int pos = raw;
    if (gather && p.key_bounds) pos = (pos >= key_lo && pos < key_hi) ? pos - key_lo : -1;
    if (pos >= capacity) pos = -1;
    *pos_out = pos;
    return (paged && pos >= 0) ? ptab[pos >> page_shift] : 0;
  };

  // Issue the copies of tile n (key `lane` at position `pos` in page `page`, from the translation stages) into ring
  // slot `slot`; returns the bitmask of keys that exist.
  // Gated kernels also fetch delta of key (lane & 15) into *dval (0 for keys that do not exist).
  auto issue_tile = [&](int n, int pos, int page, int slot, float* dval) -> unsigned {
    long long e = -1;
    if (lane < DTN && pos >= 0)
      e = paged ? (long long)page * p.k_sb + (long long)(pos & page_mask) * p.k_sn + (long long)hkv * p.k_sh
                : (long long)bk * p.k_sb + (long long)(off_k + pos) * p.k_sn + (long long)hkv * p.k_sh;
    if (KIND == KIND_GATED) {
      float dv = 0.f;
      if (lane < DTN && e >= 0) {
        const long long de = paged ? (long long)page * p.d_sb + (long long)hkv * p.d_sh +
                                         (pos & page_mask)
                                   : (long long)bk * p.d_sb + (long long)hkv * p.d_sh + off_k + pos;
        dv = float(reinterpret_cast<const TO*>(p.delta)[de]);
      }
      *dval = __shfl_sync(0xffffffffu, dv, lane & 15);
    }
    const unsigned present = __ballot_sync(0xffffffffu, e >= 0) & 0xffffu;
    // Lane l copies chunk l % CH of the rows RPI * it + l / CH: a warp instruction moves whole rows (one request per
    // row; 32-byte pieces of sixteen rows per instruction ran 4.5 times slower). The row's byte offset comes from
    // its owner lane by shuffle; everything else per copy is lane-constant or compile-time: the chunk's offset in
    // the row, the swizzled place in the tile (chunk ^ row & 7 = (chunk ^ l / CH) ^ (RPI * it & 7)) and, from the
    // ballot, whether the row exists.
    const long long rowb = e >= 0 ? e * ES : 0;  // a row that does not exist copies nothing: any valid address
    const unsigned rlo = (unsigned)rowb, rhi = (unsigned)(rowb >> 32);
    const uint32_t kd = ring_u32 + slot * 2 * SM::kTile + lane_h * SM::kRow;
    const unsigned ph = present >> lane_h;
    unroll_copy<0, DTN / RPI>([&](auto it_tag) {
      constexpr int it = decltype(it_tag)::value;
      const int src_lane = RPI * it + lane_h;
      const unsigned lo = __shfl_sync(0xffffffffu, rlo, src_lane), hi = __shfl_sync(0xffffffffu, rhi, src_lane);
      const long long rb = (long long)(((unsigned long long)hi << 32) | lo);
      const int sz = int((ph >> (RPI * it)) & 1u) * lane_sz;
      const uint32_t d = kd + (lane_x4 ^ (((RPI * it) & 7) << 4));
      cp_async16_at<it * RPI * SM::kRow>(d, lane_k + rb, sz);
      cp_async16_at<it * RPI * SM::kRow + SM::kTile>(d, lane_v + rb, sz);
    });
    return present;
  };

  constexpr int MROWS = TR ? 8 : 16;  // query rows of a KV head handled per pass over the keys
  const int n_mtiles = (p.G + MROWS - 1) / MROWS;
  for (int mt = 0; mt < n_mtiles; ++mt) {
    // ---- Q fragments of this warp (all warps hold the same rows) --------------------------------
    // TR: this lane's two rows are 2t and 2t+1 (columns of S^T); otherwise g and g + 8
    uint32_t qa[HD / 16][TR ? 2 : 4];
    if constexpr (TR) {
      // B fragments of Q^T: head columns 16 kk + 2t, +1 and 16 kk + 8 + 2t, +1 of query row g
      const int qrow = mt * 8 + g;
      const T* q0 = reinterpret_cast<const T*>(p.q) + (long long)b * p.q_sb + (long long)(hkv * p.G + qrow) * p.q_sh;
#pragma unroll
      for (int kk = 0; kk < HD / 16; ++kk) {
        const bool lo = kk * 16 + 2 * t < p.D, hi = kk * 16 + 8 + 2 * t < p.D;
        qa[kk][0] = (qrow < p.G && lo) ? *reinterpret_cast<const uint32_t*>(q0 + kk * 16 + 2 * t) : 0u;
        qa[kk][1] = (qrow < p.G && hi) ? *reinterpret_cast<const uint32_t*>(q0 + kk * 16 + 8 + 2 * t) : 0u;
      }
    } else {
      const int r0 = mt * 16 + g, r1 = r0 + 8;
      const T* q0 = reinterpret_cast<const T*>(p.q) + (long long)b * p.q_sb + (long long)(hkv * p.G + r0) * p.q_sh;
      const T* q1 = reinterpret_cast<const T*>(p.q) + (long long)b * p.q_sb + (long long)(hkv * p.G + r1) * p.q_sh;
      if constexpr (F8) {
        // step kk uses head columns 16 kk + 4t .. +3: the first two as k = 2t, 2t+1, the others as k = 2t+8, 2t+9
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t w0 = (r0 < p.G) ? *reinterpret_cast<const uint32_t*>(q0 + kk * 16 + 4 * t) : 0u;
          const uint32_t w1 = (r1 < p.G) ? *reinterpret_cast<const uint32_t*>(q1 + kk * 16 + 4 * t) : 0u;
          qa[kk][0] = fp8x2_to_f16x2<T, 0>(w0);
          qa[kk][1] = fp8x2_to_f16x2<T, 0>(w1);
          qa[kk][2] = fp8x2_to_f16x2<T, 1>(w0);
          qa[kk][3] = fp8x2_to_f16x2<T, 1>(w1);
        }
      } else {
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const bool lo = kk * 16 + 2 * t < p.D, hi = kk * 16 + 8 + 2 * t < p.D;
          qa[kk][0] = (r0 < p.G && lo) ? *reinterpret_cast<const uint32_t*>(q0 + kk * 16 + 2 * t) : 0u;
          qa[kk][1] = (r1 < p.G && lo) ? *reinterpret_cast<const uint32_t*>(q1 + kk * 16 + 2 * t) : 0u;
          qa[kk][2] = (r0 < p.G && hi) ? *reinterpret_cast<const uint32_t*>(q0 + kk * 16 + 8 + 2 * t) : 0u;
          qa[kk][3] = (r1 < p.G && hi) ? *reinterpret_cast<const uint32_t*>(q1 + kk * 16 + 8 + 2 * t) : 0u;
        }
      }
    }
    const int row0 = TR ? mt * 8 + 2 * t : mt * 16 + g, row1 = TR ? row0 + 1 : row0 + 8;  // this lane's two query rows
    const bool row0_ok = row0 < p.G, row1_ok = row1 < p.G;
    // ---- gated: alpha of the two rows, its extremes over the real rows, the running gate bound ----
    float al0 = 0.f, al1 = 0.f, a_max = 0.f, a_min = 0.f, gate_max = -INFINITY;
    // Gate decisions taken BEFORE a tile's rows are requested: with the per-tile extremes of delta in gate_ws
    // (dec_gate_ext_kernel) the bound of activations.py:265-299 is evaluated when the walk reaches a tile, and a
    // gate-skipped tile never enters the ring. Without the workspace the bound is evaluated when the tile is consumed.
    const bool gate_early = (KIND == KIND_GATED) && p.gate_ws != nullptr;
    const float2* gext = gate_early ? reinterpret_cast<const float2*>(p.gate_ws) + ((long long)b * p.Hkv + hkv) * p.n_tiles
                                    : nullptr;
    float dlq[DSTAGES];  // gated: delta of key (lane & 15) of the tiles in the ring, oldest first
#pragma unroll
    for (int i = 0; i < DSTAGES; ++i) dlq[i] = 0.f;
    const float gate_thr_log2 = (KIND == KIND_GATED) ? log2f(p.gate_thr) : 0.f;
    if (KIND == KIND_GATED) {
      const TO* ab = reinterpret_cast<const TO*>(p.alpha) + (long long)b * p.a_sb;
      if (row0_ok) al0 = float(ab[(long long)(hkv * p.G + row0) * p.a_sh]);
      if (row1_ok) al1 = float(ab[(long long)(hkv * p.G + row1) * p.a_sh]);
      a_max = fmaxf(row0_ok ? al0 : -INFINITY, row1_ok ? al1 : -INFINITY);
      a_min = fminf(row0_ok ? al0 : INFINITY, row1_ok ? al1 : INFINITY);
#pragma unroll
      for (int sft = 16; sft > 0; sft >>= 1) {
        a_max = fmaxf(a_max, __shfl_xor_sync(0xffffffffu, a_max, sft));
        a_min = fminf(a_min, __shfl_xor_sync(0xffffffffu, a_min, sft));
      }
    }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float lg_l[2] = {-INFINITY, -INFINITY};  // log2(l_run) for the skip test, refreshed after every update of l_run
    float o[TR ? HD / 16 : HD / 8][4];  // TR: O^T, 16 head columns x 8 rows per entry
#pragma unroll
    for (int j = 0; j < (TR ? HD / 16 : HD / 8); ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;

    // ---- ring prologue ----------------------------------------------------------------------------
    // without local windows the visited tiles are one descending range
    auto tile_below = [&](int n) {
      return loc_sched ? fsa_fwd_next_tile_below(sched, n, true) : (n - 1 >= sched.n_min ? n - 1 : -1);
    };
    int n_walk = fsa_fwd_next_tile_below(sched, 1 << 28, loc_sched);
    // next tile whose rows are fetched (-1: none left)
    auto next_fetch = [&]() -> int {
      while (n_walk >= 0) {
        const int n = n_walk;
        n_walk = tile_below(n_walk);
        if (gate_early) {
          const float2 de = __ldg(gext + n);
          const float gmc = fmaxf(fmaxf(a_max * de.x, a_max * de.y), fmaxf(a_min * de.x, a_min * de.y));
          const bool gskip = (gmc - gate_max) * c < gate_thr_log2;
          if (gskip) {
            if (p.tile_map && lane == 0 && mt == 0) p.tile_map[((long long)b * p.Hkv + hkv) * p.n_tiles + n] = 3;
            continue;
          }
          gate_max = fmaxf(gmc, gate_max);
        }
        return n;
      }
      return -1;
    };
    unsigned present_q[DSTAGES];  // presence masks of the tiles in the ring, oldest first
    int n_q[DSTAGES];             // their tile indices (-1: empty)
    int slot_load = 0;
    // translation pipeline: tile xa_n has its position read under way, tile xb_n its page. It is primed with the
    // first three tiles at once - three position reads in flight, then two page reads - instead of one stage per
    // dependent load: a CTA's first tile is requested a load latency earlier.
    const int x0_n = next_fetch(), x1_n = next_fetch(), x2_n = next_fetch();
    const int x0_raw = xlat_a(x0_n), x1_raw = xlat_a(x1_n), x2_raw = xlat_a(x2_n);
    int x0_pos = -1, xb_pos = -1;
    const int x0_page = xlat_b(x0_raw, &x0_pos);
    int xb_n = x1_n;
    int xb_page = xlat_b(x1_raw, &xb_pos);
    int xa_n = x2_n, xa_raw = x2_raw;
    // hands out the tile whose translation is complete and moves the two younger ones up a stage
    auto xlat_pop = [&](int* pos, int* page) -> int {
      const int n = xb_n;
      *pos = xb_pos;
      *page = xb_page;
      xb_n = xa_n;
      xb_page = xlat_b(xa_raw, &xb_pos);
      xa_n = next_fetch();
      xa_raw = xlat_a(xa_n);
      return n;
    };
#pragma unroll
    for (int s = 0; s < DSTAGES - 1; ++s) {
      present_q[s] = 0;
      int pos = x0_pos, page = x0_page;
      n_q[s] = s == 0 ? x0_n : xlat_pop(&pos, &page);
      if (n_q[s] >= 0) present_q[s] = issue_tile(n_q[s], pos, page, s, &dlq[s]);
      cp_async_commit();
    }
    present_q[DSTAGES - 1] = 0;
    n_q[DSTAGES - 1] = -1;
    slot_load = DSTAGES - 1;
    int slot = 0;
    while (n_q[0] >= 0) {
      const int n = n_q[0];
      // keep the ring full, then wait for the oldest tile
      unsigned pres_new = 0;
      int pos_new, page_new;
      const int n_new = xlat_pop(&pos_new, &page_new);
      if (n_new >= 0) pres_new = issue_tile(n_new, pos_new, page_new, slot_load, &dlq[DSTAGES - 1]);
      cp_async_commit();
      present_q[DSTAGES - 1] = pres_new;
      n_q[DSTAGES - 1] = n_new;
      slot_load = (slot_load + 1) % DSTAGES;
      cp_async_wait<DSTAGES - 1>();
      __syncwarp();
      const unsigned present = present_q[0];
#pragma unroll
      for (int i = 0; i + 1 < DSTAGES; ++i) {
        present_q[i] = present_q[i + 1];
        n_q[i] = n_q[i + 1];
      }
      const uint32_t kt = smem_u32(ring + slot * 2 * SM::kTile);
      const uint32_t vt = kt + SM::kTile;

      // ---- visibility of the 16 keys (row-uniform: every packed row is the same query position) ------
      unsigned vis = present;
      if (!gather) {
        const int mode = fsa_fwd_tile_mode(sched, n, true, local);
        if (mode != FSA_MASK_NONE) {
          const int k_idx = n * DTN + (lane & 15);
          const int diag = sk - 1;
          bool okk = k_idx < sk;
          if (mode == FSA_MASK_LOCAL || mode == FSA_MASK_LOCAL_SINK) {
            const int near = diag - k_idx;
            bool band = (near >= 0 && near < w.near_) ||
                        (near >= w.near_ + w.right && near < w.near_ + w.right + w.left);
            if (mode == FSA_MASK_LOCAL_SINK) band = band || (k_idx < w.sink && near >= 0);
            okk = okk && band;
          }
          vis &= __ballot_sync(0xffffffffu, okk) & 0xffffu;
        }
      }

      // ---- gated: bound of the gate over the tile, running maximum, skip
      // (flash_sparse_attn/ops/triton/activations.py:265-299) ------------------------------------------
      if (KIND == KIND_GATED && !gate_early) {
        float dmax = dlq[0], dmin = dlq[0];
#pragma unroll
        for (int sft = 8; sft > 0; sft >>= 1) {
          dmax = fmaxf(dmax, __shfl_xor_sync(0xffffffffu, dmax, sft));
          dmin = fminf(dmin, __shfl_xor_sync(0xffffffffu, dmin, sft));
        }
        const float gmc = fmaxf(fmaxf(a_max * dmax, a_max * dmin), fmaxf(a_min * dmax, a_min * dmin));
        const bool gate_skip = (gmc - gate_max) * c < gate_thr_log2;
        if (!gate_skip) gate_max = fmaxf(gmc, gate_max);
        if (gate_skip) {
          if (p.tile_map && lane == 0 && mt == 0) p.tile_map[((long long)b * p.Hkv + hkv) * p.n_tiles + n] = 3;
          __syncwarp();
          slot = (slot + 1) % DSTAGES;
#pragma unroll
          for (int i = 0; i + 1 < DSTAGES; ++i) dlq[i] = dlq[i + 1];
          continue;
        }
      }

      if constexpr (TR) {
        // ---- S^T = K Q^T: keys g and g + 8 (rows), query rows 2t and 2t + 1 (columns) --------------------
        float st[4] = {0.f, 0.f, 0.f, 0.f}, st_alt[4] = {0.f, 0.f, 0.f, 0.f};  // two chains of dependent MMAs
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const int r = (lane & 7) + 8 * ((lane >> 3) & 1);
          const int ch = 2 * kk + (lane >> 4);
          uint32_t a[4];
          ldsm_x4(kt + r * SM::kRow + ((ch ^ (r & 7)) << 4), a[0], a[1], a[2], a[3]);
          mma16816<TM>((kk & 1) ? st_alt : st, a, qa[kk][0], qa[kk][1]);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) st[e] += st_alt[e];
        if (KIND == KIND_GATED) {
          const bool logsig = p.flags & F_LOGSIGMOID;
          const float dk_lo = __shfl_sync(0xffffffffu, dlq[0], g), dk_hi = __shfl_sync(0xffffffffu, dlq[0], g + 8);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float x = ((e & 1) ? al1 : al0) * (e < 2 ? dk_lo : dk_hi);
            st[e] += logsig ? log_sigmoid_fast(x) : x;
          }
        }
        if (vis != 0xffffu) {
          if (!((vis >> g) & 1u)) st[0] = st[1] = -INFINITY;
          if (!((vis >> (g + 8)) & 1u)) st[2] = st[3] = -INFINITY;
        }
        float m_cur[2] = {fmaxf(st[0], st[2]), fmaxf(st[1], st[3])};
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          m_cur[r] = fmaxf(m_cur[r], __shfl_xor_sync(0xffffffffu, m_cur[r], 4));
          m_cur[r] = fmaxf(m_cur[r], __shfl_xor_sync(0xffffffffu, m_cur[r], 8));
          m_cur[r] = fmaxf(m_cur[r], __shfl_xor_sync(0xffffffffu, m_cur[r], 16));
        }
        bool skip = false;
        if (KIND != KIND_DENSE) {
          // flash_sparse_attn/ops/triton/activations.py:129-138 over the real rows of the tile
          const float v0 = (m_cur[0] - m_run[0]) * c - lg_l[0] - thr_log2;
          const float v1 = (m_cur[1] - m_run[1]) * c - lg_l[1] - thr_log2;
          const bool want = (row0_ok && v0 >= 0.f) || (row1_ok && v1 >= 0.f);
          const bool drop = (row0_ok && v0 < 0.f) || (row1_ok && v1 < 0.f);
          skip = !__any_sync(0xffffffffu, want) && __any_sync(0xffffffffu, drop);
          if (p.tile_map && lane == 0 && mt == 0)
            p.tile_map[((long long)b * p.Hkv + hkv) * p.n_tiles + n] = skip ? 2 : 1;
        }
        if (!skip) {
          float scale[2];
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            // the reference maximum moves only when it lags by more than 2^8 (always on the first tile)
            const float m_cand = fmaxf(fmaxf(m_cur[r], m_run[r]), -1e6f);
            scale[r] = 1.0f;
            if (!((m_cand - m_run[r]) * c <= 8.0f)) {
              scale[r] = ex2_approx((m_run[r] - m_cand) * c);
              m_run[r] = m_cand;
            }
          }
          const float mc0 = m_run[0] * c, mc1 = m_run[1] * c;
          const float p0 = ex2_approx(fmaf(st[0], c, -mc0)), p1 = ex2_approx(fmaf(st[1], c, -mc1));
          const float p2 = ex2_approx(fmaf(st[2], c, -mc0)), p3 = ex2_approx(fmaf(st[3], c, -mc1));
          // P^T as the B operand: (keys 2t, 2t+1 | 2t+8, 2t+9) x row g = the transposes of the two 8 x 8 blocks
          const uint32_t pb0 = movmatrix_trans(pack2<TM>(p0, p1)), pb1 = movmatrix_trans(pack2<TM>(p2, p3));
          float sum0 = p0 + p2, sum1 = p1 + p3;
#pragma unroll
          for (int sft = 4; sft <= 16; sft <<= 1) {
            sum0 += __shfl_xor_sync(0xffffffffu, sum0, sft);
            sum1 += __shfl_xor_sync(0xffffffffu, sum1, sft);
          }
          l_run[0] = l_run[0] * scale[0] + sum0;
          l_run[1] = l_run[1] * scale[1] + sum1;
          if (KIND != KIND_DENSE) {
            lg_l[0] = lg2_approx(l_run[0]);
            lg_l[1] = lg2_approx(l_run[1]);
          }
          if (__any_sync(0xffffffffu, scale[0] != 1.f || scale[1] != 1.f)) {
#pragma unroll
            for (int j = 0; j < HD / 16; ++j) {
              o[j][0] *= scale[0];
              o[j][1] *= scale[1];
              o[j][2] *= scale[0];
              o[j][3] *= scale[1];
            }
          }
          // ---- O^T += V^T P^T: 16 head columns per MMA ------------------------------------------------------
#pragma unroll
          for (int jd = 0; jd < HD / 16; ++jd) {
            const int r = (lane & 7) + 8 * (lane >> 4);
            const int ch = 2 * jd + ((lane >> 3) & 1);
            uint32_t a[4];
            ldsm_x4_t(vt + r * SM::kRow + ((ch ^ (r & 7)) << 4), a[0], a[1], a[2], a[3]);
            mma16816<TM>(o[jd], a, pb0, pb1);
          }
        }
      } else {
        // ---- S = Q K^T over this tile: 2 key groups of 8 ------------------------------------------------
        float s[2][4], s_alt[2][4];  // two accumulators per key group: half as long a chain of dependent MMAs
  #pragma unroll
        for (int j = 0; j < 2; ++j) {
          s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
          s_alt[j][0] = s_alt[j][1] = s_alt[j][2] = s_alt[j][3] = 0.f;
        }
        if constexpr (F8) {
          // one ldmatrix.x4 = four 16-byte chunks = four k-steps; every register carries the four head
          // columns 4t .. 4t+3 of its chunk for key row g
  #pragma unroll
          for (int kk = 0; kk < HD / 16; kk += 4) {
  #pragma unroll
            for (int j = 0; j < 2; ++j) {
              const int r = 8 * j + (lane & 7);
              const int ch = kk + (lane >> 3);
              uint32_t w[4];
              ldsm_x4(kt + r * SM::kRow + ((ch ^ (r & 7)) << 4), w[0], w[1], w[2], w[3]);
  #pragma unroll
              for (int i = 0; i < 4; ++i)
                mma16816<TM>((i & 1) ? s_alt[j] : s[j], qa[kk + i], fp8x2_to_f16x2<T, 0>(w[i]), fp8x2_to_f16x2<T, 1>(w[i]));
            }
          }
        } else {
  #pragma unroll
          for (int kk = 0; kk < HD / 16; kk += 2) {
  #pragma unroll
            for (int j = 0; j < 2; ++j) {
              const int r = 8 * j + (lane & 7);
              const int ch = 2 * kk + (lane >> 3);
              uint32_t b0, b1, b2, b3;
              ldsm_x4(kt + r * SM::kRow + ((ch ^ (r & 7)) << 4), b0, b1, b2, b3);
              mma16816<TM>(s[j], qa[kk], b0, b1);
              mma16816<TM>(s_alt[j], qa[kk + 1], b2, b3);
            }
          }
        }
  #pragma unroll
        for (int j = 0; j < 2; ++j)
  #pragma unroll
          for (int e = 0; e < 4; ++e) s[j][e] += s_alt[j][e];
        if (KIND == KIND_GATED) {
          // logits = (q.k + g(alpha * delta)) * scale (flash_sparse_attn/ops/triton/flash_gated_dec.py)
          const bool logsig = p.flags & F_LOGSIGMOID;
  #pragma unroll
          for (int j = 0; j < 2; ++j)
  #pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float dk = __shfl_sync(0xffffffffu, dlq[0], 8 * j + 2 * t + (e & 1));
              const float x = (e < 2 ? al0 : al1) * dk;
              float gte = x;
              if (logsig)
                gte = log_sigmoid_fast(x);
              s[j][e] += gte;
            }
        }
        // mask: element (j, e) is key 8j + 2t + (e & 1)
        if (vis != 0xffffu) {
  #pragma unroll
          for (int j = 0; j < 2; ++j)
  #pragma unroll
            for (int e = 0; e < 4; ++e)
              if (!((vis >> (8 * j + 2 * t + (e & 1))) & 1u)) s[j][e] = -INFINITY;
        }

        float m_cur[2];
        m_cur[0] = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
        m_cur[1] = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
  #pragma unroll
        for (int r = 0; r < 2; ++r) {
          m_cur[r] = fmaxf(m_cur[r], __shfl_xor_sync(0xffffffffu, m_cur[r], 1));
          m_cur[r] = fmaxf(m_cur[r], __shfl_xor_sync(0xffffffffu, m_cur[r], 2));
        }

        bool skip = false;
        if (KIND != KIND_DENSE) {
          // flash_sparse_attn/ops/triton/activations.py:129-138 over the real rows of the tile
          const float v0 = (m_cur[0] - m_run[0]) * c - lg_l[0] - thr_log2;
          const float v1 = (m_cur[1] - m_run[1]) * c - lg_l[1] - thr_log2;
          const bool want = (row0_ok && v0 >= 0.f) || (row1_ok && v1 >= 0.f);
          const bool drop = (row0_ok && v0 < 0.f) || (row1_ok && v1 < 0.f);
          skip = !__any_sync(0xffffffffu, want) && __any_sync(0xffffffffu, drop);
          if (p.tile_map && lane == 0 && mt == 0)
            p.tile_map[((long long)b * p.Hkv + hkv) * p.n_tiles + n] = skip ? 2 : 1;
        }
        if (!skip) {
          float scale[2];
          uint32_t pa[4];
  #pragma unroll
          for (int r = 0; r < 2; ++r) {
            // the reference maximum moves only when it lags by more than 2^8 (always on the first tile, where it is
            // -inf): the exponentials stay below 2^8, the sums in fp32, and the rescaling of the 16 x HD accumulator,
            // which otherwise runs on most tiles of a short walk, becomes rare
            const float m_cand = fmaxf(fmaxf(m_cur[r], m_run[r]), -1e6f);
            scale[r] = 1.0f;
            if (!((m_cand - m_run[r]) * c <= 8.0f)) {
              scale[r] = ex2_approx((m_run[r] - m_cand) * c);
              m_run[r] = m_cand;
            }
          }
          const float mc0 = m_run[0] * c, mc1 = m_run[1] * c;
          float sum0 = 0.f, sum1 = 0.f;
  #pragma unroll
          for (int j = 0; j < 2; ++j) {
            const float p0 = ex2_approx(fmaf(s[j][0], c, -mc0)), p1 = ex2_approx(fmaf(s[j][1], c, -mc0));
            const float p2 = ex2_approx(fmaf(s[j][2], c, -mc1)), p3 = ex2_approx(fmaf(s[j][3], c, -mc1));
            sum0 += p0 + p1;
            sum1 += p2 + p3;
            pa[2 * j] = pack2<TM>(p0, p1);
            pa[2 * j + 1] = pack2<TM>(p2, p3);
          }
          sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
          sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
          sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
          sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
          l_run[0] = l_run[0] * scale[0] + sum0;
          l_run[1] = l_run[1] * scale[1] + sum1;
          if (KIND != KIND_DENSE) {  // needed by the next tile's vote: its latency runs under the P V products
            lg_l[0] = lg2_approx(l_run[0]);
            lg_l[1] = lg2_approx(l_run[1]);
          }
          if (__any_sync(0xffffffffu, scale[0] != 1.f || scale[1] != 1.f)) {
  #pragma unroll
            for (int j = 0; j < HD / 8; ++j) {
              o[j][0] *= scale[0];
              o[j][1] *= scale[0];
              o[j][2] *= scale[1];
              o[j][3] *= scale[1];
            }
          }
          // ---- O += P V -----------------------------------------------------------------------------------
          if constexpr (F8) {
            // The transposing ldmatrix moves byte PAIRS: a register holds head columns (2g, 2g+1) of its
            // chunk for keys 2t and 2t+1. Even and odd columns are split into two MMAs, whose accumulators
            // o[2c] / o[2c+1] then stand for head columns 16c + 4t + {0, 2} / {1, 3}.
  #pragma unroll
            for (int jd = 0; jd < HD / 32; ++jd) {
              const int r = (lane & 7) + 8 * ((lane >> 3) & 1);
              const int ch = 2 * jd + (lane >> 4);
              uint32_t w0, w1, w2, w3;  // chunk 2jd: keys 0-7, keys 8-15; chunk 2jd+1: keys 0-7, keys 8-15
              ldsm_x4_t(vt + r * SM::kRow + ((ch ^ (r & 7)) << 4), w0, w1, w2, w3);
              mma16816<TM>(o[4 * jd], pa, fp8x2_to_f16x2<T, 2>(w0), fp8x2_to_f16x2<T, 2>(w1));
              mma16816<TM>(o[4 * jd + 1], pa, fp8x2_to_f16x2<T, 3>(w0), fp8x2_to_f16x2<T, 3>(w1));
              mma16816<TM>(o[4 * jd + 2], pa, fp8x2_to_f16x2<T, 2>(w2), fp8x2_to_f16x2<T, 2>(w3));
              mma16816<TM>(o[4 * jd + 3], pa, fp8x2_to_f16x2<T, 3>(w2), fp8x2_to_f16x2<T, 3>(w3));
            }
          } else {
  #pragma unroll
            for (int jd = 0; jd < HD / 16; ++jd) {
              const int r = (lane & 7) + 8 * ((lane >> 3) & 1);
              const int ch = 2 * jd + (lane >> 4);
              uint32_t b0, b1, b2, b3;
              ldsm_x4_t(vt + r * SM::kRow + ((ch ^ (r & 7)) << 4), b0, b1, b2, b3);
              mma16816<TM>(o[2 * jd], pa, b0, b1);
              mma16816<TM>(o[2 * jd + 1], pa, b2, b3);
            }
          }
        }
      }
      __syncwarp();
      slot = (slot + 1) % DSTAGES;
#pragma unroll
      for (int i = 0; i + 1 < DSTAGES; ++i) dlq[i] = dlq[i + 1];
    }
    cp_async_wait<0>();
    __syncthreads();  // every warp is done with its ring: the space becomes the merge buffer

    // ---- merge the four warps (flash_sparse_attn/ops/triton/flash_dec_combine.py:15-153 in spirit) -----
    float* mo = reinterpret_cast<float*>(dsm) + warp * (16 * HD + 32);
    float* mm = mo + 16 * HD;
    float* ml = mm + 16;
    if constexpr (TR) {
#pragma unroll
      for (int jd = 0; jd < HD / 16; ++jd) {
        mo[(2 * t) * HD + 16 * jd + g] = o[jd][0];
        mo[(2 * t + 1) * HD + 16 * jd + g] = o[jd][1];
        mo[(2 * t) * HD + 16 * jd + g + 8] = o[jd][2];
        mo[(2 * t + 1) * HD + 16 * jd + g + 8] = o[jd][3];
      }
    } else if constexpr (F8) {
#pragma unroll
      for (int cch = 0; cch < HD / 16; ++cch) {
        *reinterpret_cast<float4*>(mo + g * HD + 16 * cch + 4 * t) =
            make_float4(o[2 * cch][0], o[2 * cch + 1][0], o[2 * cch][1], o[2 * cch + 1][1]);
        *reinterpret_cast<float4*>(mo + (g + 8) * HD + 16 * cch + 4 * t) =
            make_float4(o[2 * cch][2], o[2 * cch + 1][2], o[2 * cch][3], o[2 * cch + 1][3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < HD / 8; ++j) {
        *reinterpret_cast<float2*>(mo + g * HD + 8 * j + 2 * t) = make_float2(o[j][0], o[j][1]);
        *reinterpret_cast<float2*>(mo + (g + 8) * HD + 8 * j + 2 * t) = make_float2(o[j][2], o[j][3]);
      }
    }
    if (TR ? g == 0 : t == 0) {
      mm[row0 - mt * MROWS] = m_run[0];
      mm[row1 - mt * MROWS] = m_run[1];
      ml[row0 - mt * MROWS] = l_run[0];
      ml[row1 - mt * MROWS] = l_run[1];
    }
    __syncthreads();
    const float* all = reinterpret_cast<const float*>(dsm);
    for (int item = tid; item < 16 * (HD / 4); item += DWARPS * 32) {
      const int r = item / (HD / 4), d0 = (item % (HD / 4)) * 4;
      const int row = mt * MROWS + r;
      if (r >= MROWS || row >= p.G || d0 >= p.D) continue;
      float m_tot = -INFINITY;
#pragma unroll
      for (int ww = 0; ww < DWARPS; ++ww) m_tot = fmaxf(m_tot, all[ww * (16 * HD + 32) + 16 * HD + r]);
      float l_tot = 0.f;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int ww = 0; ww < DWARPS; ++ww) {
        const float* base = all + ww * (16 * HD + 32);
        const float mw = base[16 * HD + r], lw = base[16 * HD + 16 + r];
        const float wgt = (mw == -INFINITY || lw == 0.f) ? 0.f : ex2_approx((mw - m_tot) * c);
        l_tot += lw * wgt;
        const float4 ov = *reinterpret_cast<const float4*>(base + r * HD + d0);
        acc.x += ov.x * wgt;
        acc.y += ov.y * wgt;
        acc.z += ov.z * wgt;
        acc.w += ov.w * wgt;
      }
      const bool dead = (l_tot == 0.f) || (l_tot != l_tot);
      const float inv = dead ? 1.f : v_scale / l_tot;
      const int head = hkv * p.G + row;
      if (p.flags & F_SPLIT) {
        const long long o_at = (long long)split * p.op_ss + ((long long)b * p.Hq + head) * p.D + d0;
        const long long l_at = (long long)split * p.lp_ss + (long long)head * p.B + b;
        const float4 ov = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
        const float lv = dead ? -INFINITY : m_tot * c + log2f(l_tot);
        if (p.peer_world > 0) {
          // the packed block of this rank, stored into the receive buffer of every rank (plain peer stores)
          const long long lse_off = p.lse_partial - p.out_partial;
          for (int r = 0; r < p.peer_world; ++r) {
            float* blk = reinterpret_cast<float*>(p.peer_base[r] + 256) + peer_slot;
            *reinterpret_cast<float4*>(blk + o_at) = ov;
            if (d0 == 0) blk[lse_off + l_at] = lv;
          }
        } else {
          *reinterpret_cast<float4*>(p.out_partial + o_at) = ov;
          if (d0 == 0) p.lse_partial[l_at] = lv;
        }
      } else {
        TO* dst = reinterpret_cast<TO*>(p.out) + (long long)b * p.o_sb + (long long)head * p.o_sh + d0;
        uint2 v;
        v.x = pack2<TO>(acc.x * inv, acc.y * inv);
        v.y = pack2<TO>(acc.z * inv, acc.w * inv);
        *reinterpret_cast<uint2*>(dst) = v;
        if (d0 == 0)
          p.lse[(long long)b * p.l_sb + (long long)head * p.l_sh] =
              dead ? -INFINITY : (m_tot * c + log2f(l_tot)) * 0.6931471805599453f;
      }
    }
    __syncthreads();
  }
  if (p.peer_world > 0) {
    // every store of this CTA is ordered before its arrivals; the last CTA counts the exchange as sent
    __threadfence_system();
    __syncthreads();
    if (tid == 0) {
      for (int r = 0; r < p.peer_world; ++r)
        atomicAdd_system(reinterpret_cast<unsigned long long*>(p.peer_base[r]) + p.peer_rank, 1ull);
      unsigned char* mine = p.peer_base[p.peer_rank];
      unsigned int* done = reinterpret_cast<unsigned int*>(mine + 136);
      if (atomicAdd(done, 1u) == gridDim.x - 1) {
        *done = 0u;
        *reinterpret_cast<volatile unsigned long long*>(mine + 128) = peer_step + 1;
      }
    }
  }
}

// One half-warp per (sequence, KV head, 16-key tile): the extremes of delta over the tile's keys, with the key
// addressing of the decode kernel (contiguous, packed, paged, gathered) and 0 for keys that do not exist (the
// reference's masked loads read 0 there, scheduler.py:2572-2600). The decode kernel takes its gate decisions from
// these before it requests a tile's rows.
template <typename TO>
__global__ void __launch_bounds__(256) dec_gate_ext_kernel(const DecKernelParams p) {
  const int lane = threadIdx.x & 31, l16 = lane & 15;
  const long long item = ((long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * 2 + (lane >> 4);
  const long long n_items = (long long)p.B * p.Hkv * p.n_tiles;
  float v = 0.f;
  if (item < n_items) {
    const int n = (int)(item % p.n_tiles);
    const int hkv = (int)((item / p.n_tiles) % p.Hkv);
    const int b = (int)(item / ((long long)p.n_tiles * p.Hkv));
    const bool gather = p.flags & F_GATHER, paged = p.flags & F_PAGED;
    const int off_k = (p.flags & F_VARLEN_K) ? p.cu_k[b] : 0;
    const int sk = (p.flags & F_USED_K) ? p.used_k[b] : ((p.flags & F_VARLEN_K) ? p.cu_k[b + 1] - off_k : p.sk);
    const int bk = (p.flags & F_VARLEN_K) ? 0 : b;
    const int capacity = paged ? p.pt_stride * p.page_size
                               : ((p.flags & F_VARLEN_K) ? p.cu_k[b + 1] - off_k : p.sk_capacity);
    const int i = n * DTN + l16;
    int pos;
    if (gather) {
      const int topk = p.gather_count ? min(p.topk, p.gather_count[b]) : p.topk;
      pos = (i < topk) ? p.gather_idx[(long long)b * p.gi_stride + i] : -1;
      if (p.key_bounds) pos = (pos >= p.key_bounds[2 * b] && pos < p.key_bounds[2 * b + 1]) ? pos - p.key_bounds[2 * b] : -1;
    } else {
      pos = (i < sk) ? i : -1;
    }
    if (pos >= 0 && pos < capacity) {
      long long de;
      if (paged) {
        const int page = p.page_table[(long long)b * p.pt_stride + pos / p.page_size];
        de = (long long)page * p.d_sb + (long long)hkv * p.d_sh + (pos % p.page_size);
      } else {
        de = (long long)bk * p.d_sb + (long long)hkv * p.d_sh + off_k + pos;
      }
      v = float(reinterpret_cast<const TO*>(p.delta)[de]);
    }
  }
  float mx = v, mn = v;
#pragma unroll
  for (int sft = 8; sft > 0; sft >>= 1) {
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, sft));
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, sft));
  }
  if (l16 == 0 && item < n_items) reinterpret_cast<float2*>(p.gate_ws)[item] = make_float2(mx, mn);
}

template <int HD, typename T, int KIND, bool TR, int OCC>
cudaError_t launch_variant(const DecKernelParams& p, cudaStream_t stream) {
  auto kern = dec_kernel<HD, T, KIND, TR, OCC>;
  // the variant for two CTAs per SM asks for enough shared memory that a third cannot join
  constexpr int ring = DecSmem<HD, sizeof(T)>::kTotal;
  constexpr int smem = (TR && OCC == 2 && ring < 80 * 1024) ? 80 * 1024 : ring;
  static std::atomic<unsigned long long> opted_in{0};  // one bit per device: the attribute is per device
  if (cudaError_t e = smem_opt_in(kern, smem, opted_in); e != cudaSuccess) return e;
  const long long grid = (long long)p.Hkv * p.B * p.num_splits;
  if (grid <= 0) return cudaSuccess;
  if (KIND == KIND_GATED && p.gate_ws) {
    const long long items = (long long)p.B * p.Hkv * p.n_tiles;
    if (items > 0) {
      dec_gate_ext_kernel<typename DecTypes<T>::out><<<(unsigned)((items + 15) / 16), 256, 0, stream>>>(p);
      if (cudaError_t e = cudaGetLastError(); e != cudaSuccess) return e;
    }
  }
  kern<<<(unsigned)grid, DWARPS * 32, smem, stream>>>(p);
  return cudaGetLastError();
}

template <int HD, typename T, int KIND>
cudaError_t launch_one(const DecKernelParams& p, cudaStream_t stream) {
  if constexpr (HD > 128) {
    // head sizes above 128: only the transposed variant (its accumulator still fits the registers: 16 x 4 per lane),
    // eight query rows per pass over the keys; the 128 KB ring leaves one CTA per SM
    return launch_variant<HD, T, KIND, true, 2>(p, stream);
  } else {
    if constexpr (sizeof(T) == 2) {
      if (p.G <= 8) {
        // Transposed products (see dec_kernel), at three or at two CTAs per SM. The grid runs in rounds of occ x SMs
        // CTAs and a CTA takes about occ times longer with occ neighbours (the step is bandwidth bound), so the cost
        // is rounds x CTAs per SM: 512 CTAs on 148 SMs are two rounds either way and run faster two per SM (92
        // against 107 us), 440 CTAs are one round of three (82 us).
        const long long sms = device_sm_count();
        const long long ctas = (long long)p.Hkv * p.B * p.num_splits;
        const long long per_sm = (ctas + sms - 1) / sms;
        auto cost = [&](long long occ) { return ((ctas + occ * sms - 1) / (occ * sms)) * (per_sm < occ ? per_sm : occ); };
        return cost(3) <= cost(2) ? launch_variant<HD, T, KIND, true, 3>(p, stream)
                                  : launch_variant<HD, T, KIND, true, 2>(p, stream);
      }
    }
    return launch_variant<HD, T, KIND, false, FSA_DEC_MINBLOCKS>(p, stream);
  }
}

}  // namespace

cudaError_t launch_dec(const DecKernelParams& p, int kind, int dtype, int head_dim, cudaStream_t stream) {
#define FSA_DEC_CASE(HD_, T_, DT_)                                               \
  if (head_dim == HD_ && dtype == DT_) {                                         \
    if (kind == KIND_DENSE) return launch_one<HD_, T_, KIND_DENSE>(p, stream);   \
    if (kind == KIND_SPARSE) return launch_one<HD_, T_, KIND_SPARSE>(p, stream); \
    if (kind == KIND_GATED) return launch_one<HD_, T_, KIND_GATED>(p, stream);   \
  }
  FSA_DEC_CASE(128, __nv_bfloat16, DT_BF16)
  FSA_DEC_CASE(128, __half, DT_FP16)
  FSA_DEC_CASE(64, __nv_bfloat16, DT_BF16)
  FSA_DEC_CASE(64, __half, DT_FP16)
  FSA_DEC_CASE(256, __nv_bfloat16, DT_BF16)
  FSA_DEC_CASE(256, __half, DT_FP16)
  FSA_DEC_CASE(128, __nv_fp8_e4m3, DT_E4M3)
  FSA_DEC_CASE(128, __nv_fp8_e5m2, DT_E5M2)
#undef FSA_DEC_CASE
  return cudaErrorInvalidValue;
}

}  // namespace fsa
