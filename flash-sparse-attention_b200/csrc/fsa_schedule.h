// Integer tile schedule shared by host and device code.
//
// These functions decide, for one query tile (forward / decode) or one key tile (backward), which
// tiles of the other operand are visited, in which phase (i.e. with which mask) and by which split.
// They restate flash_sparse_attn/ops/triton/block_info.py:5-349 and the three `create` methods of
// flash_sparse_attn/ops/triton/scheduler.py:836-948 (forward), :994-1101 (backward), :1147-1273
// (decode). Integer division truncates toward zero exactly like the Triton source (values can be
// negative before they are clamped), so plain C `/` is intentional here.
#pragma once

#if defined(__CUDACC__)
#define FSA_HD __host__ __device__ __forceinline__
#else
#define FSA_HD static inline
#endif

struct FsaWindow {
  int sink;   // prefix tokens always visible (subject to causality)
  int left;   // width of the distant band
  int right;  // gap between the near band and the distant band
  int near_;  // width of the near-diagonal band
};

// Mask applied to a visited tile (flash_sparse_attn/ops/triton/mask.py:5-104).
enum FsaMaskMode {
  FSA_MASK_NONE = 0,        // tile is fully visible: nothing masked
  FSA_MASK_SEQLEN = 1,      // rows/cols outside the sequence only
  FSA_MASK_CAUSAL = 2,      // seqlen + (near >= 0)
  FSA_MASK_LOCAL = 3,       // seqlen + near band + distant band
  FSA_MASK_LOCAL_SINK = 4,  // seqlen + near band + distant band + sink columns
};

// The nine numbers of AttnFwdBlockScheduler / AttnDecBlockScheduler (names follow the reference).
struct FsaFwdSched {
  int n_min, n_max, n_max_no_mask;
  int win_min, win_max, win_min_no_mask, win_max_no_mask;
  int sink_min, sink_max;
};
// The nine numbers of AttnBwdBlockScheduler.
struct FsaBwdSched {
  int m_min, m_max, m_min_no_mask;
  int win_min, win_max, win_min_no_mask, win_max_no_mask;
  int sink_min, sink_max;
};

FSA_HD int fsa_cdiv(int a, int b) { return (a + b - 1) / b; }
FSA_HD int fsa_imin(int a, int b) { return a < b ? a : b; }
FSA_HD int fsa_imax(int a, int b) { return a > b ? a : b; }

// Share of `total` blocks owned by split `s` of `ns`: the first total%ns splits get one extra.
FSA_HD void fsa_split_range(int total, int ns, int s, int* off, int* cnt) {
  const int base = total / ns, extra = total % ns;
  *off = (s < extra) ? s * (base + 1) : extra * (base + 1) + (s - extra) * base;
  *cnt = (s < extra) ? base + 1 : base;
}

// block_info.py:5-123
//
// `cover_single_query`: with one query position, local windows and split-KV the reference starts the
// near-diagonal range at ceil((n_idx_near + 1) / TILE_N) (block_info.py:60-64). When the near band
// does not begin on a tile boundary that drops the band's first, partial tile: those keys are visible
// in the reference's eager ground truth (tests/test_utils.py:541-563) but never visited by its
// kernel. false reproduces the reference's numbers exactly; true rounds down like the general path,
// so that the visited tiles cover the mask exactly (what the decode kernel uses).
FSA_HD void fsa_n_block_min_max(int sq, int sk, int m_block, int split_idx, FsaWindow w, int num_splits, int TN,
                                int TM, bool causal, bool local, bool split_kv, int gpack, int* o_n_min,
                                int* o_n_max, int* o_win_min, int* o_win_max, int* o_sink_min, int* o_sink_max,
                                bool cover_single_query = false) {
  int n_block_max = fsa_cdiv(sk, TN);
  int n_block_min = 0;
  int win_max = n_block_max, win_min = 0;
  int sink_min = 0, sink_max = 0;
  int n_idx = 0, n_idx_near = 0, sink_excl = 0;
  if (causal || local) {
    int m_idx_max = (m_block + 1) * TM;
    if (gpack > 1) m_idx_max = fsa_cdiv(m_idx_max, gpack);
    m_idx_max = fsa_imin(m_idx_max, sq);
    n_idx = m_idx_max + sk - sq;
    n_block_max = fsa_imin(n_block_max, fsa_cdiv(n_idx, TN));
    if (local) {
      const int n_idx_right = n_idx - w.near_ - w.right;
      win_max = fsa_imin(win_max, fsa_imax(fsa_cdiv(n_idx_right, TN), 0));
    }
  }
  if (local) {
    sink_max = fsa_imin(fsa_cdiv(w.sink, TN), fsa_imax(fsa_cdiv(n_idx, TN), 0));
    sink_excl = fsa_cdiv(w.sink, TN);
    int m_idx_min = m_block * TM;
    if (gpack > 1) m_idx_min = m_idx_min / gpack;
    n_idx = m_idx_min + sk - sq;
    n_idx_near = n_idx - w.near_;
    n_block_min = fsa_imax(n_idx_near / TN, 0);
    n_block_min = fsa_imax(n_block_min, sink_excl);
    const int n_idx_left = n_idx - w.near_ - w.right - w.left;
    win_min = fsa_imax(n_idx_left / TN, 0);
    win_min = fsa_imax(win_min, sink_excl);
  }
  if (split_kv) {
    if (local) {
      int diag_min = (sq == 1 && !cover_single_query) ? fsa_imax(fsa_cdiv(fsa_imax(n_idx_near + 1, 0), TN), 0)
                                                      : n_block_min;
      diag_min = fsa_imax(diag_min, sink_excl);
      const int diag_max = n_block_max;
      win_max = fsa_imax(win_max, win_min);
      diag_min = fsa_imax(diag_min, win_max);
      const int total = fsa_imax(win_max - win_min, 0);
      int off, cnt;
      fsa_split_range(total, num_splits, split_idx, &off, &cnt);
      const int win_min_new = win_min + off;
      win_max = fsa_imin(win_min_new + cnt, win_max);
      win_min = win_min_new;
      sink_max = (split_idx == 0) ? sink_max : 0;
      const int non_diag_max = fsa_imax(win_max, sink_max);
      n_block_max = (split_idx >= num_splits - 1) ? diag_max : non_diag_max;
      n_block_min = (split_idx >= num_splits - 1) ? diag_min : non_diag_max;
    } else {
      const int total = fsa_imax(n_block_max - n_block_min, 0);
      int off, cnt;
      fsa_split_range(total, num_splits, split_idx, &off, &cnt);
      const int n_min_new = n_block_min + off;
      n_block_max = fsa_imin(n_min_new + cnt, n_block_max);
      n_block_min = n_min_new;
      sink_max = (split_idx == 0) ? sink_max : 0;
    }
  }
  n_block_min = fsa_imin(n_block_min, n_block_max);
  if (local) {
    win_max = fsa_imax(fsa_imin(win_max, n_block_min), win_min);
    sink_max = fsa_imax(sink_max, sink_min);
  } else {
    win_min = 0;
    win_max = 0;
  }
  *o_n_min = n_block_min;
  *o_n_max = n_block_max;
  *o_win_min = win_min;
  *o_win_max = win_max;
  *o_sink_min = sink_min;
  *o_sink_max = sink_max;
}

// block_info.py:227-247
FSA_HD int fsa_n_block_min_causal_local_mask(int sq, int sk, int m_block, int n_block_min, int w_right, int w_near,
                                             int TN, int TM, bool local, int gpack) {
  int m_idx_min = m_block * TM;
  if (gpack > 1) m_idx_min = m_idx_min / gpack;
  const int n_idx = m_idx_min + sk - sq;
  const int n_idx_right = local ? n_idx - w_near - w_right : n_idx;
  return fsa_imax(n_block_min, n_idx_right / TN);
}

// block_info.py:250-271
FSA_HD int fsa_n_block_min_before_local_mask(int sq, int sk, int m_block, int n_block_min, FsaWindow w, int TN,
                                             int TM, bool local, int gpack) {
  if (!local) return n_block_min;
  int m_idx_max = (m_block + 1) * TM;
  if (gpack > 1) m_idx_max = fsa_cdiv(m_idx_max, gpack);
  m_idx_max = fsa_imin(m_idx_max, sq);
  const int n_idx = m_idx_max + sk - sq;
  const int n_idx_left = n_idx - w.near_ - w.right - w.left;
  return fsa_imax(n_block_min, fsa_cdiv(n_idx_left, TN));
}

// scheduler.py:836-948 (forward) — also used for decode with sq = 1, m_block = 0 (scheduler.py:1180-1260).
FSA_HD FsaFwdSched fsa_fwd_schedule(int sq, int sk, int m_block, int split_idx, FsaWindow w, int num_splits, int TN,
                                    int TM, bool causal, bool local, bool split_kv, int gpack,
                                    bool cover_single_query = false) {
  FsaFwdSched s;
  fsa_n_block_min_max(sq, sk, m_block, split_idx, w, num_splits, TN, TM, causal, local, split_kv, gpack, &s.n_min,
                      &s.n_max, &s.win_min, &s.win_max, &s.sink_min, &s.sink_max, cover_single_query);
  s.n_max_no_mask = fsa_n_block_min_causal_local_mask(sq, sk, m_block, s.n_min, 0, 0, TN, TM, false, gpack);
  if (split_kv) s.n_max_no_mask = fsa_imin(s.n_max_no_mask, s.n_max);
  if (local) {
    if (split_kv)
      s.n_max_no_mask = (split_idx >= num_splits - 1) ? s.n_min : s.n_max_no_mask;
    else
      s.n_max_no_mask = s.n_min;
    s.win_max_no_mask =
        fsa_n_block_min_causal_local_mask(sq, sk, m_block, s.win_min, w.right, w.near_, TN, TM, true, gpack);
    s.win_min_no_mask = fsa_n_block_min_before_local_mask(sq, sk, m_block, s.win_min, w, TN, TM, true, gpack);
    s.win_max_no_mask = fsa_imax(fsa_imin(s.win_max_no_mask, s.win_max), s.win_min);
    s.win_min_no_mask = fsa_imax(fsa_imin(s.win_min_no_mask, s.win_max_no_mask), s.win_min);
  } else {
    s.win_min = 0;
    s.win_max = 0;
    s.win_min_no_mask = 0;
    s.win_max_no_mask = 0;
  }
  return s;
}

// Decode over a gathered (top-k) key list: block_info.py:321-349, scheduler.py:1159-1176.
FSA_HD FsaFwdSched fsa_topk_schedule(int topk, int split_idx, int num_splits, int TN) {
  FsaFwdSched s;
  const int total = fsa_cdiv(topk, TN);
  int off, cnt;
  fsa_split_range(total, num_splits, split_idx, &off, &cnt);
  s.n_min = off;
  s.n_max = fsa_imin(off + cnt, total);
  s.n_max_no_mask = s.n_max;
  s.win_min = s.win_max = s.win_min_no_mask = s.win_max_no_mask = 0;
  s.sink_min = s.sink_max = 0;
  return s;
}

FSA_HD bool fsa_fwd_sched_empty(const FsaFwdSched& s) {
  return (s.n_max <= s.n_min) && (s.win_max <= s.win_min) && (s.sink_max <= s.sink_min);
}

// Mask mode of key tile `n` for this query tile, or -1 when the tile is not visited.
// Phase order follows flash_sparse_attn/ops/triton/flash_sparse_fwd.py:280-483; every phase walks
// its range downwards and the ranges themselves are disjoint and ordered, so the whole visit
// order is simply descending in n.
FSA_HD int fsa_fwd_tile_mode(const FsaFwdSched& s, int n, bool causal, bool local) {
  if (n >= s.n_min && n < s.n_max) {
    if (causal || local) {
      if (n >= s.n_max_no_mask) return local ? FSA_MASK_LOCAL : FSA_MASK_CAUSAL;
      return FSA_MASK_NONE;  // only reachable when !local
    }
    return (n == s.n_max - 1) ? FSA_MASK_SEQLEN : FSA_MASK_NONE;
  }
  if (local) {
    if (n >= s.win_min && n < s.win_max) {
      if (n >= s.win_max_no_mask) return FSA_MASK_LOCAL;
      if (n >= s.win_min_no_mask) return FSA_MASK_NONE;
      return FSA_MASK_LOCAL;
    }
    if (n >= s.sink_min && n < s.sink_max) return FSA_MASK_LOCAL_SINK;
  }
  return -1;
}

// Largest visited tile index strictly below `n` (or -1).
FSA_HD int fsa_fwd_next_tile_below(const FsaFwdSched& s, int n, bool local) {
  int best = -1;
  if (s.n_max > s.n_min) {
    const int c = fsa_imin(n, s.n_max) - 1;
    if (c >= s.n_min) best = fsa_imax(best, c);
  }
  if (local) {
    if (s.win_max > s.win_min) {
      const int c = fsa_imin(n, s.win_max) - 1;
      if (c >= s.win_min) best = fsa_imax(best, c);
    }
    if (s.sink_max > s.sink_min) {
      const int c = fsa_imin(n, s.sink_max) - 1;
      if (c >= s.sink_min) best = fsa_imax(best, c);
    }
  }
  return best;
}

// block_info.py:126-224
FSA_HD void fsa_m_block_min_max(int sq, int sk, int n_block, int split_idx, FsaWindow w, int num_splits, int TN,
                                int TM, bool causal, bool local, bool split_qo, int* o_m_min, int* o_m_max,
                                int* o_win_min, int* o_win_max, int* o_sink_min, int* o_sink_max) {
  int m_block_max = fsa_cdiv(sq, TM);
  int m_block_min = 0;
  int win_max = m_block_max, win_min = 0;
  int sink_min = 0, sink_max = 0;
  if (causal || local) {
    const int n_idx_min = n_block * TN;
    const int m_idx = n_idx_min + sq - sk;
    m_block_min = fsa_imax(m_block_min, m_idx / TM);
    if (local) {
      const int m_idx_right = m_idx + w.near_ + w.right;
      win_min = fsa_imax(win_min, m_idx_right / TM);
    }
  }
  if (local) {
    const int sink_excl = fsa_cdiv(w.sink, TN);
    const bool is_sink_block = n_block < sink_excl;
    const int n_idx_min = n_block * TN;
    const int m_idx_sink = n_idx_min + sq - sk;
    sink_min = fsa_imax(m_idx_sink / TM, 0);
    sink_max = is_sink_block ? fsa_cdiv(sq, TM) : 0;
    sink_min = is_sink_block ? sink_min : 0;
    const int n_idx_max = (n_block + 1) * TN;
    const int m_idx = n_idx_max + sq - sk;
    const int m_idx_near = m_idx + w.near_;
    m_block_max = fsa_imin(m_block_max, fsa_cdiv(m_idx_near, TM));
    const int m_idx_left = m_idx + w.near_ + w.right + w.left;
    win_max = fsa_imin(win_max, fsa_cdiv(m_idx_left, TM));
    if (is_sink_block) {
      m_block_min = 0;
      m_block_max = 0;
      win_min = 0;
      win_max = 0;
    }
  }
  if (split_qo) {
    if (local) {
      const int n_idx_max = (n_block + 1) * TN;
      const int m_idx = n_idx_max + sq - sk;
      const int m_min_no_mask = fsa_imax(m_block_min, fsa_cdiv(m_idx, TM));
      win_min = fsa_imax(win_min, m_min_no_mask);
      const int win_blocks = fsa_imax(win_max - win_min, 0);
      int off, cnt;
      fsa_split_range(win_blocks, num_splits, split_idx, &off, &cnt);
      win_min = win_min + off;
      win_max = fsa_imin(win_min + cnt, win_max);
      m_block_min = (split_idx == 0) ? m_block_min : m_block_max;
      sink_max = (split_idx == 0) ? sink_max : 0;
      sink_min = (split_idx == 0) ? sink_min : 0;
    } else {
      const int total = fsa_imax(m_block_max - m_block_min, 0);
      int off, cnt;
      fsa_split_range(total, num_splits, split_idx, &off, &cnt);
      const int m_min_new = m_block_min + off;
      m_block_max = fsa_imin(m_min_new + cnt, m_block_max);
      m_block_min = m_min_new;
    }
  }
  m_block_min = fsa_imin(m_block_min, m_block_max);
  if (local) {
    win_min = fsa_imin(fsa_imax(win_min, m_block_max), win_max);
    sink_min = fsa_imin(sink_min, sink_max);
  } else {
    win_min = 0;
    win_max = 0;
  }
  *o_m_min = m_block_min;
  *o_m_max = m_block_max;
  *o_win_min = win_min;
  *o_win_max = win_max;
  *o_sink_min = sink_min;
  *o_sink_max = sink_max;
}

// block_info.py:274-297
FSA_HD int fsa_m_block_min_causal_local_mask(int sq, int sk, int n_block, int m_block_min, int w_right, int w_near,
                                             int TN, int TM, bool causal, bool local) {
  if (!causal && !local) return m_block_min;
  const int n_idx_max = (n_block + 1) * TN;
  const int m_idx = n_idx_max + sq - sk;
  const int m_idx_right = local ? m_idx + w_near + w_right : m_idx;
  return fsa_imax(m_block_min, fsa_cdiv(m_idx_right, TM));
}

// block_info.py:300-318
FSA_HD int fsa_m_block_max_before_local_mask(int sq, int sk, int n_block, int m_block_max, FsaWindow w, int TN,
                                             int TM, bool local) {
  if (!local) return m_block_max;
  const int n_idx_min = n_block * TN;
  const int m_idx = n_idx_min + sq - sk;
  const int m_idx_left = m_idx + w.near_ + w.right + w.left;
  return fsa_imin(m_block_max, m_idx_left / TM);
}

// scheduler.py:994-1101
FSA_HD FsaBwdSched fsa_bwd_schedule(int sq, int sk, int n_block, int split_idx, FsaWindow w, int num_splits, int TN,
                                    int TM, bool causal, bool local, bool split_qo) {
  FsaBwdSched s;
  fsa_m_block_min_max(sq, sk, n_block, split_idx, w, num_splits, TN, TM, causal, local, split_qo, &s.m_min, &s.m_max,
                      &s.win_min, &s.win_max, &s.sink_min, &s.sink_max);
  s.m_min_no_mask =
      fsa_m_block_min_causal_local_mask(sq, sk, n_block, s.m_min, 0, 0, TN, TM, causal || local, false);
  if (split_qo) s.m_min_no_mask = fsa_imin(s.m_min_no_mask, s.m_max);
  if (local) {
    s.m_min_no_mask = s.m_max;
    s.win_min_no_mask =
        fsa_m_block_min_causal_local_mask(sq, sk, n_block, s.win_min, w.right, w.near_, TN, TM, false, true);
    s.win_min_no_mask = fsa_imax(s.win_min_no_mask, s.win_min);
    s.win_max_no_mask = fsa_m_block_max_before_local_mask(sq, sk, n_block, s.win_max, w, TN, TM, true);
    s.win_max_no_mask = fsa_imax(s.win_max_no_mask, s.win_min_no_mask);
    s.win_min_no_mask = fsa_imax(fsa_imin(s.win_min_no_mask, s.win_max), s.win_min);
    s.win_max_no_mask = fsa_imax(fsa_imin(s.win_max_no_mask, s.win_max), s.win_min_no_mask);
  } else {
    s.win_min_no_mask = 0;
    s.win_max_no_mask = 0;
    s.sink_min = 0;
    s.sink_max = 0;
  }
  return s;
}

// Whether query tile `m` is one of the tiles this schedule walks (the union of the phases of
// flash_sparse_attn/ops/triton/flash_sparse_bwd.py:315-464).
FSA_HD bool fsa_bwd_visits(const FsaBwdSched& s, int m, bool causal, bool local) {
  bool in = false;
  // tiles past m_max lie beyond the query rows (the reference visits them with every load masked off)
  const int m_nm = fsa_imin(s.m_min_no_mask, s.m_max);
  if (causal || local) in |= (m >= s.m_min && m < m_nm);
  if (!local) in |= (m >= ((causal || local) ? m_nm : s.m_min) && m < s.m_max);
  if (local) {
    in |= (m >= s.win_min && m < s.win_min_no_mask);
    in |= (m >= s.win_min_no_mask && m < s.win_max_no_mask);
    in |= (m >= s.win_max_no_mask && m < s.win_max);
    in |= (m >= s.sink_min && m < s.sink_max);
  }
  return in;
}

FSA_HD bool fsa_bwd_sched_empty(const FsaBwdSched& s) {
  return (s.m_max <= s.m_min) && (s.win_max <= s.win_min) && (s.sink_max <= s.sink_min);
}
