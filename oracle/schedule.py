"""CPU oracle (test infrastructure only): the reference's integer tile schedule and masks.

Plain-Python restatement of
  * flash_sparse_attn/ops/triton/block_info.py:5-349   (block ranges, split partition)
  * flash_sparse_attn/ops/triton/scheduler.py:836-948   (AttnFwdBlockScheduler.create)
  * flash_sparse_attn/ops/triton/scheduler.py:994-1101  (AttnBwdBlockScheduler.create)
  * flash_sparse_attn/ops/triton/scheduler.py:1147-1273 (AttnDecBlockScheduler.create)
  * flash_sparse_attn/ops/triton/mask.py:5-104          (apply_mask predicates)
  * the phase order of flash_sparse_fwd.py:280-483 and flash_sparse_bwd.py:315-464.

Triton's integer ``//`` truncates toward zero (C semantics) and ``tl.cdiv(x, d)`` is
``(x + d - 1) // d`` with that same division; both are reproduced here with ``_tdiv``.

Pinned by tests/test_oracle_schedule.py: for every configuration tried, the union of visited
tiles x per-phase masks equals the eager attention mask of the reference tests
(tests/test_utils.py:541-563) exactly once per (query, key) pair.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg may import this package.
"""

from dataclasses import dataclass
from typing import List, Tuple

MASK_NONE, MASK_SEQLEN, MASK_CAUSAL, MASK_LOCAL, MASK_LOCAL_SINK = 0, 1, 2, 3, 4


def _tdiv(a: int, b: int) -> int:
    """Integer division truncating toward zero."""
    q = abs(a) // abs(b)
    return q if (a >= 0) == (b > 0) else -q


def _cdiv(a: int, b: int) -> int:
    return _tdiv(a + b - 1, b)


def _split_range(total: int, ns: int, s: int) -> Tuple[int, int]:
    base, extra = total // ns, total % ns
    off = s * (base + 1) if s < extra else extra * (base + 1) + (s - extra) * base
    cnt = base + 1 if s < extra else base
    return off, cnt


@dataclass
class FwdSched:
    n_min: int
    n_max: int
    n_max_no_mask: int
    win_min: int
    win_max: int
    win_min_no_mask: int
    win_max_no_mask: int
    sink_min: int
    sink_max: int

    def as_list(self):
        return [self.n_min, self.n_max, self.n_max_no_mask, self.win_min, self.win_max, self.win_min_no_mask,
                self.win_max_no_mask, self.sink_min, self.sink_max]

    def is_empty(self):
        return self.n_max <= self.n_min and self.win_max <= self.win_min and self.sink_max <= self.sink_min


@dataclass
class BwdSched:
    m_min: int
    m_max: int
    m_min_no_mask: int
    win_min: int
    win_max: int
    win_min_no_mask: int
    win_max_no_mask: int
    sink_min: int
    sink_max: int

    def as_list(self):
        return [self.m_min, self.m_max, self.m_min_no_mask, self.win_min, self.win_max, self.win_min_no_mask,
                self.win_max_no_mask, self.sink_min, self.sink_max]

    def is_empty(self):
        return self.m_max <= self.m_min and self.win_max <= self.win_min and self.sink_max <= self.sink_min


# --------------------------------------------------------------------------------------------------
# forward / decode: key-tile ranges of one query tile (block_info.py:5-123)
# --------------------------------------------------------------------------------------------------
def n_block_min_max(sq, sk, m_block, split_idx, window, num_splits, TN, TM, causal, local, split_kv, gpack,
                    cover_single_query=False):
    sink, left, right, near = window
    n_max = _cdiv(sk, TN)
    n_min = 0
    win_max, win_min = n_max, 0
    sink_min = sink_max = 0
    n_idx = n_idx_near = sink_excl = 0
    if causal or local:
        m_idx_max = (m_block + 1) * TM
        if gpack > 1:
            m_idx_max = _cdiv(m_idx_max, gpack)
        m_idx_max = min(m_idx_max, sq)
        n_idx = m_idx_max + sk - sq
        n_max = min(n_max, _cdiv(n_idx, TN))
        if local:
            win_max = min(win_max, max(_cdiv(n_idx - near - right, TN), 0))
    if local:
        sink_max = min(_cdiv(sink, TN), max(_cdiv(n_idx, TN), 0))
        sink_excl = _cdiv(sink, TN)
        m_idx_min = m_block * TM
        if gpack > 1:
            m_idx_min = _tdiv(m_idx_min, gpack)
        n_idx = m_idx_min + sk - sq
        n_idx_near = n_idx - near
        n_min = max(max(_tdiv(n_idx_near, TN), 0), sink_excl)
        win_min = max(max(_tdiv(n_idx - near - right - left, TN), 0), sink_excl)
    if split_kv:
        if local:
            # cover_single_query=True is NOT the reference: it rounds down so that the first, partial tile of
            # the near band is visited too (the reference's rounding leaves those keys out; see the
            # decode coverage test)
            diag_min = max(_cdiv(max(n_idx_near + 1, 0), TN), 0) if (sq == 1 and not cover_single_query) else n_min
            diag_min = max(diag_min, sink_excl)
            diag_max = n_max
            win_max = max(win_max, win_min)
            diag_min = max(diag_min, win_max)
            off, cnt = _split_range(max(win_max - win_min, 0), num_splits, split_idx)
            new_min = win_min + off
            win_max = min(new_min + cnt, win_max)
            win_min = new_min
            sink_max = sink_max if split_idx == 0 else 0
            non_diag_max = max(win_max, sink_max)
            last = split_idx >= num_splits - 1
            n_max = diag_max if last else non_diag_max
            n_min = diag_min if last else non_diag_max
        else:
            off, cnt = _split_range(max(n_max - n_min, 0), num_splits, split_idx)
            new_min = n_min + off
            n_max = min(new_min + cnt, n_max)
            n_min = new_min
            sink_max = sink_max if split_idx == 0 else 0
    n_min = min(n_min, n_max)
    if local:
        win_max = max(min(win_max, n_min), win_min)
        sink_max = max(sink_max, sink_min)
    else:
        win_min = win_max = 0
    return n_min, n_max, win_min, win_max, sink_min, sink_max


def _n_min_causal_local_mask(sq, sk, m_block, n_min, w_right, w_near, TN, TM, local, gpack):
    m_idx_min = m_block * TM
    if gpack > 1:
        m_idx_min = _tdiv(m_idx_min, gpack)
    n_idx = m_idx_min + sk - sq
    n_idx_right = n_idx - w_near - w_right if local else n_idx
    return max(n_min, _tdiv(n_idx_right, TN))


def _n_min_before_local_mask(sq, sk, m_block, n_min, window, TN, TM, local, gpack):
    if not local:
        return n_min
    _, left, right, near = window
    m_idx_max = (m_block + 1) * TM
    if gpack > 1:
        m_idx_max = _cdiv(m_idx_max, gpack)
    m_idx_max = min(m_idx_max, sq)
    n_idx = m_idx_max + sk - sq
    return max(n_min, _cdiv(n_idx - near - right - left, TN))


def fwd_schedule(sq, sk, m_block, split_idx, window, num_splits, TN, TM, causal, local, split_kv, gpack=1,
                 cover_single_query=False) -> FwdSched:
    """AttnFwdBlockScheduler.create (scheduler.py:836-948); decode uses sq=1, m_block=0, causal=False,
    split_kv=True (scheduler.py:1180-1260)."""
    n_min, n_max, win_min, win_max, sink_min, sink_max = n_block_min_max(
        sq, sk, m_block, split_idx, window, num_splits, TN, TM, causal, local, split_kv, gpack, cover_single_query)
    n_max_no_mask = _n_min_causal_local_mask(sq, sk, m_block, n_min, 0, 0, TN, TM, False, gpack)
    if split_kv:
        n_max_no_mask = min(n_max_no_mask, n_max)
    if local:
        if split_kv:
            n_max_no_mask = n_min if split_idx >= num_splits - 1 else n_max_no_mask
        else:
            n_max_no_mask = n_min
        _, _, right, near = window
        wmax_nm = _n_min_causal_local_mask(sq, sk, m_block, win_min, right, near, TN, TM, True, gpack)
        wmin_nm = _n_min_before_local_mask(sq, sk, m_block, win_min, window, TN, TM, True, gpack)
        wmax_nm = max(min(wmax_nm, win_max), win_min)
        wmin_nm = max(min(wmin_nm, wmax_nm), win_min)
    else:
        win_min = win_max = wmin_nm = wmax_nm = 0
    return FwdSched(n_min, n_max, n_max_no_mask, win_min, win_max, wmin_nm, wmax_nm, sink_min, sink_max)


def topk_schedule(topk, split_idx, num_splits, TN) -> FwdSched:
    """get_topk_n_block_min_max (block_info.py:321-349) + scheduler.py:1159-1176."""
    total = _cdiv(topk, TN)
    off, cnt = _split_range(total, num_splits, split_idx)
    n_max = min(off + cnt, total)
    return FwdSched(off, n_max, n_max, 0, 0, 0, 0, 0, 0)


def fwd_tiles(s: FwdSched, causal: bool, local: bool) -> List[Tuple[int, int]]:
    """Visited key tiles of one query tile in the reference's order, with their mask mode
    (flash_sparse_fwd.py:280-483): diagonal masked -> unmasked -> window right edge -> window
    interior -> window left edge -> sink, each range descending."""
    out = []
    if causal or local:
        for n in range(s.n_max - 1, s.n_max_no_mask - 1, -1):
            out.append((n, MASK_LOCAL if local else MASK_CAUSAL))
        n_max_no_mask = s.n_max_no_mask
    else:
        # (the reference runs this step unconditionally once the tile has any work)
        out.append((s.n_max - 1, MASK_SEQLEN))
        n_max_no_mask = s.n_max - 1
    if not local:
        for n in range(n_max_no_mask - 1, s.n_min - 1, -1):
            out.append((n, MASK_NONE))
    else:
        for n in range(s.win_max - 1, s.win_max_no_mask - 1, -1):
            out.append((n, MASK_LOCAL))
        for n in range(s.win_max_no_mask - 1, s.win_min_no_mask - 1, -1):
            out.append((n, MASK_NONE))
        for n in range(s.win_min_no_mask - 1, s.win_min - 1, -1):
            out.append((n, MASK_LOCAL))
        for n in range(s.sink_max - 1, s.sink_min - 1, -1):
            out.append((n, MASK_LOCAL_SINK))
    return out


# --------------------------------------------------------------------------------------------------
# backward: query-tile ranges of one key tile (block_info.py:126-224)
# --------------------------------------------------------------------------------------------------
def m_block_min_max(sq, sk, n_block, split_idx, window, num_splits, TN, TM, causal, local, split_qo):
    sink, left, right, near = window
    m_max = _cdiv(sq, TM)
    m_min = 0
    win_max, win_min = m_max, 0
    sink_min = sink_max = 0
    if causal or local:
        m_idx = n_block * TN + sq - sk
        m_min = max(m_min, _tdiv(m_idx, TM))
        if local:
            win_min = max(win_min, _tdiv(m_idx + near + right, TM))
    if local:
        sink_excl = _cdiv(sink, TN)
        is_sink = n_block < sink_excl
        m_idx_sink = n_block * TN + sq - sk
        sink_min = max(_tdiv(m_idx_sink, TM), 0) if is_sink else 0
        sink_max = _cdiv(sq, TM) if is_sink else 0
        m_idx = (n_block + 1) * TN + sq - sk
        m_max = min(m_max, _cdiv(m_idx + near, TM))
        win_max = min(win_max, _cdiv(m_idx + near + right + left, TM))
        if is_sink:
            m_min = m_max = win_min = win_max = 0
    if split_qo:
        if local:
            m_idx = (n_block + 1) * TN + sq - sk
            m_min_no_mask = max(m_min, _cdiv(m_idx, TM))
            win_min = max(win_min, m_min_no_mask)
            off, cnt = _split_range(max(win_max - win_min, 0), num_splits, split_idx)
            win_min = win_min + off
            win_max = min(win_min + cnt, win_max)
            m_min = m_min if split_idx == 0 else m_max
            sink_max = sink_max if split_idx == 0 else 0
            sink_min = sink_min if split_idx == 0 else 0
        else:
            off, cnt = _split_range(max(m_max - m_min, 0), num_splits, split_idx)
            new_min = m_min + off
            m_max = min(new_min + cnt, m_max)
            m_min = new_min
    m_min = min(m_min, m_max)
    if local:
        win_min = min(max(win_min, m_max), win_max)
        sink_min = min(sink_min, sink_max)
    else:
        win_min = win_max = 0
    return m_min, m_max, win_min, win_max, sink_min, sink_max


def _m_min_causal_local_mask(sq, sk, n_block, m_min, w_right, w_near, TN, TM, causal, local):
    if not causal and not local:
        return m_min
    m_idx = (n_block + 1) * TN + sq - sk
    m_idx_right = m_idx + w_near + w_right if local else m_idx
    return max(m_min, _cdiv(m_idx_right, TM))


def _m_max_before_local_mask(sq, sk, n_block, m_max, window, TN, TM, local):
    if not local:
        return m_max
    _, left, right, near = window
    m_idx = n_block * TN + sq - sk
    return min(m_max, _tdiv(m_idx + near + right + left, TM))


def bwd_schedule(sq, sk, n_block, split_idx, window, num_splits, TN, TM, causal, local, split_qo) -> BwdSched:
    """AttnBwdBlockScheduler.create (scheduler.py:994-1101)."""
    m_min, m_max, win_min, win_max, sink_min, sink_max = m_block_min_max(
        sq, sk, n_block, split_idx, window, num_splits, TN, TM, causal, local, split_qo)
    m_min_no_mask = _m_min_causal_local_mask(sq, sk, n_block, m_min, 0, 0, TN, TM, causal or local, False)
    if split_qo:
        m_min_no_mask = min(m_min_no_mask, m_max)
    if local:
        _, _, right, near = window
        m_min_no_mask = m_max
        wmin_nm = _m_min_causal_local_mask(sq, sk, n_block, win_min, right, near, TN, TM, False, True)
        wmin_nm = max(wmin_nm, win_min)
        wmax_nm = _m_max_before_local_mask(sq, sk, n_block, win_max, window, TN, TM, True)
        wmax_nm = max(wmax_nm, wmin_nm)
        wmin_nm = max(min(wmin_nm, win_max), win_min)
        wmax_nm = max(min(wmax_nm, win_max), wmin_nm)
    else:
        wmin_nm = wmax_nm = 0
        sink_min = sink_max = 0
    return BwdSched(m_min, m_max, m_min_no_mask, win_min, win_max, wmin_nm, wmax_nm, sink_min, sink_max)


def bwd_tiles(s: BwdSched, causal: bool, local: bool) -> List[Tuple[int, int]]:
    """Visited query tiles of one key tile in the reference's order (flash_sparse_bwd.py:315-464):
    ascending within each phase: diagonal masked -> unmasked -> window (right-masked, interior,
    left-masked) -> sink."""
    out = []
    # without split-QO the reference leaves m_min_no_mask unclamped (scheduler.py:1041-1043): tiles in
    # [m_max, m_min_no_mask) lie past the query rows and contribute nothing, they are not listed
    m_nm = min(s.m_min_no_mask, s.m_max)
    if causal or local:
        for m in range(s.m_min, m_nm):
            out.append((m, MASK_LOCAL if local else MASK_CAUSAL))
        if not local:
            for m in range(m_nm, s.m_max):
                out.append((m, MASK_NONE))
    else:
        for m in range(s.m_min, s.m_max):
            out.append((m, MASK_NONE))
    if local:
        for m in range(s.win_min, s.win_min_no_mask):
            out.append((m, MASK_LOCAL))
        for m in range(s.win_min_no_mask, s.win_max_no_mask):
            out.append((m, MASK_NONE))
        for m in range(s.win_max_no_mask, s.win_max):
            out.append((m, MASK_LOCAL))
        for m in range(s.sink_min, s.sink_max):
            out.append((m, MASK_LOCAL_SINK))
    return out


# --------------------------------------------------------------------------------------------------
# masks (mask.py:52-102)
# --------------------------------------------------------------------------------------------------
def visible(q_idx: int, k_idx: int, sq: int, sk: int, window, mode: int) -> bool:
    """Is score (q_idx, k_idx) kept under mask `mode` (mask.py:60-102)?"""
    if mode == MASK_NONE:
        return True
    if not (k_idx < sk and q_idx < sq):
        return False
    if mode == MASK_SEQLEN:
        return True
    sink, left, right, near_w = window
    near = q_idx + (sk - sq) - k_idx
    if mode == MASK_CAUSAL:
        return near >= 0
    ok = (0 <= near < near_w) or (near_w + right <= near < near_w + right + left)
    if mode == MASK_LOCAL_SINK:
        ok = ok or (k_idx < sink and near >= 0)
    return ok


def allowed(q_idx: int, k_idx: int, sq: int, sk: int, window, causal: bool, local: bool) -> bool:
    """The attention mask of the eager reference (tests/test_utils.py:541-563)."""
    if not (k_idx < sk and q_idx < sq):
        return False
    dist = q_idx + (sk - sq) - k_idx
    if local:
        sink, left, right, near_w = window
        return (k_idx < sink and dist >= 0) or (0 <= dist < near_w) or (near_w + right <= dist < near_w + right + left)
    if causal:
        return dist >= 0
    return True
