"""CPU oracle (test infrastructure only): tile-faithful forward, backward and decode with the reference's
skip rules (softmax threshold and gate bound), returning the per-tile decision maps.

Walks the reference kernel's loop structure on the CPU, one (batch, head, query tile, split) "program"
at a time, in fp32:
  * tile schedule and phase order: oracle/schedule.py (block_info.py, scheduler.py, flash_sparse_fwd.py:280-483)
  * per-row softmax threshold: flash_sparse_attn/ops/triton/seqlen_info.py:118-153
  * one inner step: flash_sparse_attn/ops/triton/flash_sparse_fwd.py:27-88
      S = Q K^T (raw, fp32) -> mask -> online_sparse_softmax (activations.py:103-166):
      skip the tile iff max over rows of ((rowmax(S) - m) * c - log2(l) - thr_log2) < 0, NaN rows ignored
      unless all rows are NaN; otherwise m, l update with exp2, P cast to the value dtype, O += P V
  * finalize: activations.py:169-203 (dead rows -> O = 0, lse = -inf; base-2 lse when split)
  * split-KV merge: flash_sparse_attn/ops/triton/flash_fwd_combine.py:118-161
Rows and key columns outside the sequence read as zeros (the reference loads through bounds-checked
descriptors), which matters only for the skip vote of fully-visible tiles.

  * gated: flash_gated_fwd.py:27-125, :330-373 (gate added to the raw scores before the scale; the interval bound
    of activations.py:265-299 against a running scalar, first tile of a program exempt), threshold of
    seqlen_info.py:156-191
  * backward: flash_sparse_bwd.py:29-107, :315-464 and flash_gated_bwd.py:30-167 (ascending query tiles, the skip
    tests true probabilities exp2(S c - lse2); the gate bound runs per key tile over the query tiles)
  * decode: flash_sparse_dec.py:27-100, flash_gated_dec.py, block_info.py:321-349
It returns the outputs AND the per-tile decision map (1 = computed, 2 = skipped by the softmax threshold,
3 = skipped by the gate bound), which is what the
skip-set parity tests compare with the kernel's own map. The reference's tests never enable skipping
(they pass threshold -128), so for skip sets this file is the only oracle: parity of skip sets is
pinned to this restatement, not to reference outputs ("parity unpinned" by the reference itself).

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg may import this package.
"""

import numpy as np
import torch

from . import schedule as S

LOG2E = 1.44269504089
LN2 = 0.6931471805599453


def _f32(x):
    return torch.tensor(x, dtype=torch.float32)


def softmax_threshold_log2(threshold, q_idx, sq, sk, causal):
    """seqlen_info.py:118-153. q_idx: int64 tensor of (unpacked) query positions of the tile rows."""
    if causal:
        visible = (q_idx + (sk - sq) + 1).float()
    else:
        visible = torch.full(q_idx.shape, float(sk))
    with torch.no_grad():
        t = torch.clamp(torch.minimum(_f32(threshold) / visible, _f32(1.0)), min=0.0)
        return torch.log2(t)


def _tile_mask(mode, q_idx, k_idx, sq, sk, window):
    """bool [TM, TN] of kept scores for mask mode `mode` (mask.py:52-102)."""
    qi = q_idx.unsqueeze(1)
    ki = k_idx.unsqueeze(0)
    in_seq = (ki < sk) & (qi < sq)
    if mode == S.MASK_SEQLEN:
        return in_seq
    near = qi + (sk - sq) - ki
    if mode == S.MASK_CAUSAL:
        return in_seq & (near >= 0)
    sink, left, right, near_w = window
    ok = ((near >= 0) & (near < near_w)) | ((near >= near_w + right) & (near < near_w + right + left))
    if mode == S.MASK_LOCAL_SINK:
        ok = ok | ((ki < sink) & (near >= 0))
    return in_seq & ok


def _nanmax_lt0(val):
    """`tl.max(x) < 0.0` as the reference evaluates it: the maximum ignores NaN entries unless all are NaN,
    and NaN < 0 is False. Returns (skip, margin) with margin = that maximum (NaN when all entries are)."""
    good = val[~torch.isnan(val)]
    if good.numel() == 0:
        return False, float("nan")
    mx = good.max().item()
    return mx < 0.0, mx


class _Decisions:
    """Softmax-skip decisions of one run. With `force` (a tile map of another implementation run on the same
    inputs) the walk takes that map's decision for every tile it computes, so that later tiles see the same
    running state, and only records what it would have decided itself: `margin` holds, per tile, the maximum
    over rows of (log2 of the tile's largest probability bound) - (log2 threshold); the tile is skipped iff
    that is < 0. A forced decision that contradicts a margin far from 0 is a real disagreement."""

    def __init__(self, shape, force):
        self.margin = torch.full(shape, float("nan"))
        self.force = force

    def decide(self, idx, val, dense):
        if dense:
            return False
        skip, m = _nanmax_lt0(val)
        self.margin[idx] = m
        if self.force is not None and int(self.force[idx]) in (1, 2):
            return int(self.force[idx]) == 2
        return skip


def log_sigmoid(x):
    """activations.py:245-262 with FASTMATH=False: min(x, 0) - log(1 + exp(-|x|))."""
    return torch.minimum(x, _f32(0.0)) - torch.log(1.0 + torch.exp(-x.abs()))


def gate_threshold_log2(gate_threshold, q_idx, sq, sk, causal, adapt):
    """seqlen_info.py:156-191: scalar bound of one query tile (q_idx: positions of ALL tile rows, also those
    past the sequence end)."""
    g = np.float32(gate_threshold)
    if causal and adapt:
        vis = (q_idx + (sk - sq)).float() + 1.0
        g_thr = (torch.tensor(g) * vis / float(sk)).min()
    else:
        g_thr = torch.tensor(g)
    with np.errstate(all="ignore"):
        return np.float32(torch.log2(g_thr.float()).item())


def gate_step(a_max, a_min, d_max, d_min, gate_max, c, thr_log2):
    """activations.py:265-299 in fp32, operation for operation. Returns (gate_max_new, skip)."""
    f = np.float32
    with np.errstate(all="ignore"):
        a_max, a_min, d_max, d_min = f(a_max), f(a_min), f(d_max), f(d_min)
        cur = max(max(a_max * d_max, a_max * d_min), max(a_min * d_max, a_min * d_min))
        diff = f(f(cur - f(gate_max)) * f(c))
        skip = bool(diff < f(thr_log2))
    return (f(gate_max) if skip else max(cur, f(gate_max))), skip


def forward_tiled(q, k, v, softmax_scale=None, is_causal=False, window_sizes=None, softmax_threshold=1.0,
                  num_splits=1, is_split_kv=False, pack_gqa=False, tile_m=128, tile_n=128, dense=False,
                  alpha=None, delta=None, gate_threshold=None, is_logsigmoid_gate=True, is_adapt_gate=True,
                  force_map=None, return_margin=False):
    """q [B,Sq,Hq,D], k/v [B,Sk,Hkv,D] (16-bit); window_sizes int [Hkv,4] or None; gated when alpha [B,Sq,Hq]
    and delta [B,Sk,Hkv] are given (gate_threshold None = 1 / Sk, flash_gated_fwd.py:872).
    Returns (out [B,Sq,Hq,D] in q.dtype, lse [B,Hq,Sq] natural log, tile_map uint8
    [B, Hgrid, m_blocks, splits, n_blocks][, margin]); force_map / margin: see _Decisions."""
    B, sq, hq, D = q.shape
    sk, hkv = k.shape[1], k.shape[2]
    G = hq // hkv
    gpack = G if (pack_gqa and G > 1) else 1
    local = window_sizes is not None
    if softmax_scale is None:
        softmax_scale = D ** -0.5
    c = float(_f32(softmax_scale) * _f32(LOG2E))
    ns = num_splits if is_split_kv else 1
    hgrid = hkv if gpack > 1 else hq
    m_blocks = -(-sq * gpack // tile_m)
    n_blocks = -(-sk // tile_n)
    tile_map = torch.zeros(B, hgrid, m_blocks, ns, n_blocks, dtype=torch.uint8)
    dec = _Decisions(tile_map.shape, force_map)
    out_p = torch.zeros(ns, B, sq, hq, D, dtype=torch.float32)
    lse_p = torch.full((ns, B, hq, sq), float("-inf"), dtype=torch.float32)

    qf, kf, vf = q.float(), k.float(), v.float()
    gated = alpha is not None
    if gated:
        af, df = alpha.float(), delta.float()
        if gate_threshold is None:
            gate_threshold = 1.0 / sk
    for b in range(B):
        for hg in range(hgrid):
            h_kv = hg if gpack > 1 else hg // G
            window = [int(x) for x in window_sizes[h_kv].tolist()] if local else [0, 0, 0, 0]
            for mb in range(m_blocks):
                offs_m = torch.arange(mb * tile_m, (mb + 1) * tile_m)
                q_idx = offs_m // gpack
                heads = (h_kv * G + (offs_m - q_idx * gpack)) if gpack > 1 else torch.full_like(offs_m, hg)
                row_ok = q_idx < sq
                q_tile = torch.zeros(tile_m, D)
                q_tile[row_ok] = qf[b, q_idx[row_ok], heads[row_ok]]
                thr = softmax_threshold_log2(softmax_threshold, q_idx, sq, sk, is_causal)
                if gated:
                    a_tile = torch.zeros(tile_m)
                    a_tile[row_ok] = af[b, q_idx[row_ok], heads[row_ok]]
                    a_max, a_min = a_tile.max().item(), a_tile.min().item()
                    g_thr = gate_threshold_log2(gate_threshold, q_idx, sq, sk, is_causal, is_adapt_gate)
                for sp in range(ns):
                    sched = S.fwd_schedule(sq, sk, mb, sp, window, ns, tile_n, tile_m, is_causal, local,
                                           is_split_kv, gpack)
                    if sched.is_empty():
                        continue
                    m = torch.full((tile_m,), float("-inf"))
                    l = torch.zeros(tile_m)
                    acc = torch.zeros(tile_m, D)
                    gate_max, first = np.float32(float("-inf")), True
                    for n, mode in S.fwd_tiles(sched, is_causal, local):
                        k_idx = torch.arange(n * tile_n, (n + 1) * tile_n)
                        col_ok = k_idx < sk
                        if gated:
                            d_tile = torch.zeros(tile_n)
                            d_tile[col_ok] = df[b, k_idx[col_ok], h_kv]
                            gate_max, gskip = gate_step(a_max, a_min, d_tile.max().item(), d_tile.min().item(),
                                                        gate_max, c, g_thr)
                            if gskip and not first:  # the first tile of a program is never gate-skipped
                                tile_map[b, hg, mb, sp, n] = 3
                                continue
                            first = False
                        k_tile = torch.zeros(tile_n, D)
                        v_tile = torch.zeros(tile_n, D)
                        k_tile[col_ok] = kf[b, k_idx[col_ok], h_kv]
                        v_tile[col_ok] = vf[b, k_idx[col_ok], h_kv]
                        s = q_tile @ k_tile.t()
                        if gated:
                            gte = a_tile.unsqueeze(1) * d_tile.unsqueeze(0)
                            s = s + (log_sigmoid(gte) if is_logsigmoid_gate else gte)
                        if mode != S.MASK_NONE:
                            keep = _tile_mask(mode, q_idx, k_idx, sq, sk, window)
                            s = torch.where(keep, s, _f32(float("-inf")))
                        m_cur = s.max(dim=1).values
                        skip = dec.decide((b, hg, mb, sp, n), (m_cur - m) * c - torch.log2(l) - thr, dense)
                        tile_map[b, hg, mb, sp, n] = 2 if skip else 1
                        if skip:
                            continue
                        m_new = torch.maximum(m_cur, m)
                        if mode != S.MASK_NONE:
                            m_new = torch.clamp(m_new, min=-1e6)  # CHECK_INF
                        scale = torch.exp2((m - m_new) * c)
                        p = torch.exp2(s * c - (m_new * c).unsqueeze(1))
                        l = l * scale + p.sum(dim=1)
                        m = m_new
                        acc = acc * scale.unsqueeze(1) + p.to(v.dtype).float() @ v_tile
                    dead = (l == 0) | torch.isnan(l)
                    inv = torch.where(dead, _f32(1.0), 1.0 / l)
                    lse2 = torch.where(dead, _f32(float("-inf")), m * c + torch.log2(l))
                    rows = row_ok.nonzero().squeeze(1)
                    out_p[sp, b, q_idx[rows], heads[rows]] = (acc * inv.unsqueeze(1))[rows]
                    lse_p[sp, b, heads[rows], q_idx[rows]] = lse2[rows]
    # merge the splits (flash_fwd_combine.py:118-161); with one split this is the identity
    e_max = lse_p.max(dim=0).values
    w = torch.where(torch.isinf(lse_p) & (lse_p < 0), _f32(0.0), torch.exp2(lse_p - e_max.unsqueeze(0)))
    w = torch.nan_to_num(w, nan=0.0)
    e_sum = w.sum(dim=0)
    inv = torch.where((e_sum == 0) | torch.isnan(e_sum), _f32(0.0), 1.0 / e_sum)
    out = (out_p * w.permute(0, 1, 3, 2).unsqueeze(-1)).sum(dim=0) * inv.permute(0, 2, 1).unsqueeze(-1)
    lse = torch.where(e_sum > 0, (e_max + torch.log2(e_sum)) * LN2, _f32(float("-inf")))
    return (out.to(q.dtype), lse, tile_map, dec.margin) if return_margin else (out.to(q.dtype), lse, tile_map)


def backward_tiled(q, k, v, dout, softmax_scale=None, is_causal=False, window_sizes=None, softmax_threshold=1.0,
                   num_splits=1, is_split_qo=False, tile_m=128, tile_n=128, dense=False, lse=None, out=None,
                   alpha=None, delta=None, gate_threshold=None, is_logsigmoid_gate=True, is_adapt_gate=True,
                   force_map=None, return_margin=False):
    """Tile-faithful backward: one program per (batch, query head, key tile, QO split) walking its query tiles in
    ascending order (flash_sparse_bwd.py:315-464 / flash_gated_bwd.py:392-560).

    lse / out: the forward results the backward is given (natural-log lse [B,Hq,Sq], out like q). When omitted they
    are computed here without any skipping. Pre-process as flash_bwd_preprocess.py:171-195: dpsum = sum(out * dout),
    lse2 = lse * log2(e) with NaN -> 1e6 and -inf clamped to -1e6; rows past the query length read as 0 for both
    (masked loads, scheduler.py:2173-2188).
    Returns (dq, dk, dv[, dalpha, ddelta], tile_map uint8 [B, Hq, n_blocks, splits, m_blocks])."""
    B, sq, hq, D = q.shape
    sk, hkv = k.shape[1], k.shape[2]
    G = hq // hkv
    local = window_sizes is not None
    if softmax_scale is None:
        softmax_scale = D ** -0.5
    c = float(_f32(softmax_scale) * _f32(LOG2E))
    ns = num_splits if is_split_qo else 1
    m_blocks, n_blocks = -(-sq // tile_m), -(-sk // tile_n)
    gated = alpha is not None
    qf, kf, vf, dof = q.float(), k.float(), v.float(), dout.float()
    if gated:
        af, df = alpha.float(), delta.float()
        if gate_threshold is None:
            gate_threshold = 1.0 / sk
    if lse is None or out is None:
        from . import eager

        kw = dict(alpha=alpha, delta=delta, is_logsigmoid_gate=is_logsigmoid_gate) if gated else {}
        out, lse = eager.forward(q, k, v, softmax_scale, is_causal, is_local=local, window_sizes=window_sizes,
                                 return_lse=True, **kw)
    dpsum = (out.float() * dof).sum(-1).permute(0, 2, 1)  # [B,Hq,Sq]
    lse2 = torch.where(torch.isnan(lse), _f32(1e6), lse.float() * _f32(LOG2E)).clamp(min=-1e6)
    tile_map = torch.zeros(B, hq, n_blocks, ns, m_blocks, dtype=torch.uint8)
    dec = _Decisions(tile_map.shape, force_map)
    dq = torch.zeros(B, sq, hq, D)
    dk = torch.zeros(B, sk, hkv, D)
    dv = torch.zeros(B, sk, hkv, D)
    da = torch.zeros(B, sq, hq)
    dd = torch.zeros(B, sk, hkv)
    for b in range(B):
        for h in range(hq):
            h_kv = h // G
            window = [int(x) for x in window_sizes[h_kv].tolist()] if local else [0, 0, 0, 0]
            for nb in range(n_blocks):
                k_idx = torch.arange(nb * tile_n, (nb + 1) * tile_n)
                col_ok = k_idx < sk
                k_tile, v_tile = torch.zeros(tile_n, D), torch.zeros(tile_n, D)
                k_tile[col_ok] = kf[b, k_idx[col_ok], h_kv]
                v_tile[col_ok] = vf[b, k_idx[col_ok], h_kv]
                if gated:
                    d_tile = torch.zeros(tile_n)
                    d_tile[col_ok] = df[b, k_idx[col_ok], h_kv]
                    d_max, d_min = d_tile.max().item(), d_tile.min().item()
                for sp in range(ns):
                    sched = S.bwd_schedule(sq, sk, nb, sp, window, ns, tile_n, tile_m, is_causal, local, is_split_qo)
                    if sched.is_empty():
                        continue
                    acc_dk, acc_dv, acc_dd = torch.zeros(tile_n, D), torch.zeros(tile_n, D), torch.zeros(tile_n)
                    gate_max = np.float32(float("-inf"))
                    for mb, mode in S.bwd_tiles(sched, is_causal, local):
                        q_idx = torch.arange(mb * tile_m, (mb + 1) * tile_m)
                        row_ok = q_idx < sq
                        rows = q_idx[row_ok]
                        if gated:
                            a_tile = torch.zeros(tile_m)
                            a_tile[row_ok] = af[b, rows, h]
                            g_thr = gate_threshold_log2(gate_threshold, q_idx, sq, sk, is_causal, is_adapt_gate)
                            gate_max, gskip = gate_step(a_tile.max().item(), a_tile.min().item(), d_max, d_min,
                                                        gate_max, c, g_thr)
                            if gskip:
                                tile_map[b, h, nb, sp, mb] = 3
                                continue
                        q_tile, do_tile = torch.zeros(tile_m, D), torch.zeros(tile_m, D)
                        q_tile[row_ok] = qf[b, rows, h]
                        do_tile[row_ok] = dof[b, rows, h]
                        l2, dps = torch.zeros(tile_m), torch.zeros(tile_m)
                        l2[row_ok] = lse2[b, h, rows]
                        dps[row_ok] = dpsum[b, h, rows]
                        s = k_tile @ q_tile.t()  # [TN, TM]
                        ds_scale = None
                        if gated:
                            gte = d_tile.unsqueeze(1) * a_tile.unsqueeze(0)
                            if is_logsigmoid_gate:
                                ds_scale = torch.sigmoid(-gte)
                                gte = log_sigmoid(gte)
                            s = s + gte
                        if mode != S.MASK_NONE:
                            keep = _tile_mask(mode, q_idx, k_idx, sq, sk, window).t()
                            s = torch.where(keep, s, _f32(float("-inf")))
                        p_log2 = s * c - l2.unsqueeze(0)
                        thr = softmax_threshold_log2(softmax_threshold, q_idx, sq, sk, is_causal)
                        skip = dec.decide((b, h, nb, sp, mb), p_log2 - thr.unsqueeze(0), dense)
                        tile_map[b, h, nb, sp, mb] = 2 if skip else 1
                        if skip:
                            continue
                        p = torch.exp2(p_log2).to(q.dtype).float()
                        acc_dv += p @ do_tile
                        dp = v_tile @ do_tile.t()
                        ds = p * (dp - dps.unsqueeze(0)).to(q.dtype).float()
                        dq_t = ds.t() @ k_tile
                        dq[b, rows, h] += dq_t[row_ok]
                        acc_dk += ds @ q_tile
                        if gated:
                            dsg = ds * ds_scale if ds_scale is not None else ds
                            da[b, rows, h] += (dsg * d_tile.unsqueeze(1)).sum(0)[row_ok]
                            acc_dd += (dsg * a_tile.unsqueeze(0)).sum(1)
                    cols = k_idx[col_ok]
                    dk[b, cols, h_kv] += acc_dk[col_ok] * softmax_scale
                    dv[b, cols, h_kv] += acc_dv[col_ok]
                    if gated:
                        dd[b, cols, h_kv] += acc_dd[col_ok] * softmax_scale
    dq = (dq * softmax_scale).to(q.dtype)
    res = [dq, dk.to(k.dtype), dv.to(v.dtype)]
    if gated:
        res += [(da * softmax_scale).to(alpha.dtype), dd.to(delta.dtype)]
    return (*res, tile_map, dec.margin) if return_margin else (*res, tile_map)


def decode_tiled(q, k, v, softmax_scale=None, window_sizes=None, softmax_threshold=1.0, num_splits=1,
                 gather_kv_indices=None, seqused_k=None, tile_n=16, sub_splits=4, dense=False, pad_rows_vote=False,
                 alpha=None, delta=None, gate_threshold=None, is_logsigmoid_gate=True, force_map=None,
                 return_margin=False, threshold_seqlen_k=None):
    """Tile-faithful decode (flash_sparse_dec.py:27-100, :298-482; gated: flash_gated_dec.py): one query position per
    sequence, the G query heads of a KV head are the rows of one tile, the keys of a (sequence, KV head) are cut into
    num_splits * sub_splits contiguous ranges with the reference's partition (block_info.py:94-105, :321-349), every
    range runs its own online softmax over tile_n-key tiles in descending order, partials are merged as
    flash_dec_combine.py:15-153. The kernels here run tile_n = 16 with sub_splits = 4 (one range per warp).

    q [B,Hq,D]; k, v [B,Sk,Hkv,D] (logical cache); gather_kv_indices int [B,topk] (negative = masked; windows and
    sequence lengths then do not apply, flash_sparse_dec.py:321-357); seqused_k [B] or None.
    pad_rows_vote: the reference pads the G rows to TILE_M = 16 with zero rows whose vote counts (they always vote
    "keep", so with G < 16 nothing is ever skipped); False leaves them out of the vote, which is what the kernels
    here do.
    Returns (out [B,Hq,D], lse [B,Hq] natural log, tile_map uint8 [B, Hkv, tiles])."""
    B, hq, D = q.shape
    cap, hkv = k.shape[1], k.shape[2]
    G = hq // hkv
    local = window_sizes is not None and gather_kv_indices is None
    gather = gather_kv_indices is not None
    if softmax_scale is None:
        softmax_scale = D ** -0.5
    c = float(_f32(softmax_scale) * _f32(LOG2E))
    nsub = num_splits * sub_splits
    gated = alpha is not None
    rows_m = max(16, G) if pad_rows_vote else G
    topk = gather_kv_indices.shape[1] if gather else 0
    n_tiles = -(-(topk if gather else cap) // tile_n)
    tile_map = torch.zeros(B, hkv, n_tiles, dtype=torch.uint8)
    dec = _Decisions(tile_map.shape, force_map)
    out = torch.zeros(B, hq, D)
    lse = torch.full((B, hq), float("-inf"))
    qf, kf, vf = q.float(), k.float(), v.float()
    for b in range(B):
        sk = int(seqused_k[b]) if seqused_k is not None else cap
        # a shard of a longer sequence normalises the threshold by the whole length (threshold_seqlen_k)
        thr_sk = int(threshold_seqlen_k[b]) if threshold_seqlen_k is not None else sk
        thr = softmax_threshold_log2(softmax_threshold, torch.zeros(rows_m, dtype=torch.long), 1, thr_sk, False)
        g_thr_val = (1.0 / sk) if gate_threshold is None else gate_threshold
        for h_kv in range(hkv):
            window = [int(x) for x in window_sizes[h_kv].tolist()] if local else [0, 0, 0, 0]
            q_tile = torch.zeros(rows_m, D)
            q_tile[:G] = qf[b, h_kv * G:(h_kv + 1) * G]
            if gated:
                a_tile = torch.zeros(rows_m)
                a_tile[:G] = alpha[b, h_kv * G:(h_kv + 1) * G].float()
                a_max, a_min = a_tile.max().item(), a_tile.min().item()
                g_thr = gate_threshold_log2(g_thr_val, None, 1, sk, False, False)
            parts = []
            for sub in range(nsub):
                if gather:
                    sched = S.topk_schedule(topk, sub, nsub, tile_n)
                else:
                    sched = S.fwd_schedule(1, sk, 0, sub, window, nsub, tile_n, 16, False, local, True, G,
                                           cover_single_query=True)
                m = torch.full((rows_m,), float("-inf"))
                l = torch.zeros(rows_m)
                acc = torch.zeros(rows_m, D)
                gate_max, first = np.float32(float("-inf")), True
                for n, mode in S.fwd_tiles(sched, True, local):
                    slot = torch.arange(n * tile_n, (n + 1) * tile_n)
                    if gather:
                        pos = torch.full((tile_n,), -1, dtype=torch.long)
                        inr = slot < topk
                        pos[inr] = gather_kv_indices[b, slot[inr]].long()
                        valid = (pos >= 0) & (pos < cap)
                        keep_cols = valid
                    else:
                        pos = slot.clone()
                        valid = pos < sk
                        # the single query position sits at the end of the keys: near = sk - 1 - k
                        keep_cols = (_tile_mask(mode, torch.zeros(1, dtype=torch.long), pos, 1, sk, window)[0]
                                     if mode != S.MASK_NONE else torch.ones(tile_n, dtype=torch.bool))
                    k_tile, v_tile = torch.zeros(tile_n, D), torch.zeros(tile_n, D)
                    k_tile[valid] = kf[b, pos[valid], h_kv]
                    v_tile[valid] = vf[b, pos[valid], h_kv]
                    if gated:
                        d_tile = torch.zeros(tile_n)
                        d_tile[valid] = delta[b, pos[valid], h_kv].float()
                        gate_max, gskip = gate_step(a_max, a_min, d_tile.max().item(), d_tile.min().item(), gate_max, c,
                                                    g_thr)
                        if gskip and not first:
                            tile_map[b, h_kv, n] = 3
                            continue
                        first = False
                    s = q_tile @ k_tile.t()
                    if gated:
                        gte = a_tile.unsqueeze(1) * d_tile.unsqueeze(0)
                        s = s + (log_sigmoid(gte) if is_logsigmoid_gate else gte)
                    s = torch.where(keep_cols.unsqueeze(0), s, _f32(float("-inf")))
                    m_cur = s.max(dim=1).values
                    skip = dec.decide((b, h_kv, n), (m_cur - m) * c - torch.log2(l) - thr, dense)
                    tile_map[b, h_kv, n] = 2 if skip else 1
                    if skip:
                        continue
                    m_new = torch.clamp(torch.maximum(m_cur, m), min=-1e6)
                    scale = torch.exp2((m - m_new) * c)
                    p = torch.exp2(s * c - (m_new * c).unsqueeze(1))
                    l = l * scale + p.sum(dim=1)
                    m = m_new
                    acc = acc * scale.unsqueeze(1) + p.to(v.dtype).float() @ v_tile
                dead = (l == 0) | torch.isnan(l)
                inv = torch.where(dead, _f32(1.0), 1.0 / l)
                parts.append(((acc * inv.unsqueeze(1))[:G], torch.where(dead, _f32(float("-inf")), m * c + torch.log2(l))[:G]))
            o_p = torch.stack([x[0] for x in parts])  # [nsub, G, D]
            l_p = torch.stack([x[1] for x in parts])  # [nsub, G] base 2
            e_max = l_p.max(dim=0).values
            w = torch.where(torch.isinf(l_p) & (l_p < 0), _f32(0.0), torch.exp2(l_p - e_max.unsqueeze(0)))
            w = torch.nan_to_num(w, nan=0.0)
            e_sum = w.sum(dim=0)
            inv = torch.where((e_sum == 0) | torch.isnan(e_sum), _f32(0.0), 1.0 / e_sum)
            out[b, h_kv * G:(h_kv + 1) * G] = (o_p * w.unsqueeze(-1)).sum(0) * inv.unsqueeze(-1)
            lse[b, h_kv * G:(h_kv + 1) * G] = torch.where(e_sum > 0, (e_max + torch.log2(e_sum)) * LN2, _f32(float("-inf")))
    return (out.to(q.dtype), lse, tile_map, dec.margin) if return_margin else (out.to(q.dtype), lse, tile_map)
