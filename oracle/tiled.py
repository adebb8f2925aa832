"""CPU oracle (test infrastructure only): tile-faithful forward with the reference's skip rules.

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

It returns the outputs AND the per-tile decision map (1 = computed, 2 = skipped), which is what the
skip-set parity tests compare with the kernel's own map. The reference's tests never enable skipping
(they pass threshold -128), so for skip sets this file is the only oracle: parity of skip sets is
pinned to this restatement, not to reference outputs ("parity unpinned" by the reference itself).

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg may import this package.
"""

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


def forward_tiled(q, k, v, softmax_scale=None, is_causal=False, window_sizes=None, softmax_threshold=1.0,
                  num_splits=1, is_split_kv=False, pack_gqa=False, tile_m=128, tile_n=128, dense=False):
    """q [B,Sq,Hq,D], k/v [B,Sk,Hkv,D] (16-bit); window_sizes int [Hkv,4] or None.
    Returns (out [B,Sq,Hq,D] in q.dtype, lse [B,Hq,Sq] natural log, tile_map uint8
    [B, Hgrid, m_blocks, splits, n_blocks])."""
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
    out_p = torch.zeros(ns, B, sq, hq, D, dtype=torch.float32)
    lse_p = torch.full((ns, B, hq, sq), float("-inf"), dtype=torch.float32)

    qf, kf, vf = q.float(), k.float(), v.float()
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
                for sp in range(ns):
                    sched = S.fwd_schedule(sq, sk, mb, sp, window, ns, tile_n, tile_m, is_causal, local,
                                           is_split_kv, gpack)
                    if sched.is_empty():
                        continue
                    m = torch.full((tile_m,), float("-inf"))
                    l = torch.zeros(tile_m)
                    acc = torch.zeros(tile_m, D)
                    for n, mode in S.fwd_tiles(sched, is_causal, local):
                        k_idx = torch.arange(n * tile_n, (n + 1) * tile_n)
                        col_ok = k_idx < sk
                        k_tile = torch.zeros(tile_n, D)
                        v_tile = torch.zeros(tile_n, D)
                        k_tile[col_ok] = kf[b, k_idx[col_ok], h_kv]
                        v_tile[col_ok] = vf[b, k_idx[col_ok], h_kv]
                        s = q_tile @ k_tile.t()
                        if mode != S.MASK_NONE:
                            keep = _tile_mask(mode, q_idx, k_idx, sq, sk, window)
                            s = torch.where(keep, s, _f32(float("-inf")))
                        m_cur = s.max(dim=1).values
                        skip = False
                        if not dense:
                            d = (m_cur - m) * c - torch.log2(l)
                            val = d - thr
                            good = val[~torch.isnan(val)]
                            # tl.max ignores NaN unless every entry is NaN; NaN < 0 is False
                            skip = bool(good.numel() > 0 and good.max() < 0.0)
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
    return out.to(q.dtype), lse, tile_map
