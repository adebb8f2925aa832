"""CPU oracle (test infrastructure only): eager fp32 attention, the value reference.

Restates in plain PyTorch-on-CPU tensor arithmetic what the reference's tests use as ground truth:
  * tests/test_utils.py:516-565  scores, causal / flex-local masks  -> ``scores``
  * tests/test_utils.py:568-658  dense / sparse / gated forward      -> ``forward``
  * tests/test_utils.py:661-726  packed (varlen) forward              -> ``varlen_forward``
  * tests/test_utils.py:729-795  decode                               -> ``decode``, ``varlen_decode``
  * tests/test_utils.py:1716-1765 backward = autograd through forward -> ``backward``
  * tests/test_topk_gather_decode.py:97-140 top-k gathered decode     -> ``gather_decode``
  * tests/test_paged_kv.py:25-80   paged cache = logical cache        -> ``unpage``
  * flash_sparse_attn/ops/triton/utils.py:47-102 default window table -> ``window_sizes_heuristic``
  * flash_sparse_attn/ops/triton/quant.py:42-64  per-tensor FP8       -> ``quantize_fp8``

The "sparse" eager reference is the dense one (the reference's tests never enable skipping); the
tile-faithful variant with the skip rule lives in oracle/tiled.py.

Pinned by tests/test_oracle_golden.py against fixtures produced by the reference's own functions
(tests/golden/make_golden.py). Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg
may import this package; nothing in the product path does.
"""

from typing import List, Optional, Sequence

import torch
import torch.nn.functional as F


def window_sizes_heuristic(seqlen_k: int, num_heads_kv: int, equal_bandwidth: bool = True, window_near: int = 1024,
                           window_sink: int = 64) -> torch.Tensor:
    """int32 [num_heads_kv, 4] = (sink, left, right, near): shared sink and near band, the rest of
    the causal distances cut into one band per KV head (utils.py:47-102, single-rank case)."""
    near = min(max(window_near, 0), seqlen_k)
    sink = min(max(window_sink, 0), max(seqlen_k - near, 0))
    span = max(seqlen_k - sink - near, 0)
    idx = torch.arange(num_heads_kv + 1, dtype=torch.float32)
    if equal_bandwidth:
        cuts = (span * idx / num_heads_kv).to(torch.int32)
    else:
        cuts = (span * (1.0 - torch.sqrt(1.0 - idx / num_heads_kv))).to(torch.int32)
    left = cuts[1:] - cuts[:-1]
    right = cuts[:-1]
    return torch.stack([torch.full_like(left, sink), left, right, torch.full_like(left, near)], dim=1)


def allowed_mask(seqlen_q: int, seqlen_k: int, is_causal: bool, window: Optional[Sequence[int]]) -> torch.Tensor:
    """bool [seqlen_q, seqlen_k]; ``window`` = (sink, left, right, near) makes it local
    (tests/test_utils.py:541-563, mask.py:68-102)."""
    q_idx = torch.arange(seqlen_q).unsqueeze(1)
    k_idx = torch.arange(seqlen_k).unsqueeze(0)
    dist = q_idx + (seqlen_k - seqlen_q) - k_idx
    if window is not None:
        sink, left, right, near = (int(x) for x in window)
        return ((k_idx < sink) & (dist >= 0)) | ((dist >= 0) & (dist < near)) | (
            (dist >= near + right) & (dist < near + right + left))
    if is_causal:
        return dist >= 0
    return torch.ones(seqlen_q, seqlen_k, dtype=torch.bool)


def scores(q, k, softmax_scale, is_causal, is_local=False, window_sizes=None, local_seqlen_k=None,
           alpha=None, delta=None, is_logsigmoid_gate=True):
    """Masked, scaled logits [B, Hq, Sq, Sk] in fp32. q [B,Sq,Hq,D], k [B,Sk,Hkv,D];
    gated: alpha [B,Sq,Hq], delta [B,Sk,Hkv], logits = (q.k + g(alpha*delta)) * scale
    (tests/test_utils.py:516-565, :644-646)."""
    qh = q.transpose(1, 2).float()
    kh = k.transpose(1, 2).float()
    hq, hkv = qh.shape[1], kh.shape[1]
    group = hq // hkv
    kh = kh.repeat_interleave(group, dim=1)
    s = torch.matmul(qh, kh.transpose(-2, -1)) * softmax_scale
    if alpha is not None:
        a = alpha.transpose(1, 2).float()
        d = delta.transpose(1, 2).float().repeat_interleave(group, dim=1)
        raw = a.unsqueeze(-1) * d.unsqueeze(-2)
        s = s + (F.logsigmoid(raw) if is_logsigmoid_gate else raw) * softmax_scale
    sq, sk = q.shape[1], k.shape[1]
    if is_local:
        if window_sizes is None:
            window_sizes = window_sizes_heuristic(local_seqlen_k if local_seqlen_k is not None else sk, hkv)
        for h in range(hkv):
            ok = allowed_mask(sq, sk, True, window_sizes[h].tolist())
            s[:, h * group:(h + 1) * group] = s[:, h * group:(h + 1) * group].masked_fill(~ok, float("-inf"))
    elif is_causal:
        s = s.masked_fill(~allowed_mask(sq, sk, True, None), float("-inf"))
    return s


def forward(q, k, v, softmax_scale=None, is_causal=False, is_local=False, window_sizes=None, local_seqlen_k=None,
            alpha=None, delta=None, is_logsigmoid_gate=True, return_lse=False, keep_fp32=False):
    """Eager attention. Returns out [B,Sq,Hq,D] in q.dtype (fp32 if keep_fp32) and optionally the
    natural-log LSE [B,Hq,Sq]; fully masked rows give 0 / -inf
    (tests/test_utils.py:568-658: softmax, nan_to_num, matmul)."""
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** -0.5
    s = scores(q, k, softmax_scale, is_causal, is_local, window_sizes, local_seqlen_k, alpha, delta,
               is_logsigmoid_gate)
    group = q.shape[2] // k.shape[2]
    vh = v.transpose(1, 2).float().repeat_interleave(group, dim=1)
    p = torch.nan_to_num(torch.softmax(s, dim=-1), nan=0.0)
    out = torch.matmul(p, vh).transpose(1, 2).contiguous()
    if not keep_fp32:
        out = out.to(q.dtype)
    if return_lse:
        return out, torch.logsumexp(s, dim=-1)
    return out


def varlen_forward(q, k, v, cu_seqlens_q, cu_seqlens_k, softmax_scale=None, is_causal=False, is_local=False,
                   window_sizes=None, max_seqlen_k=None, alpha=None, delta=None, is_logsigmoid_gate=True,
                   seqused_q=None, seqused_k=None, return_lse=False, keep_fp32=False):
    """Packed sequences: per-sequence eager forward, local windows derived from the longest key
    sequence (tests/test_utils.py:661-726). q [Tq,Hq,D]; lse [Hq,Tq]. Rows beyond seqused_q stay 0."""
    cq, ck = cu_seqlens_q.tolist(), cu_seqlens_k.tolist()
    nb = len(cq) - 1
    if max_seqlen_k is None:
        max_seqlen_k = max(ck[i + 1] - ck[i] for i in range(nb))
    out = torch.zeros(q.shape, dtype=torch.float32 if keep_fp32 else q.dtype)
    lse = torch.full((q.shape[1], q.shape[0]), float("-inf"))
    for i in range(nb):
        lq = int(seqused_q[i]) if seqused_q is not None else cq[i + 1] - cq[i]
        lk = int(seqused_k[i]) if seqused_k is not None else ck[i + 1] - ck[i]
        if lq == 0:
            continue
        qs, ks = slice(cq[i], cq[i] + lq), slice(ck[i], ck[i] + lk)
        o, l = forward(q[qs].unsqueeze(0), k[ks].unsqueeze(0), v[ks].unsqueeze(0), softmax_scale, is_causal,
                       is_local, window_sizes, max_seqlen_k if is_local else None,
                       alpha[qs].unsqueeze(0) if alpha is not None else None,
                       delta[ks].unsqueeze(0) if delta is not None else None, is_logsigmoid_gate,
                       return_lse=True, keep_fp32=keep_fp32)
        out[qs] = o[0]
        lse[:, qs] = l[0]
    return (out, lse) if return_lse else out


def decode(q, k, v, softmax_scale=None, is_local=False, window_sizes=None, local_seqlen_k=None, seqused_k=None,
           alpha=None, delta=None, is_logsigmoid_gate=True, return_lse=False):
    """One query position per sequence: q [B,Hq,D] (alpha [B,Hq]) against k/v [B,Sk,Hkv,D]
    (delta [B,Sk,Hkv]); never causal; local windows are evaluated for a query sitting at the last
    key position (tests/test_utils.py:729-795)."""
    outs, lses = [], []
    for b in range(q.shape[0]):
        lk = int(seqused_k[b]) if seqused_k is not None else k.shape[1]
        o, l = forward(q[b:b + 1].unsqueeze(1), k[b:b + 1, :lk], v[b:b + 1, :lk], softmax_scale, False, is_local,
                       window_sizes, local_seqlen_k if local_seqlen_k is not None else k.shape[1],
                       alpha[b:b + 1].unsqueeze(1) if alpha is not None else None,
                       delta[b:b + 1, :lk] if delta is not None else None, is_logsigmoid_gate, return_lse=True)
        outs.append(o[0, 0])
        lses.append(l[0, :, 0])
    out, lse = torch.stack(outs), torch.stack(lses)
    return (out, lse) if return_lse else out


def varlen_decode(q, k, v, cu_seqlens_k, softmax_scale=None, is_local=False, window_sizes=None, max_seqlen_k=None,
                  seqused_k=None, alpha=None, delta=None, is_logsigmoid_gate=True, return_lse=False):
    """Decode against packed keys [Tk,Hkv,D] (tests/test_utils.py:729-795)."""
    ck = cu_seqlens_k.tolist()
    nb = len(ck) - 1
    if max_seqlen_k is None:
        max_seqlen_k = max(ck[i + 1] - ck[i] for i in range(nb))
    outs, lses = [], []
    for b in range(nb):
        lk = int(seqused_k[b]) if seqused_k is not None else ck[b + 1] - ck[b]
        ks = slice(ck[b], ck[b] + lk)
        o, l = forward(q[b:b + 1].unsqueeze(1), k[ks].unsqueeze(0), v[ks].unsqueeze(0), softmax_scale, False,
                       is_local, window_sizes, max_seqlen_k if is_local else None,
                       alpha[b:b + 1].unsqueeze(1) if alpha is not None else None,
                       delta[ks].unsqueeze(0) if delta is not None else None, is_logsigmoid_gate, return_lse=True)
        outs.append(o[0, 0])
        lses.append(l[0, :, 0])
    out, lse = torch.stack(outs), torch.stack(lses)
    return (out, lse) if return_lse else out


def gather_decode(q, k, v, gather_kv_indices, softmax_scale=None, alpha=None, delta=None, is_logsigmoid_gate=True,
                  return_lse=False):
    """Decode over a gathered key list: indices [B,topk] are positions in k/v [B,Sk,Hkv,D]; negative
    entries are masked; neither windows nor sequence lengths apply
    (tests/test_topk_gather_decode.py:97-140, flash_sparse_dec.py:321-357)."""
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** -0.5
    valid = gather_kv_indices >= 0
    idx = gather_kv_indices.clamp_min(0).long()
    hq, hkv = q.shape[1], k.shape[2]
    group = hq // hkv
    outs, lses = [], []
    for b in range(q.shape[0]):
        kb = k[b].index_select(0, idx[b]).float().transpose(0, 1).repeat_interleave(group, dim=0)  # [Hq,topk,D]
        vb = v[b].index_select(0, idx[b]).float().transpose(0, 1).repeat_interleave(group, dim=0)
        vb = vb.masked_fill(~valid[b][None, :, None], 0.0)
        s = torch.einsum("hd,htd->ht", q[b].float(), kb) * softmax_scale
        if alpha is not None:
            db = delta[b].index_select(0, idx[b]).float().transpose(0, 1).repeat_interleave(group, dim=0)
            raw = alpha[b].float().unsqueeze(-1) * db
            s = s + (F.logsigmoid(raw) if is_logsigmoid_gate else raw) * softmax_scale
        s = s.masked_fill(~valid[b][None, :], float("-inf"))
        p = torch.nan_to_num(torch.softmax(s, dim=-1), nan=0.0)
        outs.append(torch.einsum("ht,htd->hd", p, vb).to(q.dtype))
        lses.append(torch.logsumexp(s, dim=-1))
    out, lse = torch.stack(outs), torch.stack(lses)
    return (out, lse) if return_lse else out


def unpage(cache: torch.Tensor, page_table: torch.Tensor) -> torch.Tensor:
    """Logical [B, max_pages*page, Hkv, D] view of a paged cache [num_pages, page, Hkv, D]
    (the equivalence tests/test_paged_kv.py:25-80 relies on)."""
    b, mp = page_table.shape
    pages = cache[page_table.reshape(-1).long()]
    return pages.reshape(b, mp * cache.shape[1], *cache.shape[2:])


def backward(q, k, v, dout, softmax_scale=None, is_causal=False, is_local=False, window_sizes=None,
             local_seqlen_k=None, alpha=None, delta=None, is_logsigmoid_gate=True):
    """Gradients by autograd through the fp32 eager forward (tests/test_utils.py:1716-1765).
    Returns (dq, dk, dv) or (dq, dk, dv, dalpha, ddelta), in fp32."""
    leaves = [t.detach().float().requires_grad_(True) for t in (q, k, v)]
    gate = []
    if alpha is not None:
        gate = [t.detach().float().requires_grad_(True) for t in (alpha, delta)]
    out = forward(leaves[0], leaves[1], leaves[2], softmax_scale if softmax_scale is not None else q.shape[-1] ** -0.5,
                  is_causal, is_local, window_sizes, local_seqlen_k, gate[0] if gate else None,
                  gate[1] if gate else None, is_logsigmoid_gate, keep_fp32=True)
    grads = torch.autograd.grad(out, leaves + gate, dout.float())
    return tuple(grads)


def varlen_backward(q, k, v, dout, cu_seqlens_q, cu_seqlens_k, softmax_scale=None, is_causal=False, is_local=False,
                    window_sizes=None, max_seqlen_k=None, alpha=None, delta=None, is_logsigmoid_gate=True):
    """Packed-sequence gradients, one sequence at a time."""
    cq, ck = cu_seqlens_q.tolist(), cu_seqlens_k.tolist()
    nb = len(cq) - 1
    if max_seqlen_k is None:
        max_seqlen_k = max(ck[i + 1] - ck[i] for i in range(nb))
    outs: List[torch.Tensor] = [torch.zeros(t.shape) for t in (q, k, v)]
    if alpha is not None:
        outs += [torch.zeros(alpha.shape), torch.zeros(delta.shape)]
    for i in range(nb):
        qs, ks = slice(cq[i], cq[i + 1]), slice(ck[i], ck[i + 1])
        g = backward(q[qs].unsqueeze(0), k[ks].unsqueeze(0), v[ks].unsqueeze(0), dout[qs].unsqueeze(0),
                     softmax_scale, is_causal, is_local, window_sizes, max_seqlen_k if is_local else None,
                     alpha[qs].unsqueeze(0) if alpha is not None else None,
                     delta[ks].unsqueeze(0) if delta is not None else None, is_logsigmoid_gate)
        outs[0][qs], outs[1][ks], outs[2][ks] = g[0][0], g[1][0], g[2][0]
        if alpha is not None:
            outs[3][qs], outs[4][ks] = g[3][0], g[4][0]
    return tuple(outs)


_FP8_MAX = {torch.float8_e5m2: 57344.0, torch.float8_e4m3fn: 448.0}


def quantize_fp8(x: torch.Tensor, dtype: torch.dtype = torch.float8_e5m2):
    """Per-tensor FP8: scale = FP8_MAX / amax(|x|); returns (x*scale as fp8, amax/FP8_MAX in x.dtype)
    (quant.py:42-64)."""
    amax = x.float().abs().max()
    scale = _FP8_MAX[dtype] / amax
    return (x.float() * scale).to(dtype), (amax / _FP8_MAX[dtype]).to(x.dtype).reshape(1)
