"""Seeded synthetic workloads with the shapes and value distributions of the benchmark configurations.

Shared by the GPU tests, the benchmarks and the script that runs another implementation of the
operators on the same tensors, so this module imports nothing but torch: every tensor is drawn on the
device from ``torch.Generator(device).manual_seed(seed)`` in a fixed order, which makes two processes on the
same GPU model produce identical inputs.

    C2   sparse causal + 1024-token window, forward/backward: B2 S4096 Hq32 Hkv8 D128, iid N(0, 1)
    C3   gated, per-KV-head windows from {512, 1024, 2048, 4096}: B4 S8192 Hq32 Hkv8 D128
    C4   16 packed sequences with lengths uniform in [256, 4096], Hq32 Hkv8 D128
    C5   top-k decode: B64, contexts uniform in [4096, 131072], Hq64 Hkv8 D128, 256-token pages, top-k 2048
    S16K causal B1 S16384 Hq32 Hkv8 D128, iid or "llm-like"

"llm-like" follows the recipe of the reference's benchmark input generator (tests/test_utils.py:231-329 of the
reference): smooth sinusoidal position features shared by queries and keys, a latent per 1024-token block and KV
head added to both, a sink latent on the first 64 keys, plus noise - attention mass concentrates on the own
block and on the sink, which is what makes tile skipping trigger; iid inputs skip nothing.
"""

import math

import torch

BF16 = torch.bfloat16


def _gen(device, seed):
    return torch.Generator(device=device).manual_seed(seed)


def _randn(g, *shape, dtype=BF16):
    return torch.randn(*shape, generator=g, device=g.device, dtype=dtype)


def iid_qkv(device, seed, b, sq, sk, hq, hkv, d, with_dout=True, dtype=BF16):
    g = _gen(device, seed)
    q, k, v = _randn(g, b, sq, hq, d, dtype=dtype), _randn(g, b, sk, hkv, d, dtype=dtype), _randn(g, b, sk, hkv, d, dtype=dtype)
    do = _randn(g, b, sq, hq, d, dtype=dtype) if with_dout else None
    return q, k, v, do


def position_features(seqlen, head_dim, device, dtype=BF16):
    pairs = (head_dim + 1) // 2
    period = max(float(seqlen), 1024.0)
    freqs = torch.exp(torch.linspace(math.log(1.0 / period), math.log(1.0 / 64.0), pairs, device=device, dtype=torch.float32))
    ang = torch.arange(seqlen, device=device, dtype=torch.float32)[:, None] * freqs[None, :]
    return torch.cat([ang.sin(), ang.cos()], dim=-1)[:, :head_dim].to(dtype)


def llm_like_qkv(device, seed, b, sq, sk, hq, hkv, d, with_dout=True, dtype=BF16, block=1024, sink=64):
    """Queries / keys = 0.35 noise + 0.65 position features + 0.75 block latent (+ sink latent: 0.45 on every
    query, 1.10 on the first `sink` keys, whose values are scaled by 1.15)."""
    g = _gen(device, seed)
    group = hq // hkv
    kv_of = torch.arange(hq, device=device) // group
    pos_k = position_features(sk, d, device, dtype)
    pos_q = pos_k[sk - sq:]
    q, k, v = _randn(g, b, sq, hq, d, dtype=dtype), _randn(g, b, sk, hkv, d, dtype=dtype), _randn(g, b, sk, hkv, d, dtype=dtype)
    q.mul_(0.35).add_(pos_q[None, :, None, :], alpha=0.65)
    k.mul_(0.35).add_(pos_k[None, :, None, :], alpha=0.65)
    blk_k = torch.arange(sk, device=device) // block
    blk_q = (torch.arange(sq, device=device) + (sk - sq)) // block
    latent = _randn(g, b, (sk + block - 1) // block, hkv, d, dtype=dtype)
    q.add_(latent[:, blk_q][:, :, kv_of, :], alpha=0.75)
    k.add_(latent[:, blk_k], alpha=0.75)
    n_sink = min(sink, sk)
    if n_sink > 0:
        s_lat = _randn(g, b, hkv, d, dtype=dtype)
        q.add_(s_lat[:, None, kv_of, :], alpha=0.45)
        k[:, :n_sink].add_(s_lat[:, None, :, :], alpha=1.10)
        v[:, :n_sink].mul_(1.15)
    do = _randn(g, b, sq, hq, d, dtype=dtype) if with_dout else None
    return q, k, v, do


# ---------------------------------------------------------------------------------------------------------
def c2(device, seed=0, batch=2, seqlen=4096, data="iid"):
    hq, hkv, d = 32, 8, 128
    make = iid_qkv if data == "iid" else llm_like_qkv
    q, k, v, do = make(device, seed, batch, seqlen, seqlen, hq, hkv, d)
    ws = torch.tensor([[0, 1024, 0, 0]] * hkv, dtype=torch.int32, device=device)
    kw = dict(is_causal=True, window_sizes=ws, softmax_threshold=1.0, is_split_kv=True, is_split_qo=True)
    return dict(q=q, k=k, v=v, dout=do, kwargs=kw)


def s16k(device, seed=0, seqlen=16384, data="iid", threshold=1.0):
    hq, hkv, d = 32, 8, 128
    make = iid_qkv if data == "iid" else llm_like_qkv
    q, k, v, do = make(device, seed, 1, seqlen, seqlen, hq, hkv, d)
    return dict(q=q, k=k, v=v, dout=do, kwargs=dict(is_causal=True, softmax_threshold=threshold))


def c3(device, seed=0, batch=4, seqlen=8192):
    hq, hkv, d = 32, 8, 128
    g = _gen(device, seed)
    q, k, v = _randn(g, batch, seqlen, hq, d), _randn(g, batch, seqlen, hkv, d), _randn(g, batch, seqlen, hkv, d)
    alpha, delta = _randn(g, batch, seqlen, hq), _randn(g, batch, seqlen, hkv)
    do = _randn(g, batch, seqlen, hq, d)
    pick = torch.randint(0, 4, (hkv,), generator=torch.Generator().manual_seed(seed))
    widths = torch.tensor([512, 1024, 2048, 4096])[pick]
    ws = torch.zeros(hkv, 4, dtype=torch.int32)
    ws[:, 1] = widths.to(torch.int32)
    kw = dict(is_causal=True, window_sizes=ws.to(device))  # thresholds and gate options at their defaults
    return dict(q=q, k=k, v=v, alpha=alpha, delta=delta, dout=do, kwargs=kw, widths=widths.tolist())


def c4(device, seed=0, n_seq=16, lo=256, hi=4096):
    hq, hkv, d = 32, 8, 128
    lens = torch.randint(lo, hi + 1, (n_seq,), generator=torch.Generator().manual_seed(seed))
    cu = torch.zeros(n_seq + 1, dtype=torch.int32)
    cu[1:] = lens.cumsum(0).to(torch.int32)
    total = int(cu[-1])
    g = _gen(device, seed)
    q, k, v, do = _randn(g, total, hq, d), _randn(g, total, hkv, d), _randn(g, total, hkv, d), _randn(g, total, hq, d)
    cu_d = cu.to(device)
    kw = dict(cu_seqlens_q=cu_d, cu_seqlens_k=cu_d, max_seqlen_q=int(lens.max()), max_seqlen_k=int(lens.max()),
              is_causal=True, softmax_threshold=1.0, is_split_kv=True, is_split_qo=True)
    return dict(q=q, k=k, v=v, dout=do, kwargs=kw, lens=lens.tolist(), cu=cu)


def c5_indices(seed=0, batch=64, ctx_lo=4096, ctx_hi=131072, topk=2048, page=256):
    """Context lengths, the permuted page table and the seeded top-k positions (host tensors)."""
    g = torch.Generator().manual_seed(seed)
    ctx = torch.randint(ctx_lo, ctx_hi + 1, (batch,), generator=g)
    pages_per = (ctx + page - 1) // page
    n_pages = int(pages_per.sum())
    table = torch.zeros(batch, int(pages_per.max()), dtype=torch.int32)
    perm = torch.randperm(n_pages, generator=g).to(torch.int32)
    o = 0
    for b in range(batch):
        n = int(pages_per[b])
        table[b, :n] = perm[o:o + n]
        o += n
    idx = torch.stack([torch.randperm(int(ctx[b]), generator=g)[:topk].to(torch.int32) for b in range(batch)])
    return ctx, n_pages, table, idx


def c5(device, seed=0, batch=64, ctx_lo=4096, ctx_hi=131072, topk=2048, page=256, paged=True):
    """paged=True: KV in `page`-token pages behind a permuted page table. paged=False: the same logical cache as
    one contiguous [batch, max ctx, Hkv, D] tensor (for implementations without a paged gather)."""
    hq, hkv, d = 64, 8, 128
    ctx, n_pages, table, idx = c5_indices(seed, batch, ctx_lo, ctx_hi, topk, page)
    g = _gen(device, seed)
    q = _randn(g, batch, hq, d)
    kp, vp = _randn(g, n_pages, page, hkv, d), _randn(g, n_pages, page, hkv, d)
    used = ctx.to(torch.int32).to(device)
    idx_d, table_d = idx.to(device), table.to(device)
    nbytes = batch * hkv * topk * d * 2 * 2 + batch * topk * 4 + 2 * batch * hq * d * 2
    if paged:
        kw = dict(page_table=table_d, gather_kv_indices=idx_d, seqused_k=used)
        return dict(q=q, k=kp, v=vp, kwargs=kw, ctx=ctx, bytes=nbytes)
    smax = table.shape[1] * page
    flat = table_d.long().clamp_(min=0)
    k = kp[flat].reshape(batch, smax, hkv, d)  # logical position p of sequence b = row p % page of page table[b, p // page]
    v = vp[flat].reshape(batch, smax, hkv, d)
    del kp, vp
    return dict(q=q, k=k, v=v, kwargs=dict(gather_kv_indices=idx_d, seqused_k=used), ctx=ctx, bytes=nbytes)


def causal_flops(b, hq, s, d):
    """Dense-causal forward FLOPs (the "effective" figure): 4 * D * B * Hq * S (S + 1) / 2."""
    return 4.0 * d * b * hq * s * (s + 1) / 2
