"""Host logic of context-parallel decode on CPU ranks (gloo, world size 2): index localisation partitions
the top-k set exactly, and all-gather + log-sum-exp merge of per-shard partials reproduces the
single-device result. The per-shard partial and the merge are computed by the CPU oracle here; on GPUs the
same driver runs the CUDA decode kernel and combine kernel (tests/test_dec_gpu.py covers those)."""

import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _oracle_partial(q, k, v, idx, scale, threshold=None, sk_global=None):
    """One KV split of the decode in the wire format: normalised partial output and base-2 log-sum-exp
    (flash_sparse_dec.py:485-489). With a threshold the shard runs the tile-faithful decode, its skip bound
    normalised by the length of the whole sequence."""
    from flash_sparse_attn.ops.triton import context_parallel as cp
    from oracle import eager, tiled

    if threshold is None:
        out, lse = eager.gather_decode(q, k, v, idx, scale, return_lse=True)
    else:
        out, lse, _ = tiled.decode_tiled(q, k, v, scale, softmax_threshold=threshold, gather_kv_indices=idx,
                                         threshold_seqlen_k=torch.full((q.shape[0],), sk_global))
    lse2 = lse * 1.4426950408889634
    return cp.pack_partials(out.float().unsqueeze(0), lse2.t().contiguous().unsqueeze(0))  # [1, B*Hq*(D+1)]


def _oracle_combine(shape):
    """flash_dec_combine.py:15-153 in torch: weights exp2(lse - max), -inf partials contribute 0."""
    from flash_sparse_attn.ops.triton import context_parallel as cp

    def combine(packed, parts):
        return _merge(*cp.unpack_partials(packed, parts, *shape))

    return combine


def _merge(out_p, lse_p):
    m = lse_p.max(dim=0).values
    w = torch.where(torch.isinf(lse_p) & (lse_p < 0), torch.zeros_like(lse_p), torch.exp2(lse_p - m))
    s = w.sum(dim=0)
    out = (out_p * w.permute(0, 2, 1).unsqueeze(-1)).sum(dim=0) / s.t().unsqueeze(-1)
    return out, ((m + torch.log2(s)) * 0.6931471805599453).t()


def _worker(rank, world, port, ret):
    sys.path.insert(0, os.path.join(ROOT, "flash-sparse-attention_b200"))
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from flash_sparse_attn.ops.triton import context_parallel as cp
    from oracle import eager

    g = torch.Generator().manual_seed(0)
    b, sk, hq, hkv, d, topk = 3, 1000, 8, 2, 64, 96
    q = torch.randn(b, hq, d, generator=g).to(torch.bfloat16)
    k = torch.randn(b, sk, hkv, d, generator=g).to(torch.bfloat16)
    v = torch.randn(b, sk, hkv, d, generator=g).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(sk, generator=g)[:topk] for _ in range(b)]).to(torch.int32)
    idx[:, 3::17] = -1
    scale = d ** -0.5
    lo, hi = cp.shard_bounds(sk, world, rank, align=256)
    local = cp.localize_indices(idx, lo, hi)
    # partition property: every valid index is kept by exactly one rank
    kept = (local >= 0).to(torch.int32)
    dist.all_reduce(kept)
    assert torch.equal(kept, (idx >= 0).to(torch.int32))
    assert torch.equal(local[local >= 0] + lo, idx[(idx >= lo) & (idx < hi)])
    out, lse = cp.context_parallel_decode(
        lambda: _oracle_partial(q, k[:, lo:hi], v[:, lo:hi], local, scale), _oracle_combine((b, hq, d)))
    ref, ref_lse = eager.gather_decode(q, k, v, idx, scale, return_lse=True)
    ok = torch.allclose(out, ref.float(), atol=1e-2) and torch.allclose(lse, ref_lse, atol=1e-4)
    # with the softmax threshold on: peaked queries so that tiles are skipped; every shard normalises the
    # threshold by the whole length, and the merged result stays within tolerance of the exact one
    qp = (k[:, -1].repeat_interleave(hq // hkv, dim=1).float() * 3).to(torch.bfloat16)
    out_t, _ = cp.context_parallel_decode(
        lambda: _oracle_partial(qp, k[:, lo:hi], v[:, lo:hi], local, scale, threshold=1.0, sk_global=sk),
        _oracle_combine((b, hq, d)))
    ref_t = eager.gather_decode(qp, k, v, idx, scale)
    ok = ok and torch.allclose(out_t, ref_t.float(), atol=2e-2, rtol=2e-2)
    ret[rank] = bool(ok)
    dist.destroy_process_group()


def test_context_parallel_decode_gloo_world2():
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    assert ret.get(0) is True and ret.get(1) is True


def test_shard_bounds_cover_the_sequence():
    from flash_sparse_attn.ops.triton import context_parallel as cp

    for sk in (1, 255, 256, 4096, 131072, 100000):
        for world in (1, 2, 4, 8):
            bounds = [cp.shard_bounds(sk, world, r) for r in range(world)]
            assert bounds[0][0] == 0 and max(hi for _, hi in bounds) == sk
            for (a, b_), (c, d_) in zip(bounds, bounds[1:]):
                assert b_ == c or (b_ == sk and c == sk)
            assert all(lo % 256 == 0 or lo == sk for lo, _ in bounds)
