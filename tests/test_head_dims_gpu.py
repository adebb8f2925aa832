"""Head sizes other than 64 / 128 (any multiple of 16, the reference's contract `assert_inputs.py:39-40`): up to
128 forward, backward and decode run on the 64- or 128-wide kernels with the missing columns loaded as zeros; up to
256 the forward and the decode run on 256-wide kernels. Results are compared with the eager oracle."""

import pytest
import torch

from fixtures import assert_close, seeded_qkv
from oracle import eager

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ops():
    import flash_sparse_attn as fsa

    return fsa


@pytest.mark.parametrize("head_dim", [16, 32, 48, 80, 96, 112])
@pytest.mark.parametrize("kind", ["dense", "sparse", "gated"])
def test_forward_backward_other_head_dims(head_dim, kind):
    fsa = _ops()
    b, s, hq, hkv = 2, 384, 4, 2
    q, k, v = seeded_qkv(head_dim, b, s, s, hq, hkv, head_dim)
    g = torch.Generator().manual_seed(3)
    do = torch.randn(b, s, hq, head_dim, generator=g).to(torch.bfloat16)
    a, d = torch.randn(b, s, hq, generator=g).to(torch.bfloat16), torch.randn(b, s, hkv, generator=g).to(torch.bfloat16)
    gate = dict(alpha=a, delta=d) if kind == "gated" else {}
    ref_out = eager.forward(q, k, v, None, True, **gate)
    ref_grads = eager.backward(q, k, v, do, None, True, **gate)
    leaves = [t.to(DEV).requires_grad_(True) for t in ((q, k, v, a, d) if kind == "gated" else (q, k, v))]
    kw = {}
    if kind != "dense":
        kw["softmax_threshold"] = -128.0
    if kind == "gated":
        kw["gate_threshold"] = -128.0
    fn = {"dense": fsa.flash_dense_attn_func, "sparse": fsa.flash_sparse_attn_func,
          "gated": fsa.flash_gated_attn_func}[kind]
    out = fn(*leaves, is_causal=True, **kw)
    out.backward(do.to(DEV))
    torch.cuda.synchronize()
    fsa.check_status()
    assert out.shape == (b, s, hq, head_dim)
    assert_close(f"hd{head_dim}-{kind}-out", out, ref_out)
    for name, t, r in zip(("dq", "dk", "dv", "dalpha", "ddelta"), leaves, ref_grads):
        assert_close(f"hd{head_dim}-{kind}-{name}", t.grad, r, rtol=2.5e-2, atol=2.5e-2)


@pytest.mark.parametrize("head_dim", [32, 96])
def test_split_paths_other_head_dims(head_dim):
    """Split-KV forward (fp32 partials + combine) and split-QO backward (fp32 dK/dV partials)."""
    fsa = _ops()
    b, s, hq, hkv = 1, 1024, 4, 2
    q, k, v = seeded_qkv(head_dim + 1, b, s, s, hq, hkv, head_dim)
    do = torch.randn(b, s, hq, head_dim, generator=torch.Generator().manual_seed(4)).to(torch.bfloat16)
    ref_out = eager.forward(q, k, v, None, True)
    ref = eager.backward(q, k, v, do, None, True)
    leaves = [t.to(DEV).requires_grad_(True) for t in (q, k, v)]
    out = fsa.flash_sparse_attn_func(*leaves, is_causal=True, softmax_threshold=-128.0, is_split_kv=True,
                                     is_split_qo=True, num_splits=3)
    out.backward(do.to(DEV))
    torch.cuda.synchronize()
    fsa.check_status()
    assert_close(f"hd{head_dim}-split-out", out, ref_out)
    for name, t, r in zip(("dq", "dk", "dv"), leaves, ref):
        assert_close(f"hd{head_dim}-split-{name}", t.grad, r, rtol=2.5e-2, atol=2.5e-2)


@pytest.mark.parametrize("head_dim", [32, 80, 96])
@pytest.mark.parametrize("mode", ["plain", "gather_split"])
def test_decode_other_head_dims(head_dim, mode):
    fsa = _ops()
    b, sk, hq, hkv = 2, 1024, 16, 2
    g = torch.Generator().manual_seed(head_dim)
    mk = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16)  # noqa: E731
    q, k, v = mk(b, hq, head_dim), mk(b, sk, hkv, head_dim), mk(b, sk, hkv, head_dim)
    if mode == "plain":
        ref = eager.decode(q, k, v)
        out = fsa.flash_sparse_attn_with_kvcache_func(q.to(DEV), k.to(DEV), v.to(DEV), softmax_threshold=-128.0)
    else:
        idx = torch.stack([torch.randperm(sk, generator=g)[:512] for _ in range(b)]).to(torch.int32)
        ref = eager.gather_decode(q, k, v, idx)
        out = fsa.flash_sparse_attn_with_kvcache_func(q.to(DEV), k.to(DEV), v.to(DEV), gather_kv_indices=idx.to(DEV),
                                                      softmax_threshold=-128.0, num_splits=4)
    torch.cuda.synchronize()
    fsa.check_status()
    assert_close(f"hd{head_dim}-decode-{mode}", out, ref, rtol=2.5e-2, atol=2.5e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("hq,hkv", [(8, 2), (16, 2), (24, 2)])
@pytest.mark.parametrize("head_dim", [160, 192, 256])
@pytest.mark.parametrize("mode", ["plain_split", "local", "paged_gather", "gated", "skip"])
def test_decode_head_dims_above_128(mode, head_dim, hq, hkv, dtype):
    """Decode at head sizes 160 / 192 / 256 (16-bit inputs): the 256-wide transposed kernel, eight query rows of a
    KV head per pass over the keys (4, 8 and 12 query heads per KV head: one and two passes), against the eager
    oracle. Forward and backward stay at head sizes up to 128."""
    fsa = _ops()
    b, sk = 2, 1200
    g = torch.Generator().manual_seed(head_dim + hq)
    mk = lambda *s: torch.randn(*s, generator=g).to(dtype)  # noqa: E731
    q, k, v = mk(b, hq, head_dim), mk(b, sk, hkv, head_dim), mk(b, sk, hkv, head_dim)
    if mode == "plain_split":
        ref = eager.decode(q, k, v)
        out = fsa.flash_dense_attn_with_kvcache_func(q.to(DEV), k.to(DEV), v.to(DEV), num_splits=3)
    elif mode == "local":
        ws = torch.tensor([[32, 200, 100, 160], [0, 300, 0, 64]], dtype=torch.int32)
        ref = eager.decode(q, k, v, is_local=True, window_sizes=ws)
        out = fsa.flash_sparse_attn_with_kvcache_func(q.to(DEV), k.to(DEV), v.to(DEV), window_sizes=ws.to(DEV),
                                                      softmax_threshold=-128.0)
    elif mode == "paged_gather":
        page = 64
        n_pages = b * (1216 // page)
        kc, vc = mk(n_pages + 3, page, hkv, head_dim), mk(n_pages + 3, page, hkv, head_dim)
        table = torch.randperm(n_pages + 3, generator=g)[:n_pages].reshape(b, -1).to(torch.int32)
        kl, vl = eager.unpage(kc, table), eager.unpage(vc, table)
        idx = torch.stack([torch.randperm(sk, generator=g)[:256] for _ in range(b)]).to(torch.int32)
        idx[:, 3::17] = -1
        ref = eager.gather_decode(q, kl, vl, idx)
        out = fsa.flash_sparse_attn_with_kvcache_func(q.to(DEV), kc.to(DEV), vc.to(DEV), page_table=table.to(DEV),
                                                      gather_kv_indices=idx.to(DEV), softmax_threshold=-128.0)
    elif mode == "gated":
        a, d = mk(b, hq), mk(b, sk, hkv)
        ref = eager.decode(q, k, v, alpha=a, delta=d)
        out = fsa.flash_gated_attn_with_kvcache_func(q.to(DEV), k.to(DEV), v.to(DEV), a.to(DEV), d.to(DEV),
                                                     softmax_threshold=-128.0, gate_threshold=-128.0)
    else:  # peaked queries with the threshold on: tiles are skipped, the result stays close
        q = (k[:, -1].float().repeat_interleave(hq // hkv, dim=1) * 3).to(dtype)
        ref = eager.decode(q, k, v)
        out = fsa.flash_sparse_attn_with_kvcache_func(q.to(DEV), k.to(DEV), v.to(DEV), softmax_threshold=1.0)
    torch.cuda.synchronize()
    fsa.check_status()
    assert_close(f"hd{head_dim}-decode-{mode}", out, ref, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("head_dim", [160, 192, 256])
@pytest.mark.parametrize("mode", ["dense", "causal_sparse", "local_split", "gated", "varlen", "pack_gqa", "paged", "skip"])
def test_forward_head_dims_above_128(mode, head_dim, dtype):
    """Forward at head sizes 160 / 192 / 256: the 256-wide kernel (one query tile per CTA, one stage of K and V),
    against the eager oracle, with a ragged sequence length (several key tiles, a partial last tile)."""
    fsa = _ops()
    b, s, hq, hkv = 2, 600, 4, 2
    g = torch.Generator().manual_seed(head_dim)
    mk = lambda *sh: torch.randn(*sh, generator=g).to(dtype)  # noqa: E731
    q, k, v = mk(b, s, hq, head_dim), mk(b, s, hkv, head_dim), mk(b, s, hkv, head_dim)
    with torch.no_grad():
        if mode == "dense":
            ref = eager.forward(q, k, v, None, False)
            out = fsa.flash_dense_attn_func(q.to(DEV), k.to(DEV), v.to(DEV), is_causal=False)
        elif mode == "causal_sparse":
            ref = eager.forward(q, k, v, None, True)
            out = fsa.flash_sparse_attn_func(q.to(DEV), k.to(DEV), v.to(DEV), is_causal=True, softmax_threshold=-128.0)
        elif mode == "local_split":
            ws = torch.tensor([[16, 100, 50, 120], [0, 200, 0, 64]], dtype=torch.int32)
            ref = eager.forward(q, k, v, None, True, is_local=True, window_sizes=ws)
            out = fsa.flash_sparse_attn_func(q.to(DEV), k.to(DEV), v.to(DEV), is_causal=True, window_sizes=ws.to(DEV),
                                             softmax_threshold=-128.0, is_split_kv=True, num_splits=2)
        elif mode == "gated":
            a, d = mk(b, s, hq), mk(b, s, hkv)
            ref = eager.forward(q, k, v, None, True, alpha=a, delta=d)
            out = fsa.flash_gated_attn_func(q.to(DEV), k.to(DEV), v.to(DEV), a.to(DEV), d.to(DEV), is_causal=True,
                                            softmax_threshold=-128.0, gate_threshold=-128.0)
        elif mode == "varlen":
            lens = [600, 333]
            cu = torch.tensor([0, 600, 933], dtype=torch.int32)
            qp, kp, vp = mk(933, hq, head_dim), mk(933, hkv, head_dim), mk(933, hkv, head_dim)
            ref = torch.cat([eager.forward(qp[None, cu[i]:cu[i + 1]], kp[None, cu[i]:cu[i + 1]], vp[None, cu[i]:cu[i + 1]],
                                           None, True)[0] for i in range(2)])
            out = fsa.flash_sparse_attn_varlen_func(qp.to(DEV), kp.to(DEV), vp.to(DEV), cu.to(DEV), cu.to(DEV),
                                                    max(lens), max(lens), is_causal=True, softmax_threshold=-128.0)
        elif mode == "pack_gqa":
            ref = eager.forward(q[:, :5], k, v, None, True)
            out = fsa.flash_sparse_attn_func(q[:, :5].to(DEV), k.to(DEV), v.to(DEV), is_causal=True,
                                             softmax_threshold=-128.0, pack_gqa=True)
        elif mode == "paged":
            page, max_pages = 64, 10
            kc, vc = mk(b * max_pages + 3, page, hkv, head_dim), mk(b * max_pages + 3, page, hkv, head_dim)
            table = torch.randperm(b * max_pages + 3, generator=g)[: b * max_pages].reshape(b, max_pages).to(torch.int32)
            used = torch.tensor([max_pages * page - 37, 333], dtype=torch.int32)
            kl, vl = eager.unpage(kc, table), eager.unpage(vc, table)
            qs = q[:, :200]
            ref = torch.stack([eager.forward(qs[i:i + 1], kl[i:i + 1, :used[i]], vl[i:i + 1, :used[i]], None, True)[0]
                               for i in range(b)])
            out = fsa.flash_sparse_attn_func(qs.to(DEV), kc.to(DEV), vc.to(DEV), is_causal=True,
                                             softmax_threshold=-128.0, page_table=table.to(DEV),
                                             seqused_k=used.to(DEV))
        else:  # peaked queries with the threshold on: tiles are skipped, the result stays close
            q = (k.float().repeat_interleave(hq // hkv, dim=2) * 3).to(dtype)
            ref = eager.forward(q, k, v, None, True)
            out = fsa.flash_sparse_attn_func(q.to(DEV), k.to(DEV), v.to(DEV), is_causal=True, softmax_threshold=1.0)
    torch.cuda.synchronize()
    fsa.check_status()
    assert out.shape == ref.shape
    assert_close(f"hd{head_dim}-fwd-{mode}", out, ref, rtol=3e-2, atol=3e-2)


def test_head_dims_above_128_backward_is_refused():
    """The backward kernels stop at head size 128: the forward runs, the backward raises."""
    fsa = _ops()
    q = torch.randn(1, 256, 4, 192, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    out = fsa.flash_sparse_attn_func(q, q.detach(), q.detach(), is_causal=True)
    with pytest.raises((AssertionError, RuntimeError)):
        out.sum().backward()
    qd = torch.randn(2, 4, 320, device=DEV, dtype=torch.bfloat16)
    kd = torch.randn(2, 64, 4, 320, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(AssertionError):
        fsa.flash_sparse_attn_with_kvcache_func(qd, kd, kd)
    with pytest.raises(AssertionError):
        fsa.flash_sparse_attn_func(kd, kd, kd)
