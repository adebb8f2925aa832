"""GPU parity of the backward pass (through the C ABI) against the CPU oracle (autograd through the
eager fp32 forward, as the reference's tests do: tests/test_utils.py:1716-1765) and the golden
fixture. Tolerances: rtol 1.6e-2 / atol 1e-5 with the reference's mean-difference rule."""

import itertools

import pytest
import torch

from fixtures import assert_close, load, seeded_qkv
from oracle import eager

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ops():
    import flash_sparse_attn as fsa

    return fsa


def _run(fn, q, k, v, do, **kw):
    qg, kg, vg = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
    kw = {n: (t.to(DEV) if isinstance(t, torch.Tensor) else t) for n, t in kw.items()}
    out = fn(qg, kg, vg, **kw)
    out.backward(do.to(DEV))
    torch.cuda.synchronize()
    _ops().check_status()
    return qg.grad, kg.grad, vg.grad


def test_golden_backward():
    fsa = _ops()
    g = load("bwd_causal")
    dq, dk, dv = _run(fsa.flash_dense_attn_func, g["q"], g["k"], g["v"], g["dout"], is_causal=True)
    assert_close("dq", dq, g["dq_dense"])
    assert_close("dk", dk, g["dk_dense"])
    assert_close("dv", dv, g["dv_dense"])
    dq, dk, dv = _run(fsa.flash_sparse_attn_func, g["q"], g["k"], g["v"], g["dout"], is_causal=True,
                      softmax_threshold=-128.0)
    assert_close("dq-sparse", dq, g["dq_dense"])
    assert_close("dk-sparse", dk, g["dk_dense"])
    assert_close("dv-sparse", dv, g["dv_dense"])


# the reference's backward grid (tests/test_sparse_base_backward.py): causal x local x split_qo x head_dim
@pytest.mark.parametrize("kind", ["dense", "sparse"])
@pytest.mark.parametrize("causal,local", [(False, False), (True, False), (False, True), (True, True)])
@pytest.mark.parametrize("split", [False, True])
@pytest.mark.parametrize("head_dim", [64, 128])
def test_backward_grid(kind, causal, local, split, head_dim):
    fsa = _ops()
    b, s, hq, hkv = 2, 1024, 8, 2
    q, k, v = seeded_qkv(0, b, s, s, hq, hkv, head_dim)
    do = torch.randn(b, s, hq, head_dim, generator=torch.Generator().manual_seed(9)).to(torch.bfloat16)
    ws = torch.tensor([[32, 200, 100, 160], [0, 300, 0, 64]], dtype=torch.int32) if local else None
    ref = eager.backward(q, k, v, do, None, causal, is_local=local, window_sizes=ws)
    fn = fsa.flash_dense_attn_func if kind == "dense" else fsa.flash_sparse_attn_func
    kw = {} if kind == "dense" else {"softmax_threshold": -128.0}
    got = _run(fn, q, k, v, do, is_causal=causal, window_sizes=ws, is_split_qo=split, num_splits=3 if split else None,
               **kw)
    for name, a, r in zip(("dq", "dk", "dv"), got, ref):
        assert_close(f"{kind}-{name}", a, r)


@pytest.mark.parametrize("sq,sk", [(77, 300), (300, 300), (129, 1000), (513, 513)])
@pytest.mark.parametrize("causal", [False, True])
def test_backward_ragged(sq, sk, causal):
    fsa = _ops()
    q, k, v = seeded_qkv(1, 2, sq, sk, 4, 2, 128, torch.float16)
    do = torch.randn(2, sq, 4, 128, generator=torch.Generator().manual_seed(3)).to(torch.float16)
    ref = eager.backward(q, k, v, do, None, causal)
    got = _run(fsa.flash_sparse_attn_func, q, k, v, do, is_causal=causal, softmax_threshold=-128.0)
    for name, a, r in zip(("dq", "dk", "dv"), got, ref):
        assert_close(name, a, r)


def test_backward_varlen():
    fsa = _ops()
    lens_q, lens_k = [5, 130, 257, 64], [70, 130, 300, 64]
    cq = torch.tensor([0] + list(itertools.accumulate(lens_q)), dtype=torch.int32)
    ck = torch.tensor([0] + list(itertools.accumulate(lens_k)), dtype=torch.int32)
    g = torch.Generator().manual_seed(3)
    q = torch.randn(sum(lens_q), 4, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(sum(lens_k), 2, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(sum(lens_k), 2, 128, generator=g).to(torch.bfloat16)
    do = torch.randn(sum(lens_q), 4, 128, generator=g).to(torch.bfloat16)
    ref = eager.varlen_backward(q, k, v, do, cq, ck, None, True)
    qg, kg, vg = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
    out = fsa.flash_sparse_attn_varlen_func(qg, kg, vg, cq.to(DEV), ck.to(DEV), max(lens_q), max(lens_k),
                                            is_causal=True, softmax_threshold=-128.0)
    out.backward(do.to(DEV))
    torch.cuda.synchronize()
    fsa.check_status()
    for name, a, r in zip(("dq", "dk", "dv"), (qg.grad, kg.grad, vg.grad), ref):
        assert_close("varlen-" + name, a, r)


def test_backward_skip_is_small_and_recorded():
    """With the threshold on and peaked scores the backward skips tiles; the gradients stay within
    tolerance of the exact ones (skipped probabilities are below threshold / visible length)."""
    from flash_sparse_attn.ops.triton.flash_bwd import tile_map_numel

    fsa = _ops()
    s, hq, hkv, d = 1536, 4, 2, 128
    g = torch.Generator().manual_seed(5)
    base = torch.randn(1, s, hkv, d, generator=g)
    q = (base.repeat_interleave(hq // hkv, dim=2) * 3 + torch.randn(1, s, hq, d, generator=g) * 0.3).to(torch.bfloat16)
    k = (base + torch.randn(1, s, hkv, d, generator=g) * 0.1).to(torch.bfloat16)
    v = torch.randn(1, s, hkv, d, generator=g).to(torch.bfloat16)
    do = torch.randn(1, s, hq, d, generator=g).to(torch.bfloat16)
    ref = eager.backward(q, k, v, do, None, True)
    from flash_sparse_attn.ops.triton import flash_bwd, flash_fwd

    qd, kd, vd, dod = (t.to(DEV) for t in (q, k, v, do))
    out, lse, *_ = flash_fwd.attn_forward("sparse", qd, kd, vd, is_causal=True, softmax_threshold=1.0)
    tmap = torch.zeros(tile_map_numel(1, s, s, hq), dtype=torch.uint8, device=DEV)
    dq, dk, dv = flash_bwd.attn_backward("sparse", qd, kd, vd, out, dod, lse, is_causal=True, softmax_threshold=1.0,
                                         tile_map=tmap)
    torch.cuda.synchronize()
    fsa.check_status()
    assert (tmap == 2).sum().item() > 0 and (tmap == 1).sum().item() > 0
    # visited tiles are exactly the causal lower triangle of 12 x 12 tiles per head
    assert (tmap != 0).sum().item() == hq * 12 * 13 // 2
    for name, a, r in zip(("dq", "dk", "dv"), (dq, dk, dv), ref):
        assert_close("skip-" + name, a, r, rtol=3e-2, atol=3e-2)


def test_c2_full_size_backward_properties():
    """Headline configuration: dK/dV are bitwise reproducible (fixed in-CTA reduction order), dQ is
    reproducible to fp32-reduction noise, gradients are linear in dO, and one (batch, KV head) slice
    matches the CPU oracle."""
    fsa = _ops()
    b, s, hq, hkv, d = 2, 4096, 32, 8, 128
    g = torch.Generator(device=DEV).manual_seed(0)
    mk = lambda *sh: torch.randn(*sh, generator=g, device=DEV, dtype=torch.bfloat16)  # noqa: E731
    q, k, v, do1, do2 = mk(b, s, hq, d), mk(b, s, hkv, d), mk(b, s, hkv, d), mk(b, s, hq, d), mk(b, s, hq, d)
    ws = torch.tensor([[0, 1024, 0, 0]] * hkv, dtype=torch.int32, device=DEV)

    def grads(do):
        qg, kg, vg = (t.detach().requires_grad_(True) for t in (q, k, v))
        out = fsa.flash_sparse_attn_func(qg, kg, vg, is_causal=True, window_sizes=ws, softmax_threshold=1.0,
                                         is_split_kv=True, is_split_qo=True)
        out.backward(do)
        return qg.grad, kg.grad, vg.grad

    a, a2, c = grads(do1), grads(do1), grads(do2)
    both = grads((do1.float() + do2.float()).to(torch.bfloat16))
    torch.cuda.synchronize()
    fsa.check_status()
    assert torch.equal(a[1], a2[1]) and torch.equal(a[2], a2[2])
    assert (a[0].float() - a2[0].float()).abs().max().item() < 2e-2
    for i in range(3):
        lin = (both[i].float() - (a[i].float() + c[i].float())).abs().max().item()
        assert lin < 0.25, lin
    qs, ks, vs, dos = q[:1, :, 4:8].cpu(), k[:1, :, 1:2].cpu(), v[:1, :, 1:2].cpu(), do1[:1, :, 4:8].cpu()
    ref = eager.backward(qs, ks, vs, dos, None, True, is_local=True, window_sizes=ws[:1].cpu())
    assert_close("c2-dq", a[0][:1, :, 4:8], ref[0])
    assert_close("c2-dk", a[1][:1, :, 1:2], ref[1])
    assert_close("c2-dv", a[2][:1, :, 1:2], ref[2])


# ---------------------------------------------------------------------------------------------------
# deterministic dQ: key tiles add their dQ tiles in a fixed (descending) order
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("case", ["causal", "noncausal", "local_split", "gqa_hd64"])
def test_deterministic_dq_is_bitwise_reproducible(case):
    fsa = _ops()
    hd = 64 if case == "gqa_hd64" else 128
    b, s, hq, hkv = 2, 2048, 8, 2
    q, k, v = seeded_qkv(5, b, s, s, hq, hkv, hd)
    do = torch.randn(b, s, hq, hd, generator=torch.Generator().manual_seed(6)).to(torch.bfloat16)
    kw = dict(is_causal=case != "noncausal", softmax_threshold=-128.0)
    ws = None
    if case == "local_split":
        ws = torch.tensor([[32, 200, 100, 160], [0, 300, 0, 64]], dtype=torch.int32)
        kw.update(window_sizes=ws, is_split_qo=True, num_splits=3)
    ref = eager.backward(q, k, v, do, None, kw["is_causal"], is_local=ws is not None, window_sizes=ws)
    fsa.set_deterministic(True)
    try:
        runs = [_run(fsa.flash_sparse_attn_func, q, k, v, do, **kw) for _ in range(3)]
    finally:
        fsa.set_deterministic(False)
    for name, a, r in zip(("dq", "dk", "dv"), runs[0], ref):
        assert_close(f"det-{case}-{name}", a, r)
    for other in runs[1:]:
        for name, a, o in zip(("dq", "dk", "dv"), runs[0], other):
            assert torch.equal(a, o), f"{case}: {name} differs between two deterministic runs"


def test_deterministic_dq_varlen_and_skipped_tiles():
    """Packed sequences of different lengths, and a run in which tiles are skipped (a skipped tile still
    has to pass its turn on)."""
    fsa = _ops()
    lens = [300, 1000, 129, 2048]
    cu = torch.tensor([0] + list(itertools.accumulate(lens)), dtype=torch.int32)
    g = torch.Generator().manual_seed(8)
    q = (torch.randn(sum(lens), 8, 128, generator=g) * 2.5).to(torch.bfloat16)
    k = (torch.randn(sum(lens), 2, 128, generator=g) * 2.5).to(torch.bfloat16)
    v = torch.randn(sum(lens), 2, 128, generator=g).to(torch.bfloat16)
    do = torch.randn(sum(lens), 8, 128, generator=g).to(torch.bfloat16)
    fsa.set_deterministic(True)
    try:
        outs = []
        for _ in range(2):
            qg, kg, vg = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
            out = fsa.flash_sparse_attn_varlen_func(qg, kg, vg, cu.to(DEV), cu.to(DEV), max(lens), max(lens),
                                                    is_causal=True, softmax_threshold=1.0)
            out.backward(do.to(DEV))
            torch.cuda.synchronize()
            fsa.check_status()
            outs.append((qg.grad, kg.grad, vg.grad))
    finally:
        fsa.set_deterministic(False)
    for a, o in zip(outs[0], outs[1]):
        assert torch.equal(a, o)
    ref = eager.varlen_backward(q, k, v, do, cu, cu, None, True)
    for name, a, r in zip(("dq", "dk", "dv"), outs[0], ref):
        # the eager oracle keeps the probability mass that the skipped tiles drop (threshold 1.0: up to
        # 1 / visible_len per row and tile), so the element-wise bound is the skip error, not rounding
        assert_close("det-varlen-" + name, a, r, rtol=5e-2, atol=5e-2, ew_rtol=5e-2, ew_atol=1e-1)
