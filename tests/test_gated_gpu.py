"""GPU parity of the gated operators against the golden fixtures (reference's eager gated forward) and
the CPU oracle: logits = (q.k + g(alpha_i * delta_j)) * scale, g = logsigmoid or identity."""

import pytest
import torch

from fixtures import assert_close, load, seeded_qkv
from oracle import eager

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ops():
    import flash_sparse_attn as fsa

    return fsa


def _sync():
    torch.cuda.synchronize()
    _ops().check_status()


def _gates(seed, b, sq, sk, hq, hkv, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(b, sq, hq, generator=g).to(dtype), torch.randn(b, sk, hkv, generator=g).to(dtype)


@pytest.mark.parametrize("name", ["fwd_nc", "fwd_causal", "fwd_causal_sq_lt_sk"])
def test_golden_gated_forward(name):
    fsa = _ops()
    g = load(name)
    q, k, v, a, d = (g[n].to(DEV) for n in ("q", "k", "v", "alpha", "delta"))
    causal = bool(g["causal"])
    out, lse = fsa.flash_gated_attn_func(q, k, v, a, d, is_causal=causal, softmax_threshold=-128.0,
                                         gate_threshold=-128.0, return_lse=True)
    _sync()
    assert_close(name + "-gated", out, g["out_gated"])
    assert torch.allclose(lse.cpu(), g["lse_gated"], rtol=0, atol=2e-3)
    out = fsa.flash_gated_attn_func(q, k, v, a, d, is_causal=causal, softmax_threshold=-128.0, gate_threshold=-128.0,
                                    is_logsigmoid_gate=False)
    _sync()
    assert_close(name + "-gated-linear", out, g["out_gated_lin"])


def test_golden_gated_varlen():
    fsa = _ops()
    g = load("fwd_varlen")
    q, k, v, a, d = (g[n].to(DEV) for n in ("q", "k", "v", "alpha", "delta"))
    cu = g["cu_seqlens"].to(torch.int32).to(DEV)
    out = fsa.flash_gated_attn_varlen_func(q, k, v, a, d, cu, cu, 160, 160, is_causal=True, softmax_threshold=-128.0,
                                           gate_threshold=-128.0)
    _sync()
    assert_close("gated-varlen", out, g["out_gated"])


# the reference's gated forward grid (tests/test_gated_base_forward.py) adds is_logsigmoid_gate
@pytest.mark.parametrize("causal,local", [(False, False), (True, False), (True, True)])
@pytest.mark.parametrize("split", [False, True])
@pytest.mark.parametrize("head_dim", [64, 128])
@pytest.mark.parametrize("pack_gqa", [False, True])
@pytest.mark.parametrize("logsig", [True, False])
def test_gated_forward_grid(causal, local, split, head_dim, pack_gqa, logsig):
    fsa = _ops()
    b, s, hq, hkv = 2, 1024, 8, 2
    q, k, v = seeded_qkv(0, b, s, s, hq, hkv, head_dim)
    a, d = _gates(1, b, s, s, hq, hkv)
    ws = torch.tensor([[32, 200, 100, 160], [0, 300, 0, 64]], dtype=torch.int32) if local else None
    ref = eager.forward(q, k, v, None, causal, is_local=local, window_sizes=ws, alpha=a, delta=d,
                        is_logsigmoid_gate=logsig)
    out = fsa.flash_gated_attn_func(q.to(DEV), k.to(DEV), v.to(DEV), a.to(DEV), d.to(DEV), is_causal=causal,
                                    window_sizes=ws.to(DEV) if local else None, softmax_threshold=-128.0,
                                    gate_threshold=-128.0, is_logsigmoid_gate=logsig, is_split_kv=split,
                                    num_splits=3 if split else None, pack_gqa=pack_gqa)
    _sync()
    assert_close("gated-fwd", out, ref)


def test_gate_skip_triggers_and_stays_close():
    """With the default gate threshold, tiles whose gate bound is far below the running maximum are
    skipped (map value 3); their weight is bounded by the threshold, so the output stays close."""
    from flash_sparse_attn.ops.triton.flash_fwd import attn_forward, tile_map_numel

    b, s, hq, hkv, d = 1, 2048, 2, 2, 128
    q, k, v = seeded_qkv(3, b, s, s, hq, hkv, d)
    g = torch.Generator().manual_seed(4)
    alpha = torch.full((b, s, hq), 4.0)
    # keys of the last 256 positions carry a large positive delta, everything else strongly negative
    delta = torch.full((b, s, hkv), -32.0)
    delta[:, -256:] = 6.0
    alpha, delta = alpha.to(torch.bfloat16), delta.to(torch.bfloat16)
    ref = eager.forward(q, k, v, None, True, alpha=alpha, delta=delta, is_logsigmoid_gate=False)
    tmap = torch.zeros(tile_map_numel(b, s, s, hq, hkv), dtype=torch.uint8, device=DEV)
    out, *_ = attn_forward("gated", q.to(DEV), k.to(DEV), v.to(DEV), alpha=alpha.transpose(1, 2).contiguous().to(DEV),
                           delta=delta.transpose(1, 2).contiguous().to(DEV), is_causal=True, softmax_threshold=0.0,
                           gate_threshold=None, is_logsigmoid_gate=False, is_adapt_gate=True, tile_map=tmap)
    _sync()
    assert (tmap == 3).sum().item() > 0
    # rows in the last 256 positions see the boosted keys: everything else is negligible there
    assert_close("gate-skip", out[:, -200:], ref[:, -200:], rtol=3e-2, atol=3e-2)


# ---------------------------------------------------------------------------------------------------
# gated decode
# ---------------------------------------------------------------------------------------------------
def test_golden_gated_decode():
    fsa = _ops()
    g = load("decode")
    q, k, v, a, d = (g[n].to(DEV) for n in ("q", "k", "v", "alpha", "delta"))
    out = fsa.flash_gated_attn_with_kvcache_func(q, k, v, a, d, softmax_threshold=-128.0, gate_threshold=-128.0)
    _sync()
    assert_close("gated-decode", out, g["out_gated"])


@pytest.mark.parametrize("logsig", [True, False])
@pytest.mark.parametrize("local", [False, True])
@pytest.mark.parametrize("head_dim", [64, 128])
@pytest.mark.parametrize("mode", ["plain", "gather", "paged", "varlen"])
def test_gated_decode_grid(logsig, local, head_dim, mode):
    fsa = _ops()
    b, sk, hq, hkv = 2, 1024, 16, 2
    g = torch.Generator().manual_seed(11)
    mk = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16)  # noqa: E731
    q, k, v, a, d = mk(b, hq, head_dim), mk(b, sk, hkv, head_dim), mk(b, sk, hkv, head_dim), mk(b, hq), mk(b, sk, hkv)
    ws = torch.tensor([[32, 200, 100, 160], [0, 300, 0, 64]], dtype=torch.int32) if local else None
    kw = dict(softmax_threshold=-128.0, gate_threshold=-128.0, is_logsigmoid_gate=logsig)
    if mode == "gather":
        if local:
            pytest.skip("windows do not apply to gathered keys")
        idx = torch.stack([torch.randperm(sk, generator=g)[:128] for _ in range(b)]).to(torch.int32)
        idx[:, 2::13] = -1
        ref = eager.gather_decode(q, k, v, idx, alpha=a, delta=d, is_logsigmoid_gate=logsig)
        out = fsa.flash_gated_attn_with_kvcache_func(q.to(DEV), k.to(DEV), v.to(DEV), a.to(DEV), d.to(DEV),
                                                     gather_kv_indices=idx.to(DEV), **kw)
    elif mode == "paged":
        page = 64
        kc, vc, dc = k.reshape(b * sk // page, page, hkv, head_dim), v.reshape(b * sk // page, page, hkv, head_dim), \
            d.reshape(b * sk // page, page, hkv)
        perm = torch.randperm(b * sk // page, generator=g)
        table = torch.empty(b * sk // page, dtype=torch.int32)
        table[perm] = torch.arange(b * sk // page, dtype=torch.int32)   # logical page i lives at physical perm^-1
        kp, vp, dp = torch.empty_like(kc), torch.empty_like(vc), torch.empty_like(dc)
        kp[table.long()], vp[table.long()], dp[table.long()] = kc, vc, dc
        table = table.reshape(b, sk // page)
        ref = eager.decode(q, k, v, is_local=local, window_sizes=ws, alpha=a, delta=d, is_logsigmoid_gate=logsig)
        out = fsa.flash_gated_attn_with_kvcache_func(q.to(DEV), kp.to(DEV), vp.to(DEV), a.to(DEV), dp.to(DEV),
                                                     page_table=table.to(DEV),
                                                     window_sizes=ws.to(DEV) if local else None, **kw)
    elif mode == "varlen":
        lens = [1024, 700]
        cu = torch.tensor([0, 1024, 1724], dtype=torch.int32)
        kp, vp, dp = mk(1724, hkv, head_dim), mk(1724, hkv, head_dim), mk(1724, hkv)
        ref = eager.varlen_decode(q, kp, vp, cu, is_local=local, window_sizes=ws, alpha=a, delta=dp,
                                  is_logsigmoid_gate=logsig)
        out = fsa.flash_gated_attn_varlen_with_kvcache_func(q.to(DEV), kp.to(DEV), vp.to(DEV), a.to(DEV), dp.to(DEV),
                                                            cu.to(DEV), max(lens),
                                                            window_sizes=ws.to(DEV) if local else None, **kw)
    else:
        ref = eager.decode(q, k, v, is_local=local, window_sizes=ws, alpha=a, delta=d, is_logsigmoid_gate=logsig)
        out = fsa.flash_gated_attn_with_kvcache_func(q.to(DEV), k.to(DEV), v.to(DEV), a.to(DEV), d.to(DEV),
                                                     window_sizes=ws.to(DEV) if local else None, **kw)
    _sync()
    assert_close(f"gated-decode-{mode}", out, ref, rtol=2.5e-2, atol=2.5e-2)


# ---------------------------------------------------------------------------------------------------
# gated backward: dq, dk, dv, dalpha, ddelta
# ---------------------------------------------------------------------------------------------------
def _run_gated_bwd(fn, q, k, v, a, d, do, *extra, **kw):
    leaves = [t.to(DEV).requires_grad_(True) for t in (q, k, v, a, d)]
    kw = {n: (t.to(DEV) if isinstance(t, torch.Tensor) else t) for n, t in kw.items()}
    extra = [t.to(DEV) if isinstance(t, torch.Tensor) else t for t in extra]
    out = fn(*leaves, *extra, softmax_threshold=-128.0, gate_threshold=-128.0, **kw)
    out.backward(do.to(DEV))
    _sync()
    return [t.grad for t in leaves]


_GNAMES = ("dq", "dk", "dv", "dalpha", "ddelta")


def test_golden_gated_backward():
    fsa = _ops()
    g = load("bwd_causal")
    got = _run_gated_bwd(fsa.flash_gated_attn_func, g["q"], g["k"], g["v"], g["alpha"], g["delta"], g["dout"],
                         is_causal=True)
    for name, t, key in zip(_GNAMES, got, ("dq_gated", "dk_gated", "dv_gated", "da_gated", "dd_gated")):
        assert_close("golden-gated-" + name, t, g[key])


# the reference's gated backward grid (tests/test_gated_base_backward.py): causal x local x split_qo x gate form
@pytest.mark.parametrize("causal,local", [(False, False), (True, False), (False, True), (True, True)])
@pytest.mark.parametrize("split", [False, True])
@pytest.mark.parametrize("logsig", [True, False])
@pytest.mark.parametrize("head_dim", [64, 128])
def test_gated_backward_grid(causal, local, split, logsig, head_dim):
    fsa = _ops()
    b, s, hq, hkv = 2, 640, 8, 2
    q, k, v = seeded_qkv(0, b, s, s, hq, hkv, head_dim)
    a, d = _gates(5, b, s, s, hq, hkv)
    do = torch.randn(b, s, hq, head_dim, generator=torch.Generator().manual_seed(9)).to(torch.bfloat16)
    ws = torch.tensor([[32, 200, 100, 160], [0, 300, 0, 64]], dtype=torch.int32) if local else None
    ref = eager.backward(q, k, v, do, None, causal, is_local=local, window_sizes=ws, alpha=a, delta=d,
                         is_logsigmoid_gate=logsig)
    got = _run_gated_bwd(fsa.flash_gated_attn_func, q, k, v, a, d, do, is_causal=causal, window_sizes=ws,
                         is_split_qo=split, num_splits=3 if split else None, is_logsigmoid_gate=logsig)
    for name, t, r in zip(_GNAMES, got, ref):
        assert_close("gated-" + name, t, r, rtol=2.5e-2, atol=2.5e-2)


@pytest.mark.parametrize("sq,sk", [(77, 300), (300, 300), (129, 1000)])
@pytest.mark.parametrize("causal", [False, True])
def test_gated_backward_ragged(sq, sk, causal):
    fsa = _ops()
    q, k, v = seeded_qkv(1, 2, sq, sk, 4, 2, 128, torch.float16)
    a, d = _gates(6, 2, sq, sk, 4, 2, torch.float16)
    do = torch.randn(2, sq, 4, 128, generator=torch.Generator().manual_seed(3)).to(torch.float16)
    ref = eager.backward(q, k, v, do, None, causal, alpha=a, delta=d)
    got = _run_gated_bwd(fsa.flash_gated_attn_func, q, k, v, a, d, do, is_causal=causal)
    for name, t, r in zip(_GNAMES, got, ref):
        assert_close("gated-ragged-" + name, t, r, rtol=2.5e-2, atol=2.5e-2)


def test_gated_backward_varlen():
    import itertools

    fsa = _ops()
    lens_q, lens_k = [5, 130, 257, 64], [70, 130, 300, 64]
    cq = torch.tensor([0] + list(itertools.accumulate(lens_q)), dtype=torch.int32)
    ck = torch.tensor([0] + list(itertools.accumulate(lens_k)), dtype=torch.int32)
    g = torch.Generator().manual_seed(3)
    mk = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16)  # noqa: E731
    q, k, v, do = mk(sum(lens_q), 4, 128), mk(sum(lens_k), 2, 128), mk(sum(lens_k), 2, 128), mk(sum(lens_q), 4, 128)
    a, d = mk(sum(lens_q), 4), mk(sum(lens_k), 2)
    ref = eager.varlen_backward(q, k, v, do, cq, ck, None, True, alpha=a, delta=d)
    got = _run_gated_bwd(fsa.flash_gated_attn_varlen_func, q, k, v, a, d, do, cq, ck, max(lens_q), max(lens_k),
                         is_causal=True)
    for name, t, r in zip(_GNAMES, got, ref):
        assert_close("gated-varlen-" + name, t, r, rtol=2.5e-2, atol=2.5e-2)


def test_gated_backward_gate_skip_is_recorded():
    """Keys whose delta pushes the gate far below the running bound are skipped (tile map value 3) and
    the gradients stay close to the exact ones."""
    from flash_sparse_attn.ops.triton import flash_bwd, flash_fwd

    b, s, hq, hkv, hd = 1, 1024, 4, 2, 128
    q, k, v = seeded_qkv(2, b, s, s, hq, hkv, hd)
    # The bound runs over the query tiles of ONE key tile (flash_gated_bwd.py:406-432): the first query
    # tile (alpha = 0, gate bound 0) sets it, the others (alpha = 4 against delta = -64) fall far below.
    a = torch.full((b, s, hq), 4.0)
    a[:, :128] = 0.0
    a = a.to(torch.bfloat16)
    d = torch.zeros(b, s, hkv)
    d[:, 256:512] = -64.0
    d = d.to(torch.bfloat16)
    do = torch.randn(b, s, hq, hd, generator=torch.Generator().manual_seed(4)).to(torch.bfloat16)
    ref = eager.backward(q, k, v, do, None, False, alpha=a, delta=d)
    at, dt = a.transpose(1, 2).contiguous().to(DEV), d.transpose(1, 2).contiguous().to(DEV)
    qd, kd, vd, dod = (t.to(DEV) for t in (q, k, v, do))
    out, lse, *_ = flash_fwd.attn_forward("gated", qd, kd, vd, alpha=at, delta=dt, softmax_threshold=-128.0,
                                          gate_threshold=-128.0)
    tmap = torch.zeros(flash_bwd.tile_map_numel(b, s, s, hq), dtype=torch.uint8, device=DEV)
    got = flash_bwd.attn_backward("gated", qd, kd, vd, out, dod, lse, alpha=at, delta=dt, softmax_threshold=-128.0,
                                  gate_threshold=1e-6, tile_map=tmap)
    _sync()
    tm = tmap.cpu().reshape(b, hq, 8, 1, 8)
    assert (tm[:, :, 2:4, :, 1:] == 3).all(), "key tiles 2 and 3 are gate-skipped after their first query tile"
    assert (tm[:, :, 2:4, :, 0] == 1).all() and (tm[:, :, :2] == 1).all() and (tm[:, :, 4:] == 1).all()
    got = list(got)
    got[3], got[4] = got[3].transpose(1, 2), got[4].transpose(1, 2)
    for name, t, r in zip(_GNAMES, got, ref):
        assert_close("gated-skip-" + name, t, r, rtol=2.5e-2, atol=2.5e-2)
