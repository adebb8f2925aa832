"""Pin the CPU oracle to fixtures produced by the reference's own eager functions
(tests/golden/make_golden.py)."""

import torch

from fixtures import assert_close, load
from oracle import eager, tiled

SCALE = 64 ** -0.5


def _regen(seed, shape, decode=False):
    b, s, hq, hkv, d = shape
    torch.manual_seed(int(seed))
    if decode:
        q = torch.randn(b, hq, d, dtype=torch.bfloat16)
    else:
        q = torch.randn(b, s, hq, d, dtype=torch.bfloat16)
    k = torch.randn(b, s, hkv, d, dtype=torch.bfloat16)
    v = torch.randn(b, s, hkv, d, dtype=torch.bfloat16)
    return q, k, v


def test_forward_matches_reference():
    for name in ("fwd_nc", "fwd_causal", "fwd_causal_sq_lt_sk"):
        g = load(name)
        causal = bool(g["causal"])
        out, lse = eager.forward(g["q"], g["k"], g["v"], SCALE, causal, return_lse=True)
        assert torch.equal(out, g["out_dense"]) and torch.equal(out, g["out_sparse"]), name
        assert torch.allclose(lse, g["lse_dense"], rtol=0, atol=1e-6)
        og, lg = eager.forward(g["q"], g["k"], g["v"], SCALE, causal, alpha=g["alpha"], delta=g["delta"],
                               return_lse=True)
        assert torch.equal(og, g["out_gated"]), name
        assert torch.allclose(lg, g["lse_gated"], rtol=0, atol=1e-6)
        ol = eager.forward(g["q"], g["k"], g["v"], SCALE, causal, alpha=g["alpha"], delta=g["delta"],
                           is_logsigmoid_gate=False)
        assert torch.equal(ol, g["out_gated_lin"]), name


def test_local_forward_matches_reference():
    g = load("fwd_local")
    q, k, v = _regen(g["seed"], g["shape"].tolist())
    assert abs(q.float().sum().item() - g["q_sum"]) < 1e-3 and abs(v.float().sum().item() - g["v_sum"]) < 1e-3
    ws = eager.window_sizes_heuristic(k.shape[1], k.shape[2])
    assert torch.equal(ws, g["window_sizes"].to(torch.int32))
    out, lse = eager.forward(q, k, v, SCALE, True, is_local=True, return_lse=True)
    assert torch.equal(out, g["out"])
    assert torch.allclose(lse, g["lse"], rtol=0, atol=1e-6)
    # explicit window table == heuristic table
    out2 = eager.forward(q, k, v, SCALE, True, is_local=True, window_sizes=ws)
    assert torch.equal(out2, g["out"])


def test_varlen_matches_reference():
    g = load("fwd_varlen")
    cu = g["cu_seqlens"]
    out = eager.varlen_forward(g["q"], g["k"], g["v"], cu, cu, SCALE, True)
    assert torch.equal(out, g["out_sparse"])
    og = eager.varlen_forward(g["q"], g["k"], g["v"], cu, cu, SCALE, True, alpha=g["alpha"], delta=g["delta"])
    assert torch.equal(og, g["out_gated"])


def test_decode_matches_reference():
    g = load("decode")
    assert torch.equal(eager.decode(g["q"], g["k"], g["v"], SCALE), g["out_dense"])
    assert torch.equal(eager.decode(g["q"], g["k"], g["v"], SCALE, alpha=g["alpha"], delta=g["delta"]), g["out_gated"])
    assert torch.equal(eager.varlen_decode(g["q"], g["k_packed"], g["v_packed"], g["cu_seqlens"], SCALE),
                       g["out_varlen"])
    got = eager.gather_decode(g["q"], g["k"], g["v"], g["gather_idx"], SCALE)
    assert_close("gather", got, g["out_gather"], rtol=1e-2, atol=1e-2)
    assert (got.float() - g["out_gather"].float()).abs().max() <= 2 ** -6
    gl = load("decode_local")
    q, k, v = _regen(gl["seed"], gl["shape"].tolist(), decode=True)
    assert abs(k.float().sum().item() - gl["k_sum"]) < 1e-3
    assert torch.equal(eager.decode(q, k, v, SCALE, is_local=True), gl["out"])


def test_backward_matches_reference():
    g = load("bwd_causal")
    dq, dk, dv = eager.backward(g["q"], g["k"], g["v"], g["dout"], SCALE, True)
    for n, t in (("dq", dq), ("dk", dk), ("dv", dv)):
        assert torch.allclose(t, g[f"{n}_dense"], rtol=1e-5, atol=1e-6), n
    gr = eager.backward(g["q"], g["k"], g["v"], g["dout"], SCALE, True, alpha=g["alpha"], delta=g["delta"])
    for n, t in zip(("dq", "dk", "dv", "da", "dd"), gr):
        assert torch.allclose(t, g[f"{n}_gated"], rtol=1e-5, atol=1e-6), n


def test_paged_view_roundtrip():
    torch.manual_seed(0)
    cache = torch.randn(12, 32, 2, 16)
    table = torch.randperm(12).reshape(3, 4).to(torch.int32)
    logical = eager.unpage(cache, table)
    assert logical.shape == (3, 128, 2, 16)
    assert torch.equal(logical[1, 40], cache[table[1, 1], 8])


def test_tiled_equals_eager_when_skipping_is_off():
    """With the threshold disabled the tile-faithful walk must reproduce the eager result
    (the reference's own tests run exactly this configuration, tests/test_utils.py:837)."""
    g = load("fwd_causal_sq_lt_sk")
    for tile in ((64, 64), (128, 128), (32, 64)):
        out, lse, tmap = tiled.forward_tiled(g["q"], g["k"], g["v"], SCALE, True, softmax_threshold=-128.0,
                                             tile_m=tile[0], tile_n=tile[1])
        assert_close("tiled", out, g["out_sparse"])
        assert (tmap != 2).all()
    gl = load("fwd_local")
    q, k, v = _regen(gl["seed"], gl["shape"].tolist())
    q, k, v = q[:, :700], k[:, :700], v[:, :700]
    ws = torch.tensor([[16, 100, 50, 130], [0, 200, 0, 64]], dtype=torch.int32)
    ref = eager.forward(q, k, v, SCALE, True, is_local=True, window_sizes=ws)
    for ns in (1, 3):
        out, lse, tmap = tiled.forward_tiled(q, k, v, SCALE, True, window_sizes=ws, softmax_threshold=-128.0,
                                             num_splits=ns, is_split_kv=ns > 1)
        assert_close(f"tiled-local-{ns}", out, ref)


def test_tiled_skips_on_peaked_scores():
    """A strongly peaked score distribution must trigger the skip rule for far-away tiles, and the
    result must stay close to the eager one (skipped mass is below the threshold by construction)."""
    torch.manual_seed(0)
    s, d = 512, 64
    base = torch.randn(1, s, 1, d)
    q = (base * 4).to(torch.bfloat16)   # q_i . k_i large, q_i . k_j small
    k = base.to(torch.bfloat16)
    v = torch.randn(1, s, 1, d).to(torch.bfloat16)
    out, lse, tmap = tiled.forward_tiled(q, k, v, d ** -0.5, True, softmax_threshold=1.0, tile_m=64, tile_n=64)
    assert (tmap == 2).sum() > 0
    ref = eager.forward(q, k, v, d ** -0.5, True)
    assert (out.float() - ref.float()).abs().max() < 2e-2
