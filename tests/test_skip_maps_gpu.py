"""Which tiles the kernels skip, against the tile-faithful CPU restatement (oracle/tiled.py), for the forward, the
backward and the decode, sparse and gated.

Three statements per case:
  1. visited tiles (integer schedule): equal bit for bit;
  2. gate-skipped tiles (map value 3): equal bit for bit - the bound is fp32 arithmetic on 16-bit extremes with no
     matrix product in it;
  3. softmax-threshold decisions (1 = computed, 2 = skipped): the restatement is run a second time FOLLOWING the
     kernel's decisions (so that every tile sees the kernel's running state) and records its own margin per tile
     (log2 of the largest probability bound minus the log2 threshold; skip iff < 0). Every kernel decision must
     agree with the sign of that margin unless |margin| < MARGIN_TOL: only ties within fp32 / exp2-approximation
     noise may differ. In addition the free-running restatement must agree on >= 99.9 % of the tiles.
Inputs: "peaked" queries aligned with their keys, and the llm-like generator of benchmarks/workloads.py (the
distribution of the reference's benchmark inputs), because iid inputs skip nothing.
"""

import importlib.util
import os

import pytest
import torch

from fixtures import assert_close
from oracle import eager, tiled

pytestmark = pytest.mark.gpu
DEV = "cuda"
MARGIN_TOL = 2.0 ** -5   # log2 units: 2 % in probability
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _workloads():
    spec = importlib.util.spec_from_file_location(
        "fsa_workloads", os.path.join(ROOT, "flash-sparse-attention_b200", "benchmarks", "workloads.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _inputs(kind, seed, s, hq, hkv, d):
    if kind == "llm":
        q, k, v, do = _workloads().llm_like_qkv("cpu", seed, 1, s, s, hq, hkv, d)
        return q, k, v, do
    g = torch.Generator().manual_seed(seed)
    base = torch.randn(1, s, hkv, d, generator=g)
    q = base.repeat_interleave(hq // hkv, dim=2) * 3 + torch.randn(1, s, hq, d, generator=g) * 0.3
    k = base + torch.randn(1, s, hkv, d, generator=g) * 0.1
    v = torch.randn(1, s, hkv, d, generator=g)
    do = torch.randn(1, s, hq, d, generator=g)
    return tuple(t.to(torch.bfloat16) for t in (q, k, v, do))


def _gates(seed, s, hq, hkv, n_tile=128):
    """alpha in [2, 8]; delta per 128-key tile either 'hot' (around +4) or 'cold' (around -60): once a hot tile has
    set the running bound (up to 32), the bound of a cold tile (about -114) lies more than the 81 below it that the
    default threshold 1 / Sk asks for at head size 128 ((bound - running) * scale * log2(e) < log2(threshold))."""
    g = torch.Generator().manual_seed(seed)
    alpha = torch.rand(1, s, hq, generator=g) * 6 + 2
    hot = torch.rand(1, -(-s // n_tile), hkv, generator=g) < 0.4
    hot[:, -1] = True
    level = torch.where(hot, torch.tensor(4.0), torch.tensor(-60.0)).repeat_interleave(n_tile, dim=1)[:, :s]
    delta = level + torch.randn(1, s, hkv, generator=g)
    return alpha.to(torch.bfloat16), delta.to(torch.bfloat16)


def _status():
    import flash_sparse_attn as fsa

    torch.cuda.synchronize()
    fsa.check_status()


def _compare(tag, got_map, free_map, margin):
    assert torch.equal(got_map != 0, free_map != 0), f"{tag}: visited tiles differ"
    assert torch.equal(got_map == 3, free_map == 3), f"{tag}: gate-skipped tiles differ"
    decided = (got_map == 1) | (got_map == 2)
    would_skip = margin < 0
    wrong = decided & ((got_map == 2) != would_skip) & ~(margin.abs() < MARGIN_TOL) & ~torch.isnan(margin)
    assert not wrong.any(), (f"{tag}: {int(wrong.sum())} decisions contradict the restatement away from a tie, e.g. margin "
                             f"{margin[wrong][:4].tolist()} with map {got_map[wrong][:4].tolist()}")
    agree = (got_map == free_map).float().mean().item()
    assert agree >= 0.999, f"{tag}: free-running agreement {agree:.4f}"
    return int((got_map == 2).sum()), int((got_map == 3).sum())


FWD_CASES = [("peaked", False, 1), ("peaked", True, 1), ("peaked", False, 3), ("llm", False, 1), ("llm", True, 2)]


@pytest.mark.parametrize("data,local,splits", FWD_CASES)
def test_forward_softmax_skip_map(data, local, splits):
    from flash_sparse_attn.ops.triton.flash_fwd import attn_forward, tile_map_numel

    s, hq, hkv, d = 2048 if data == "llm" else 1536, 4, 2, 128
    q, k, v, _ = _inputs(data, 5, s, hq, hkv, d)
    ws = torch.tensor([[64, 400, 200, 300], [0, 600, 0, 256]], dtype=torch.int32) if local else None
    kw = dict(window_sizes=ws, softmax_threshold=1.0, num_splits=splits, is_split_kv=splits > 1)
    tmap = torch.zeros(tile_map_numel(1, s, s, hq, hkv, False, splits), dtype=torch.uint8, device=DEV)
    out, *_ = attn_forward("sparse", q.to(DEV), k.to(DEV), v.to(DEV), is_causal=True,
                           window_sizes=ws.to(DEV) if local else None, is_local=local, softmax_threshold=1.0,
                           is_split_kv=splits > 1, num_splits=splits if splits > 1 else None, tile_map=tmap)
    _status()
    ref, _, free_map = tiled.forward_tiled(q, k, v, None, True, **kw)
    got_map = tmap.cpu().reshape(free_map.shape)
    _, _, _, margin = tiled.forward_tiled(q, k, v, None, True, force_map=got_map, return_margin=True, **kw)
    n_skip, _ = _compare(f"fwd-{data}", got_map, free_map, margin)
    assert n_skip > 0, "inputs must trigger skipping"
    assert_close("fwd-skip-out", out, ref)


@pytest.mark.parametrize("data,local", [("peaked", False), ("llm", True)])
def test_gated_forward_skip_maps(data, local):
    from flash_sparse_attn.ops.triton.flash_fwd import attn_forward, tile_map_numel

    s, hq, hkv, d = 1536, 4, 2, 128
    q, k, v, _ = _inputs(data, 6, s, hq, hkv, d)
    alpha, delta = _gates(7, s, hq, hkv)
    ws = torch.tensor([[64, 400, 200, 300], [0, 600, 0, 256]], dtype=torch.int32) if local else None
    kw = dict(window_sizes=ws, softmax_threshold=1.0, alpha=alpha, delta=delta)
    tmap = torch.zeros(tile_map_numel(1, s, s, hq, hkv), dtype=torch.uint8, device=DEV)
    out, *_ = attn_forward("gated", q.to(DEV), k.to(DEV), v.to(DEV), alpha=alpha.transpose(1, 2).contiguous().to(DEV),
                           delta=delta.transpose(1, 2).contiguous().to(DEV), is_causal=True,
                           window_sizes=ws.to(DEV) if local else None, is_local=local, softmax_threshold=1.0,
                           gate_threshold=None, tile_map=tmap)
    _status()
    ref, _, free_map = tiled.forward_tiled(q, k, v, None, True, **kw)
    got_map = tmap.cpu().reshape(free_map.shape)
    _, _, _, margin = tiled.forward_tiled(q, k, v, None, True, force_map=got_map, return_margin=True, **kw)
    _, n_gate = _compare(f"gated-fwd-{data}", got_map, free_map, margin)
    assert n_gate > 0, "inputs must trigger gate skipping"
    assert_close("gated-fwd-skip-out", out, ref)


@pytest.mark.parametrize("data,causal,local,splits", [("peaked", True, False, 1), ("peaked", False, False, 1),
                                                      ("llm", True, True, 1), ("llm", True, False, 2)])
def test_backward_softmax_skip_map(data, causal, local, splits):
    from flash_sparse_attn.ops.triton import flash_bwd, flash_fwd

    s, hq, hkv, d = (1536 if causal else 1400), 4, 2, 128   # non-causal: a ragged last tile in both directions
    q, k, v, do = _inputs(data, 8, s, hq, hkv, d)
    ws = torch.tensor([[64, 400, 200, 300], [0, 600, 0, 256]], dtype=torch.int32) if local else None
    qd, kd, vd, dod = (t.to(DEV) for t in (q, k, v, do))
    # the forward that feeds the backward runs WITHOUT skipping, so that out / lse are the exact ones on both sides
    out, lse, *_ = flash_fwd.attn_forward("sparse", qd, kd, vd, is_causal=causal, is_local=local,
                                          window_sizes=ws.to(DEV) if local else None, softmax_threshold=-128.0)
    tmap = torch.zeros(flash_bwd.tile_map_numel(1, s, s, hq, splits), dtype=torch.uint8, device=DEV)
    got = flash_bwd.attn_backward("sparse", qd, kd, vd, out, dod, lse, is_causal=causal, is_local=local,
                                  window_sizes=ws.to(DEV) if local else None, softmax_threshold=1.0,
                                  is_split_qo=splits > 1, num_splits=splits if splits > 1 else None, tile_map=tmap)
    _status()
    kw = dict(window_sizes=ws, softmax_threshold=1.0, num_splits=splits, is_split_qo=splits > 1, lse=lse.cpu(),
              out=out.cpu())
    *ref, free_map = tiled.backward_tiled(q, k, v, do, None, causal, **kw)
    got_map = tmap.cpu().reshape(free_map.shape)
    *_, margin = tiled.backward_tiled(q, k, v, do, None, causal, force_map=got_map, return_margin=True, **kw)
    n_skip, _ = _compare(f"bwd-{data}", got_map, free_map, margin)
    assert n_skip > 0, "inputs must trigger skipping"
    for name, a, r in zip(("dq", "dk", "dv"), got, ref):
        assert_close(f"bwd-skip-{name}", a, r, rtol=3e-2, atol=3e-2, ew_atol=3e-2)


@pytest.mark.parametrize("data", ["peaked", "llm"])
def test_gated_backward_skip_maps(data):
    from flash_sparse_attn.ops.triton import flash_bwd, flash_fwd

    s, hq, hkv, d = 1280, 4, 2, 128
    q, k, v, do = _inputs(data, 9, s, hq, hkv, d)
    # the backward bound runs over the QUERY tiles of one key tile: alpha per 128-row tile 'hot' or 'cold'
    delta, alpha = _gates(10, s, hkv, hq)   # roles swapped: per-tile levels on alpha, positive delta in [2, 8]
    at, dt = alpha.transpose(1, 2).contiguous().to(DEV), delta.transpose(1, 2).contiguous().to(DEV)
    qd, kd, vd, dod = (t.to(DEV) for t in (q, k, v, do))
    out, lse, *_ = flash_fwd.attn_forward("gated", qd, kd, vd, alpha=at, delta=dt, is_causal=True,
                                          softmax_threshold=-128.0, gate_threshold=-128.0)
    tmap = torch.zeros(flash_bwd.tile_map_numel(1, s, s, hq), dtype=torch.uint8, device=DEV)
    got = list(flash_bwd.attn_backward("gated", qd, kd, vd, out, dod, lse, alpha=at, delta=dt, is_causal=True,
                                       softmax_threshold=1.0, gate_threshold=None, tile_map=tmap))
    _status()
    kw = dict(softmax_threshold=1.0, alpha=alpha, delta=delta, lse=lse.cpu(), out=out.cpu())
    *ref, free_map = tiled.backward_tiled(q, k, v, do, None, True, **kw)
    got_map = tmap.cpu().reshape(free_map.shape)
    *_, margin = tiled.backward_tiled(q, k, v, do, None, True, force_map=got_map, return_margin=True, **kw)
    _, n_gate = _compare(f"gated-bwd-{data}", got_map, free_map, margin)
    assert n_gate > 0, "inputs must trigger gate skipping"
    got[3], got[4] = got[3].transpose(1, 2), got[4].transpose(1, 2)
    for name, a, r in zip(("dq", "dk", "dv", "dalpha", "ddelta"), got, ref):
        assert_close(f"gated-bwd-skip-{name}", a, r, rtol=3e-2, atol=3e-2, ew_atol=3e-2, ew_rtol=3e-2)


@pytest.mark.parametrize("mode,group,splits", [("plain", 16, 1), ("plain", 4, 2), ("gather", 16, 1), ("local", 8, 2)])
def test_decode_softmax_skip_map(mode, group, splits):
    """Rows that pad the G heads to 16 take no part in the kernel's vote (pad_rows_vote=False); with G = 16 that is
    also the reference's behaviour, with fewer heads the reference never skips (its zero rows always vote keep)."""
    from flash_sparse_attn.ops.triton.flash_dec import attn_decode

    g = torch.Generator().manual_seed(11)
    b, sk, hkv, d = 2, 3000, 2, 128
    hq = hkv * group
    k = torch.randn(b, sk, hkv, d, generator=g)
    q = (k[:, -1].repeat_interleave(group, dim=1) * 3 + torch.randn(b, hq, d, generator=g) * 0.2).to(torch.bfloat16)
    k = k.to(torch.bfloat16)
    v = torch.randn(b, sk, hkv, d, generator=g).to(torch.bfloat16)
    kw, okw = {}, {}
    n_tiles = -(-sk // 16)
    if mode == "gather":
        idx = torch.stack([torch.randperm(sk, generator=g)[:700] for _ in range(b)]).to(torch.int32)
        idx[:, -1] = sk - 1   # the peak sits in the first tile the walk visits (it descends from the last slot)
        idx[:, 5] = -1
        kw["gather_kv_indices"] = idx.to(DEV)
        okw["gather_kv_indices"] = idx
        n_tiles = -(-700 // 16)
    if mode == "local":
        ws = torch.tensor([[32, 700, 100, 500], [0, 900, 0, 260]], dtype=torch.int32)
        kw.update(window_sizes=ws.to(DEV), is_local=True)
        okw["window_sizes"] = ws
    tmap = torch.zeros(b * hkv * n_tiles, dtype=torch.uint8, device=DEV)
    out, _ = attn_decode("sparse", q.to(DEV), k.to(DEV), v.to(DEV), softmax_threshold=1.0, num_splits=splits,
                         tile_map=tmap, **kw)
    _status()
    okw.update(softmax_threshold=1.0, num_splits=splits, pad_rows_vote=(group == 16))
    ref, _, free_map = tiled.decode_tiled(q, k, v, **okw)
    got_map = tmap.cpu().reshape(free_map.shape)
    _, _, _, margin = tiled.decode_tiled(q, k, v, force_map=got_map, return_margin=True, **okw)
    n_skip, _ = _compare(f"dec-{mode}", got_map, free_map, margin)
    assert n_skip > 0, "inputs must trigger skipping"
    assert_close("dec-skip-out", out, ref)


def test_gated_decode_skip_maps():
    from flash_sparse_attn.ops.triton.flash_dec import attn_decode

    g = torch.Generator().manual_seed(12)
    b, sk, hkv, group, d = 2, 2048, 2, 16, 128
    hq = hkv * group
    k = torch.randn(b, sk, hkv, d, generator=g).to(torch.bfloat16)
    q = torch.randn(b, hq, d, generator=g).to(torch.bfloat16)
    v = torch.randn(b, sk, hkv, d, generator=g).to(torch.bfloat16)
    alpha = (torch.rand(b, hq, generator=g) * 6 + 2).to(torch.bfloat16)
    hot = torch.rand(b, sk // 16, hkv, generator=g) < 0.3
    delta = (torch.where(hot, torch.tensor(4.0), torch.tensor(-60.0)).repeat_interleave(16, dim=1)
             + torch.randn(b, sk, hkv, generator=g)).to(torch.bfloat16)
    tmap = torch.zeros(b * hkv * (sk // 16), dtype=torch.uint8, device=DEV)
    out, _ = attn_decode("gated", q.to(DEV), k.to(DEV), v.to(DEV), alpha=alpha.to(DEV),
                         delta=delta.transpose(1, 2).contiguous().to(DEV), softmax_threshold=1.0, gate_threshold=None,
                         num_splits=1, tile_map=tmap)
    _status()
    okw = dict(softmax_threshold=1.0, alpha=alpha, delta=delta, pad_rows_vote=True)
    ref, _, free_map = tiled.decode_tiled(q, k, v, **okw)
    got_map = tmap.cpu().reshape(free_map.shape)
    _, _, _, margin = tiled.decode_tiled(q, k, v, force_map=got_map, return_margin=True, **okw)
    _, n_gate = _compare("gated-dec", got_map, free_map, margin)
    assert n_gate > 0, "inputs must trigger gate skipping"
    assert_close("gated-dec-skip-out", out, ref)
