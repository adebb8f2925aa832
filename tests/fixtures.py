"""Helpers shared by the tests: golden fixture loading, comparison with the reference's tolerance rule."""

import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# tolerances of the reference's own tests (tests/test_utils.py:35-54, :798-820, :1285-1291)
RTOL, ATOL = 1.6e-2, 1.0e-5
FP8_TOL = 1.5e-1


def load(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    out = {}
    for k in z.files:
        a = z[k]
        if a.dtype == np.uint16:
            out[k] = torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
        elif a.ndim == 0:
            out[k] = a.item()
        else:
            out[k] = torch.from_numpy(a.copy())
    return out


def assert_close(name, got, ref, rtol=RTOL, atol=ATOL):
    """The reference's acceptance rule: elementwise allclose, or, failing that, mean absolute
    difference <= atol or mean relative difference <= rtol (tests/test_utils.py:798-820)."""
    got_f, ref_f = got.detach().float().cpu(), ref.detach().float().cpu()
    assert got_f.shape == ref_f.shape, f"{name}: shape {tuple(got_f.shape)} vs {tuple(ref_f.shape)}"
    assert not torch.isnan(got_f).any(), f"{name}: NaN in result"
    if torch.allclose(got_f, ref_f, rtol=rtol, atol=atol):
        return
    diff = (got_f - ref_f).abs()
    finite = torch.isfinite(ref_f)
    assert torch.equal(torch.isfinite(got_f), finite), f"{name}: infinities differ"
    diff = diff[finite]
    mean_abs = diff.mean().item()
    mean_rel = mean_abs / max(ref_f[finite].abs().mean().item(), 1e-6)
    assert mean_abs <= atol or mean_rel <= rtol, (
        f"{name}: mean_abs_diff={mean_abs:.6f} mean_rel_diff={mean_rel:.6f} max_abs_diff={diff.max().item():.6f}")


def seeded_qkv(seed, b, sq, sk, hq, hkv, d, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(b, sq, hq, d, generator=g).to(dtype)
    k = torch.randn(b, sk, hkv, d, generator=g).to(dtype)
    v = torch.randn(b, sk, hkv, d, generator=g).to(dtype)
    return q, k, v
