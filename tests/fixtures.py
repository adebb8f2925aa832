"""Helpers shared by the tests: golden fixture loading, comparison with an element-wise bound plus the
reference's tolerance rule."""

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


# element-wise bound for 16-bit outputs and gradients; FP8 paths state their own (FP8_TOL)
EW_RTOL, EW_ATOL = 2.0e-2, 2.0e-2


def assert_close(name, got, ref, rtol=RTOL, atol=ATOL, ew_rtol=None, ew_atol=None):
    """Two checks, both must hold.

    1. Element-wise: |got - ref| <= ew_atol + ew_rtol * |ref| for EVERY element (default 2e-2 / 2e-2 for
       bf16 / fp16 results; a caller that passes rtol >= 1e-1, the FP8 tests, gets that value here too).
       One wrong tile among hundreds trips this.
    2. The reference's own acceptance rule (tests/test_utils.py:798-820): allclose(rtol, atol), or mean
       absolute difference <= atol, or mean relative difference <= rtol.
    """
    got_f, ref_f = got.detach().float().cpu(), ref.detach().float().cpu()
    assert got_f.shape == ref_f.shape, f"{name}: shape {tuple(got_f.shape)} vs {tuple(ref_f.shape)}"
    assert not torch.isnan(got_f).any(), f"{name}: NaN in result"
    finite = torch.isfinite(ref_f)
    assert torch.equal(torch.isfinite(got_f), finite), f"{name}: infinities differ"
    if ew_rtol is None:
        ew_rtol = rtol if rtol >= 1e-1 else EW_RTOL
    if ew_atol is None:
        ew_atol = atol if atol >= 1e-1 else EW_ATOL
    diff = (got_f - ref_f).abs()[finite]
    if diff.numel() == 0:
        return
    bound = ew_atol + ew_rtol * ref_f[finite].abs()
    excess = diff - bound
    worst = int(excess.argmax())
    assert excess[worst] <= 0, (
        f"{name}: element-wise bound (rtol {ew_rtol}, atol {ew_atol}) broken by {int((excess > 0).sum())} of "
        f"{diff.numel()} elements; worst |diff|={diff[worst].item():.5f} at |ref|={ref_f[finite][worst].abs().item():.5f}; "
        f"max_abs_diff={diff.max().item():.5f}")
    if torch.allclose(got_f, ref_f, rtol=rtol, atol=atol):
        return
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
