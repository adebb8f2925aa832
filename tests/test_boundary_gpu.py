"""Behaviour of the C-ABI boundary on a GPU: the sticky status word, several devices in one process."""

import pytest
import torch

from fixtures import seeded_qkv

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_status_word_injected_from_the_host():
    """The abort path without any device wait running out: the host sets the status word, the next launches find it
    set, drain at once (no output is written), check_status() raises and clears the word, and the call after that
    computes normally."""
    import flash_sparse_attn as fsa
    from flash_sparse_attn import _lib

    q, k, v = (t.to(DEV) for t in seeded_qkv(3, 1, 256, 256, 4, 2, 128))
    good = fsa.flash_sparse_attn_func(q, k, v, is_causal=True)
    torch.cuda.synchronize()
    fsa.check_status()
    word = _lib.status_word(torch.device(DEV, torch.cuda.current_device()))
    word.fill_(7)
    out = torch.full_like(q, 3.0)
    lse = torch.zeros(1, 4, 256, dtype=torch.float32, device=DEV)
    fsa.flash_sparse_attn_func(q, k, v, is_causal=True, out=out, lse=lse)
    torch.cuda.synchronize()
    assert bool((out == 3.0).all()), "a kernel launched with the status word set must not write its output"
    with pytest.raises(RuntimeError, match="device status"):
        fsa.check_status()
    fsa.check_status()  # cleared by the raise
    again = fsa.flash_sparse_attn_func(q, k, v, is_causal=True)
    torch.cuda.synchronize()
    fsa.check_status()
    assert torch.equal(again, good)
    # backward: same contract
    qg = q.clone().requires_grad_(True)
    o = fsa.flash_sparse_attn_func(qg, k, v, is_causal=True)
    word.fill_(1)
    o.backward(torch.ones_like(o))
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="device status"):
        fsa.check_status()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_devices_in_one_process():
    """Forward, backward and decode on cuda:0 and then cuda:1 from one process: the opt-in to large dynamic
    shared memory is per device."""
    import flash_sparse_attn as fsa
    from oracle import eager

    q, k, v = seeded_qkv(5, 1, 384, 384, 4, 2, 128)
    ref = eager.forward(q, k, v, None, True)
    for dev in ("cuda:0", "cuda:1"):
        qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
        out = fsa.flash_sparse_attn_func(qd, kd, vd, is_causal=True)
        out.backward(torch.ones_like(out))
        dec = fsa.flash_sparse_attn_with_kvcache_func(qd[:, -1].detach(), kd.detach(), vd.detach())
        torch.cuda.synchronize(dev)
        fsa.check_status()
        assert (out.float().cpu() - ref.float()).abs().max().item() < 2e-2
        assert torch.isfinite(qd.grad).all() and torch.isfinite(dec).all()
