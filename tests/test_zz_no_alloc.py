"""fsa_decode_static_scratch: the decode entry point for callers that cannot allocate device memory
(serving loops whose KV pool owns the whole GPU, frozen memory plans, code that cannot afford the
implicit synchronisation of cudaMalloc). Its split workspace is a fixed array inside the library.

Checked here through the C ABI: it gives the same result as the regular entry point (which gets its
workspace from the caller) on two consecutive calls - the second call finds the first call's leftovers
in the shared array and must not be affected by them - and it refuses requests that do not fit.
The file name keeps it last in collection order, so a failure here cannot hide other tests.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _inputs(seed, b, sk, hq, hkv, d):
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).to(DEV)  # noqa: E731
    return mk(b, hq, d), mk(b, sk, hkv, d), mk(b, sk, hkv, d)


def test_static_scratch_decode_matches_regular_entry_point_twice():
    import flash_sparse_attn as fsa
    from flash_sparse_attn import static_scratch
    from flash_sparse_attn.ops.triton.flash_dec import attn_decode

    assert static_scratch.scratch_bytes() == 16 * 1024 * 1024
    # two different problems back to back: the second one reuses (and partly overlaps) the bytes the
    # first one left in the shared workspace
    for call, (seed, b, sk, hq, hkv, d, ns) in enumerate([(11, 8, 3000, 32, 4, 128, 4), (12, 5, 1777, 16, 2, 64, 3)]):
        q, k, v = _inputs(seed, b, sk, hq, hkv, d)
        ref_out, ref_lse = attn_decode("sparse", q, k, v, softmax_threshold=1.0, num_splits=ns)
        out = torch.empty_like(q)
        lse = torch.empty(b, hq, dtype=torch.float32, device=DEV)
        torch.cuda.synchronize()
        free_before, torch_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
        static_scratch.decode_static_scratch("sparse", q, k, v, out, lse, num_splits=ns, softmax_threshold=1.0)
        torch.cuda.synchronize()
        fsa.check_status()
        if call > 0:  # the first call on a device may load the workspace; later ones take no memory at all
            assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the device's free memory"
            assert torch.cuda.memory_allocated() == torch_before, "the call allocated through torch"
        # same kernels, same split count, same arithmetic: bit-identical
        assert torch.equal(out, ref_out), f"call {call}: outputs differ"
        assert torch.equal(lse, ref_lse), f"call {call}: lse differs"


def test_static_scratch_rejects_oversized_requests():
    from flash_sparse_attn import static_scratch

    q, k, v = _inputs(13, 64, 256, 64, 8, 128)
    out = torch.empty_like(q)
    lse = torch.empty(64, 64, dtype=torch.float32, device=DEV)
    # 16 splits x 64 x 64 x 129 floats = 33.8 MB > 16 MiB
    with pytest.raises(RuntimeError, match="built-in workspace"):
        static_scratch.decode_static_scratch("dense", q, k, v, out, lse, num_splits=16)
