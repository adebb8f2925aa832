"""Top-k position selection (the step in front of the gathered decode): the CPU restatement against the
golden fixture produced by the reference's flash_sparse_attn/utils/mask.py:20-44, and the CUDA kernel
(through the C ABI) against both. Index work: every comparison is bit-exact."""

import numpy as np
import pytest
import torch

from fixtures import load
from oracle import topk as oracle_topk

DEV = "cuda"


def test_oracle_matches_reference_golden():
    g = load("topk")
    for name in "abcd":
        scores, k, ref = g[f"{name}_scores"], int(g[f"{name}_k"]), g[f"{name}_idx"]
        got = oracle_topk.topk_indices(scores.float().numpy(), k)
        assert np.array_equal(got, ref.numpy()), name


def test_oracle_tie_rule_and_specials():
    x = np.array([[1.0, 3.0, 3.0, 3.0, 0.5, 3.0, np.inf, -np.inf, np.nan, 2.0]], dtype=np.float32)
    # NaN first, then +inf, then the lowest positions among the equal 3.0s
    assert oracle_topk.topk_indices(x, 4).tolist() == [[1, 2, 6, 8]]
    assert oracle_topk.topk_indices(x, 10).tolist() == [list(range(10))]


@pytest.mark.gpu
def test_kernel_matches_reference_golden():
    from flash_sparse_attn.utils.mask import topk_indices

    g = load("topk")
    for name in "abcd":
        scores, k, ref = g[f"{name}_scores"], int(g[f"{name}_k"]), g[f"{name}_idx"]
        got = topk_indices(scores.to(DEV), k)
        torch.cuda.synchronize()
        assert got.dtype == torch.int64 and got.shape == ref.shape
        assert torch.equal(got.cpu(), ref), name


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,n,k", [(3, 1, 1), (5, 513, 1), (4, 1000, 1000), (8, 4096, 2048), (2, 131072, 2048),
                                      (7, 777, 300)])
def test_kernel_matches_oracle_with_ties(dtype, rows, n, k):
    """16-bit scores have many equal values: the lowest positions at the threshold are taken, and the selected
    VALUES are the multiset torch.topk selects."""
    from flash_sparse_attn.utils.mask import topk_indices

    g = torch.Generator().manual_seed(rows * 1000 + n + k)
    x = torch.randn(rows, n, generator=g).to(dtype)
    ref = oracle_topk.topk_indices(x.float().numpy(), k)
    for out_dtype in (torch.int32, torch.int64):
        got = topk_indices(x.to(DEV), k, dtype=out_dtype)
        torch.cuda.synchronize()
        assert got.dtype == out_dtype
        assert np.array_equal(got.cpu().numpy().astype(np.int64), ref)
    vals = torch.gather(x.float(), 1, torch.from_numpy(ref))
    assert torch.equal(vals.sort(dim=1).values, torch.topk(x.float(), k, dim=1).values.sort(dim=1).values)


@pytest.mark.gpu
def test_kernel_specials_strided_rows_and_decode_hand_over():
    from flash_sparse_attn import flash_sparse_attn_with_kvcache_func
    from flash_sparse_attn.utils.mask import topk_indices
    from oracle import eager

    x = torch.tensor([[1.0, 3.0, 3.0, 3.0, 0.5, 3.0, float("inf"), float("-inf"), float("nan"), 2.0]])
    assert topk_indices(x.to(DEV), 4).cpu().tolist() == [[1, 2, 6, 8]]
    # rows that are a strided view (batch, kv head, key) with padding between rows
    big = torch.randn(2, 3, 1100, generator=torch.Generator().manual_seed(1))
    view = big[..., :1000]
    got = topk_indices(view.to(DEV)[..., :1000], 64)
    assert np.array_equal(got.cpu().numpy(), oracle_topk.topk_indices(view.numpy(), 64))
    # the int32 result feeds the gathered decode directly
    b, sk, hq, hkv, d = 2, 2048, 16, 2, 128
    g = torch.Generator().manual_seed(5)
    mk = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16)  # noqa: E731
    q, k, v, bias = mk(b, hq, d), mk(b, sk, hkv, d), mk(b, sk, hkv, d), torch.randn(b, sk, generator=g)
    idx = topk_indices(bias.to(DEV), 256, dtype=torch.int32)
    out = flash_sparse_attn_with_kvcache_func(q.to(DEV), k.to(DEV), v.to(DEV), gather_kv_indices=idx,
                                              softmax_threshold=-128.0)
    torch.cuda.synchronize()
    ref = eager.gather_decode(q, k, v, torch.from_numpy(oracle_topk.topk_indices(bias.numpy(), 256)).to(torch.int32))
    assert torch.allclose(out.float().cpu(), ref.float(), rtol=2.5e-2, atol=2.5e-2)
