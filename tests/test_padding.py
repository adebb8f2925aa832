"""Padded batch <-> packed tokens (flash_sparse_attn/utils/padding.py) against outputs of the reference's own
functions (tests/golden/padding.npz, made by tests/golden/make_golden.py): index work, every comparison exact."""

import pytest
import torch

from fixtures import load

B, S = 3, 17


def _pad():
    from flash_sparse_attn.utils import padding

    return padding


@pytest.mark.parametrize("name", ["right", "left"])
def test_unpad_and_pad_match_the_reference(name):
    P, g = _pad(), load("padding")
    mask, unused, x = g[f"{name}_mask"], g[f"{name}_unused"], g[f"{name}_x"]
    for tag, um in (("", None), ("_u", unused)):
        packed, idx, cu, mx, used = P.unpad_input(x, mask, um)
        assert torch.equal(packed, g[f"{name}{tag}_packed"]) and torch.equal(idx, g[f"{name}{tag}_idx"])
        assert cu.dtype == torch.int32 and torch.equal(cu, g[f"{name}{tag}_cu"])
        assert isinstance(mx, int) and mx == int(g[f"{name}{tag}_max"])
        assert used.dtype == torch.int32 and torch.equal(used, g[f"{name}{tag}_used"])
    packed, idx, cu, mx, _ = P.unpad_input(x, mask)
    assert torch.equal(P.pad_input(packed, idx, B, S), g[f"{name}_repadded"])
    # a round trip keeps the selected tokens and zeroes the rest
    assert torch.equal(P.pad_input(packed, idx, B, S), x * mask[:, :, None, None].to(x.dtype))
    i2, cu2, mx2 = P.get_unpad_data(mask)
    assert torch.equal(i2, idx) and torch.equal(cu2, cu) and mx2 == mx


@pytest.mark.parametrize("name", ["right", "left"])
@pytest.mark.parametrize("ql", [S, 1, 5])
def test_upad_input_matches_the_reference(name, ql):
    P, g = _pad(), load("padding")
    pre = f"{name}_q{ql}"
    qo, ko, vo, iq, (cq, ck), (mq, mk) = P.upad_input(g[pre + "_q"], g[f"{name}_k"], g[f"{name}_v"], g[f"{name}_mask"],
                                                     ql, P.unpad_input)
    for got, key in ((qo, "_qo"), (ko, "_ko"), (vo, "_vo"), (iq, "_iq"), (cq, "_cq"), (ck, "_ck")):
        assert got.dtype == g[pre + key].dtype and torch.equal(got, g[pre + key]), key
    assert (mq, mk) == (int(g[pre + "_mq"]), int(g[pre + "_mk"]))


def test_empty_sequence_in_batch():
    P = _pad()
    mask = torch.tensor([[1, 1, 0], [0, 0, 0], [1, 0, 0]], dtype=torch.int32)
    x = torch.arange(18, dtype=torch.float32).view(3, 3, 2)
    packed, idx, cu, mx, used = P.unpad_input(x, mask)
    assert cu.tolist() == [0, 2, 2, 3] and mx == 2 and used.tolist() == [2, 0, 1] and idx.tolist() == [0, 1, 6]
    assert torch.equal(P.pad_input(packed, idx, 3, 3), x * mask[:, :, None].float())
