"""Host heuristics of the operator layer agree with the reference's (golden table)."""

import torch

from fixtures import load
from flash_sparse_attn.ops.triton import utils


def test_window_sizes_heuristic():
    g = load("heuristics")
    for row in g["windows"].tolist():
        sk, hkv = row[0], row[1]
        want = torch.tensor(row[2:2 + 4 * hkv], dtype=torch.int32).reshape(hkv, 4)
        got = utils.window_sizes_heuristic(sk, hkv, torch.device("cpu"))
        assert got.dtype == torch.int32 and torch.equal(got, want), (sk, hkv)


def test_num_splits_heuristic():
    g = load("heuristics")
    for sq, sk, sms, tm, tn, loc, hkv, want in g["splits"].tolist():
        assert utils.num_splits_heuristic(sq, sk, sms, tm, tn, bool(loc), hkv) == want
