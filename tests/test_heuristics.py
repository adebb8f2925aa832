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


def test_decode_num_splits():
    """The decode's own split rule (not the reference's): fill one wave of CTA slots at most, and cut long
    contexts into about six waves so that sequences of unequal length even out."""
    from flash_sparse_attn.ops.triton.flash_dec import decode_num_splits

    sms = 148
    assert decode_num_splits(64, 8, 2048, sms) == 1      # 512 CTAs already exceed the 296 slots
    assert decode_num_splits(16, 8, 2048, sms) == 2      # 128 CTAs: two splits stay inside one wave, three do not
    assert decode_num_splits(8, 8, 2048, sms) == 4
    assert decode_num_splits(1, 8, 2048, sms) == 4       # never below 512 keys per CTA
    assert decode_num_splits(64, 8, 131072, sms) == 4    # long contexts: about six waves
    assert decode_num_splits(4, 8, 131072, sms) == 32    # capped
    assert decode_num_splits(2, 8, 300, sms) == 1
    assert decode_num_splits(1, 1, 0, sms) == 1
    for batch in (1, 3, 17, 64, 300):
        for keys in (1, 511, 512, 5000, 1 << 20):
            assert 1 <= decode_num_splits(batch, 8, keys, sms) <= max(32, 2 * sms)
