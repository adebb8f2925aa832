"""Routing of the Hugging Face glue (CPU: the operators are replaced by recorders) and, on a GPU, its three routes
against the eager oracle."""

import pytest
import torch

from flash_sparse_attn.integrations import modeling_flash_sparse_attention_utils as M


def _recorders(monkeypatch):
    calls = []

    def batched(q, k, v, **kw):
        calls.append(("batched", q.shape, kw))
        return torch.zeros_like(q)

    def packed(q, k, v, **kw):
        calls.append(("packed", q.shape, kw))
        return torch.zeros_like(q)

    from flash_sparse_attn.utils.padding import pad_input, unpad_input

    monkeypatch.setattr(M, "lazy_import_flash_sparse_attention",
                        lambda impl=None, force_import=False: ((batched, packed, pad_input, unpad_input, None),
                                                               M._process_flash_sparse_attention_kwargs))
    return calls


def test_routes_on_cpu(monkeypatch):
    calls = _recorders(monkeypatch)
    q = torch.zeros(2, 6, 4, 8)
    kv = torch.zeros(2, 6, 2, 8)
    # route 3: no mask
    out = M._flash_sparse_attention_forward(q, kv, kv, None, None, 6, 6, True)
    assert calls[-1][0] == "batched" and calls[-1][2]["is_causal"] is True and out.shape == q.shape
    # route 1: padding mask -> packed tokens, scattered back
    mask = torch.tensor([[1, 1, 1, 1, 0, 0], [1, 1, 1, 1, 1, 1]])
    out = M._flash_sparse_attention_forward(q, kv, kv, mask, None, 6, 6, True)
    name, shape, kw = calls[-1]
    assert name == "packed" and shape[0] == 10 and kw["cu_seqlens_q"].tolist() == [0, 4, 10] and kw["max_seqlen_k"] == 6
    assert out.shape == q.shape
    # route 2: one flattened row with restarting position ids
    q1, kv1 = torch.zeros(1, 7, 4, 8), torch.zeros(1, 7, 2, 8)
    pos = torch.tensor([[0, 1, 2, 0, 1, 0, 1]])
    out = M._flash_sparse_attention_forward(q1, kv1, kv1, None, None, 7, 7, True, position_ids=pos)
    name, shape, kw = calls[-1]
    assert name == "packed" and kw["cu_seqlens_q"].tolist() == [0, 3, 5, 7] and kw["max_seqlen_q"] == 3
    assert out.shape == q1.shape
    # route 2 with pre-computed lengths
    cu = torch.tensor([0, 2, 7])
    M._flash_sparse_attention_forward(q1, kv1, kv1, None, None, 7, 7, True, cu_seq_lens_q=cu, cu_seq_lens_k=cu,
                                      max_length_q=5, max_length_k=5)
    assert calls[-1][0] == "packed" and calls[-1][2]["cu_seqlens_k"].dtype == torch.int32
    # single query position is never causal; window only when the keys exceed it
    M._flash_sparse_attention_forward(q[:, :1], kv, kv, None, None, 1, 6, True, window_size=4)
    kw = calls[-1][2]
    assert kw["is_causal"] is False and kw["window_sizes"].tolist() == [[0, 0, 0, 4]] * 2
    M._flash_sparse_attention_forward(q, kv, kv, None, None, 6, 6, True, window_size=64)
    assert "window_sizes" not in calls[-1][2]
    # what the operators cannot express is refused, not ignored
    with pytest.raises(ValueError):
        M._flash_sparse_attention_forward(q, kv, kv, None, torch.zeros(2, 1, 6, 6), 6, 6, True)
    with pytest.raises(ValueError):
        M._flash_sparse_attention_forward(q, kv, kv, mask, torch.zeros(2, 1, 6, 6), 6, 6, True)
    with pytest.raises(ValueError):
        M._flash_sparse_attention_forward(q, kv, kv, None, None, 6, 6, True, softcap=30.0)
    assert not M._is_packed_sequence(torch.arange(7)[None], 1) and M._is_packed_sequence(pos, 1)


@pytest.mark.gpu
def test_routes_against_the_oracle():
    from flash_sparse_attn.integrations.flash_sparse_attention import flash_sparse_attention_forward
    from oracle import eager

    g = torch.Generator().manual_seed(0)
    b, s, hq, hkv, d = 2, 200, 4, 2, 64
    q = torch.randn(b, hq, s, d, generator=g).to(torch.bfloat16)
    k = torch.randn(b, hkv, s, d, generator=g).to(torch.bfloat16)
    v = torch.randn(b, hkv, s, d, generator=g).to(torch.bfloat16)
    module = torch.nn.Module()
    module.is_causal = True
    dev = "cuda"
    qn, kn, vn = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    # no padding
    out, _ = flash_sparse_attention_forward(module, q.to(dev), k.to(dev), v.to(dev), None)
    ref = eager.forward(qn, kn, vn, None, True)
    assert (out.float().cpu() - ref.float()).abs().max().item() < 2e-2
    # right padding: sequence 0 has 150 tokens
    mask = torch.ones(b, s, dtype=torch.int64)
    mask[0, 150:] = 0
    out, _ = flash_sparse_attention_forward(module, q.to(dev), k.to(dev), v.to(dev), mask.to(dev))
    ref0 = eager.forward(qn[:1, :150], kn[:1, :150], vn[:1, :150], None, True)
    assert (out[0, :150].float().cpu() - ref0[0].float()).abs().max().item() < 2e-2
    assert (out[0, 150:] == 0).all()
    assert (out[1].float().cpu() - ref[1].float()).abs().max().item() < 2e-2
    # packed row: two sequences of 120 and 80 tokens, sliding window 64
    pos = torch.cat([torch.arange(120), torch.arange(80)])[None]
    out, _ = flash_sparse_attention_forward(module, q[:1].to(dev), k[:1].to(dev), v[:1].to(dev), None,
                                            position_ids=pos.to(dev), window_size=64)
    ws = torch.tensor([[0, 0, 0, 64]] * hkv, dtype=torch.int32)
    for lo, hi in ((0, 120), (120, 200)):
        r = eager.forward(qn[:1, lo:hi], kn[:1, lo:hi], vn[:1, lo:hi], None, True, is_local=True, window_sizes=ws)
        assert (out[0, lo:hi].float().cpu() - r[0].float()).abs().max().item() < 2e-2
