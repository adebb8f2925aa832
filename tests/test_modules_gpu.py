"""The attention layer (projections -> gated operator -> output projection) against the same layer computed
with the eager oracle: outputs and the gradients of the input and of every projection weight."""

import pytest
import torch

from fixtures import assert_close
from oracle import eager


def _layer(hidden=256, heads=4, kv_heads=2, head_dim=64, seed=0):
    from flash_sparse_attn.modules.flash_sparse_attention import FlashSparseAttention, FlashSparseAttentionConfig

    torch.manual_seed(seed)
    cfg = FlashSparseAttentionConfig(hidden, heads, kv_heads, head_dim, softmax_threshold=-128.0, gate_threshold=-128.0)
    return FlashSparseAttention(cfg, layer_idx=3)


def test_layer_parameters_match_the_reference_names():
    layer = _layer()
    names = sorted(n for n, _ in layer.named_parameters())
    assert names == sorted(f"{p}_proj.weight" for p in "qkvado")
    assert layer.a_proj.weight.shape == (4, 256) and layer.d_proj.weight.shape == (2, 256)
    assert layer.scaling == 64**-0.5 and layer.is_causal and layer.layer_idx == 3


@pytest.mark.gpu
def test_layer_matches_eager():
    layer = _layer().to("cuda", torch.bfloat16)
    b, s = 2, 200
    x = (0.5 * torch.randn(b, s, 256, generator=torch.Generator().manual_seed(1))).to(torch.bfloat16)
    xg = x.cuda().requires_grad_(True)
    out, (k_states, v_states) = layer(xg)
    dy = torch.randn(b, s, 256, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
    out.backward(dy.cuda())
    torch.cuda.synchronize()
    assert k_states.shape == (b, s, 2, 64) and v_states.shape == (b, s, 2, 64)

    # the same layer on the CPU: bf16 projections (rounded like the GPU's), eager fp32 gated attention
    w = {n: p.detach().cpu().clone().requires_grad_(True) for n, p in layer.named_parameters()}
    xr = x.clone().requires_grad_(True)
    lin = lambda n: torch.nn.functional.linear(xr, w[n + "_proj.weight"])  # noqa: E731
    q = lin("q").view(b, s, 4, 64)
    k = lin("k").view(b, s, 2, 64)
    v = lin("v").view(b, s, 2, 64)
    o = eager.forward(q, k, v, softmax_scale=64**-0.5, is_causal=True, alpha=lin("a"), delta=lin("d"))
    ref = torch.nn.functional.linear(o.to(torch.bfloat16).view(b, s, -1), w["o_proj.weight"])
    ref.backward(dy)

    assert_close("layer-out", out, ref, rtol=3e-2, atol=3e-2)
    assert_close("layer-dx", xg.grad, xr.grad, rtol=3e-2, atol=3e-2)
    for n, p in layer.named_parameters():
        assert_close("layer-d" + n, p.grad, w[n].grad, rtol=3e-2, atol=3e-2)
