"""`flash_sparse_attention_forward`: the attention-interface function a Hugging Face model registers (same name,
arguments and return value as flash_sparse_attn/integrations/flash_sparse_attention.py:13-117 of the reference):
query / key / value arrive as [batch, heads, positions, head_dim] and leave as (output [batch, positions, heads,
head_dim], None)."""

import logging
from typing import Optional

import torch

from .modeling_flash_sparse_attention_utils import _flash_sparse_attention_forward

logger = logging.getLogger(__name__)


def flash_sparse_attention_forward(module: torch.nn.Module, query: torch.Tensor, key: torch.Tensor,
                                   value: torch.Tensor, attention_mask: Optional[torch.Tensor],
                                   attention_bias: Optional[torch.Tensor] = None, scaling: Optional[float] = None,
                                   window_size: Optional[int] = None, softcap: Optional[float] = None, **kwargs):
    if kwargs.get("output_attentions", False) or kwargs.get("head_mask") is not None:
        logger.warning("`flash_sparse_attention` supports neither `output_attentions=True` nor `head_mask`.")
    if any(dim == 0 for dim in query.shape):
        raise ValueError("flash_sparse_attention does not support inputs with a zero-sized dimension")
    query_len, key_len = query.shape[2], key.shape[2]
    query, key, value = query.transpose(1, 2), key.transpose(1, 2), value.transpose(1, 2)
    target_dtype = None
    if query.dtype == torch.float32:  # activations silently kept in fp32 (PEFT, autocast): find the model's type
        if torch.is_autocast_enabled():
            target_dtype = torch.get_autocast_gpu_dtype()
        elif hasattr(getattr(module, "config", None), "_pre_quantization_dtype"):
            target_dtype = module.config._pre_quantization_dtype
        else:
            target_dtype = next(m for m in module.modules() if isinstance(m, torch.nn.Linear)).weight.dtype
    is_causal = kwargs.pop("is_causal", None)
    if is_causal is None:
        is_causal = getattr(module, "is_causal", True)
    out = _flash_sparse_attention_forward(query, key, value, attention_mask, attention_bias, query_length=query_len,
                                          key_length=key_len, is_causal=is_causal, softmax_scale=scaling,
                                          softcap=softcap, window_size=window_size, target_dtype=target_dtype,
                                          implementation="flash_sparse_attn", **kwargs)
    return out, None
