"""Glue between Hugging Face style attention modules and the attention operators.

Plays the role of flash_sparse_attn/integrations/modeling_flash_sparse_attention_utils.py:463-640 of the reference
(`_flash_sparse_attention_forward` and its helpers) with the same entry-point names and argument lists, so that a
model file written against the reference imports and calls it unchanged. Three routes, chosen like there:

  1. a 2-D padding mask [batch, key_len]: tokens are packed (utils.padding.upad_input), the packed operator runs,
     the result is scattered back (pad_input);
  2. packed sequences - either pre-computed cu_seq_lens_{q,k} / max_length_{q,k}, or position ids that restart
     inside a single flattened row (`_is_packed_sequence`) - go to the packed operator as they are;
  3. otherwise the batched operator.

Differences from the reference, on purpose: its route 3 still passes (attention_mask, attention_bias) positionally
to an operator that no longer has those parameters (lines 629-636 there; the call fails with the current operator
signature). Here route 3 calls the operator with keywords only; a dense 4-D mask or a bias tensor is refused with
an explanation, because the operators have no such inputs. `window_size` becomes a sliding window on every KV head
(`window_sizes` rows [0, 0, 0, window_size]) when the key length exceeds it; `softcap` and `s_aux` are refused when
set (no operator support); `deterministic` follows flash_sparse_attn.set_deterministic / FSA_DETERMINISTIC.
"""

import logging
from typing import Optional, TypedDict

import torch

logger = logging.getLogger(__name__)


class FlashSparseAttentionKwargs(TypedDict, total=False):
    """Optional packed-sequence arguments a model may pass through (same keys as the reference's TypedDict)."""

    cu_seq_lens_q: Optional[torch.LongTensor]
    cu_seq_lens_k: Optional[torch.LongTensor]
    max_length_q: Optional[int]
    max_length_k: Optional[int]


def lazy_import_flash_sparse_attention(implementation: Optional[str] = None, force_import: bool = False):
    """((batched op, packed op, pad_input, unpad_input, create_mask), kwargs builder) - the tuple the reference's
    function of this name returns. Nothing is lazy here: the package is importable or the call fails loudly."""
    from flash_sparse_attn import flash_sparse_attn_func, flash_sparse_attn_varlen_func
    from flash_sparse_attn.utils.padding import pad_input, unpad_input

    return (flash_sparse_attn_func, flash_sparse_attn_varlen_func, pad_input, unpad_input, None), \
        _process_flash_sparse_attention_kwargs


def _is_packed_sequence(position_ids, batch_size):
    """True when ONE flattened row holds several sequences: its position ids are not 0, 1, 2, ... from their minimum."""
    if position_ids is None:
        return False
    steps = torch.arange(position_ids.shape[1], device=position_ids.device) + position_ids.min()
    return bool(batch_size == 1 and (steps - position_ids).abs().sum().bool())


def prepare_fsa_kwargs_from_position_ids(position_ids):
    """((cu_seqlens_q, cu_seqlens_k), (max_q, max_k)) of a flattened row: a sequence starts wherever the id is 0."""
    flat = position_ids.reshape(-1)
    starts = (flat == 0).nonzero().reshape(-1).to(torch.int32)
    cu = torch.cat([starts, torch.tensor([flat.numel()], dtype=torch.int32, device=flat.device)])
    longest = int(cu.diff().max().item())
    return (cu, cu), (longest, longest)


def _prepare_from_posids(query, key, value, position_ids):
    flatten = lambda t: t.contiguous().view(-1, t.size(-2), t.size(-1))  # noqa: E731
    cu, longest = prepare_fsa_kwargs_from_position_ids(position_ids)
    return flatten(query), flatten(key), flatten(value), cu, longest


def fsa_peft_integration_check(q, k, v, bias, target_dtype=None):
    """fp32 activations (layer norms kept in fp32 by PEFT) are cast back to the model's 16-bit type."""
    if target_dtype is not None and q.dtype == torch.float32:
        logger.warning("Casting fp32 inputs back to %s for flash_sparse_attn compatibility.", target_dtype)
        q, k, v = q.to(target_dtype), k.to(target_dtype), v.to(target_dtype)
        bias = bias.to(target_dtype) if bias is not None else None
    return q, k, v, bias


def _process_flash_sparse_attention_kwargs(query_length, key_length, is_causal, softmax_scale=None, window_size=None,
                                           softcap=None, deterministic=None, s_aux=None, num_heads_kv=None,
                                           device=None, **kwargs):
    """Operator keywords for one call. A single query position is never causal (the operators say the same)."""
    if softcap is not None or s_aux is not None:
        raise ValueError("flash_sparse_attn operators have no softcap / s_aux inputs; use another attention backend")
    out = {"is_causal": bool(is_causal) and query_length != 1, "softmax_scale": softmax_scale}
    if window_size is not None and key_length > window_size:
        if num_heads_kv is None:
            raise ValueError("window_size needs the number of KV heads")
        ws = torch.zeros((num_heads_kv, 4), dtype=torch.int32, device=device)
        ws[:, 3] = int(window_size)  # (sink, left, right, near): the window_size most recent keys of every query
        out["window_sizes"] = ws
    return out


def _flash_sparse_attention_forward(query_states, key_states, value_states, attention_mask, attention_bias,
                                    query_length, key_length, is_causal, position_ids=None, softmax_scale=None,
                                    window_size=None, softcap=None, deterministic=None, cu_seq_lens_q=None,
                                    cu_seq_lens_k=None, max_length_q=None, max_length_k=None, target_dtype=None,
                                    implementation=None, **kwargs):
    """query [B, Sq, Hq, D], key / value [B, Sk, Hkv, D] -> attention output [B, Sq, Hq, D]."""
    if attention_mask is not None and attention_mask.dim() == 2 and attention_bias is not None:
        raise ValueError("If shape of attention_mask is (batch_size, seq_len), attention_bias has to be None.")
    (fsa_fn, fsa_varlen_fn, pad_fn, unpad_fn, _), make_kwargs = lazy_import_flash_sparse_attention(implementation)
    from flash_sparse_attn.utils.padding import upad_input

    query_states, key_states, value_states, attention_bias = fsa_peft_integration_check(
        query_states, key_states, value_states, attention_bias, target_dtype)
    flash_kwargs = make_kwargs(query_length=query_length, key_length=key_length, is_causal=is_causal,
                               softmax_scale=softmax_scale, window_size=window_size, softcap=softcap,
                               deterministic=deterministic, s_aux=kwargs.get("s_aux"),
                               num_heads_kv=key_states.shape[-2], device=query_states.device)
    batch = query_states.size(0)
    packed_by_ids = _is_packed_sequence(position_ids, batch_size=batch)
    packed_by_kwargs = all(x is not None for x in (cu_seq_lens_q, cu_seq_lens_k, max_length_q, max_length_k))

    def first(x):
        return x[0] if isinstance(x, tuple) else x

    if attention_mask is not None and attention_mask.dim() == 2:  # route 1: right- or left-padded batch
        q, k, v, indices_q, (cu_q, cu_k), (max_q, max_k) = upad_input(
            query_states, key_states, value_states, attention_mask, query_length, unpad_fn)
        out = first(fsa_varlen_fn(q, k, v, cu_seqlens_q=cu_q, cu_seqlens_k=cu_k, max_seqlen_q=max_q,
                                  max_seqlen_k=max_k, **flash_kwargs))
        return pad_fn(out, indices_q, batch, query_length)
    if packed_by_kwargs or packed_by_ids:  # route 2: sequences already flattened into one row
        if cu_seq_lens_q is None or cu_seq_lens_k is None:
            q, k, v, (cu_seq_lens_q, cu_seq_lens_k), (max_length_q, max_length_k) = _prepare_from_posids(
                query_states, key_states, value_states, position_ids)
        else:
            q, k, v = (t.reshape(-1, t.size(-2), t.size(-1)) for t in (query_states, key_states, value_states))
        out = first(fsa_varlen_fn(q, k, v, cu_seqlens_q=cu_seq_lens_q.to(torch.int32),
                                  cu_seqlens_k=cu_seq_lens_k.to(torch.int32), max_seqlen_q=int(max_length_q),
                                  max_seqlen_k=int(max_length_k), **flash_kwargs))
        return out.view(batch, -1, out.size(-2), out.size(-1))
    if attention_bias is not None or (attention_mask is not None and attention_mask.dim() > 2):  # route 3
        raise ValueError("flash_sparse_attn operators take no dense mask / bias tensor: pass a 2-D padding mask, "
                         "packed-sequence arguments, is_causal and window_size instead")
    return first(fsa_fn(query_states, key_states, value_states, **flash_kwargs))
