"""Padded batch <-> packed tokens: the data format on either side of the varlen operators.

Same functions, argument order and return tuples as flash_sparse_attn/utils/padding.py:7-179 of the
reference (which the model integration calls to route right-padded batches to the ``*_varlen_func``
operators): a boolean / 0-1 ``attention_mask [batch, seqlen]`` selects the tokens that are kept, packed
tensors are ``[total_tokens, ...]`` with ``cu_seqlens`` int32 ``[batch + 1]``.
"""

import torch


def _lengths_to_cu(lengths: torch.Tensor) -> torch.Tensor:
    cu = torch.zeros(lengths.numel() + 1, dtype=torch.int32, device=lengths.device)
    cu[1:] = torch.cumsum(lengths, dim=0, dtype=torch.int32)
    return cu


def index_first_axis(tensor, indices):
    """Rows ``indices`` of ``tensor`` with its first two axes (batch, position) flattened into one."""
    return tensor.reshape(-1, *tensor.shape[2:])[indices]


def get_unpad_data(attention_mask):
    """(flat indices of the kept tokens, cu_seqlens int32 [batch + 1], longest sequence as a python int)."""
    lengths = attention_mask.sum(dim=-1, dtype=torch.int32)
    indices = torch.nonzero(attention_mask.flatten(), as_tuple=False).flatten()
    return indices, _lengths_to_cu(lengths), int(lengths.max().item())


def unpad_input(hidden_states, attention_mask, unused_mask=None):
    """Pack ``hidden_states [batch, seqlen, ...]``. Tokens of ``unused_mask`` are allocated in the packed
    layout as well (they count in ``cu_seqlens``) but not in the returned used lengths.
    Returns (packed, indices, cu_seqlens, max_seqlen, used_lengths int32 [batch])."""
    allocated = attention_mask if unused_mask is None else attention_mask + unused_mask
    indices, cu_seqlens, max_seqlen = get_unpad_data(allocated)
    used = attention_mask.sum(dim=-1, dtype=torch.int32)
    return index_first_axis(hidden_states, indices), indices, cu_seqlens, max_seqlen, used


def pad_input(hidden_states, indices, batch, seqlen):
    """Scatter packed rows back to ``[batch, seqlen, ...]``; positions that were not kept are zero."""
    out = hidden_states.new_zeros((batch * seqlen, *hidden_states.shape[1:]))
    out[indices] = hidden_states
    return out.view(batch, seqlen, *hidden_states.shape[1:])


def upad_input(query_layer, key_layer, value_layer, attention_mask, query_length, unpad_input_func):
    """Pack q, k, v of one attention call with a single pass over the mask. The mask describes the key
    positions; queries are the last ``query_length`` of them (all of them in prefill, one in decode).
    Returns (q, k, v, indices_q, (cu_seqlens_q, cu_seqlens_k), (max_seqlen_q, max_seqlen_k))."""
    indices_k, cu_k, max_k = get_unpad_data(attention_mask)
    mask_len = attention_mask.shape[-1]
    if key_layer.shape[1] > mask_len:  # a cache longer than the mask: only the described part is used
        key_layer, value_layer = key_layer[:, :mask_len], value_layer[:, :mask_len]
    batch, kv_len = key_layer.shape[0], key_layer.shape[1]
    key_layer = index_first_axis(key_layer, indices_k)
    value_layer = index_first_axis(value_layer, indices_k)
    if query_length == kv_len:
        query_layer, indices_q, cu_q, max_q = index_first_axis(query_layer, indices_k), indices_k, cu_k, max_k
    elif query_length == 1:
        cu_q = torch.arange(batch + 1, dtype=torch.int32, device=query_layer.device)
        indices_q, max_q = cu_q[:-1], 1
        query_layer = query_layer.squeeze(1)
    else:
        query_layer, indices_q, cu_q, max_q, *_ = unpad_input_func(query_layer, attention_mask[:, -query_length:])
    return query_layer, key_layer, value_layer, indices_q, (cu_q, cu_k), (max_q, max_k)
