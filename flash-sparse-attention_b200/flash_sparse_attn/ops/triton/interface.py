"""Operator API: the twelve ``flash_{dense,sparse,gated}_attn{,_varlen}{,_with_kvcache}_func``
entry points with the signatures, defaults and return conventions of the reference's
flash_sparse_attn/ops/triton/interface.py:935-2052, backed by the sm_100a kernels in
``libfsa_b200.so``.

Argument normalisation that the reference does in its autograd Functions is kept
(interface.py:317-436): a single query position disables causality, ``window_sizes`` implies
``is_local``, ``num_splits`` implies both split modes, ``is_quant`` without scales quantises the
inputs first, ``tile_mn`` is handed to the backward with its two entries swapped, and backward
returns ``None`` for every non-tensor argument.
"""

from typing import Optional, Tuple, Union

import torch

from flash_sparse_attn.ops.triton import quant
from flash_sparse_attn.ops.triton.flash_bwd import attn_backward
from flash_sparse_attn.ops.triton.flash_dec import attn_decode
from flash_sparse_attn.ops.triton.flash_fwd import attn_forward
from flash_sparse_attn.ops.triton.utils import ensure_contiguous

_Out = Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]
_NONES = (None,) * 30


def _normalise(single_query: bool, is_causal, window_sizes, is_local, num_splits, is_split_kv, is_split_qo):
    if single_query:
        is_causal = False
    if window_sizes is not None:
        is_local = True
    if num_splits is not None:
        is_split_kv = True
        is_split_qo = True
    return is_causal, is_local, is_split_kv, is_split_qo


def _maybe_quantize(is_quant, query, key, value, query_scale, key_scale, value_scale, cu_q=None, cu_k=None, max_q=None,
                    max_k=None, block_ok=True):
    if is_quant and (query_scale is None or key_scale is None or value_scale is None):
        if quant.block_scaled_enabled() and block_ok and query.shape[-1] == 128:
            # internal format (not in the reference): e4m3 with one scale per 128 positions and head
            query, query_scale = quant.quantize_fp8_blockwise(query, cu_seqlens=cu_q, max_seqlen=max_q)
            key, key_scale = quant.quantize_fp8_blockwise(key, cu_seqlens=cu_k, max_seqlen=max_k)
            value, value_scale = quant.quantize_fp8_blockwise(value, cu_seqlens=cu_k, max_seqlen=max_k)
            return query, key, value, query_scale, key_scale, value_scale
        query, query_scale = quant.quantize_fp8(query)
        key, key_scale = quant.quantize_fp8(key)
        value, value_scale = quant.quantize_fp8(value)
    return query, key, value, query_scale, key_scale, value_scale


def _swap(tile_mn):
    return (tile_mn[1], tile_mn[0]) if tile_mn is not None else None


class _AttnFunc(torch.autograd.Function):
    """Shared forward/backward for the batched and packed, dense / sparse / gated operators."""

    @staticmethod
    def forward(ctx, kind, varlen, query, key, value, alpha, delta, cu_seqlens_q, cu_seqlens_k, max_seqlen_q,
                max_seqlen_k, is_causal, softmax_scale, query_scale, key_scale, value_scale, window_sizes,
                softmax_threshold, gate_threshold, is_logsigmoid_gate, is_adapt_gate, is_local, is_quant,
                is_split_kv, is_split_qo, pack_gqa, num_splits, page_table, seqused_q, seqused_k, out, lse,
                is_autotune, tile_mn, skip_checks, return_lse):
        single = (max_seqlen_q == 1) if varlen else (query.shape[1] == 1)
        is_causal, is_local, is_split_kv, is_split_qo = _normalise(
            single, is_causal, window_sizes, is_local, num_splits, is_split_kv, is_split_qo
        )
        query, key, value, query_scale, key_scale, value_scale = _maybe_quantize(
            is_quant, query, key, value, query_scale, key_scale, value_scale, cu_seqlens_q, cu_seqlens_k,
            max_seqlen_q, max_seqlen_k, block_ok=(kind != "gated" and not pack_gqa and page_table is None)
        )
        if kind == "gated":
            # kernels read alpha as [.., heads, positions] rows, like the reference's transposed copies
            alpha = alpha.transpose(-2, -1).contiguous()
            delta = delta.transpose(-2, -1).contiguous()

        out, lse, softmax_scale, softmax_threshold, gate_threshold = attn_forward(
            kind, query, key, value, alpha=alpha, delta=delta, cu_seqlens_q=cu_seqlens_q,
            cu_seqlens_k=cu_seqlens_k, max_seqlen_q=max_seqlen_q, max_seqlen_k=max_seqlen_k, is_causal=is_causal,
            softmax_scale=softmax_scale, query_scale=query_scale, key_scale=key_scale, value_scale=value_scale,
            window_sizes=window_sizes, softmax_threshold=softmax_threshold, gate_threshold=gate_threshold,
            is_logsigmoid_gate=is_logsigmoid_gate, is_adapt_gate=is_adapt_gate, is_local=is_local,
            is_quant=is_quant, is_split_kv=is_split_kv, pack_gqa=pack_gqa, num_splits=num_splits,
            page_table=page_table, seqused_q=seqused_q, seqused_k=seqused_k, out=out, lse=lse,
            is_autotune=is_autotune, tile_mn=tile_mn, skip_checks=skip_checks,
        )

        ctx.save_for_backward(query, key, value, alpha, delta, out, lse, cu_seqlens_q, cu_seqlens_k, seqused_q,
                              seqused_k)
        ctx.kind, ctx.varlen = kind, varlen
        ctx.max_seqlen_q, ctx.max_seqlen_k = max_seqlen_q, max_seqlen_k
        ctx.is_causal = is_causal
        ctx.softmax_scale = softmax_scale
        ctx.query_scale, ctx.key_scale, ctx.value_scale = query_scale, key_scale, value_scale
        ctx.window_sizes = window_sizes
        ctx.softmax_threshold, ctx.gate_threshold = softmax_threshold, gate_threshold
        ctx.is_logsigmoid_gate, ctx.is_adapt_gate = is_logsigmoid_gate, is_adapt_gate
        ctx.is_local, ctx.is_quant, ctx.is_split_qo = is_local, is_quant, is_split_qo
        ctx.num_splits, ctx.is_autotune = num_splits, is_autotune
        ctx.tile_mn = _swap(tile_mn)
        ctx.skip_checks = skip_checks

        if return_lse:
            ctx.mark_non_differentiable(lse)  # no gradient flows through the log-sum-exp
            return out, lse
        return out

    @staticmethod
    def backward(ctx, dout, *args):
        (query, key, value, alpha, delta, out, lse, cu_seqlens_q, cu_seqlens_k, seqused_q,
         seqused_k) = ctx.saved_tensors
        grads = attn_backward(
            ctx.kind, query, key, value, out, dout.contiguous(), lse, alpha=alpha, delta=delta,
            cu_seqlens_q=cu_seqlens_q, cu_seqlens_k=cu_seqlens_k, max_seqlen_q=ctx.max_seqlen_q,
            max_seqlen_k=ctx.max_seqlen_k, is_causal=ctx.is_causal, softmax_scale=ctx.softmax_scale,
            query_scale=ctx.query_scale, key_scale=ctx.key_scale, value_scale=ctx.value_scale,
            window_sizes=ctx.window_sizes, softmax_threshold=ctx.softmax_threshold,
            gate_threshold=ctx.gate_threshold, is_logsigmoid_gate=ctx.is_logsigmoid_gate,
            is_adapt_gate=ctx.is_adapt_gate, is_local=ctx.is_local, is_quant=ctx.is_quant,
            seqused_q=seqused_q, seqused_k=seqused_k, is_split_qo=ctx.is_split_qo, num_splits=ctx.num_splits,
            is_autotune=ctx.is_autotune, tile_mn=ctx.tile_mn, skip_checks=ctx.skip_checks,
        )
        dq, dk, dv = grads[:3]
        da = dd = None
        if ctx.kind == "gated":
            da = grads[3].transpose(-2, -1).contiguous()
            dd = grads[4].transpose(-2, -1).contiguous()
        # (kind, varlen, q, k, v, alpha, delta, then 29 non-differentiable arguments)
        return (None, None, dq, dk, dv, da, dd) + (None,) * 29


def _contig(*ts):
    return tuple(t.contiguous() if isinstance(t, torch.Tensor) else t for t in ts)


def _apply(kind, varlen, query, key, value, alpha, delta, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
           is_causal, softmax_scale, query_scale, key_scale, value_scale, window_sizes, softmax_threshold,
           gate_threshold, is_logsigmoid_gate, is_adapt_gate, is_local, is_quant, is_split_kv, is_split_qo, pack_gqa,
           num_splits, page_table, seqused_q, seqused_k, out, lse, is_autotune, tile_mn, skip_checks, return_lse):
    (query, key, value, alpha, delta, cu_seqlens_q, cu_seqlens_k, query_scale, key_scale, value_scale, window_sizes,
     page_table, seqused_q, seqused_k, out, lse) = _contig(
        query, key, value, alpha, delta, cu_seqlens_q, cu_seqlens_k, query_scale, key_scale, value_scale,
        window_sizes, page_table, seqused_q, seqused_k, out, lse)
    return _AttnFunc.apply(kind, varlen, query, key, value, alpha, delta, cu_seqlens_q, cu_seqlens_k, max_seqlen_q,
                           max_seqlen_k, is_causal, softmax_scale, query_scale, key_scale, value_scale, window_sizes,
                           softmax_threshold, gate_threshold, is_logsigmoid_gate, is_adapt_gate, is_local, is_quant,
                           is_split_kv, is_split_qo, pack_gqa, num_splits, page_table, seqused_q, seqused_k, out,
                           lse, is_autotune, tile_mn, skip_checks, return_lse)


# ----------------------------------------------------------------------------------------------------
# dense
# ----------------------------------------------------------------------------------------------------
def flash_dense_attn_func(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    is_causal: bool = False,
    softmax_scale: Optional[float] = None,
    query_scale: Optional[torch.Tensor] = None,
    key_scale: Optional[torch.Tensor] = None,
    value_scale: Optional[torch.Tensor] = None,
    window_sizes: Optional[torch.Tensor] = None,
    is_local: bool = False,
    is_quant: bool = False,
    is_split_kv: bool = False,
    is_split_qo: bool = False,
    pack_gqa: bool = False,
    num_splits: Optional[int] = None,
    page_table: Optional[torch.Tensor] = None,
    seqused_k: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    lse: Optional[torch.Tensor] = None,
    is_autotune: bool = True,
    tile_mn: Optional[Tuple[int, int]] = None,
    skip_checks: bool = False,
    return_lse: bool = False,
) -> _Out:
    """Dense attention, ``query [B, Sq, Hq, D]``, ``key/value [B, Sk, Hkv, D]`` (or paged cache +
    ``page_table``). Returns ``out`` or ``(out, lse)``; same contract as the reference's
    flash_dense_attn_func (interface.py:935-1013)."""
    return _apply("dense", False, query, key, value, None, None, None, None, None, None, is_causal, softmax_scale,
                  query_scale, key_scale, value_scale, window_sizes, None, None, True, True, is_local, is_quant,
                  is_split_kv, is_split_qo, pack_gqa, num_splits, page_table, None, seqused_k, out, lse, is_autotune,
                  tile_mn, skip_checks, return_lse)


def flash_dense_attn_varlen_func(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    cu_seqlens_k: torch.Tensor,
    max_seqlen_q: int,
    max_seqlen_k: int,
    is_causal: bool = False,
    softmax_scale: Optional[float] = None,
    query_scale: Optional[torch.Tensor] = None,
    key_scale: Optional[torch.Tensor] = None,
    value_scale: Optional[torch.Tensor] = None,
    window_sizes: Optional[torch.Tensor] = None,
    is_local: bool = False,
    is_quant: bool = False,
    is_split_kv: bool = False,
    is_split_qo: bool = False,
    pack_gqa: bool = False,
    num_splits: Optional[int] = None,
    seqused_q: Optional[torch.Tensor] = None,
    seqused_k: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    lse: Optional[torch.Tensor] = None,
    is_autotune: bool = True,
    tile_mn: Optional[Tuple[int, int]] = None,
    skip_checks: bool = False,
    return_lse: bool = False,
) -> _Out:
    """Dense attention over packed sequences: ``query [Tq, Hq, D]``, ``key/value [Tk, Hkv, D]``,
    int32 ``cu_seqlens_{q,k} [B + 1]``; ``lse`` is ``[Hq, Tq]``."""
    return _apply("dense", True, query, key, value, None, None, cu_seqlens_q, cu_seqlens_k, max_seqlen_q,
                  max_seqlen_k, is_causal, softmax_scale, query_scale, key_scale, value_scale, window_sizes, None,
                  None, True, True, is_local, is_quant, is_split_kv, is_split_qo, pack_gqa, num_splits, None,
                  seqused_q, seqused_k, out, lse, is_autotune, tile_mn, skip_checks, return_lse)


# ----------------------------------------------------------------------------------------------------
# sparse (softmax-threshold tile skipping)
# ----------------------------------------------------------------------------------------------------
def flash_sparse_attn_func(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    is_causal: bool = False,
    softmax_scale: Optional[float] = None,
    query_scale: Optional[torch.Tensor] = None,
    key_scale: Optional[torch.Tensor] = None,
    value_scale: Optional[torch.Tensor] = None,
    window_sizes: Optional[torch.Tensor] = None,
    softmax_threshold: Optional[float] = None,
    is_local: bool = False,
    is_quant: bool = False,
    is_split_kv: bool = False,
    is_split_qo: bool = False,
    pack_gqa: bool = False,
    num_splits: Optional[int] = None,
    page_table: Optional[torch.Tensor] = None,
    seqused_k: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    lse: Optional[torch.Tensor] = None,
    is_autotune: bool = True,
    tile_mn: Optional[Tuple[int, int]] = None,
    skip_checks: bool = False,
    return_lse: bool = False,
) -> _Out:
    """Sparse attention: like the dense operator, plus skipping of key tiles whose largest
    estimated probability stays below ``softmax_threshold`` times the uniform weight
    (default 1.0; ``<= 0`` disables skipping). Reference: interface.py:1280-1361."""
    return _apply("sparse", False, query, key, value, None, None, None, None, None, None, is_causal, softmax_scale,
                  query_scale, key_scale, value_scale, window_sizes, softmax_threshold, None, True, True, is_local,
                  is_quant, is_split_kv, is_split_qo, pack_gqa, num_splits, page_table, None, seqused_k, out, lse,
                  is_autotune, tile_mn, skip_checks, return_lse)


def flash_sparse_attn_varlen_func(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    cu_seqlens_k: torch.Tensor,
    max_seqlen_q: int,
    max_seqlen_k: int,
    is_causal: bool = False,
    softmax_scale: Optional[float] = None,
    query_scale: Optional[torch.Tensor] = None,
    key_scale: Optional[torch.Tensor] = None,
    value_scale: Optional[torch.Tensor] = None,
    window_sizes: Optional[torch.Tensor] = None,
    softmax_threshold: Optional[float] = None,
    is_local: bool = False,
    is_quant: bool = False,
    is_split_kv: bool = False,
    is_split_qo: bool = False,
    pack_gqa: bool = False,
    num_splits: Optional[int] = None,
    seqused_q: Optional[torch.Tensor] = None,
    seqused_k: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    lse: Optional[torch.Tensor] = None,
    is_autotune: bool = True,
    tile_mn: Optional[Tuple[int, int]] = None,
    skip_checks: bool = False,
    return_lse: bool = False,
) -> _Out:
    """Packed-sequence form of :func:`flash_sparse_attn_func` (reference: interface.py:1451-1544)."""
    return _apply("sparse", True, query, key, value, None, None, cu_seqlens_q, cu_seqlens_k, max_seqlen_q,
                  max_seqlen_k, is_causal, softmax_scale, query_scale, key_scale, value_scale, window_sizes,
                  softmax_threshold, None, True, True, is_local, is_quant, is_split_kv, is_split_qo, pack_gqa,
                  num_splits, None, seqused_q, seqused_k, out, lse, is_autotune, tile_mn, skip_checks, return_lse)


# ----------------------------------------------------------------------------------------------------
# gated (additive gate g(alpha_i * delta_j) + gate-bound tile skipping)
# ----------------------------------------------------------------------------------------------------
def flash_gated_attn_func(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    alpha: torch.Tensor,
    delta: torch.Tensor,
    is_causal: bool = False,
    softmax_scale: Optional[float] = None,
    query_scale: Optional[torch.Tensor] = None,
    key_scale: Optional[torch.Tensor] = None,
    value_scale: Optional[torch.Tensor] = None,
    window_sizes: Optional[torch.Tensor] = None,
    softmax_threshold: Optional[float] = None,
    gate_threshold: Optional[float] = None,
    is_logsigmoid_gate: bool = True,
    is_adapt_gate: bool = True,
    is_local: bool = False,
    is_quant: bool = False,
    is_split_kv: bool = False,
    is_split_qo: bool = False,
    pack_gqa: bool = False,
    num_splits: Optional[int] = None,
    page_table: Optional[torch.Tensor] = None,
    seqused_k: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    lse: Optional[torch.Tensor] = None,
    is_autotune: bool = True,
    tile_mn: Optional[Tuple[int, int]] = None,
    skip_checks: bool = False,
    return_lse: bool = False,
) -> _Out:
    """Gated attention: logits ``(q.k + g(alpha_i * delta_j)) * scale`` with ``alpha [B, Sq, Hq]``,
    ``delta [B, Sk, Hkv]`` and ``g`` = logsigmoid (default) or identity. Reference:
    interface.py:1638-1734."""
    return _apply("gated", False, query, key, value, alpha, delta, None, None, None, None, is_causal, softmax_scale,
                  query_scale, key_scale, value_scale, window_sizes, softmax_threshold, gate_threshold,
                  is_logsigmoid_gate, is_adapt_gate, is_local, is_quant, is_split_kv, is_split_qo, pack_gqa,
                  num_splits, page_table, None, seqused_k, out, lse, is_autotune, tile_mn, skip_checks, return_lse)


def flash_gated_attn_varlen_func(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    alpha: torch.Tensor,
    delta: torch.Tensor,
    cu_seqlens_q: torch.Tensor,
    cu_seqlens_k: torch.Tensor,
    max_seqlen_q: int,
    max_seqlen_k: int,
    is_causal: bool = False,
    softmax_scale: Optional[float] = None,
    query_scale: Optional[torch.Tensor] = None,
    key_scale: Optional[torch.Tensor] = None,
    value_scale: Optional[torch.Tensor] = None,
    window_sizes: Optional[torch.Tensor] = None,
    softmax_threshold: Optional[float] = None,
    gate_threshold: Optional[float] = None,
    is_logsigmoid_gate: bool = True,
    is_adapt_gate: bool = True,
    is_local: bool = False,
    is_quant: bool = False,
    is_split_kv: bool = False,
    is_split_qo: bool = False,
    pack_gqa: bool = False,
    num_splits: Optional[int] = None,
    seqused_q: Optional[torch.Tensor] = None,
    seqused_k: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    lse: Optional[torch.Tensor] = None,
    is_autotune: bool = True,
    tile_mn: Optional[Tuple[int, int]] = None,
    skip_checks: bool = False,
    return_lse: bool = False,
) -> _Out:
    """Packed-sequence form of :func:`flash_gated_attn_func` (``alpha [Tq, Hq]``, ``delta [Tk, Hkv]``)."""
    return _apply("gated", True, query, key, value, alpha, delta, cu_seqlens_q, cu_seqlens_k, max_seqlen_q,
                  max_seqlen_k, is_causal, softmax_scale, query_scale, key_scale, value_scale, window_sizes,
                  softmax_threshold, gate_threshold, is_logsigmoid_gate, is_adapt_gate, is_local, is_quant,
                  is_split_kv, is_split_qo, pack_gqa, num_splits, None, seqused_q, seqused_k, out, lse, is_autotune,
                  tile_mn, skip_checks, return_lse)


# ----------------------------------------------------------------------------------------------------
# decode (one query position per sequence against a KV cache; no autograd)
# ----------------------------------------------------------------------------------------------------
def _decode(kind, query, key, value, alpha, delta, cu_seqlens_k, max_seqlen_k, softmax_scale, query_scale, key_scale,
            value_scale, window_sizes, softmax_threshold, gate_threshold, is_logsigmoid_gate, is_local, is_quant,
            num_splits, page_table, gather_kv_indices, seqused_k, out, lse, is_autotune, tile_mn, skip_checks,
            return_lse):
    query, key, value, query_scale, key_scale, value_scale = _maybe_quantize(
        is_quant, query, key, value, query_scale, key_scale, value_scale, block_ok=False  # decode: per tensor only
    )
    if window_sizes is not None:
        is_local = True
    if kind == "gated":
        delta = delta.transpose(-2, -1).contiguous()
    out, lse = attn_decode(
        kind, query, key, value, alpha=alpha, delta=delta, cu_seqlens_k=cu_seqlens_k, max_seqlen_k=max_seqlen_k,
        softmax_scale=softmax_scale, query_scale=query_scale, key_scale=key_scale, value_scale=value_scale,
        window_sizes=window_sizes, softmax_threshold=softmax_threshold, gate_threshold=gate_threshold,
        is_logsigmoid_gate=is_logsigmoid_gate, is_local=is_local, is_quant=is_quant, num_splits=num_splits,
        page_table=page_table, gather_kv_indices=gather_kv_indices, seqused_k=seqused_k, out=out, lse=lse,
        is_autotune=is_autotune, tile_mn=tile_mn, skip_checks=skip_checks,
    )
    return (out, lse) if return_lse else out


def flash_dense_attn_with_kvcache_func(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    softmax_scale: Optional[float] = None,
    query_scale: Optional[torch.Tensor] = None,
    key_scale: Optional[torch.Tensor] = None,
    value_scale: Optional[torch.Tensor] = None,
    window_sizes: Optional[torch.Tensor] = None,
    is_local: bool = False,
    is_quant: bool = False,
    num_splits: Optional[int] = None,
    page_table: Optional[torch.Tensor] = None,
    gather_kv_indices: Optional[torch.Tensor] = None,
    seqused_k: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    lse: Optional[torch.Tensor] = None,
    is_autotune: bool = True,
    tile_mn: Optional[Tuple[int, int]] = None,
    skip_checks: bool = False,
    return_lse: bool = False,
) -> _Out:
    """Dense decode: ``query [B, Hq, D]`` against ``key/value [B, Sk, Hkv, D]``, a paged cache
    ``[num_pages, page, Hkv, D]`` + ``page_table [B, max_pages]``, and/or ``gather_kv_indices
    [B, topk]`` (logical positions, negative = masked)."""
    return _decode("dense", query, key, value, None, None, None, None, softmax_scale, query_scale, key_scale,
                   value_scale, window_sizes, None, None, True, is_local, is_quant, num_splits, page_table,
                   gather_kv_indices, seqused_k, out, lse, is_autotune, tile_mn, skip_checks, return_lse)


def flash_dense_attn_varlen_with_kvcache_func(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    cu_seqlens_k: torch.Tensor,
    max_seqlen_k: int,
    softmax_scale: Optional[float] = None,
    query_scale: Optional[torch.Tensor] = None,
    key_scale: Optional[torch.Tensor] = None,
    value_scale: Optional[torch.Tensor] = None,
    window_sizes: Optional[torch.Tensor] = None,
    is_local: bool = False,
    is_quant: bool = False,
    seqused_k: Optional[torch.Tensor] = None,
    gather_kv_indices: Optional[torch.Tensor] = None,
    num_splits: Optional[int] = None,
    out: Optional[torch.Tensor] = None,
    lse: Optional[torch.Tensor] = None,
    is_autotune: bool = True,
    tile_mn: Optional[Tuple[int, int]] = None,
    skip_checks: bool = False,
    return_lse: bool = False,
) -> _Out:
    """Dense decode against packed keys/values ``[Tk, Hkv, D]`` addressed by ``cu_seqlens_k``."""
    return _decode("dense", query, key, value, None, None, cu_seqlens_k, max_seqlen_k, softmax_scale, query_scale,
                   key_scale, value_scale, window_sizes, None, None, True, is_local, is_quant, num_splits, None,
                   gather_kv_indices, seqused_k, out, lse, is_autotune, tile_mn, skip_checks, return_lse)


def flash_sparse_attn_with_kvcache_func(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    softmax_scale: Optional[float] = None,
    query_scale: Optional[torch.Tensor] = None,
    key_scale: Optional[torch.Tensor] = None,
    value_scale: Optional[torch.Tensor] = None,
    window_sizes: Optional[torch.Tensor] = None,
    softmax_threshold: Optional[float] = None,
    is_local: bool = False,
    is_quant: bool = False,
    num_splits: Optional[int] = None,
    page_table: Optional[torch.Tensor] = None,
    gather_kv_indices: Optional[torch.Tensor] = None,
    seqused_k: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    lse: Optional[torch.Tensor] = None,
    is_autotune: bool = True,
    tile_mn: Optional[Tuple[int, int]] = None,
    skip_checks: bool = False,
    return_lse: bool = False,
) -> _Out:
    """Sparse decode (reference: interface.py:1364-1448). Unlike the reference, a paged cache and
    ``gather_kv_indices`` may be combined: each index is a logical position that is translated
    through the page table."""
    return _decode("sparse", query, key, value, None, None, None, None, softmax_scale, query_scale, key_scale,
                   value_scale, window_sizes, softmax_threshold, None, True, is_local, is_quant, num_splits,
                   page_table, gather_kv_indices, seqused_k, out, lse, is_autotune, tile_mn, skip_checks, return_lse)


def flash_sparse_attn_varlen_with_kvcache_func(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    cu_seqlens_k: torch.Tensor,
    max_seqlen_k: int,
    softmax_scale: Optional[float] = None,
    query_scale: Optional[torch.Tensor] = None,
    key_scale: Optional[torch.Tensor] = None,
    value_scale: Optional[torch.Tensor] = None,
    window_sizes: Optional[torch.Tensor] = None,
    softmax_threshold: Optional[float] = None,
    is_local: bool = False,
    is_quant: bool = False,
    seqused_k: Optional[torch.Tensor] = None,
    gather_kv_indices: Optional[torch.Tensor] = None,
    num_splits: Optional[int] = None,
    out: Optional[torch.Tensor] = None,
    lse: Optional[torch.Tensor] = None,
    is_autotune: bool = True,
    tile_mn: Optional[Tuple[int, int]] = None,
    skip_checks: bool = False,
    return_lse: bool = False,
) -> _Out:
    """Sparse decode against packed keys/values (reference: interface.py:1547-1635)."""
    return _decode("sparse", query, key, value, None, None, cu_seqlens_k, max_seqlen_k, softmax_scale, query_scale,
                   key_scale, value_scale, window_sizes, softmax_threshold, None, True, is_local, is_quant,
                   num_splits, None, gather_kv_indices, seqused_k, out, lse, is_autotune, tile_mn, skip_checks,
                   return_lse)


def flash_gated_attn_with_kvcache_func(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    alpha: torch.Tensor,
    delta: torch.Tensor,
    softmax_scale: Optional[float] = None,
    query_scale: Optional[torch.Tensor] = None,
    key_scale: Optional[torch.Tensor] = None,
    value_scale: Optional[torch.Tensor] = None,
    window_sizes: Optional[torch.Tensor] = None,
    softmax_threshold: Optional[float] = None,
    gate_threshold: Optional[float] = None,
    is_logsigmoid_gate: bool = True,
    is_local: bool = False,
    is_quant: bool = False,
    num_splits: Optional[int] = None,
    page_table: Optional[torch.Tensor] = None,
    gather_kv_indices: Optional[torch.Tensor] = None,
    seqused_k: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    lse: Optional[torch.Tensor] = None,
    is_autotune: bool = True,
    tile_mn: Optional[Tuple[int, int]] = None,
    skip_checks: bool = False,
    return_lse: bool = False,
) -> _Out:
    """Gated decode: ``alpha [B, Hq]``, ``delta [B, Sk, Hkv]``."""
    return _decode("gated", query, key, value, alpha, delta, None, None, softmax_scale, query_scale, key_scale,
                   value_scale, window_sizes, softmax_threshold, gate_threshold, is_logsigmoid_gate, is_local,
                   is_quant, num_splits, page_table, gather_kv_indices, seqused_k, out, lse, is_autotune, tile_mn,
                   skip_checks, return_lse)


def flash_gated_attn_varlen_with_kvcache_func(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    alpha: torch.Tensor,
    delta: torch.Tensor,
    cu_seqlens_k: torch.Tensor,
    max_seqlen_k: int,
    softmax_scale: Optional[float] = None,
    query_scale: Optional[torch.Tensor] = None,
    key_scale: Optional[torch.Tensor] = None,
    value_scale: Optional[torch.Tensor] = None,
    window_sizes: Optional[torch.Tensor] = None,
    softmax_threshold: Optional[float] = None,
    gate_threshold: Optional[float] = None,
    is_logsigmoid_gate: bool = True,
    is_local: bool = False,
    is_quant: bool = False,
    seqused_k: Optional[torch.Tensor] = None,
    gather_kv_indices: Optional[torch.Tensor] = None,
    num_splits: Optional[int] = None,
    out: Optional[torch.Tensor] = None,
    lse: Optional[torch.Tensor] = None,
    is_autotune: bool = True,
    tile_mn: Optional[Tuple[int, int]] = None,
    skip_checks: bool = False,
    return_lse: bool = False,
) -> _Out:
    """Gated decode against packed keys/values (``delta [Tk, Hkv]``)."""
    return _decode("gated", query, key, value, alpha, delta, cu_seqlens_k, max_seqlen_k, softmax_scale, query_scale,
                   key_scale, value_scale, window_sizes, softmax_threshold, gate_threshold, is_logsigmoid_gate,
                   is_local, is_quant, num_splits, None, gather_kv_indices, seqused_k, out, lse, is_autotune,
                   tile_mn, skip_checks, return_lse)


# ----------------------------------------------------------------------------------------------------
# the reference's autograd Function names (interface.py:45, :163, :317, :439, :597, :745 there): callers that use
# `FlashSparseAttnFunc.apply(q, k, v, is_causal, ...)` with the positional list of the matching *_func keep working
# ----------------------------------------------------------------------------------------------------
class _FunctionAlias:
    """`apply(*positional)` forwards to the operator, which takes the same positional list and runs the one shared
    autograd Function of this module."""

    def __init__(self, name, fn):
        self.__name__ = name
        self._fn = fn

    def apply(self, *args, **kwargs):
        return self._fn(*args, **kwargs)

    __call__ = apply


FlashDenseAttnFunc = _FunctionAlias("FlashDenseAttnFunc", flash_dense_attn_func)
FlashDenseAttnVarlenFunc = _FunctionAlias("FlashDenseAttnVarlenFunc", flash_dense_attn_varlen_func)
FlashSparseAttnFunc = _FunctionAlias("FlashSparseAttnFunc", flash_sparse_attn_func)
FlashSparseAttnVarlenFunc = _FunctionAlias("FlashSparseAttnVarlenFunc", flash_sparse_attn_varlen_func)
FlashGatedAttnFunc = _FunctionAlias("FlashGatedAttnFunc", flash_gated_attn_func)
FlashGatedAttnVarlenFunc = _FunctionAlias("FlashGatedAttnVarlenFunc", flash_gated_attn_varlen_func)
