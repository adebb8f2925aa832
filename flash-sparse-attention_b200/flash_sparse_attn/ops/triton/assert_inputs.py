"""Input contract of the operators, raised as AssertionError like the reference's
flash_sparse_attn/ops/triton/assert_inputs.py:6-318 (skipped when ``skip_checks=True``).

Same checks and messages as the reference, with three differences: head sizes above 256 - above 128 in the
backward pass and with FP8 inputs - are refused here (the reference admits up to 512), a page table may be
combined with gather_kv_indices (the reference rejects that, :303-305; here the gathered position goes through
the page table), and the shapes of the gate vectors, of caller-provided out / lse buffers and of the page table
are checked as well, because the kernels take their strides on trust."""

import torch

_FP8 = (torch.float8_e5m2, torch.float8_e4m3fn)
_F16 = (torch.float16, torch.bfloat16)
MAX_HEAD_DIM = 128
MAX_HEAD_DIM_WIDE = 256  # forward and decode with 16-bit inputs (FP8: head size 128); the backward stops at 128


def _same_device(device, *tensors):
    for t in tensors:
        if t is not None:
            assert t.device == device, "All inputs must be on the same device"


def _int32(*tensors, what):
    for t in tensors:
        if t is not None:
            assert t.dtype == torch.int32, f"{what} must be int32"


def _check_qkv(query, key, value, query_scale, key_scale, value_scale, num_heads_q, num_heads_kv, head_dim, is_quant,
               device, max_head_dim=MAX_HEAD_DIM):
    _same_device(device, query, key, value)
    if is_quant:
        assert query.dtype in _FP8, "Input dtype must be float8_e5m2 or float8_e4m3fn"
        assert query_scale is not None and key_scale is not None and value_scale is not None, (
            "Scale tensors must be provided for quantized inputs"
        )
        assert query_scale.dtype in (torch.float16, torch.bfloat16, torch.float32), (
            "Scale tensors must be float16, bfloat16, or float32"
        )
        assert query_scale.dtype == key_scale.dtype == value_scale.dtype, "All scale tensors must have the same dtype"
        _same_device(device, query_scale, key_scale, value_scale)
    else:
        assert query.dtype in _F16, "Input dtype must be float16 or bfloat16"
    assert query.dtype == key.dtype == value.dtype, "All inputs must have the same dtype"
    assert num_heads_q % num_heads_kv == 0, "num_heads_q must be divisible by num_heads_kv"
    assert head_dim % 16 == 0, "head_dim must be a multiple of 16 for efficient memory access"
    assert head_dim <= 512, "head_dim must be less than or equal to 512 for efficient memory access"
    if is_quant:
        max_head_dim = min(max_head_dim, MAX_HEAD_DIM)
    assert head_dim <= max_head_dim, f"head_dim must be less than or equal to {max_head_dim} in this build"


def _check_paged(page_size, tile_mn, page_table=None, batch=None):
    if page_size is not None:
        assert page_size in (32, 64, 128, 256), "paged KV page_size must be one of 32, 64, 128, or 256"
        if tile_mn is not None:
            assert tile_mn[1] == page_size, "paged KV requires tile_mn[1] == page_size"
    if page_table is not None:
        assert page_table.ndim == 2 and page_table.stride(1) == 1, "page_table must be [batch, max_pages] with unit stride"
        if batch is not None:
            assert page_table.shape[0] == batch, "page_table must have one row per sequence"


def _check_gate(alpha, delta, alpha_shape=None, delta_shape=None):
    """alpha / delta as the launchers receive them: position-contiguous [.., heads, positions]."""
    if alpha is None and delta is None:
        return
    assert alpha is not None and delta is not None, "alpha and delta must be given together"
    assert (alpha.shape[-1] == 1 or alpha.stride(-1) == 1) and (delta.shape[-1] == 1 or delta.stride(-1) == 1), (
        "alpha and delta must be contiguous along positions")
    if alpha_shape is not None:
        assert tuple(alpha.shape) == tuple(alpha_shape), f"alpha must have shape {tuple(alpha_shape)}"
    if delta_shape is not None:
        assert tuple(delta.shape) == tuple(delta_shape), f"delta must have shape {tuple(delta_shape)}"


def check_out_buffers(out, lse, out_shape, out_dtype, lse_shape):
    """Caller-provided result buffers (written in place and returned by identity)."""
    if out is not None:
        assert tuple(out.shape) == tuple(out_shape) and out.dtype == out_dtype, (
            f"out must have shape {tuple(out_shape)} and dtype {out_dtype}")
        assert out.shape[-1] == 1 or out.stride(-1) == 1, "out must be contiguous along head_dim"
    if lse is not None:
        assert tuple(lse.shape) == tuple(lse_shape) and lse.dtype == torch.float32, (
            f"lse must have shape {tuple(lse_shape)} and dtype float32")
        assert lse.shape[-1] == 1 or lse.stride(-1) == 1, "lse must be contiguous along its last dimension"


def _check_windows(window_sizes):
    if window_sizes is not None:
        assert window_sizes.dtype == torch.int32, "window_sizes must be int32"
        assert window_sizes.ndim == 2 and window_sizes.shape[1] == 4, (
            "window_sizes must have shape [num_kv_heads, 4] with columns "
            "[window_sink, window_left, window_right, window_near]"
        )


def assert_fwd_inputs(query, key, value, query_scale=None, key_scale=None, value_scale=None, window_sizes=None,
                      alpha=None, delta=None, cu_seqlens_q=None, cu_seqlens_k=None, seqused_q=None, seqused_k=None,
                      num_heads_q=None, num_heads_kv=None, head_dim=None, page_size=None, tile_mn=None,
                      is_quant=False, device=None, page_table=None):
    _check_qkv(query, key, value, query_scale, key_scale, value_scale, num_heads_q, num_heads_kv, head_dim, is_quant,
               device, max_head_dim=MAX_HEAD_DIM_WIDE)
    _check_paged(page_size, tile_mn, page_table, query.shape[0] if cu_seqlens_q is None else None)
    _check_gate(alpha, delta)
    _same_device(device, alpha, delta, cu_seqlens_q, cu_seqlens_k, seqused_q, seqused_k, page_table)
    _int32(page_table, what="page_table")
    _int32(cu_seqlens_q, cu_seqlens_k, what="cu_seqlens_q and cu_seqlens_k")
    _int32(seqused_q, seqused_k, what="seqused_q and seqused_k")
    _check_windows(window_sizes)


def assert_bwd_inputs(query, key, value, out, dout, lse, query_scale=None, key_scale=None, value_scale=None,
                      window_sizes=None, alpha=None, delta=None, cu_seqlens_q=None, cu_seqlens_k=None,
                      seqused_q=None, seqused_k=None, num_heads_q=None, num_heads_kv=None, head_dim=None,
                      is_quant=False, device=None):
    _check_qkv(query, key, value, query_scale, key_scale, value_scale, num_heads_q, num_heads_kv, head_dim, is_quant,
               device)
    _same_device(device, out, dout, lse, alpha, delta, cu_seqlens_q, cu_seqlens_k, seqused_q, seqused_k)
    _check_gate(alpha, delta)
    assert dout.dtype in _F16, "dout dtype must be float16 or bfloat16"
    if not is_quant:
        assert query.dtype == out.dtype == dout.dtype, "All inputs must have the same dtype"
    assert out.shape == dout.shape, "out and dout must have the same shape"
    assert lse.dtype == torch.float32, "lse must be float32"
    _int32(cu_seqlens_q, cu_seqlens_k, what="cu_seqlens_q and cu_seqlens_k")
    _int32(seqused_q, seqused_k, what="seqused_q and seqused_k")
    _check_windows(window_sizes)


def assert_dec_inputs(query, key, value, query_scale=None, key_scale=None, value_scale=None, window_sizes=None,
                      alpha=None, delta=None, cu_seqlens_k=None, seqused_k=None, page_table=None,
                      gather_kv_indices=None, num_heads_q=None, num_heads_kv=None, head_dim=None, page_size=None,
                      is_quant=False, device=None, tile_mn=None):
    _check_qkv(query, key, value, query_scale, key_scale, value_scale, num_heads_q, num_heads_kv, head_dim, is_quant,
               device, max_head_dim=MAX_HEAD_DIM_WIDE)
    _check_paged(page_size, tile_mn, page_table, query.shape[0])
    _check_gate(alpha, delta)
    if gather_kv_indices is not None:
        assert gather_kv_indices.ndim == 2 and gather_kv_indices.shape[0] == query.shape[0], (
            "gather_kv_indices must be [batch, topk]")
    _same_device(device, alpha, delta, cu_seqlens_k, seqused_k, page_table, gather_kv_indices)
    _int32(cu_seqlens_k, what="cu_seqlens_k")
    _int32(seqused_k, what="seqused_k")
    _int32(page_table, what="page_table")
    _int32(gather_kv_indices, what="gather_kv_indices")
    _check_windows(window_sizes)
