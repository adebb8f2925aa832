"""Input contract of the operators, raised as AssertionError like the reference's
flash_sparse_attn/ops/triton/assert_inputs.py:6-318 (skipped when ``skip_checks=True``)."""

import torch

_FP8 = (torch.float8_e5m2, torch.float8_e4m3fn)
_F16 = (torch.float16, torch.bfloat16)


def _same_device(device, *tensors):
    for t in tensors:
        if t is not None:
            assert t.device == device, "All inputs must be on the same device"


def _int32(*tensors, what):
    for t in tensors:
        if t is not None:
            assert t.dtype == torch.int32, f"{what} must be int32"


def _check_qkv(query, key, value, query_scale, key_scale, value_scale, num_heads_q, num_heads_kv, head_dim, is_quant,
               device):
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
                      is_quant=False, device=None):
    _check_qkv(query, key, value, query_scale, key_scale, value_scale, num_heads_q, num_heads_kv, head_dim, is_quant,
               device)
    if page_size is not None:
        assert page_size in (32, 64, 128, 256), "paged KV page_size must be one of 32, 64, 128, or 256"
    _same_device(device, alpha, delta, cu_seqlens_q, cu_seqlens_k, seqused_q, seqused_k)
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
    assert dout.dtype in _F16, "dout dtype must be float16 or bfloat16"
    assert lse.dtype == torch.float32, "lse must be float32"
    _int32(cu_seqlens_q, cu_seqlens_k, what="cu_seqlens_q and cu_seqlens_k")
    _int32(seqused_q, seqused_k, what="seqused_q and seqused_k")
    _check_windows(window_sizes)


def assert_dec_inputs(query, key, value, query_scale=None, key_scale=None, value_scale=None, window_sizes=None,
                      alpha=None, delta=None, cu_seqlens_k=None, seqused_k=None, page_table=None,
                      gather_kv_indices=None, num_heads_q=None, num_heads_kv=None, head_dim=None, page_size=None,
                      is_quant=False, device=None):
    _check_qkv(query, key, value, query_scale, key_scale, value_scale, num_heads_q, num_heads_kv, head_dim, is_quant,
               device)
    if page_size is not None:
        assert page_size in (32, 64, 128, 256), "paged KV page_size must be one of 32, 64, 128, or 256"
    _same_device(device, alpha, delta, cu_seqlens_k, seqused_k, page_table, gather_kv_indices)
    _int32(cu_seqlens_k, what="cu_seqlens_k")
    _int32(seqused_k, what="seqused_k")
    _int32(page_table, what="page_table")
    _int32(gather_kv_indices, what="gather_kv_indices")
    _check_windows(window_sizes)
