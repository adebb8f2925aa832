"""Per-tensor FP8 quantisation with the contract of flash_sparse_attn/ops/triton/quant.py:42-64, and the
widening cast the quantised operators use on their inputs. Both run as CUDA kernels of the library
(``fsa_quantize_fp8``: absolute maximum, then scaled cast; ``fsa_fp8_widen``), without host
synchronisation.

Block-scaled FP8 (``quantize_fp8_blockwise`` / ``dequantize_fp8_blockwise``, ``set_block_scaled``) is an internal
format that the reference does not have: one fp32 scale per (sequence, head, block of 128 positions) instead of one
per tensor, so an outlier only costs its own block its resolution. The forward kernels take the scales per tile
(``query_scale`` / ``key_scale`` / ``value_scale`` with more than one element select this path); the backward runs on
the de-quantised tensors like the per-tensor path."""

import ctypes

from typing import Optional

import torch

from flash_sparse_attn import _lib

_FP8 = (torch.float8_e5m2, torch.float8_e4m3fn)


def quantize_fp8(x: torch.Tensor, dtype: torch.dtype = torch.float8_e5m2):
    """Returns ``(x_fp8, scale)`` with ``x_fp8 = (x * FP8_MAX / amax).to(dtype)`` and
    ``scale = amax / FP8_MAX`` as a one-element tensor of ``x.dtype`` (so ``x ~ x_fp8 * scale``)."""
    assert x.is_cuda and x.dtype in (torch.float16, torch.bfloat16, torch.float32)
    assert dtype in _FP8
    xc = x.contiguous()
    x_fp8 = torch.empty_like(xc, dtype=dtype)
    scale = torch.empty(1, dtype=x.dtype, device=x.device)
    amax = torch.empty(1, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.load().fsa_quantize_fp8(xc.data_ptr(), x_fp8.data_ptr(), scale.data_ptr(), amax.data_ptr(),
                                          xc.numel(), _lib.dtype_code(x.dtype), _lib.dtype_code(dtype),
                                          _lib.current_stream_ptr(x.device))
    _lib.check(rc, "fsa_quantize_fp8")
    return x_fp8, scale


def widen_fp8(x: torch.Tensor, dtype: torch.dtype = torch.bfloat16, scale: Optional[torch.Tensor] = None):
    """``(x.float() * scale).to(dtype)`` for an FP8 tensor; with ``scale=None`` the values are kept as
    they are (exact in bf16 and fp16)."""
    assert x.is_cuda and x.dtype in _FP8 and dtype in (torch.bfloat16, torch.float16)
    xc = x.contiguous()
    out = torch.empty_like(xc, dtype=dtype)
    if scale is not None:
        scale = scale.reshape(-1)[:1].to(dtype)
    with torch.cuda.device(x.device):
        rc = _lib.load().fsa_fp8_widen(xc.data_ptr(), out.data_ptr(), _lib.ptr(scale), xc.numel(),
                                       _lib.dtype_code(x.dtype), _lib.dtype_code(dtype),
                                       _lib.current_stream_ptr(x.device))
    _lib.check(rc, "fsa_fp8_widen")
    return out


def scales_f32(query_scale, key_scale, value_scale, device):
    """The three per-tensor scales as one fp32 device tensor (what the kernels read)."""
    return torch.stack([torch.as_tensor(t, device=device).reshape(-1)[0].float()
                        for t in (query_scale, key_scale, value_scale)])


_block_scaled = False


def set_block_scaled(enabled: bool = True):
    """With this switch on, ``is_quant=True`` without scales quantises q, k, v to block-scaled e4m3 (scales per 128
    positions and head) instead of the reference's per-tensor e5m2. Off by default: the operators then behave like
    the reference's."""
    global _block_scaled
    _block_scaled = bool(enabled)


def block_scaled_enabled() -> bool:
    return _block_scaled


def is_block_scale(scale) -> bool:
    return isinstance(scale, torch.Tensor) and scale.numel() > 1


def _block_args(x16, x8, scales, cu_seqlens, max_seqlen, dequantize):
    a = _lib.FsaBlockQuantArgs()
    a.x16, a.x8, a.scales = x16.data_ptr(), x8.data_ptr(), scales.data_ptr()
    a.cu_seqlens = _lib.ptr(cu_seqlens)
    if cu_seqlens is None:
        a.batch, a.seqlen, a.heads, a.head_dim = x16.shape
        a.x_stride_b, a.x_stride_s, a.x_stride_h = x16.stride(0), x16.stride(1), x16.stride(2)
        a.q_stride_b, a.q_stride_s, a.q_stride_h = x8.stride(0), x8.stride(1), x8.stride(2)
    else:
        a.batch, a.seqlen = cu_seqlens.numel() - 1, int(max_seqlen)
        a.heads, a.head_dim = x16.shape[1], x16.shape[2]
        a.x_stride_b, a.x_stride_s, a.x_stride_h = 0, x16.stride(0), x16.stride(1)
        a.q_stride_b, a.q_stride_s, a.q_stride_h = 0, x8.stride(0), x8.stride(1)
    a.x_dtype, a.fp8_dtype = _lib.dtype_code(x16.dtype), _lib.dtype_code(x8.dtype)
    a.dequantize = int(dequantize)
    return a


def quantize_fp8_blockwise(x: torch.Tensor, dtype: torch.dtype = torch.float8_e4m3fn,
                           cu_seqlens: Optional[torch.Tensor] = None, max_seqlen: Optional[int] = None):
    """``x [B, S, H, D]`` (or packed ``[T, H, D]`` with ``cu_seqlens`` / ``max_seqlen``) -> ``(x_fp8, scales)`` with
    ``scales [B, H, ceil(S / 128)]`` fp32: per block of 128 positions of one sequence and head,
    ``scale = max|x| / FP8_MAX`` (0 for an all-zero block) and ``x_fp8 = rne(x / scale)``."""
    assert x.is_cuda and x.dtype in (torch.float16, torch.bfloat16) and dtype in _FP8
    xc = x.contiguous()
    x8 = torch.empty_like(xc, dtype=dtype)
    if cu_seqlens is None:
        batch, seqlen, heads = xc.shape[0], xc.shape[1], xc.shape[2]
    else:
        batch, seqlen, heads = cu_seqlens.numel() - 1, int(max_seqlen), xc.shape[1]
    # blocks that do not exist (shorter sequences of a packed batch) keep scale 0, like all-zero blocks
    scales = torch.zeros((batch, heads, -(-seqlen // 128)), dtype=torch.float32, device=x.device)
    a = _block_args(xc, x8, scales, cu_seqlens, max_seqlen, False)
    with torch.cuda.device(x.device):
        rc = _lib.load().fsa_quantize_fp8_blockwise(ctypes.byref(a), _lib.current_stream_ptr(x.device))
    _lib.check(rc, "fsa_quantize_fp8_blockwise")
    return x8, scales


def dequantize_fp8_blockwise(x8: torch.Tensor, scales: torch.Tensor, dtype: torch.dtype = torch.bfloat16,
                             cu_seqlens: Optional[torch.Tensor] = None, max_seqlen: Optional[int] = None):
    """The inverse map: ``(x8.float() * scale of its block).to(dtype)``."""
    assert x8.is_cuda and x8.dtype in _FP8 and dtype in (torch.float16, torch.bfloat16)
    xc = x8.contiguous()
    out = torch.zeros_like(xc, dtype=dtype)
    a = _block_args(out, xc, scales.contiguous(), cu_seqlens, max_seqlen, True)
    with torch.cuda.device(x8.device):
        rc = _lib.load().fsa_quantize_fp8_blockwise(ctypes.byref(a), _lib.current_stream_ptr(x8.device))
    _lib.check(rc, "fsa_quantize_fp8_blockwise")
    return out
