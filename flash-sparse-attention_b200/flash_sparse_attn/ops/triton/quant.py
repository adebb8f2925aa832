"""Per-tensor FP8 quantisation with the contract of flash_sparse_attn/ops/triton/quant.py:42-64, and the
widening cast the quantised operators use on their inputs. Both run as CUDA kernels of the library
(``fsa_quantize_fp8``: absolute maximum, then scaled cast; ``fsa_fp8_widen``), without host
synchronisation."""

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
