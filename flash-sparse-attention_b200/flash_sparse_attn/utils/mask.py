"""Top-k position selection with the contract of the reference's ``flash_sparse_attn/utils/mask.py:20-44``.

``topk_indices`` is the step in front of the gathered decode: from a score per key position (the
attention bias of the reference's dynamic-mask models) it returns the ``window_size`` positions with the
largest scores, in ascending order - what ``gather_kv_indices`` of
``flash_sparse_attn_with_kvcache_func`` takes. It runs as one CUDA kernel of the library
(``fsa_topk_indices``: radix select + ordered compaction), without host synchronisation.
"""

import torch

from flash_sparse_attn import _lib


def topk_indices(attention_bias: torch.Tensor, window_size: int, dtype: torch.dtype = torch.int64, **kwargs) -> torch.Tensor:
    """``attention_bias`` ``[..., key_len]`` (bf16 / fp16 / fp32, CUDA) -> ``[..., window_size]`` ascending
    positions of the largest entries (``dtype`` int64 like ``torch.topk``, or int32 to feed
    ``gather_kv_indices`` directly). Ties at the threshold take the lowest positions."""
    if not attention_bias.is_cuda:
        raise RuntimeError("flash_sparse_attn (B200 build) only runs on CUDA tensors; there is no CPU path")
    assert dtype in (torch.int32, torch.int64)
    x = attention_bias.detach()
    n = x.shape[-1]
    assert 0 < window_size <= n, "window_size must be in [1, key_len]"
    x2 = x.reshape(-1, n)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    out = torch.empty((x2.shape[0], window_size), dtype=dtype, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.load().fsa_topk_indices(x2.data_ptr(), _lib.dtype_code(x2.dtype), x2.shape[0], n, x2.stride(0),
                                          window_size, out.data_ptr(), int(dtype == torch.int64),
                                          _lib.current_stream_ptr(x.device))
    _lib.check(rc, "fsa_topk_indices")
    return out.reshape(*x.shape[:-1], window_size)
