"""Device-side steps in front of a (top-k) decode: appending the new key / value rows to the cache and cutting
global top-k positions down to one shard of a sharded cache. Thin wrappers of ``fsa_kv_append`` and
``fsa_localize_indices``; neither has a counterpart in the reference, which leaves cache management to its caller
(the cache layouts are the ones its decode operators read: contiguous ``[B, Sk, Hkv, D]`` or paged
``[pages, page_size, Hkv, D]`` with ``page_table [B, max_pages]``)."""

import ctypes
from typing import Optional

import torch

from flash_sparse_attn import _lib


def append_kv(key_new: torch.Tensor, value_new: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor,
              seqused_k: torch.Tensor, page_table: Optional[torch.Tensor] = None,
              free_pages: Optional[torch.Tensor] = None, free_count: Optional[torch.Tensor] = None,
              pos_ws: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Write ``key_new / value_new [B, T, Hkv, D]`` at positions ``seqused_k[b] .. + T`` of the cache and advance
    ``seqused_k`` (int32 [B], in place). Paged caches take missing pages (page-table entries < 0) from the stack
    ``free_pages`` (int32) of height ``free_count`` (int32 [1], decremented in place). Rows without room are dropped
    and reported by ``flash_sparse_attn.check_status()`` (status 3). No host synchronisation. Returns ``seqused_k``."""
    if not key_new.is_cuda:
        raise RuntimeError("flash_sparse_attn (B200 build) only runs on CUDA tensors; there is no CPU path")
    device = key_new.device
    batch, new_tokens, heads_kv, head_dim = key_new.shape
    assert value_new.shape == key_new.shape and value_new.stride() == key_new.stride()
    assert value_cache.shape == key_cache.shape and value_cache.stride() == key_cache.stride()
    assert key_cache.dtype == key_new.dtype == value_new.dtype == value_cache.dtype
    assert seqused_k.dtype == torch.int32 and seqused_k.numel() == batch and seqused_k.is_contiguous()
    assert key_new.stride(-1) == 1 and key_cache.stride(-1) == 1
    if pos_ws is None:
        pos_ws = torch.empty(batch, dtype=torch.int32, device=device)
    a = _lib.FsaKvAppendArgs()
    a.k_new, a.v_new, a.k_cache, a.v_cache = (t.data_ptr() for t in (key_new, value_new, key_cache, value_cache))
    a.seqused_k, a.pos_ws = seqused_k.data_ptr(), pos_ws.data_ptr()
    a.page_table, a.free_pages, a.free_count = _lib.ptr(page_table), _lib.ptr(free_pages), _lib.ptr(free_count)
    a.status = _lib.status_word(device).data_ptr()
    a.new_stride_b, a.new_stride_s, a.new_stride_h = key_new.stride(0), key_new.stride(1), key_new.stride(2)
    a.cache_stride_b, a.cache_stride_s, a.cache_stride_h = key_cache.stride(0), key_cache.stride(1), key_cache.stride(2)
    a.batch, a.new_tokens, a.heads_kv, a.head_dim = batch, new_tokens, heads_kv, head_dim
    if page_table is not None:
        assert page_table.dtype == torch.int32 and page_table.shape[0] == batch and page_table.stride(1) == 1
        a.page_size, a.page_table_stride = key_cache.shape[1], page_table.stride(0)
    else:
        a.capacity = key_cache.shape[1]
    a.dtype = _lib.dtype_code(key_new.dtype)
    with torch.cuda.device(device):
        rc = _lib.load().fsa_kv_append(ctypes.byref(a), _lib.current_stream_ptr(device))
    _lib.check(rc, "fsa_kv_append")
    return seqused_k


def localize_indices(gather_kv_indices: torch.Tensor, key_bounds: torch.Tensor, out: Optional[torch.Tensor] = None,
                     count: Optional[torch.Tensor] = None):
    """Global top-k positions ``[B, topk]`` (int32) -> ``(local, count)``: per row the positions inside
    ``[lo, hi) = key_bounds[b]`` shifted by ``-lo``, moved to the front in their original order, the rest ``-1``;
    ``count [B]`` says how many. ``out`` / ``count`` may be supplied so that the call allocates nothing."""
    device = gather_kv_indices.device
    rows, topk = gather_kv_indices.shape
    assert gather_kv_indices.dtype == torch.int32 and gather_kv_indices.stride(1) == 1
    assert key_bounds.dtype == torch.int32 and tuple(key_bounds.shape) == (rows, 2) and key_bounds.is_contiguous()
    out = torch.empty((rows, topk), dtype=torch.int32, device=device) if out is None else out
    count = torch.empty(rows, dtype=torch.int32, device=device) if count is None else count
    with torch.cuda.device(device):
        rc = _lib.load().fsa_localize_indices(gather_kv_indices.data_ptr(), gather_kv_indices.stride(0),
                                              key_bounds.data_ptr(), out.data_ptr(), out.stride(0), count.data_ptr(),
                                              rows, topk, _lib.current_stream_ptr(device))
    _lib.check(rc, "fsa_localize_indices")
    return out, count
