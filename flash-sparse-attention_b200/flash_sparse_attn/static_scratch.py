"""Python access to ``fsa_decode_static_scratch``: split-KV decode whose split workspace is a fixed
16 MiB array inside the library, for callers that cannot allocate device memory at call time.

Unlike the regular operators this helper takes pre-made output buffers and allocates nothing itself.
"""

import ctypes

import torch

from flash_sparse_attn import _lib


def scratch_bytes() -> int:
    lib = _lib.load()
    lib.fsa_static_scratch_bytes.restype = ctypes.c_size_t
    return int(lib.fsa_static_scratch_bytes())


def decode_static_scratch(kind: str, query, key, value, out, lse, num_splits: int, softmax_scale=None,
                          softmax_threshold: float = 1.0, page_table=None, gather_kv_indices=None, seqused_k=None):
    """Split-KV decode of ``query [B, Hq, D]`` against ``key/value`` ([B, Sk, Hkv, D] or a paged cache with
    ``page_table``) into the caller's ``out [B, Hq, D]`` / ``lse [B, Hq]``. Raises RuntimeError when
    ``num_splits * B * Hq * (D + 1)`` floats exceed the built-in workspace. The first call on a device loads the
    workspace (16 MiB of device memory, an implicit synchronisation): make it at start-up, before a memory pool
    takes the rest of the GPU and outside stream capture; later calls allocate nothing. Overlapping calls on one
    GPU must be ordered by the caller."""
    if value.stride() != key.stride() or value.shape != key.shape:
        raise ValueError("value must have key's shape and strides (the C ABI passes one set of strides for both)")
    want = torch.bfloat16 if query.dtype in (torch.float8_e4m3fn, torch.float8_e5m2) else query.dtype
    if out.dtype != want or tuple(out.shape) != tuple(query.shape) or out.stride(-1) != 1:
        raise ValueError(f"out must be a {want} tensor shaped like query with a contiguous last dimension")
    if lse.dtype != torch.float32 or tuple(lse.shape) != tuple(query.shape[:2]):
        raise ValueError("lse must be a float32 tensor of shape [batch, heads_q]")
    if query.stride(-1) != 1 or key.stride(-1) != 1:
        raise ValueError("query, key and value must be contiguous along head_dim")
    lib = _lib.load()
    lib.fsa_decode_static_scratch.restype = ctypes.c_int
    lib.fsa_decode_static_scratch.argtypes = [ctypes.POINTER(_lib.FsaDecArgs), ctypes.c_void_p]
    device = query.device
    batch, heads_q, head_dim = query.shape
    a = _lib.FsaDecArgs()
    a.q, a.k, a.v = query.data_ptr(), key.data_ptr(), value.data_ptr()
    a.out, a.lse = out.data_ptr(), lse.data_ptr()
    a.seqused_k = _lib.ptr(seqused_k)
    a.page_table, a.gather_kv_indices = _lib.ptr(page_table), _lib.ptr(gather_kv_indices)
    a.status = _lib.status_word(device).data_ptr()
    a.q_stride_b, a.q_stride_h = query.stride(0), query.stride(1)
    a.k_stride_b, a.k_stride_s, a.k_stride_h = key.stride(0), key.stride(1), key.stride(2)
    a.o_stride_b, a.o_stride_h = out.stride(0), out.stride(1)
    a.lse_stride_b, a.lse_stride_h = lse.stride(0), lse.stride(1)
    a.batch, a.heads_q, a.heads_kv, a.head_dim = batch, heads_q, key.shape[2], head_dim
    if page_table is not None:
        a.num_pages, a.page_size, a.page_table_stride = key.shape[0], key.shape[1], page_table.stride(0)
        a.seqlen_k = page_table.shape[1] * key.shape[1]
    else:
        a.seqlen_k = key.shape[1]
    if gather_kv_indices is not None:
        a.topk, a.gather_stride = gather_kv_indices.shape[-1], gather_kv_indices.stride(0)
    a.num_splits = int(num_splits)
    a.kind = {"dense": _lib.KIND_DENSE, "sparse": _lib.KIND_SPARSE}[kind]
    a.dtype = _lib.dtype_code(query.dtype)
    a.softmax_scale = float(softmax_scale if softmax_scale is not None else head_dim ** -0.5)
    a.softmax_threshold = float(softmax_threshold)
    with torch.cuda.device(device):
        rc = lib.fsa_decode_static_scratch(ctypes.byref(a), _lib.current_stream_ptr(device))
    _lib.check(rc, "fsa_decode_static_scratch")
    return out, lse
