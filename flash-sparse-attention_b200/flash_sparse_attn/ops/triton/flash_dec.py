"""Host launcher of the decode pass.

Serves the dense and sparse kv-cache operators (contiguous, packed, paged and / or gathered keys); it
plays the role of ``_flash_{dense,sparse}_attn_decode`` / ``..._varlen_decode`` of the reference
(flash_sparse_attn/ops/triton/flash_sparse_dec.py:519-744, :747-952). Shapes only decide the launch
(no device data is read on the host, nothing synchronises), so the call can be captured into a CUDA
graph once the output buffers are passed in, as the reference's README describes for decode.
"""

import ctypes
from typing import Optional, Tuple

import torch

from flash_sparse_attn import _lib
from flash_sparse_attn.ops.triton import assert_inputs, quant, utils

_KIND = {"dense": _lib.KIND_DENSE, "sparse": _lib.KIND_SPARSE, "gated": _lib.KIND_GATED}
KEYS_PER_WARP_TILE = 16
WARPS = 4


def decode_num_splits(batch: int, num_heads_kv: int, keys: int, num_sms: int) -> int:
    """Number of KV splits when the caller gives none. One CTA serves (sequence, KV head, split), two CTAs share
    an SM, and every split costs a share of a second (combine) launch plus per-CTA set-up: about 10 us on a
    2048-key step. Two rules, the larger result wins (measured on paged caches with contexts of 4K-128K keys):

    * fill: an under-occupied grid is split until it fills ONE wave of CTA slots, never beyond it (a second, partly
      filled wave costs more than the idle slots) and never below 512 keys per CTA (128 per warp);
    * balance: long contexts (at least 2048 keys per split) are cut until the grid holds about six waves, which evens
      out sequences of unequal length - 64 sequences of 4K-128K keys run in 2.50 ms with 4 splits against 3.22 ms with
      one, a single 66K sequence in 57 us with 32 splits against 126 us with 8.
    """
    slots = 2 * max(num_sms, 1)
    ctas = max(batch * num_heads_kv, 1)
    fill = min(slots // ctas, keys // (WARPS * 128))
    balance = min(32, keys // 2048, -(-6 * slots // ctas))
    return max(1, fill, balance)


def attn_decode(
    kind: str,
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    alpha: Optional[torch.Tensor] = None,
    delta: Optional[torch.Tensor] = None,
    cu_seqlens_k: Optional[torch.Tensor] = None,
    max_seqlen_k: Optional[int] = None,
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
    tile_map: Optional[torch.Tensor] = None,
    partial_only: bool = False,
    workspace: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
    threshold_seqlen_k: Optional[torch.Tensor] = None,
    key_range=None,
    packed_partials: Optional[torch.Tensor] = None,
    gather_count: Optional[torch.Tensor] = None,
    peers=None,
):
    """Returns ``(out, lse)``; with ``partial_only`` returns ``(out_partial [ns,B,Hq,D] fp32,
    lse_partial [ns,Hq,B] fp32 base-2)`` instead (used by context-parallel decode).
    ``workspace`` optionally supplies the two partial buffers so that no allocation happens.
    For a shard of a longer key sequence: ``threshold_seqlen_k`` (int32 [B]) is the key count that normalises the
    softmax threshold (the whole sequence's, so that a shard skips by the same bound as an unsharded call);
    ``key_range`` (int32 [B, 2] of (lo, hi) per sequence, or one (lo, hi) tuple) makes gathered positions outside
    [lo, hi) masked and addresses the others at position - lo. ``packed_partials`` (fp32, at least splits * B * Hq * (D + 1) elements) receives the partials
    of every split as one block - outputs then log-sum-exps - so that they travel in a single all-gather.
    ``gather_count`` (int32 [B]): only that many leading entries of each row of ``gather_kv_indices`` can be valid
    (see ``flash_sparse_attn.utils.kvcache.localize_indices``); the kernel visits only the tiles that hold them."""
    if not query.is_cuda:
        raise RuntimeError("flash_sparse_attn (B200 build) only runs on CUDA tensors; there is no CPU path")
    device = query.device
    batch, num_heads_q, head_dim = query.shape
    varlen = cu_seqlens_k is not None
    page_size = None
    if varlen:
        total_k, num_heads_kv, _ = key.shape
        seqlen_k = int(max_seqlen_k)
    elif page_table is not None:
        _, page_size, num_heads_kv, _ = key.shape
        seqlen_k = page_table.shape[1] * page_size
        total_k = 0
    else:
        _, seqlen_k, num_heads_kv, _ = key.shape
        total_k = 0
    softmax_scale = softmax_scale if softmax_scale is not None else 1.0 / (head_dim**0.5)
    softmax_threshold = softmax_threshold if softmax_threshold is not None else 1.0
    if kind == "gated":
        gate_threshold = gate_threshold if gate_threshold is not None else 1.0 / max(seqlen_k, 1)
    else:
        gate_threshold = 0.0
    is_gather = gather_kv_indices is not None
    if is_local and window_sizes is None:
        window_sizes = utils.window_sizes_heuristic(seqlen_k, num_heads_kv, device)

    if not skip_checks:
        assert_inputs.assert_dec_inputs(
            query, key, value, query_scale=query_scale, key_scale=key_scale, value_scale=value_scale,
            window_sizes=window_sizes, alpha=alpha, delta=delta, cu_seqlens_k=cu_seqlens_k, seqused_k=seqused_k,
            page_table=page_table, gather_kv_indices=gather_kv_indices, num_heads_q=num_heads_q,
            num_heads_kv=num_heads_kv, head_dim=head_dim, page_size=page_size, is_quant=is_quant, device=device,
            tile_mn=tile_mn,
        )
        assert_inputs.check_out_buffers(out, lse, query.shape, torch.bfloat16 if is_quant else query.dtype,
                                        query.shape[:2])

    qkv_scale = None
    if is_quant:
        # FP8 query and cache: widened (exactly) to bf16 before the kernel; scales as in the forward
        qkv_scale = quant.scales_f32(query_scale, key_scale, value_scale, device)
        native = head_dim == 128 and query.dtype == key.dtype == value.dtype
        if not native:  # other head sizes / mixed formats: widen the tensors and run the 16-bit kernel
            query, key, value = (quant.widen_fp8(t, torch.bfloat16) for t in (query, key, value))

    out_dtype = torch.bfloat16 if is_quant else query.dtype
    keys = gather_kv_indices.shape[-1] if is_gather else seqlen_k
    if num_splits is None:
        num_splits = decode_num_splits(batch, num_heads_kv, keys, utils.device_num_sms(device))
    num_splits = max(1, int(num_splits))

    if out is None and not partial_only:
        out = torch.empty(query.shape, dtype=out_dtype, device=device)
    if lse is None and not partial_only:
        lse = torch.empty((batch, num_heads_q), dtype=torch.float32, device=device)
    a = _lib.FsaDecArgs()
    a.q, a.k, a.v = query.data_ptr(), key.data_ptr(), value.data_ptr()
    a.out, a.lse = _lib.ptr(out), _lib.ptr(lse)
    a.cu_seqlens_k, a.seqused_k = _lib.ptr(cu_seqlens_k), _lib.ptr(seqused_k)
    a.page_table, a.gather_kv_indices = _lib.ptr(page_table), _lib.ptr(gather_kv_indices)
    a.window_sizes = _lib.ptr(window_sizes)
    a.status = _lib.status_word(device).data_ptr()
    a.tile_map = _lib.ptr(tile_map)
    a.q_stride_b, a.q_stride_h = query.stride(0), query.stride(1)
    if varlen:
        a.k_stride_b, a.k_stride_s, a.k_stride_h = 0, key.stride(0), key.stride(1)
    else:
        a.k_stride_b, a.k_stride_s, a.k_stride_h = key.stride(0), key.stride(1), key.stride(2)
    if value.stride() != key.stride():
        raise RuntimeError("key and value must share one memory layout")
    if out is not None:
        a.o_stride_b, a.o_stride_h = out.stride(0), out.stride(1)
        a.lse_stride_b, a.lse_stride_h = lse.stride(0), lse.stride(1)
    a.batch, a.seqlen_k, a.total_k = batch, seqlen_k, total_k
    a.heads_q, a.heads_kv, a.head_dim = num_heads_q, num_heads_kv, head_dim
    if is_gather:
        a.topk, a.gather_stride = gather_kv_indices.shape[-1], gather_kv_indices.stride(0)
    if page_table is not None:
        a.num_pages, a.page_size, a.page_table_stride = key.shape[0], page_size, page_table.stride(0)
    a.window_stride = window_sizes.stride(0) if window_sizes is not None else 0
    a.num_splits = num_splits
    a.partial_only = int(partial_only)
    a.kind = _KIND[kind]
    a.dtype = _lib.dtype_code(query.dtype)
    a.flags = (_lib.F_LOCAL if is_local else 0) | (_lib.F_LOGSIGMOID if is_logsigmoid_gate else 0)
    if kind == "gated":
        # alpha [B, Hq]; delta [B, Hkv, Sk] / [Hkv, Tk] / paged [pages, Hkv, page] (positions contiguous)
        alpha, delta = alpha.to(out_dtype).contiguous(), delta.to(out_dtype).contiguous()
        keep_alive = (alpha, delta)  # noqa: F841  (the launch below is asynchronous)
        a.alpha, a.delta = alpha.data_ptr(), delta.data_ptr()
        a.alpha_stride_b, a.alpha_stride_h = alpha.stride(0), alpha.stride(1)
        a.delta_stride_b, a.delta_stride_h = (0, delta.stride(0)) if varlen else (delta.stride(0), delta.stride(1))
    a.softmax_scale = float(softmax_scale)
    a.softmax_threshold = float(softmax_threshold)
    a.gate_threshold = float(gate_threshold)
    a.qkv_scale = _lib.ptr(qkv_scale)
    a.thr_seqlen_k = _lib.ptr(threshold_seqlen_k)
    a.gather_count = _lib.ptr(gather_count)
    if key_range is not None:
        if not isinstance(key_range, torch.Tensor):  # one (lo, hi) for every sequence
            key_range = torch.tensor([[int(key_range[0]), int(key_range[1])]] * batch, dtype=torch.int32, device=device)
        assert key_range.dtype == torch.int32 and tuple(key_range.shape) == (batch, 2) and key_range.is_contiguous()
        a.key_bounds = key_range.data_ptr()

    # split partials [splits, B, Hq, D] / [splits, Hq, B] (base-2 lse): the caller's, or sized by the library
    lib = _lib.load()
    ws = _lib.FsaDecWorkspace()
    _lib.check(lib.fsa_decode_workspace_bytes(ctypes.byref(a), ctypes.byref(ws)), "fsa_decode_workspace_bytes")
    gate_ws = _lib.workspace(ws.gate_ws, device)  # gated kind: extremes of delta per 16-key tile
    a.gate_ws = _lib.ptr(gate_ws)
    out_partial = lse_partial = None
    if packed_partials is not None:
        # one buffer [splits, B*Hq*(D+1)]: the partial outputs of a split followed by its log-sum-exps
        per = batch * num_heads_q * (head_dim + 1)
        assert packed_partials.dtype == torch.float32 and packed_partials.numel() >= num_splits * per
        flat = packed_partials.view(-1)
        out_partial, lse_partial = flat, flat[batch * num_heads_q * head_dim:]
        a.out_partial_stride = a.lse_partial_stride = per
    elif workspace is not None:
        out_partial, lse_partial = workspace
    else:
        if ws.out_partial:
            out_partial = _lib.workspace(ws.out_partial, device).view(num_splits, batch, num_heads_q, head_dim)
            lse_partial = _lib.workspace(ws.lse_partial, device).view(num_splits, num_heads_q, batch)
    a.out_partial, a.lse_partial = _lib.ptr(out_partial), _lib.ptr(lse_partial)
    if peers is not None:
        # `peers`: the FsaPeerArgs of a context-parallel group - the kernel stores the packed partials into the
        # receive buffer of every rank and counts its arrivals there (context_parallel.PeerExchange)
        assert partial_only and packed_partials is not None
        a.peers = ctypes.cast(ctypes.pointer(peers), ctypes.c_void_p)
    _lib.attach_profile_events(a)

    with torch.cuda.device(device):
        rc = lib.fsa_decode(ctypes.byref(a), _lib.current_stream_ptr(device))
    _lib.check(rc, f"fsa_decode[{kind}]")
    if partial_only:
        return out_partial, lse_partial
    return out, lse


def combine_partials(out_partial: torch.Tensor, lse_partial: torch.Tensor, dtype: torch.dtype, out=None, lse=None):
    """Merge partial decode results ``[P, B, Hq, D]`` / ``[P, Hq, B]`` (base-2 lse) into ``(out [B,Hq,D],
    lse [B,Hq])`` with the library's combine kernel."""
    parts, batch, heads, head_dim = out_partial.shape
    device = out_partial.device
    out = torch.empty((batch, heads, head_dim), dtype=dtype, device=device) if out is None else out
    lse = torch.empty((batch, heads), dtype=torch.float32, device=device) if lse is None else lse
    with torch.cuda.device(device):
        rc = _lib.load().fsa_combine(out_partial.data_ptr(), lse_partial.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                     parts, batch, heads, head_dim, _lib.dtype_code(dtype), 0, 0,
                                     _lib.current_stream_ptr(device))
    _lib.check(rc, "fsa_combine")
    return out, lse


def combine_packed_partials(packed: torch.Tensor, parts: int, batch: int, heads: int, head_dim: int,
                            dtype: torch.dtype, out=None, lse=None):
    """Merge `parts` partials stored as blocks of B*Hq*(D+1) floats (outputs, then base-2 log-sum-exps [Hq, B]):
    the layout ``attn_decode(..., packed_partials=...)`` writes and an all-gather of it concatenates."""
    device = packed.device
    per = batch * heads * (head_dim + 1)
    flat = packed.view(-1)
    assert flat.numel() >= parts * per
    out = torch.empty((batch, heads, head_dim), dtype=dtype, device=device) if out is None else out
    lse = torch.empty((batch, heads), dtype=torch.float32, device=device) if lse is None else lse
    with torch.cuda.device(device):
        rc = _lib.load().fsa_combine(flat.data_ptr(), flat[batch * heads * head_dim:].data_ptr(), out.data_ptr(),
                                     lse.data_ptr(), parts, batch, heads, head_dim, _lib.dtype_code(dtype), per, per,
                                     _lib.current_stream_ptr(device))
    _lib.check(rc, "fsa_combine")
    return out, lse
