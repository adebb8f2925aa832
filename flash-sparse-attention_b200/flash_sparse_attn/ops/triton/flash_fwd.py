"""Host launchers of the forward pass.

One implementation serves the dense, sparse and gated operators, batched and packed (varlen); it
plays the role of ``_flash_{dense,sparse,gated}_attn_forward`` / ``..._varlen_forward`` of the
reference (flash_sparse_attn/ops/triton/flash_sparse_fwd.py:520-758, :761-988 and the dense / gated
twins): resolve defaults, pick the number of KV splits, allocate outputs and split workspaces with
PyTorch, then make ONE call into the C ABI (``fsa_fwd``) which launches the sm_100a kernel and, when
split, the combine kernel. No host synchronisation happens here.
"""

import ctypes
from typing import Optional, Tuple

import torch

from flash_sparse_attn import _lib
from flash_sparse_attn.ops.triton import assert_inputs, quant, utils

TILE_M = 128
TILE_N = 128

_KIND = {"dense": _lib.KIND_DENSE, "sparse": _lib.KIND_SPARSE, "gated": _lib.KIND_GATED}


def _require_cuda(t: torch.Tensor):
    if not t.is_cuda:
        raise RuntimeError("flash_sparse_attn (B200 build) only runs on CUDA tensors; there is no CPU path")


def attn_forward(
    kind: str,
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    alpha: Optional[torch.Tensor] = None,
    delta: Optional[torch.Tensor] = None,
    cu_seqlens_q: Optional[torch.Tensor] = None,
    cu_seqlens_k: Optional[torch.Tensor] = None,
    max_seqlen_q: Optional[int] = None,
    max_seqlen_k: Optional[int] = None,
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
    pack_gqa: bool = False,
    num_splits: Optional[int] = None,
    page_table: Optional[torch.Tensor] = None,
    seqused_q: Optional[torch.Tensor] = None,
    seqused_k: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    lse: Optional[torch.Tensor] = None,
    is_autotune: bool = True,
    tile_mn: Optional[Tuple[int, int]] = None,
    skip_checks: bool = False,
    tile_map: Optional[torch.Tensor] = None,
):
    """Returns ``(out, lse, softmax_scale, softmax_threshold, gate_threshold)``.

    ``is_autotune`` and ``tile_mn`` are accepted for signature compatibility; the kernels use one
    tile shape (128 x 128), so they have no effect. ``tile_map`` (uint8, zero-initialised, sized with
    ``tile_map_numel``) optionally receives which tiles were computed / skipped.
    """
    _require_cuda(query)
    device = query.device
    varlen = cu_seqlens_q is not None
    if varlen:
        total_q, num_heads_q, head_dim = query.shape
        total_k, num_heads_kv, _ = key.shape
        batch = cu_seqlens_q.shape[0] - 1
        seqlen_q, seqlen_k = int(max_seqlen_q), int(max_seqlen_k)
        page_size = None
    else:
        batch, seqlen_q, num_heads_q, head_dim = query.shape
        total_q = total_k = 0
        if page_table is not None:
            _, page_size, num_heads_kv, _ = key.shape
            seqlen_k = page_table.shape[1] * page_size
        else:
            page_size = None
            _, seqlen_k, num_heads_kv, _ = key.shape

    softmax_scale = softmax_scale if softmax_scale is not None else 1.0 / (head_dim**0.5)
    softmax_threshold = softmax_threshold if softmax_threshold is not None else 1.0
    if kind == "gated":
        gate_threshold = gate_threshold if gate_threshold is not None else 1.0 / max(seqlen_k, 1)
    else:
        gate_threshold = 0.0
    group = num_heads_q // num_heads_kv
    group_packed = group if pack_gqa else 1
    if is_local and window_sizes is None:
        window_sizes = utils.window_sizes_heuristic(seqlen_k, num_heads_kv, device)

    if not skip_checks:
        assert_inputs.assert_fwd_inputs(
            query, key, value, query_scale=query_scale, key_scale=key_scale, value_scale=value_scale,
            window_sizes=window_sizes, alpha=alpha, delta=delta, cu_seqlens_q=cu_seqlens_q,
            cu_seqlens_k=cu_seqlens_k, seqused_q=seqused_q, seqused_k=seqused_k, num_heads_q=num_heads_q,
            num_heads_kv=num_heads_kv, head_dim=head_dim, page_size=page_size, tile_mn=tile_mn, is_quant=is_quant,
            device=device, page_table=page_table,
        )
        assert_inputs.check_out_buffers(
            out, lse, query.shape, torch.bfloat16 if is_quant else query.dtype,
            (num_heads_q, total_q) if varlen else (batch, num_heads_q, seqlen_q))

    qkv_scale = None
    block_scales = None
    if is_quant and quant.is_block_scale(key_scale):
        # block-scaled FP8 (scales per 128 positions and head): native kernels only; the scales go in per tile
        if head_dim != 128 or kind == "gated" or pack_gqa or page_table is not None:
            raise RuntimeError("block-scaled FP8 needs head_dim 128, the dense or sparse kind, no packed GQA, no paging")
        sq, sk, sv = (t.float().contiguous() for t in (query_scale, key_scale, value_scale))
        block_scales = (sq, sk, sv)
    elif is_quant:
        # FP8 inputs: widened (exactly) to bf16 in one pass; the per-tensor scales stay on the device and
        # enter the kernel as in scheduler.py:298-307 (logit scale *= q_scale * k_scale, out *= v_scale)
        qkv_scale = quant.scales_f32(query_scale, key_scale, value_scale, device)
        native = head_dim == 128 and query.dtype == key.dtype == value.dtype
        if not native:  # other head sizes / mixed formats: widen (exactly) to bf16 and use the 16-bit kernel
            query, key, value = (quant.widen_fp8(t, torch.bfloat16) for t in (query, key, value))

    if is_split_kv and num_splits is None:
        num_splits = utils.num_splits_heuristic(
            seqlen_q=seqlen_q * group_packed, seqlen_k=seqlen_k, num_SMs=utils.device_num_sms(device),
            TILE_M=TILE_M, TILE_N=TILE_N, is_local=is_local, num_heads_kv=num_heads_kv,
        )
        # The reference's rule only looks at the query tiles of ONE (batch, head). When batch x heads
        # already gives every SM several CTAs, splitting only adds fp32 partial traffic: keep one split.
        m_pairs = -(-seqlen_q * group_packed // (2 * TILE_M))
        ctas = batch * (num_heads_kv if group_packed > 1 else num_heads_q) * m_pairs
        if ctas >= 2 * utils.device_num_sms(device):
            num_splits = 1
    elif not is_split_kv:
        num_splits = 1
    # a single split is the unsplit kernel (same schedule, no workspace, no combine pass)
    use_split = bool(is_split_kv) and num_splits > 1

    out_dtype = torch.bfloat16 if is_quant else query.dtype
    if out is None:
        out = torch.empty_like(query, dtype=out_dtype)
    if lse is None:
        lse_shape = (num_heads_q, total_q) if varlen else (batch, num_heads_q, seqlen_q)
        lse = torch.empty(lse_shape, dtype=torch.float32, device=device)

    a = _lib.FsaFwdArgs()
    a.q, a.k, a.v = query.data_ptr(), key.data_ptr(), value.data_ptr()
    a.out, a.lse = out.data_ptr(), lse.data_ptr()
    a.alpha, a.delta = _lib.ptr(alpha), _lib.ptr(delta)
    a.cu_seqlens_q, a.cu_seqlens_k = _lib.ptr(cu_seqlens_q), _lib.ptr(cu_seqlens_k)
    a.seqused_q, a.seqused_k = _lib.ptr(seqused_q), _lib.ptr(seqused_k)
    a.page_table, a.window_sizes = _lib.ptr(page_table), _lib.ptr(window_sizes)
    a.status = _lib.status_word(device).data_ptr()
    a.tile_map = _lib.ptr(tile_map)
    a.qkv_scale = _lib.ptr(qkv_scale)
    if block_scales is not None:
        a.q_block_scale, a.k_block_scale, a.v_block_scale = (t.data_ptr() for t in block_scales)
    if varlen:
        a.q_stride_b, a.q_stride_s, a.q_stride_h = 0, query.stride(0), query.stride(1)
        a.k_stride_b, a.k_stride_s, a.k_stride_h = 0, key.stride(0), key.stride(1)
        a.v_stride_b, a.v_stride_s, a.v_stride_h = 0, value.stride(0), value.stride(1)
        a.o_stride_b, a.o_stride_s, a.o_stride_h = 0, out.stride(0), out.stride(1)
        a.lse_stride_b, a.lse_stride_h = 0, lse.stride(0)
    else:
        a.q_stride_b, a.q_stride_s, a.q_stride_h = query.stride(0), query.stride(1), query.stride(2)
        a.k_stride_b, a.k_stride_s, a.k_stride_h = key.stride(0), key.stride(1), key.stride(2)
        a.v_stride_b, a.v_stride_s, a.v_stride_h = value.stride(0), value.stride(1), value.stride(2)
        a.o_stride_b, a.o_stride_s, a.o_stride_h = out.stride(0), out.stride(1), out.stride(2)
        a.lse_stride_b, a.lse_stride_h = lse.stride(0), lse.stride(1)
    if kind == "gated":
        # alpha [B, Hq, Sq] / [Hq, Tq], delta [B, Hkv, Sk] / [Hkv, Tk] / paged [pages, Hkv, page] (position contiguous)
        if alpha.dtype != out_dtype or delta.dtype != out_dtype:
            alpha, delta = alpha.to(out_dtype), delta.to(out_dtype)
            a.alpha, a.delta = alpha.data_ptr(), delta.data_ptr()
        a.alpha_stride_b, a.alpha_stride_h = (0, alpha.stride(0)) if varlen else (alpha.stride(0), alpha.stride(1))
        a.delta_stride_b, a.delta_stride_h = (0, delta.stride(0)) if varlen else (delta.stride(0), delta.stride(1))
    a.batch, a.seqlen_q, a.seqlen_k = batch, seqlen_q, seqlen_k
    a.total_q, a.total_k = total_q, total_k
    a.heads_q, a.heads_kv, a.head_dim = num_heads_q, num_heads_kv, head_dim
    if page_table is not None:
        a.num_pages, a.page_size, a.page_table_stride = key.shape[0], page_size, page_table.stride(0)
    a.window_stride = window_sizes.stride(0) if window_sizes is not None else 0
    a.num_splits = num_splits if use_split else 1
    a.tile_m, a.tile_n = TILE_M, TILE_N
    a.kind = _KIND[kind]
    a.dtype = _lib.dtype_code(query.dtype)
    flags = 0
    if is_causal:
        flags |= _lib.F_CAUSAL
    if is_local:
        flags |= _lib.F_LOCAL
    if use_split:
        flags |= _lib.F_SPLIT
    if pack_gqa and group > 1:
        flags |= _lib.F_PACK_GQA
    if is_logsigmoid_gate:
        flags |= _lib.F_LOGSIGMOID
    if is_adapt_gate:
        flags |= _lib.F_ADAPT_GATE
    a.flags = flags
    a.softmax_scale = float(softmax_scale)
    a.softmax_threshold = float(softmax_threshold)
    a.gate_threshold = float(gate_threshold)

    # caller-owned workspaces, sized by the library: split-KV partials [splits, rows, Hq, D] / [splits, Hq, rows]
    # and the gated kind's per-tile extremes
    lib = _lib.load()
    ws = _lib.FsaFwdWorkspace()
    _lib.check(lib.fsa_fwd_workspace_bytes(ctypes.byref(a), ctypes.byref(ws)), "fsa_fwd_workspace_bytes")
    out_partial, lse_partial = _lib.workspace(ws.out_partial, device), _lib.workspace(ws.lse_partial, device)
    gate_ws = _lib.workspace(ws.gate_ws, device)
    if lse_partial is not None and varlen and seqused_q is not None:
        lse_partial.fill_(float("-inf"))  # rows past seqused_q are never written
    a.out_partial, a.lse_partial, a.gate_ws = _lib.ptr(out_partial), _lib.ptr(lse_partial), _lib.ptr(gate_ws)
    _lib.attach_profile_events(a)

    with torch.cuda.device(device):
        rc = lib.fsa_fwd(ctypes.byref(a), _lib.current_stream_ptr(device))
    _lib.check(rc, f"fsa_fwd[{kind}]")
    return out, lse, softmax_scale, softmax_threshold, gate_threshold


def tile_map_numel(batch, seqlen_q, seqlen_k, num_heads_q, num_heads_kv, pack_gqa=False, num_splits=1):
    """Number of bytes of the optional forward tile map (one per batch, grid head, query tile, split,
    key tile)."""
    group = num_heads_q // num_heads_kv
    gpack = group if pack_gqa else 1
    hgrid = num_heads_kv if gpack > 1 else num_heads_q
    m_blocks = -(-seqlen_q * gpack // TILE_M)
    n_blocks = -(-seqlen_k // TILE_N)
    return batch * hgrid * m_blocks * max(num_splits, 1) * n_blocks
