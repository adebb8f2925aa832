"""Host launcher of the backward pass.

Serves the dense, sparse and gated operators, batched and packed; it plays the role of
``_flash_{dense,sparse,gated}_attn_backward`` / ``..._varlen_backward`` of the reference
(flash_sparse_attn/ops/triton/flash_sparse_bwd.py:491-748, :751-1026, flash_gated_bwd.py:682-1298):
resolve defaults, pick the
number of QO splits, allocate gradients and fp32 workspaces with PyTorch and make ONE call into the C
ABI (``fsa_bwd``), which runs the pre-pass, the sm_100a main kernel, the dQ post-pass and the
reduction over splits. No host synchronisation happens here.
"""

import ctypes
from typing import Optional, Tuple

import torch

from flash_sparse_attn import _lib
from flash_sparse_attn.ops.triton import assert_inputs, quant, utils

TILE_M = 128
TILE_N = 128
_KIND = {"dense": _lib.KIND_DENSE, "sparse": _lib.KIND_SPARSE, "gated": _lib.KIND_GATED}


def _dequantize(x: torch.Tensor, scale: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    # saved tensors of a quantised forward are FP8; the backward runs on their de-quantised values in
    # the gradient dtype (flash_sparse_attn/ops/triton/scheduler.py:2133-2148)
    return quant.widen_fp8(x, dtype, scale)


def attn_backward(
    kind: str,
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    out: torch.Tensor,
    dout: torch.Tensor,
    lse: torch.Tensor,
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
    seqused_q: Optional[torch.Tensor] = None,
    seqused_k: Optional[torch.Tensor] = None,
    is_split_qo: bool = False,
    num_splits: Optional[int] = None,
    is_autotune: bool = True,
    tile_mn: Optional[Tuple[int, int]] = None,
    skip_checks: bool = False,
    tile_map: Optional[torch.Tensor] = None,
    deterministic: Optional[bool] = None,
):
    """Returns ``(dq, dk, dv)`` (plus ``(dalpha, ddelta)`` for the gated kind) in ``dout.dtype``.

    ``deterministic`` (default: the package-wide switch ``flash_sparse_attn.set_deterministic``) makes dQ
    bitwise reproducible: the key tiles add their dQ tiles in a fixed order instead of in the order the
    CTAs happen to run (dK and dV always are; for the gated kind dalpha keeps its fp32 atomics)."""
    if deterministic is None:
        deterministic = utils.deterministic_enabled()
    if not query.is_cuda:
        raise RuntimeError("flash_sparse_attn (B200 build) only runs on CUDA tensors; there is no CPU path")
    device = query.device
    varlen = cu_seqlens_q is not None
    if varlen:
        total_q, num_heads_q, head_dim = query.shape
        total_k, num_heads_kv, _ = key.shape
        batch = cu_seqlens_q.shape[0] - 1
        seqlen_q, seqlen_k = int(max_seqlen_q), int(max_seqlen_k)
    else:
        batch, seqlen_q, num_heads_q, head_dim = query.shape
        _, seqlen_k, num_heads_kv, _ = key.shape
        total_q = total_k = 0
    softmax_scale = softmax_scale if softmax_scale is not None else 1.0 / (head_dim**0.5)
    softmax_threshold = softmax_threshold if softmax_threshold is not None else 1.0
    if kind == "gated":
        gate_threshold = gate_threshold if gate_threshold is not None else 1.0 / max(seqlen_k, 1)
    if is_local and window_sizes is None:
        window_sizes = utils.window_sizes_heuristic(seqlen_k, num_heads_kv, device)

    if not skip_checks:
        assert_inputs.assert_bwd_inputs(
            query, key, value, out, dout, lse, query_scale=query_scale, key_scale=key_scale,
            value_scale=value_scale, window_sizes=window_sizes, alpha=alpha, delta=delta,
            cu_seqlens_q=cu_seqlens_q, cu_seqlens_k=cu_seqlens_k, seqused_q=seqused_q, seqused_k=seqused_k,
            num_heads_q=num_heads_q, num_heads_kv=num_heads_kv, head_dim=head_dim, is_quant=is_quant, device=device,
        )

    if is_quant and quant.is_block_scale(key_scale):
        query = quant.dequantize_fp8_blockwise(query, query_scale, dout.dtype, cu_seqlens_q, max_seqlen_q)
        key = quant.dequantize_fp8_blockwise(key, key_scale, dout.dtype, cu_seqlens_k, max_seqlen_k)
        value = quant.dequantize_fp8_blockwise(value, value_scale, dout.dtype, cu_seqlens_k, max_seqlen_k)
    elif is_quant:
        query = _dequantize(query, query_scale, dout.dtype)
        key = _dequantize(key, key_scale, dout.dtype)
        value = _dequantize(value, value_scale, dout.dtype)

    if is_split_qo and num_splits is None:
        # roles of the two sequence axes are swapped with respect to the forward heuristic
        num_splits = utils.num_splits_heuristic(
            seqlen_q=seqlen_k, seqlen_k=seqlen_q, num_SMs=utils.device_num_sms(device), TILE_M=TILE_N,
            TILE_N=TILE_M, is_local=is_local, num_heads_kv=num_heads_kv,
        )
        # one CTA per (key tile, KV head, batch): when that already oversubscribes the SMs, splitting the
        # query range only adds fp32 partials of dK/dV
        if batch * num_heads_kv * (-(-seqlen_k // TILE_N)) >= 2 * utils.device_num_sms(device):
            num_splits = 1
    elif not is_split_qo:
        num_splits = 1
    use_split = bool(is_split_qo) and num_splits > 1

    dq = torch.empty_like(query, dtype=dout.dtype)
    dk = torch.empty_like(key, dtype=dout.dtype)
    dv = torch.empty_like(value, dtype=dout.dtype)
    lib = _lib.load()
    da = dd = None
    if kind == "gated":
        # alpha [B, Hq, Sq] / [Hq, Tq], delta [B, Hkv, Sk] / [Hkv, Tk] (position contiguous), 16-bit like dout
        alpha = alpha.to(dout.dtype).contiguous()
        delta = delta.to(dout.dtype).contiguous()
        da = torch.empty_like(alpha)
        dd = torch.empty_like(delta)
    if seqused_k is not None or seqused_q is not None:
        # rows outside the used part of a sequence receive no gradient
        dq.zero_()
        dk.zero_()
        dv.zero_()
        if kind == "gated":
            da.zero_()
            dd.zero_()

    a = _lib.FsaBwdArgs()
    a.q, a.k, a.v = query.data_ptr(), key.data_ptr(), value.data_ptr()
    a.out, a.dout, a.lse = out.data_ptr(), dout.data_ptr(), lse.data_ptr()
    a.dq, a.dk, a.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    a.cu_seqlens_q, a.cu_seqlens_k = _lib.ptr(cu_seqlens_q), _lib.ptr(cu_seqlens_k)
    a.seqused_q, a.seqused_k = _lib.ptr(seqused_q), _lib.ptr(seqused_k)
    a.window_sizes = _lib.ptr(window_sizes)
    a.status = _lib.status_word(device).data_ptr()
    a.tile_map = _lib.ptr(tile_map)

    def strides(t):
        return (0, t.stride(0), t.stride(1)) if varlen else (t.stride(0), t.stride(1), t.stride(2))

    a.q_stride_b, a.q_stride_s, a.q_stride_h = strides(query)
    a.k_stride_b, a.k_stride_s, a.k_stride_h = strides(key)
    a.v_stride_b, a.v_stride_s, a.v_stride_h = strides(value)
    a.o_stride_b, a.o_stride_s, a.o_stride_h = strides(out)
    a.do_stride_b, a.do_stride_s, a.do_stride_h = strides(dout)
    a.dq_stride_b, a.dq_stride_s, a.dq_stride_h = strides(dq)
    a.dk_stride_b, a.dk_stride_s, a.dk_stride_h = strides(dk)
    if varlen:
        a.lse_stride_b, a.lse_stride_h = 0, lse.stride(0)
    else:
        a.lse_stride_b, a.lse_stride_h = lse.stride(0), lse.stride(1)
    a.batch, a.seqlen_q, a.seqlen_k = batch, seqlen_q, seqlen_k
    a.total_q, a.total_k = total_q, total_k
    a.heads_q, a.heads_kv, a.head_dim = num_heads_q, num_heads_kv, head_dim
    a.window_stride = window_sizes.stride(0) if window_sizes is not None else 0
    a.num_splits = num_splits if use_split else 1
    a.tile_m, a.tile_n = TILE_M, TILE_N
    a.kind = _KIND[kind]
    a.dtype = _lib.dtype_code(dout.dtype)
    flags = 0
    if is_causal:
        flags |= _lib.F_CAUSAL
    if is_local:
        flags |= _lib.F_LOCAL
    if use_split:
        flags |= _lib.F_SPLIT
    a.flags = flags
    a.softmax_scale = float(softmax_scale)
    a.softmax_threshold = float(softmax_threshold)
    a.gate_threshold = float(gate_threshold) if gate_threshold is not None else 0.0
    if deterministic:
        a.flags |= _lib.F_DETERMINISTIC
    if kind == "gated":
        a.alpha, a.delta, a.dalpha, a.ddelta = alpha.data_ptr(), delta.data_ptr(), da.data_ptr(), dd.data_ptr()
        a.alpha_stride_b, a.alpha_stride_h = (0, alpha.stride(0)) if varlen else (alpha.stride(0), alpha.stride(1))
        a.delta_stride_b, a.delta_stride_h = (0, delta.stride(0)) if varlen else (delta.stride(0), delta.stride(1))
        a.delta_numel = delta.numel()
        if is_logsigmoid_gate:
            a.flags |= _lib.F_LOGSIGMOID
        if is_adapt_gate:
            a.flags |= _lib.F_ADAPT_GATE

    # caller-owned workspaces, sized by the library (fp32 unless noted): lse2 / dpsum [Hq, R], dq_accum [Hq, R, 64 | 128]
    # with R tile-padded rows; split-QO partials of dK / dV (/ ddelta); gated: alpha copy (16-bit) and dalpha
    # accumulator [Hq, R]; deterministic: visiting order (uint16) and turn counters (int32)
    ws = _lib.FsaBwdWorkspace()
    _lib.check(lib.fsa_bwd_workspace_bytes(ctypes.byref(a), ctypes.byref(ws)), "fsa_bwd_workspace_bytes")
    bufs = {name: _lib.workspace(getattr(ws, name), device, torch.uint8) for name, _ in ws._fields_}
    if seqused_k is not None or seqused_q is not None:
        for name in ("dk_partial", "dv_partial", "dd_partial"):  # rows outside the used part receive no gradient
            if bufs[name] is not None:
                bufs[name].zero_()
    for name, buf in bufs.items():
        setattr(a, name, _lib.ptr(buf))
    _lib.attach_profile_events(a)

    with torch.cuda.device(device):
        rc = lib.fsa_bwd(ctypes.byref(a), _lib.current_stream_ptr(device))
    _lib.check(rc, f"fsa_bwd[{kind}]")
    if kind == "gated":
        return dq, dk, dv, da, dd
    return dq, dk, dv


def tile_map_numel(batch, seqlen_q, seqlen_k, num_heads_q, num_splits=1):
    """Bytes of the optional backward tile map: one per (batch, query head, key tile, split, query tile)."""
    return batch * num_heads_q * (-(-seqlen_k // TILE_N)) * max(num_splits, 1) * (-(-seqlen_q // TILE_M))
