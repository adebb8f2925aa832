"""ctypes binding of libfsa_b200.so (the C ABI declared in include/fsa_b200.h).

The library is the only compute path of this package: there is no eager or CPU fallback. Loading
fails loudly when the shared object has not been built (``python build.py`` in the directory that
holds ``csrc/``), and every entry point raises on a non-zero status.
"""

import ctypes
import os
from ctypes import POINTER, c_float, c_int, c_int32, c_int64, c_size_t, c_uint32, c_uint8, c_void_p

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(os.path.dirname(_HERE), "libfsa_b200.so")

ABI_VERSION = 2

KIND_DENSE, KIND_SPARSE, KIND_GATED = 0, 1, 2
DT_BF16, DT_FP16, DT_E4M3, DT_E5M2, DT_F32 = 0, 1, 2, 3, 4

F_CAUSAL = 1 << 0
F_LOCAL = 1 << 1
F_SPLIT = 1 << 2
F_PACK_GQA = 1 << 3
F_LOGSIGMOID = 1 << 4
F_ADAPT_GATE = 1 << 5
F_DETERMINISTIC = 1 << 6


class FsaFwdArgs(ctypes.Structure):
    _fields_ = [
        ("q", c_void_p),
        ("k", c_void_p),
        ("v", c_void_p),
        ("out", c_void_p),
        ("lse", c_void_p),
        ("out_partial", c_void_p),
        ("lse_partial", c_void_p),
        ("alpha", c_void_p),
        ("delta", c_void_p),
        ("cu_seqlens_q", c_void_p),
        ("cu_seqlens_k", c_void_p),
        ("seqused_q", c_void_p),
        ("seqused_k", c_void_p),
        ("page_table", c_void_p),
        ("window_sizes", c_void_p),
        ("status", c_void_p),
        ("tile_map", c_void_p),
        ("q_stride_b", c_int64),
        ("q_stride_s", c_int64),
        ("q_stride_h", c_int64),
        ("k_stride_b", c_int64),
        ("k_stride_s", c_int64),
        ("k_stride_h", c_int64),
        ("v_stride_b", c_int64),
        ("v_stride_s", c_int64),
        ("v_stride_h", c_int64),
        ("o_stride_b", c_int64),
        ("o_stride_s", c_int64),
        ("o_stride_h", c_int64),
        ("lse_stride_b", c_int64),
        ("lse_stride_h", c_int64),
        ("alpha_stride_b", c_int64),
        ("alpha_stride_h", c_int64),
        ("delta_stride_b", c_int64),
        ("delta_stride_h", c_int64),
        ("batch", c_int32),
        ("seqlen_q", c_int32),
        ("seqlen_k", c_int32),
        ("total_q", c_int32),
        ("total_k", c_int32),
        ("heads_q", c_int32),
        ("heads_kv", c_int32),
        ("head_dim", c_int32),
        ("num_pages", c_int32),
        ("page_size", c_int32),
        ("page_table_stride", c_int32),
        ("window_stride", c_int32),
        ("num_splits", c_int32),
        ("tile_m", c_int32),
        ("tile_n", c_int32),
        ("kind", c_int32),
        ("dtype", c_int32),
        ("flags", c_uint32),
        ("softmax_scale", c_float),
        ("softmax_threshold", c_float),
        ("gate_threshold", c_float),
        ("qkv_scale", c_void_p),
        ("gate_ws", c_void_p),
        ("q_block_scale", c_void_p),
        ("k_block_scale", c_void_p),
        ("v_block_scale", c_void_p),
        ("ev_before", c_void_p),
        ("ev_after", c_void_p),
    ]


class FsaBlockQuantArgs(ctypes.Structure):
    _fields_ = [
        ("x16", c_void_p),
        ("x8", c_void_p),
        ("scales", c_void_p),
        ("cu_seqlens", c_void_p),
        ("x_stride_b", c_int64),
        ("x_stride_s", c_int64),
        ("x_stride_h", c_int64),
        ("q_stride_b", c_int64),
        ("q_stride_s", c_int64),
        ("q_stride_h", c_int64),
        ("batch", c_int32),
        ("seqlen", c_int32),
        ("heads", c_int32),
        ("head_dim", c_int32),
        ("x_dtype", c_int32),
        ("fp8_dtype", c_int32),
        ("dequantize", c_int32),
    ]


class FsaBwdArgs(ctypes.Structure):
    _fields_ = [
        ("q", c_void_p),
        ("k", c_void_p),
        ("v", c_void_p),
        ("out", c_void_p),
        ("dout", c_void_p),
        ("lse", c_void_p),
        ("dq", c_void_p),
        ("dk", c_void_p),
        ("dv", c_void_p),
        ("lse2_ws", c_void_p),
        ("dpsum_ws", c_void_p),
        ("dq_accum", c_void_p),
        ("dk_partial", c_void_p),
        ("dv_partial", c_void_p),
        ("cu_seqlens_q", c_void_p),
        ("cu_seqlens_k", c_void_p),
        ("seqused_q", c_void_p),
        ("seqused_k", c_void_p),
        ("window_sizes", c_void_p),
        ("status", c_void_p),
        ("tile_map", c_void_p),
        ("q_stride_b", c_int64),
        ("q_stride_s", c_int64),
        ("q_stride_h", c_int64),
        ("k_stride_b", c_int64),
        ("k_stride_s", c_int64),
        ("k_stride_h", c_int64),
        ("v_stride_b", c_int64),
        ("v_stride_s", c_int64),
        ("v_stride_h", c_int64),
        ("o_stride_b", c_int64),
        ("o_stride_s", c_int64),
        ("o_stride_h", c_int64),
        ("do_stride_b", c_int64),
        ("do_stride_s", c_int64),
        ("do_stride_h", c_int64),
        ("dq_stride_b", c_int64),
        ("dq_stride_s", c_int64),
        ("dq_stride_h", c_int64),
        ("dk_stride_b", c_int64),
        ("dk_stride_s", c_int64),
        ("dk_stride_h", c_int64),
        ("lse_stride_b", c_int64),
        ("lse_stride_h", c_int64),
        ("batch", c_int32),
        ("seqlen_q", c_int32),
        ("seqlen_k", c_int32),
        ("total_q", c_int32),
        ("total_k", c_int32),
        ("heads_q", c_int32),
        ("heads_kv", c_int32),
        ("head_dim", c_int32),
        ("window_stride", c_int32),
        ("num_splits", c_int32),
        ("tile_m", c_int32),
        ("tile_n", c_int32),
        ("kind", c_int32),
        ("dtype", c_int32),
        ("flags", c_uint32),
        ("softmax_scale", c_float),
        ("softmax_threshold", c_float),
        ("gate_threshold", c_float),
        ("alpha", c_void_p),
        ("delta", c_void_p),
        ("dalpha", c_void_p),
        ("ddelta", c_void_p),
        ("alpha_ws", c_void_p),
        ("da_accum", c_void_p),
        ("dd_partial", c_void_p),
        ("alpha_stride_b", c_int64),
        ("alpha_stride_h", c_int64),
        ("delta_stride_b", c_int64),
        ("delta_stride_h", c_int64),
        ("delta_numel", c_int64),
        ("dq_order", c_void_p),
        ("dq_turn", c_void_p),
        ("gate_ws", c_void_p),
        ("ev_before", c_void_p),
        ("ev_after", c_void_p),
    ]


class FsaDecArgs(ctypes.Structure):
    _fields_ = [
        ("q", c_void_p),
        ("k", c_void_p),
        ("v", c_void_p),
        ("out", c_void_p),
        ("lse", c_void_p),
        ("out_partial", c_void_p),
        ("lse_partial", c_void_p),
        ("cu_seqlens_k", c_void_p),
        ("seqused_k", c_void_p),
        ("page_table", c_void_p),
        ("gather_kv_indices", c_void_p),
        ("window_sizes", c_void_p),
        ("alpha", c_void_p),
        ("delta", c_void_p),
        ("status", c_void_p),
        ("tile_map", c_void_p),
        ("q_stride_b", c_int64),
        ("q_stride_h", c_int64),
        ("k_stride_b", c_int64),
        ("k_stride_s", c_int64),
        ("k_stride_h", c_int64),
        ("o_stride_b", c_int64),
        ("o_stride_h", c_int64),
        ("lse_stride_b", c_int64),
        ("lse_stride_h", c_int64),
        ("alpha_stride_b", c_int64),
        ("alpha_stride_h", c_int64),
        ("delta_stride_b", c_int64),
        ("delta_stride_h", c_int64),
        ("batch", c_int32),
        ("seqlen_k", c_int32),
        ("total_k", c_int32),
        ("heads_q", c_int32),
        ("heads_kv", c_int32),
        ("head_dim", c_int32),
        ("topk", c_int32),
        ("gather_stride", c_int32),
        ("num_pages", c_int32),
        ("page_size", c_int32),
        ("page_table_stride", c_int32),
        ("window_stride", c_int32),
        ("num_splits", c_int32),
        ("partial_only", c_int32),
        ("kind", c_int32),
        ("dtype", c_int32),
        ("flags", c_uint32),
        ("softmax_scale", c_float),
        ("softmax_threshold", c_float),
        ("gate_threshold", c_float),
        ("qkv_scale", c_void_p),
        ("thr_seqlen_k", c_void_p),
        ("key_bounds", c_void_p),
        ("gather_count", c_void_p),
        ("out_partial_stride", c_int64),
        ("lse_partial_stride", c_int64),
        ("gate_ws", c_void_p),
        ("ev_before", c_void_p),
        ("ev_after", c_void_p),
        ("peers", c_void_p),
    ]


class FsaKvAppendArgs(ctypes.Structure):
    _fields_ = [
        ("k_new", c_void_p),
        ("v_new", c_void_p),
        ("k_cache", c_void_p),
        ("v_cache", c_void_p),
        ("seqused_k", c_void_p),
        ("page_table", c_void_p),
        ("free_pages", c_void_p),
        ("free_count", c_void_p),
        ("pos_ws", c_void_p),
        ("status", c_void_p),
        ("new_stride_b", c_int64),
        ("new_stride_s", c_int64),
        ("new_stride_h", c_int64),
        ("cache_stride_b", c_int64),
        ("cache_stride_s", c_int64),
        ("cache_stride_h", c_int64),
        ("batch", c_int32),
        ("new_tokens", c_int32),
        ("heads_kv", c_int32),
        ("head_dim", c_int32),
        ("capacity", c_int32),
        ("page_size", c_int32),
        ("page_table_stride", c_int32),
        ("dtype", c_int32),
    ]


PEER_MAX_RANKS = 16


class FsaIpcHandle(ctypes.Structure):
    _fields_ = [("bytes", ctypes.c_ubyte * 64)]


class FsaPeerArgs(ctypes.Structure):
    _fields_ = [("region", c_void_p * PEER_MAX_RANKS), ("world", c_int32), ("rank", c_int32), ("block_floats", c_int64)]


class FsaFwdWorkspace(ctypes.Structure):
    _fields_ = [("out_partial", c_size_t), ("lse_partial", c_size_t), ("gate_ws", c_size_t)]


class FsaBwdWorkspace(ctypes.Structure):
    _fields_ = [(n, c_size_t) for n in ("lse2_ws", "dpsum_ws", "dq_accum", "dk_partial", "dv_partial", "alpha_ws",
                                        "da_accum", "dd_partial", "gate_ws", "dq_order", "dq_turn")]


class FsaDecWorkspace(ctypes.Structure):
    _fields_ = [("out_partial", c_size_t), ("lse_partial", c_size_t), ("gate_ws", c_size_t)]


_lib = None


def lib_path() -> str:
    return _LIB_PATH


def load():
    """Load the shared library (once) and declare the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise RuntimeError(
            f"{_LIB_PATH} is missing: build it with `python build.py` next to csrc/ "
            "(this package has no fallback path)"
        )
    lib = ctypes.CDLL(_LIB_PATH)
    lib.fsa_abi_version.restype = c_int
    lib.fsa_status_string.restype = ctypes.c_char_p
    lib.fsa_status_string.argtypes = [c_int]
    lib.fsa_fwd.restype = c_int
    lib.fsa_fwd.argtypes = [POINTER(FsaFwdArgs), c_void_p]
    lib.fsa_fwd_tile_map_bytes.restype = c_size_t
    lib.fsa_fwd_tile_map_bytes.argtypes = [POINTER(FsaFwdArgs)]
    lib.fsa_bwd.restype = c_int
    lib.fsa_bwd.argtypes = [POINTER(FsaBwdArgs), c_void_p]
    lib.fsa_bwd_padded_rows.restype = c_int64
    lib.fsa_bwd_padded_rows.argtypes = [c_int, c_int, c_int, c_int]
    lib.fsa_decode.restype = c_int
    lib.fsa_decode.argtypes = [POINTER(FsaDecArgs), c_void_p]
    lib.fsa_combine.restype = c_int
    lib.fsa_combine.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int64,
                                c_int64, c_void_p]
    lib.fsa_quantize_fp8.restype = c_int
    lib.fsa_quantize_fp8.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]
    lib.fsa_fp8_widen.restype = c_int
    lib.fsa_fp8_widen.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p]
    lib.fsa_topk_indices.restype = c_int
    lib.fsa_topk_indices.argtypes = [c_void_p, c_int, c_int, c_int, c_int64, c_int, c_void_p, c_int, c_void_p]
    lib.fsa_quantize_fp8_blockwise.restype = c_int
    lib.fsa_quantize_fp8_blockwise.argtypes = [POINTER(FsaBlockQuantArgs), c_void_p]
    lib.fsa_kv_append.restype = c_int
    lib.fsa_kv_append.argtypes = [POINTER(FsaKvAppendArgs), c_void_p]
    lib.fsa_localize_indices.restype = c_int
    lib.fsa_localize_indices.argtypes = [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_int, c_int, c_void_p]
    lib.fsa_peer_region_bytes.restype = c_int
    lib.fsa_peer_region_bytes.argtypes = [c_int, c_int64, POINTER(c_int64)]
    lib.fsa_peer_alloc.restype = c_int
    lib.fsa_peer_alloc.argtypes = [c_int64, POINTER(c_void_p), POINTER(FsaIpcHandle)]
    lib.fsa_peer_open.restype = c_int
    lib.fsa_peer_open.argtypes = [POINTER(FsaIpcHandle), POINTER(c_void_p)]
    lib.fsa_peer_close.restype = c_int
    lib.fsa_peer_close.argtypes = [c_void_p]
    lib.fsa_peer_free.restype = c_int
    lib.fsa_peer_free.argtypes = [c_void_p]
    lib.fsa_peer_push.restype = c_int
    lib.fsa_peer_push.argtypes = [POINTER(FsaPeerArgs), c_void_p, c_void_p]
    lib.fsa_peer_combine.restype = c_int
    lib.fsa_peer_combine.argtypes = [POINTER(FsaPeerArgs), c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                     c_void_p, c_void_p]
    lib.fsa_fwd_workspace_bytes.restype = c_int
    lib.fsa_fwd_workspace_bytes.argtypes = [POINTER(FsaFwdArgs), POINTER(FsaFwdWorkspace)]
    lib.fsa_bwd_workspace_bytes.restype = c_int
    lib.fsa_bwd_workspace_bytes.argtypes = [POINTER(FsaBwdArgs), POINTER(FsaBwdWorkspace)]
    lib.fsa_decode_workspace_bytes.restype = c_int
    lib.fsa_decode_workspace_bytes.argtypes = [POINTER(FsaDecArgs), POINTER(FsaDecWorkspace)]
    lib.fsa_debug_fwd_schedule.restype = None
    lib.fsa_debug_fwd_schedule.argtypes = [c_int] * 4 + [POINTER(c_int32)] + [c_int] * 7 + [POINTER(c_int32)]
    lib.fsa_debug_bwd_schedule.restype = None
    lib.fsa_debug_bwd_schedule.argtypes = [c_int] * 4 + [POINTER(c_int32)] + [c_int] * 6 + [POINTER(c_int32)]
    if lib.fsa_abi_version() != ABI_VERSION:
        raise RuntimeError("libfsa_b200.so ABI version mismatch: rebuild the library")
    _lib = lib
    return lib


def check(code: int, what: str):
    if code != 0:
        msg = load().fsa_status_string(code).decode()
        raise RuntimeError(f"{what} failed: {msg} (code {code})")


def ptr(t):
    return None if t is None else t.data_ptr()


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.bfloat16:
        return DT_BF16
    if dt == torch.float16:
        return DT_FP16
    if dt == torch.float8_e4m3fn:
        return DT_E4M3
    if dt == torch.float8_e5m2:
        return DT_E5M2
    if dt == torch.float32:
        return DT_F32
    raise TypeError(f"unsupported dtype {dt}")


_status_words = {}


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 error word shared by all launches (zeroed once, never reallocated)."""
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    t = _status_words.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[key] = t
    return t


def check_status(device=None):
    """Synchronise and raise if any kernel launched so far gave up on a bounded wait."""
    for key, t in list(_status_words.items()):
        if device is not None and torch.device(device).type != key[0]:
            continue
        v = int(t.item())
        if v != 0:
            t.zero_()
            raise RuntimeError(f"fsa kernel reported device status {v} (a pipeline wait expired)")


_profile = {"before": None, "after": None}


def set_profile_events(before=None, after=None):
    """Have the next operator calls of this process record `before` / `after` (torch.cuda.Event, already recorded
    once so that their handles exist) around their main kernel; None, None switches it off. The pair is Python
    state of this module (process-wide rather than per thread: autograd runs a backward call on a thread of its
    own) and travels in the argument block of each call (`ev_before` / `ev_after`); the library keeps no state."""
    _profile["before"] = before.cuda_event if before is not None else None
    _profile["after"] = after.cuda_event if after is not None else None


def attach_profile_events(args):
    args.ev_before = _profile["before"]
    args.ev_after = _profile["after"]


def workspace(nbytes: int, device, dtype=torch.float32):
    """A caller-owned workspace of `nbytes` bytes (size from fsa_*_workspace_bytes) viewed as `dtype`, or None."""
    if nbytes == 0:
        return None
    return torch.empty(nbytes // torch.empty((), dtype=dtype).element_size(), dtype=dtype, device=device)


def current_stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def debug_fwd_schedule(sq, sk, m_block, split_idx, window, num_splits, tile_n, tile_m, causal, local, split, gpack,
                       cover_single_query=False):
    lib = load()
    w = (c_int32 * 4)(*[int(x) for x in window])
    out = (c_int32 * 9)()
    lib.fsa_debug_fwd_schedule(sq, sk, m_block, split_idx, w, num_splits, tile_n, tile_m, int(causal), int(local),
                               int(split) | (2 if cover_single_query else 0), gpack, out)
    return list(out)


def debug_bwd_schedule(sq, sk, n_block, split_idx, window, num_splits, tile_n, tile_m, causal, local, split):
    lib = load()
    w = (c_int32 * 4)(*[int(x) for x in window])
    out = (c_int32 * 9)()
    lib.fsa_debug_bwd_schedule(sq, sk, n_block, split_idx, w, num_splits, tile_n, tile_m, int(causal), int(local),
                               int(split), out)
    return list(out)
