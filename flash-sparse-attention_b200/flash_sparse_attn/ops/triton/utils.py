"""Host-side helpers with the behaviour of flash_sparse_attn/ops/triton/utils.py."""

import functools
import os
from typing import Optional

import torch


def ensure_contiguous(fn):
    """Decorator: make every tensor argument contiguous before calling ``fn(ctx, ...)``
    (reference: flash_sparse_attn/ops/triton/utils.py:26-44)."""

    @functools.wraps(fn)
    def wrapper(ctx, *args, **kwargs):
        fix = lambda x: x.contiguous() if isinstance(x, torch.Tensor) else x  # noqa: E731
        return fn(ctx, *[fix(a) for a in args], **{k: fix(v) for k, v in kwargs.items()})

    return wrapper


def _cdiv(a: int, b: int) -> int:
    return -(-a // b)


@functools.lru_cache(maxsize=4096)
def window_sizes_heuristic(
    seqlen_k: int,
    num_heads_kv: int,
    device: torch.device,
    equal_bandwidth: bool = True,
    window_near: int = 1024,
    window_sink: int = 64,
    num_heads_kv_global: Optional[int] = None,
    tp_rank: Optional[int] = None,
    tp_size: Optional[int] = None,
) -> torch.Tensor:
    """Default flex-window table, int32 ``[num_heads_kv, 4]`` with columns (sink, left, right, near).

    Every KV head sees the sink prefix and the near-diagonal band; the remaining causal distances
    are cut into one distant band per (global) KV head, of equal width (``equal_bandwidth``) or of
    equal causal area. Same numbers as flash_sparse_attn/ops/triton/utils.py:47-102.
    """
    n_global = num_heads_kv if num_heads_kv_global is None else num_heads_kv_global
    rank = tp_rank or 0
    if tp_size is not None and tp_size > n_global:
        first_head = (rank // (tp_size // n_global)) * num_heads_kv
    else:
        first_head = rank * num_heads_kv

    near = min(max(window_near, 0), seqlen_k)
    sink = min(max(window_sink, 0), max(seqlen_k - near, 0))
    span = max(seqlen_k - sink - near, 0)

    edges = torch.arange(num_heads_kv + 1, dtype=torch.float32) + first_head
    if equal_bandwidth:
        cuts = (span * edges / n_global).to(torch.int32)
    else:
        cuts = (span * (1.0 - torch.sqrt(1.0 - edges / n_global))).to(torch.int32)
    left = cuts[1:] - cuts[:-1]
    right = cuts[:-1]
    table = torch.stack([torch.full_like(left, sink), left, right, torch.full_like(left, near)], dim=1)
    return table.to(device)


@functools.lru_cache(maxsize=4096)
def num_splits_heuristic(
    seqlen_q: int,
    seqlen_k: int,
    num_SMs: int,
    TILE_M: int,
    TILE_N: int,
    is_local: bool = False,
    num_heads_kv: int = 1,
    window_near: int = 1024,
    window_sink: int = 64,
) -> int:
    """Number of KV (or QO) splits: 1 when there are at most four key tiles to share, otherwise
    enough to fill the SMs, capped by a power of two and by the tile count
    (flash_sparse_attn/ops/triton/utils.py:105-152)."""
    m_blocks = _cdiv(seqlen_q, TILE_M)
    n_blocks = _cdiv(seqlen_k, TILE_N)
    usable = n_blocks
    if is_local:
        near = min(max(window_near, 0), seqlen_k)
        sink = min(max(window_sink, 0), max(seqlen_k - near, 0))
        span = max(seqlen_k - sink - near, 0)
        widest_band = _cdiv(span, max(num_heads_kv, 1))
        per_tile = _cdiv(widest_band, TILE_N) + (1 if near > 0 else 0) + _cdiv(sink, TILE_N)
        usable = min(n_blocks, max(per_tile, 1))
    if usable <= 4:
        return 1
    pow2_cap = 1 << (max(num_SMs, 1).bit_length() - 1)
    return max(1, min(num_SMs // max(m_blocks, 1), pow2_cap, usable))


@functools.lru_cache(maxsize=16)
def device_num_sms(device: torch.device) -> int:
    return torch.cuda.get_device_properties(device).multi_processor_count


_DETERMINISTIC = os.environ.get("FSA_DETERMINISTIC", "0") not in ("", "0", "false", "False")


def set_deterministic(enabled: bool) -> None:
    """Package-wide default of the backward's deterministic dQ accumulation (also set by the
    environment variable ``FSA_DETERMINISTIC=1``). The reference has no such switch: its dQ is summed
    with atomics in arrival order (flash_sparse_attn/ops/triton/scheduler.py:2190-2192)."""
    global _DETERMINISTIC
    _DETERMINISTIC = bool(enabled)


def deterministic_enabled() -> bool:
    return _DETERMINISTIC
