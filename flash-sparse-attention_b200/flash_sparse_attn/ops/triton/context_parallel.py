"""Context-parallel decode: the KV sequence of every request is sharded across GPUs.

Not part of the reference (it has no multi-GPU code); it is built from the same pieces as its split-KV
decode: every rank produces the partial result of its key range exactly like one KV split
(flash_sparse_attn/ops/triton/flash_sparse_dec.py:485-489 - base-2 log-sum-exp partials), one NCCL
all-gather lands all partials in local memory (2.1 MB per rank at batch 64, 64 heads, head_dim 128),
and the decode combine (flash_dec_combine.py:15-153) merges them. No other collective is needed.

Sharding convention: rank r owns the logical key positions [lo_r, hi_r) of every sequence and holds them
as a local cache whose position 0 is global position lo_r. Gathered (top-k) indices are global positions;
each rank keeps the ones inside its range and masks the others (-1), so the union over ranks is exactly the
original index set.
"""

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def shard_bounds(seqlen_k: int, world_size: int, rank: int, align: int = 256) -> Tuple[int, int]:
    """Contiguous, `align`-aligned (page-aligned) key range of `rank`; the last rank takes the remainder."""
    per = -(-seqlen_k // world_size)
    per = -(-per // align) * align
    lo = min(rank * per, seqlen_k)
    hi = min(lo + per, seqlen_k)
    return lo, hi


def localize_indices(gather_kv_indices: torch.Tensor, lo: int, hi: int) -> torch.Tensor:
    """Global top-k positions -> positions inside the local shard [lo, hi); everything else becomes -1."""
    inside = (gather_kv_indices >= lo) & (gather_kv_indices < hi)
    return torch.where(inside, gather_kv_indices - lo, torch.full_like(gather_kv_indices, -1))


def context_parallel_decode(
    partial_fn: Callable[..., Tuple[torch.Tensor, torch.Tensor]],
    combine_fn: Callable[[torch.Tensor, torch.Tensor], Tuple[torch.Tensor, torch.Tensor]],
    group: Optional[dist.ProcessGroup] = None,
    **partial_kwargs,
):
    """Run `partial_fn(**partial_kwargs)` -> (out_partial [P, B, Hq, D] fp32, lse_partial [P, Hq, B] fp32,
    base 2) on this rank's shard, all-gather the partials of all ranks, and merge them with `combine_fn`.
    Returns (out [B, Hq, D], lse [B, Hq]) - identical on every rank."""
    out_p, lse_p = partial_fn(**partial_kwargs)
    world = dist.get_world_size(group)
    if world == 1:
        return combine_fn(out_p, lse_p)
    # concatenation along the partial axis: rank r's partials land at [r * P, (r + 1) * P)
    out_all = torch.empty((world * out_p.shape[0],) + tuple(out_p.shape[1:]), dtype=out_p.dtype, device=out_p.device)
    lse_all = torch.empty((world * lse_p.shape[0],) + tuple(lse_p.shape[1:]), dtype=lse_p.dtype, device=lse_p.device)
    dist.all_gather_into_tensor(out_all, out_p.contiguous(), group=group)
    dist.all_gather_into_tensor(lse_all, lse_p.contiguous(), group=group)
    return combine_fn(out_all, lse_all)


def flash_sparse_attn_with_kvcache_cp(query, key_local, value_local, shard_lo: int, shard_hi: int,
                                      gather_kv_indices=None, seqused_k_local=None, page_table=None,
                                      softmax_scale=None, softmax_threshold=None, num_splits: int = 1, kind="sparse",
                                      group=None):
    """Sparse (or dense) decode with the KV sequence sharded over the ranks of `group`.
    `key_local/value_local` hold this rank's positions [shard_lo, shard_hi) (contiguous [B, S_local, Hkv, D]
    or paged with `page_table`); `gather_kv_indices` are global positions."""
    from flash_sparse_attn.ops.triton.flash_dec import attn_decode, combine_partials

    idx = localize_indices(gather_kv_indices, shard_lo, shard_hi) if gather_kv_indices is not None else None
    return context_parallel_decode(
        lambda **kw: attn_decode(kind, query, key_local, value_local, partial_only=True, **kw),
        lambda o, l: combine_partials(o, l, query.dtype),
        group=group, gather_kv_indices=idx, seqused_k=seqused_k_local, page_table=page_table,
        softmax_scale=softmax_scale, softmax_threshold=softmax_threshold, num_splits=num_splits,
    )
