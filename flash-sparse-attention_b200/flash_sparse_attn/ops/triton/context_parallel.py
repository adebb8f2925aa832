"""Context-parallel decode: the KV sequence of every request is sharded across GPUs.

Not part of the reference (it has no multi-GPU code); it is built from the same pieces as its split-KV
decode: every rank produces the partial result of its key range exactly like one KV split
(flash_sparse_attn/ops/triton/flash_sparse_dec.py:485-489 - base-2 log-sum-exp partials), ONE NCCL
all-gather lands all partials in local memory (2.1 MB per rank at batch 64, 64 heads, head_dim 128),
and the decode combine (flash_dec_combine.py:15-153) merges them. No other collective is needed.

Sharding convention: rank r owns the logical key positions [lo_r, hi_r) of every sequence (one (lo, hi) pair per
sequence, so that sequences of different lengths can each be cut into equal parts) and holds them as a local cache
whose position 0 is global position lo_r. Gathered (top-k) indices arrive as GLOBAL positions; one small kernel
(fsa_localize_indices) keeps the ones inside [lo_r, hi_r), shifts them and moves them to the front of the row, and
the decode kernel visits only the tiles that hold them, so a rank's work shrinks with the number of shards. The
union over ranks is exactly the original index set and the step runs no eager index arithmetic. (The decode kernel
can also mask and shift global positions itself, FsaDecArgs.key_bounds, without the compaction.) The softmax threshold is normalised by the length of the WHOLE sequence on every rank
(FsaDecArgs.thr_seqlen_k); each shard still compares against its own running maximum and sum, so with a
positive threshold a shard can keep a tile that the unsharded call would skip or the other way round - the
difference is bounded by the threshold mass, as between different split counts on one GPU.

Wire format: one fp32 block of B*Hq*(D+1) elements per (rank, split): the partial outputs [B, Hq, D] followed by
the base-2 log-sum-exps [Hq, B]. The all-gather concatenates the blocks of all ranks; the combine kernel reads
them in place.

Exchange: with `exchange="peer"` (ranks on the GPUs of one node, one process per GPU) the all-gather is replaced by
the library's own kernels: every rank stores its block straight into the receive buffers of all ranks over NVLink
(`fsa_peer_push`: plain peer stores into memory mapped through CUDA IPC, an arrival counter per sender) and the
combine kernel waits, bounded, for the arrivals of the step (`fsa_peer_combine`). No multicast is involved. With
`exchange="fused"` the decode kernel itself stores its partials into the peers' buffers and counts the arrivals of its
CTAs (no push kernel): the step is localise -> decode -> combine. The default `exchange="nccl"` keeps the single NCCL
all-gather.
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
    """Global top-k positions -> positions inside the local shard [lo, hi); everything else becomes -1.
    (What the decode kernel does for `key_range = (lo, hi)`; kept for host-side checks.)"""
    inside = (gather_kv_indices >= lo) & (gather_kv_indices < hi)
    return torch.where(inside, gather_kv_indices - lo, torch.full_like(gather_kv_indices, -1))


def pack_partials(out_partial: torch.Tensor, lse_partial: torch.Tensor) -> torch.Tensor:
    """[P, B, Hq, D] and [P, Hq, B] -> the wire format [P, B*Hq*(D+1)]."""
    parts = out_partial.shape[0]
    return torch.cat([out_partial.reshape(parts, -1), lse_partial.reshape(parts, -1)], dim=1).contiguous()


def unpack_partials(packed: torch.Tensor, parts: int, batch: int, heads: int, head_dim: int):
    blocks = packed.view(parts, batch * heads * (head_dim + 1))
    n = batch * heads * head_dim
    return blocks[:, :n].reshape(parts, batch, heads, head_dim), blocks[:, n:].reshape(parts, heads, batch)


def context_parallel_decode(
    partial_fn: Callable[[], torch.Tensor],
    combine_fn: Callable[[torch.Tensor, int], Tuple[torch.Tensor, torch.Tensor]],
    group: Optional[dist.ProcessGroup] = None,
    gathered: Optional[torch.Tensor] = None,
):
    """`partial_fn()` -> this rank's partials in the wire format [P, B*Hq*(D+1)] (fp32); one all-gather; then
    `combine_fn(all_partials, world * P)` -> (out [B, Hq, D], lse [B, Hq]), identical on every rank.
    `gathered` optionally supplies the receive buffer (world * P blocks) so that the step allocates nothing."""
    packed = partial_fn()
    world = dist.get_world_size(group)
    parts = packed.shape[0]
    if world == 1:
        return combine_fn(packed, parts)
    if gathered is None:
        gathered = torch.empty((world * parts, packed.shape[1]), dtype=packed.dtype, device=packed.device)
    # concatenation along the partial axis: rank r's blocks land at [r * P, (r + 1) * P)
    dist.all_gather_into_tensor(gathered, packed, group=group)
    return combine_fn(gathered, world * parts)


class ContextParallelDecoder:
    """Sparse (or dense) decode with the KV sequence sharded over the ranks of `group`, with every buffer of the
    step allocated once: decode kernel (partials in the wire format) -> one all-gather -> combine kernel.

    `key_local / value_local` hold this rank's positions [shard_lo, shard_hi) (contiguous [B, S_local, Hkv, D], or
    paged with `page_table`); `shard_lo` may also be an int32 [B, 2] tensor of per-sequence (lo, hi) bounds; `gather_kv_indices` are GLOBAL positions; `seqused_k_global` (int32 [B]) the lengths
    of the whole sequences (normalises the softmax threshold; in gather mode it is all the kernel needs to know
    about lengths), `seqused_k_local` the number of valid keys in the local shard (full-context mode)."""

    def __init__(self, batch: int, heads_q: int, head_dim: int, dtype: torch.dtype, device, num_splits: int = 1,
                 group=None, exchange: str = "nccl"):
        assert exchange in ("nccl", "peer", "fused")
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.batch, self.heads, self.head_dim, self.dtype, self.ns = batch, heads_q, head_dim, dtype, num_splits
        per = batch * heads_q * (head_dim + 1)
        self.send = torch.empty((num_splits, per), dtype=torch.float32, device=device)
        self.recv = torch.empty((self.world * num_splits, per), dtype=torch.float32, device=device)
        self.out = torch.empty((batch, heads_q, head_dim), dtype=dtype, device=device)
        self.lse = torch.empty((batch, heads_q), dtype=torch.float32, device=device)
        self._bounds = self._bounds_key = self._idx = self._count = None
        self.peers = None
        self.fused = exchange == "fused" and self.world > 1
        if exchange in ("peer", "fused") and self.world > 1:
            self.peers = PeerExchange(num_splits * per, device, group)
        self._arrivals = 0

    def partial(self, query, key_local, value_local, shard_lo, shard_hi, gather_kv_indices=None,
                seqused_k_global=None, seqused_k_local=None, page_table=None, softmax_scale=None,
                softmax_threshold=None, kind="sparse"):
        from flash_sparse_attn.ops.triton.flash_dec import attn_decode
        from flash_sparse_attn.utils.kvcache import localize_indices as localize_on_device

        gather = gather_kv_indices is not None
        idx = count = None
        if gather:
            # one small kernel: this shard's positions, shard-local, at the front of every row, and how many - the
            # decode kernel then only visits the tiles that hold them (its work shrinks with the number of shards)
            if isinstance(shard_lo, torch.Tensor):
                bounds = shard_lo
            else:
                if self._bounds is None or self._bounds_key != (shard_lo, shard_hi):
                    self._bounds = torch.tensor([[int(shard_lo), int(shard_hi)]] * self.batch, dtype=torch.int32,
                                                device=query.device)
                    self._bounds_key = (shard_lo, shard_hi)
                bounds = self._bounds
            if self._idx is None or self._idx.shape != gather_kv_indices.shape:
                self._idx = torch.empty_like(gather_kv_indices)
                self._count = torch.empty(self.batch, dtype=torch.int32, device=query.device)
            idx, count = localize_on_device(gather_kv_indices, bounds, out=self._idx, count=self._count)
        attn_decode(kind, query, key_local, value_local, partial_only=True, num_splits=self.ns,
                    packed_partials=self.send, gather_kv_indices=idx, gather_count=count,
                    seqused_k=seqused_k_global if gather else seqused_k_local,
                    threshold_seqlen_k=None if gather else seqused_k_global, page_table=page_table,
                    softmax_scale=softmax_scale, softmax_threshold=softmax_threshold,
                    peers=self.peers.args if self.fused else None)
        # arrivals a rank counts per step when the decode kernel stores the partials itself: its CTAs
        self._arrivals = self.batch * key_local.shape[-2] * self.ns
        return self.send

    def exchange(self):
        if self.world == 1:
            return self.send
        if self.peers is not None:
            if not self.fused:
                self.peers.push(self.send)
            return None  # the partials are in the peer region; combine() waits for them
        dist.all_gather_into_tensor(self.recv, self.send, group=self.group)
        return self.recv

    def combine(self, packed):
        from flash_sparse_attn.ops.triton.flash_dec import combine_packed_partials

        if packed is None:
            return self.peers.combine(self.out, self.lse, self.ns, self.batch, self.heads, self.head_dim,
                                      arrivals=self._arrivals if self.fused else 0)
        return combine_packed_partials(packed, packed.shape[0], self.batch, self.heads, self.head_dim, self.dtype,
                                       out=self.out, lse=self.lse)

    def __call__(self, *args, **kwargs):
        self.partial(*args, **kwargs)
        return self.combine(self.exchange())


class PeerExchange:
    """The receive region of this rank and the mapped regions of the others (see the module docstring). Set-up is
    collective over `group` (one all-gather of the 64-byte handles through the process group) and synchronises;
    `push` / `combine` only enqueue kernels and can be captured in a CUDA graph. Every rank must run the same
    sequence of push / combine pairs."""

    def __init__(self, block_floats: int, device, group=None):
        import ctypes

        from flash_sparse_attn import _lib

        self._lib = _lib
        self.device = torch.device(device)
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        assert self.world <= _lib.PEER_MAX_RANKS and block_floats % 4 == 0
        lib = _lib.load()
        nbytes = ctypes.c_int64()
        _lib.check(lib.fsa_peer_region_bytes(self.world, block_floats, ctypes.byref(nbytes)), "fsa_peer_region_bytes")
        own, handle = ctypes.c_void_p(), _lib.FsaIpcHandle()
        with torch.cuda.device(self.device):
            _lib.check(lib.fsa_peer_alloc(nbytes.value, ctypes.byref(own), ctypes.byref(handle)), "fsa_peer_alloc")
        self._own = own.value
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle.bytes), group=group)
        self.args = _lib.FsaPeerArgs()
        self.args.world, self.args.rank, self.args.block_floats = self.world, self.rank, block_floats
        self._opened = []
        with torch.cuda.device(self.device):
            for r in range(self.world):
                if r == self.rank:
                    self.args.region[r] = self._own
                    continue
                h = _lib.FsaIpcHandle()
                ctypes.memmove(h.bytes, handles[r], 64)
                ptr = ctypes.c_void_p()
                _lib.check(lib.fsa_peer_open(ctypes.byref(h), ctypes.byref(ptr)), "fsa_peer_open")
                self.args.region[r] = ptr.value
                self._opened.append(ptr.value)
        dist.barrier(group=group)  # every region is zeroed and mapped before anybody sends

    def push(self, block: torch.Tensor):
        import ctypes

        assert block.dtype == torch.float32 and block.is_contiguous() and block.numel() == self.args.block_floats
        with torch.cuda.device(self.device):
            rc = self._lib.load().fsa_peer_push(ctypes.byref(self.args), block.data_ptr(),
                                                self._lib.current_stream_ptr(self.device))
        self._lib.check(rc, "fsa_peer_push")

    def combine(self, out, lse, partials_per_rank, batch, heads, head_dim, arrivals: int = 0):
        import ctypes

        status = self._lib.status_word(self.device)
        with torch.cuda.device(self.device):
            rc = self._lib.load().fsa_peer_combine(ctypes.byref(self.args), out.data_ptr(), lse.data_ptr(),
                                                   partials_per_rank, batch, heads, head_dim,
                                                   self._lib.dtype_code(out.dtype), arrivals, status.data_ptr(),
                                                   self._lib.current_stream_ptr(self.device))
        self._lib.check(rc, "fsa_peer_combine")
        return out, lse

    def close(self):
        """Unmap the other ranks' regions and free this rank's (after all ranks have finished their last step)."""
        lib = self._lib.load()
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            for ptr in self._opened:
                lib.fsa_peer_close(ptr)
            self._opened = []
            if self._own:
                lib.fsa_peer_free(self._own)
                self._own = None


def flash_sparse_attn_with_kvcache_cp(query, key_local, value_local, shard_lo: int, shard_hi: int,
                                      gather_kv_indices=None, seqused_k_local=None, page_table=None,
                                      softmax_scale=None, softmax_threshold=None, num_splits: int = 1, kind="sparse",
                                      group=None, seqused_k_global=None):
    """One-shot form of ContextParallelDecoder (allocates its buffers on every call)."""
    dec = ContextParallelDecoder(query.shape[0], query.shape[1], query.shape[2],
                                 torch.bfloat16 if query.dtype.itemsize == 1 else query.dtype, query.device,
                                 num_splits=num_splits, group=group)
    out, lse = dec(query, key_local, value_local, shard_lo, shard_hi, gather_kv_indices=gather_kv_indices,
                   seqused_k_global=seqused_k_global, seqused_k_local=seqused_k_local, page_table=page_table,
                   softmax_scale=softmax_scale, softmax_threshold=softmax_threshold, kind=kind)
    return out, lse
