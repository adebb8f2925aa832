"""GPU parity of the decode operators (through the C ABI) against the CPU oracle and the golden
fixtures: contiguous, packed, paged and gathered KV, their combination, local windows, splits."""

import pytest
import torch

from fixtures import assert_close, load
from oracle import eager

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ops():
    import flash_sparse_attn as fsa

    return fsa


def _sync():
    torch.cuda.synchronize()
    _ops().check_status()


def _qkv(seed, b, sk, hq, hkv, d, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(b, hq, d, generator=g).to(dtype), torch.randn(b, sk, hkv, d, generator=g).to(dtype),
            torch.randn(b, sk, hkv, d, generator=g).to(dtype))


def test_golden_decode():
    fsa = _ops()
    g = load("decode")
    q, k, v = (g[n].to(DEV) for n in ("q", "k", "v"))
    out, lse = fsa.flash_dense_attn_with_kvcache_func(q, k, v, return_lse=True)
    _sync()
    assert_close("dense", out, g["out_dense"])
    out = fsa.flash_sparse_attn_with_kvcache_func(q, k, v, softmax_threshold=-128.0)
    _sync()
    assert_close("sparse", out, g["out_dense"])
    cu = g["cu_seqlens"].to(torch.int32).to(DEV)
    out = fsa.flash_sparse_attn_varlen_with_kvcache_func(q, g["k_packed"].to(DEV), g["v_packed"].to(DEV), cu, 200,
                                                         softmax_threshold=-128.0)
    _sync()
    assert_close("varlen", out, g["out_varlen"])
    out = fsa.flash_sparse_attn_with_kvcache_func(q, k, v, softmax_threshold=-128.0,
                                                  gather_kv_indices=g["gather_idx"].to(torch.int32).to(DEV))
    _sync()
    assert_close("gather", out, g["out_gather"], rtol=2.5e-2, atol=2.5e-2)


def test_golden_local_decode():
    fsa = _ops()
    g = load("decode_local")
    b, s, hq, hkv, d = g["shape"].tolist()
    torch.manual_seed(int(g["seed"]))
    q = torch.randn(b, hq, d, dtype=torch.bfloat16)
    k = torch.randn(b, s, hkv, d, dtype=torch.bfloat16)
    v = torch.randn(b, s, hkv, d, dtype=torch.bfloat16)
    for ns in (None, 1, 3):
        out = fsa.flash_sparse_attn_with_kvcache_func(q.to(DEV), k.to(DEV), v.to(DEV), is_local=True,
                                                      softmax_threshold=-128.0, num_splits=ns)
        _sync()
        assert_close(f"local-{ns}", out, g["out"])


# the reference's decode grid (tests/test_sparse_base_decode.py): output buffers x local x head_dim
@pytest.mark.parametrize("kind", ["dense", "sparse"])
@pytest.mark.parametrize("use_buffers", [False, True])
@pytest.mark.parametrize("local", [False, True])
@pytest.mark.parametrize("head_dim", [64, 128])
@pytest.mark.parametrize("hq,hkv", [(32, 2), (8, 8), (6, 2)])
def test_decode_grid(kind, use_buffers, local, head_dim, hq, hkv):
    fsa = _ops()
    b, sk = 2, 1500
    q, k, v = _qkv(0, b, sk, hq, hkv, head_dim)
    ws = torch.tensor([[32, 200, 100, 160]] * hkv, dtype=torch.int32) if local else None
    if local:
        ws[-1] = torch.tensor([0, 300, 0, 64], dtype=torch.int32)
    ref, ref_lse = eager.decode(q, k, v, is_local=local, window_sizes=ws, return_lse=True)
    out_buf = torch.empty(b, hq, head_dim, dtype=torch.bfloat16, device=DEV) if use_buffers else None
    lse_buf = torch.empty(b, hq, dtype=torch.float32, device=DEV) if use_buffers else None
    fn = fsa.flash_dense_attn_with_kvcache_func if kind == "dense" else fsa.flash_sparse_attn_with_kvcache_func
    kw = {} if kind == "dense" else {"softmax_threshold": -128.0}
    out, lse = fn(q.to(DEV), k.to(DEV), v.to(DEV), window_sizes=ws.to(DEV) if local else None, out=out_buf,
                  lse=lse_buf, return_lse=True, **kw)
    _sync()
    if use_buffers:
        assert out.data_ptr() == out_buf.data_ptr() and lse.data_ptr() == lse_buf.data_ptr()
    assert_close("decode", out, ref)
    assert torch.allclose(lse.cpu(), ref_lse, rtol=0, atol=2e-3)


@pytest.mark.parametrize("page_size", [32, 64, 128, 256])
@pytest.mark.parametrize("with_gather", [False, True])
def test_paged_and_gathered_decode(page_size, with_gather):
    """Permuted page table (tests/test_paged_kv.py) and random top-k lists with masked entries
    (tests/test_topk_gather_decode.py:36-52), alone and combined."""
    fsa = _ops()
    b, hq, hkv, d = 3, 16, 2, 128
    max_pages = 2048 // page_size
    num_pages = b * max_pages + 7
    g = torch.Generator().manual_seed(page_size)
    q = torch.randn(b, hq, d, generator=g).to(torch.bfloat16)
    kc = torch.randn(num_pages, page_size, hkv, d, generator=g).to(torch.bfloat16)
    vc = torch.randn(num_pages, page_size, hkv, d, generator=g).to(torch.bfloat16)
    table = torch.randperm(num_pages, generator=g)[: b * max_pages].reshape(b, max_pages).to(torch.int32)
    used = torch.tensor([2048, 1111, 300], dtype=torch.int32)
    kl, vl = eager.unpage(kc, table), eager.unpage(vc, table)
    if with_gather:
        topk = 256
        idx = torch.full((b, topk), -1, dtype=torch.int32)
        for i in range(b):
            n = min(topk, int(used[i]))
            idx[i, :n] = torch.randperm(int(used[i]), generator=g)[:n].to(torch.int32)
            idx[i, i::23] = -1
        ref = eager.gather_decode(q, kl, vl, idx)
        out = fsa.flash_sparse_attn_with_kvcache_func(q.to(DEV), kc.to(DEV), vc.to(DEV), page_table=table.to(DEV),
                                                      gather_kv_indices=idx.to(DEV), softmax_threshold=-128.0)
    else:
        ref = eager.decode(q, kl, vl, seqused_k=used)
        out = fsa.flash_sparse_attn_with_kvcache_func(q.to(DEV), kc.to(DEV), vc.to(DEV), page_table=table.to(DEV),
                                                      seqused_k=used.to(DEV), softmax_threshold=-128.0)
    _sync()
    assert_close("paged", out, ref, rtol=2.5e-2, atol=2.5e-2)


def test_contiguous_topk_equals_regular_decode():
    """Gathering positions 0..Sk-1 in order is the plain decode (tests/test_topk_gather_decode.py:321-397)."""
    fsa = _ops()
    q, k, v = _qkv(3, 2, 777, 8, 2, 128)
    idx = torch.arange(777, dtype=torch.int32).repeat(2, 1)
    a = fsa.flash_dense_attn_with_kvcache_func(q.to(DEV), k.to(DEV), v.to(DEV), num_splits=1)
    b_ = fsa.flash_dense_attn_with_kvcache_func(q.to(DEV), k.to(DEV), v.to(DEV), gather_kv_indices=idx.to(DEV),
                                                num_splits=1)
    _sync()
    assert torch.equal(a, b_)


def test_decode_is_graph_capturable():
    """The decode call does no host synchronisation or allocation once buffers are supplied, so it
    can be captured and replayed (the usage README.md:136-164 of the reference describes)."""
    fsa = _ops()
    q, k, v = _qkv(4, 4, 2048, 16, 2, 128)
    q, k, v = q.to(DEV), k.to(DEV), v.to(DEV)
    out = torch.empty_like(q)
    lse = torch.empty(4, 16, dtype=torch.float32, device=DEV)
    fsa.flash_sparse_attn_with_kvcache_func(q, k, v, out=out, lse=lse, num_splits=1)  # warm-up outside capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fsa.flash_sparse_attn_with_kvcache_func(q, k, v, out=out, lse=lse, num_splits=1)
    out.zero_()
    graph.replay()
    _sync()
    ref = eager.decode(q.cpu(), k.cpu(), v.cpu())
    assert_close("graph", out, ref)


def test_decode_skip_map():
    """Peaked scores trigger the skip rule per 16-key warp tile; the result stays within tolerance."""
    from flash_sparse_attn.ops.triton.flash_dec import attn_decode

    g = torch.Generator().manual_seed(7)
    b, sk, hq, hkv, d = 2, 4096, 16, 2, 128
    k = torch.randn(b, sk, hkv, d, generator=g)
    q = (k[:, -1].repeat_interleave(hq // hkv, dim=1) * 3).to(torch.bfloat16)
    k = k.to(torch.bfloat16)
    v = torch.randn(b, sk, hkv, d, generator=g).to(torch.bfloat16)
    tmap = torch.zeros(b * hkv * (sk // 16), dtype=torch.uint8, device=DEV)
    out, _ = attn_decode("sparse", q.to(DEV), k.to(DEV), v.to(DEV), softmax_threshold=1.0, num_splits=2, tile_map=tmap)
    _sync()
    assert (tmap == 2).sum().item() > 0 and (tmap != 0).all()
    ref = eager.decode(q, k, v)
    assert_close("skip", out, ref, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("mode", ["gather", "full"])
@pytest.mark.parametrize("splits", [1, 2])
def test_sharded_decode_pieces_on_one_gpu(mode, splits):
    """The per-rank pieces of context-parallel decode, run one after the other on a single GPU: every 'rank' decodes
    its key range into the wire format (global top-k positions localised inside the kernel via key_range, threshold
    normalised by the whole length), the blocks are concatenated as an all-gather would, one combine merges them."""
    from flash_sparse_attn.ops.triton import context_parallel as cp
    from flash_sparse_attn.ops.triton.flash_dec import attn_decode, combine_packed_partials
    from flash_sparse_attn.utils.kvcache import localize_indices

    g = torch.Generator().manual_seed(21)
    b, sk, hq, hkv, d, topk, world = 3, 2300, 16, 2, 128, 384, 3
    q = torch.randn(b, hq, d, generator=g).to(torch.bfloat16).to(DEV)
    k = torch.randn(b, sk, hkv, d, generator=g).to(torch.bfloat16).to(DEV)
    v = torch.randn(b, sk, hkv, d, generator=g).to(torch.bfloat16).to(DEV)
    idx = torch.stack([torch.randperm(sk, generator=g)[:topk] for _ in range(b)]).to(torch.int32).to(DEV)
    idx[:, 7::23] = -1
    used = torch.full((b,), sk, dtype=torch.int32, device=DEV)
    per = b * hq * (d + 1)
    recv = torch.empty(world * splits, per, dtype=torch.float32, device=DEV)
    for r in range(world):
        lo, hi = cp.shard_bounds(sk, world, r)
        send = recv[r * splits:(r + 1) * splits]
        kl, vl = k[:, lo:hi].contiguous(), v[:, lo:hi].contiguous()
        if mode == "gather" and r == 1:   # masking and shifting inside the decode kernel
            attn_decode("sparse", q, kl, vl, partial_only=True, num_splits=splits, packed_partials=send,
                        gather_kv_indices=idx, key_range=(lo, hi), seqused_k=used, softmax_threshold=-128.0)
        elif mode == "gather":            # compacted by fsa_localize_indices: only the tiles that hold indices
            bounds = torch.tensor([[lo, hi]] * b, dtype=torch.int32, device=DEV)
            local, count = localize_indices(idx, bounds)
            attn_decode("sparse", q, kl, vl, partial_only=True, num_splits=splits, packed_partials=send,
                        gather_kv_indices=local, gather_count=count, seqused_k=used, softmax_threshold=-128.0)
        else:
            attn_decode("sparse", q, kl, vl, partial_only=True, num_splits=splits, packed_partials=send,
                        threshold_seqlen_k=used, softmax_threshold=-128.0)
    out, lse = combine_packed_partials(recv, world * splits, b, hq, d, torch.bfloat16)
    kw = dict(gather_kv_indices=idx) if mode == "gather" else {}
    ref, ref_lse = attn_decode("sparse", q, k, v, softmax_threshold=-128.0, num_splits=1, **kw)
    _sync()
    assert_close(f"sharded-{mode}", out, ref)
    assert torch.allclose(lse, ref_lse, rtol=0, atol=2e-3)


@pytest.mark.parametrize("fused", [False, True])
def test_peer_exchange_kernels_single_rank(fused):
    """The peer-exchange kernels of the context-parallel decode with a group of one rank (no second GPU, no IPC
    mapping): partials go through the region's two alternating receive buffers, the arrival counters and the
    device-side step counter, eagerly and as a replayed CUDA graph. `fused`: the decode kernel stores the partials
    into the region itself; otherwise fsa_peer_push does."""
    import ctypes

    from flash_sparse_attn import _lib
    from flash_sparse_attn.ops.triton.flash_dec import attn_decode

    lib = _lib.load()
    g = torch.Generator().manual_seed(33)
    b, sk, hq, hkv, d, topk, splits = 3, 1500, 16, 2, 128, 256, 2
    q = torch.randn(b, hq, d, generator=g).to(torch.bfloat16).to(DEV)
    k = torch.randn(b, sk, hkv, d, generator=g).to(torch.bfloat16).to(DEV)
    v = torch.randn(b, sk, hkv, d, generator=g).to(torch.bfloat16).to(DEV)
    idx = torch.stack([torch.randperm(sk, generator=g)[:topk] for _ in range(b)]).to(torch.int32).to(DEV)
    per = b * hq * (d + 1)
    nbytes = ctypes.c_int64()
    assert lib.fsa_peer_region_bytes(1, splits * per, ctypes.byref(nbytes)) == 0
    region, handle = ctypes.c_void_p(), _lib.FsaIpcHandle()
    assert lib.fsa_peer_alloc(nbytes.value, ctypes.byref(region), ctypes.byref(handle)) == 0
    try:
        args = _lib.FsaPeerArgs()
        args.region[0], args.world, args.rank, args.block_floats = region.value, 1, 0, splits * per
        send = torch.empty(splits, per, dtype=torch.float32, device=DEV)
        out = torch.empty(b, hq, d, dtype=torch.bfloat16, device=DEV)
        lse = torch.empty(b, hq, dtype=torch.float32, device=DEV)
        status = _lib.status_word(torch.device(DEV))

        def step(qq):
            attn_decode("sparse", qq, k, v, partial_only=True, num_splits=splits, packed_partials=send,
                        gather_kv_indices=idx, softmax_threshold=-128.0, peers=args if fused else None)
            stream = _lib.current_stream_ptr(torch.device(DEV))
            if not fused:
                assert lib.fsa_peer_push(ctypes.byref(args), send.data_ptr(), stream) == 0
            arrivals = b * hkv * splits if fused else 0
            assert lib.fsa_peer_combine(ctypes.byref(args), out.data_ptr(), lse.data_ptr(), splits, b, hq, d,
                                        _lib.dtype_code(torch.bfloat16), arrivals, status.data_ptr(), stream) == 0

        qs = [q, (q.float() * 0.5).to(torch.bfloat16), (q.float() * -1.0).to(torch.bfloat16)]
        for qq in qs:  # three steps: both receive buffers, different data each time
            step(qq)
            ref, ref_lse = attn_decode("sparse", qq, k, v, gather_kv_indices=idx, softmax_threshold=-128.0, num_splits=1)
            _sync()
            assert_close("peer-single", out, ref)
            assert torch.allclose(lse, ref_lse, rtol=0, atol=2e-3)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step(q)
        ref, _ = attn_decode("sparse", q, k, v, gather_kv_indices=idx, softmax_threshold=-128.0, num_splits=1)
        for _ in range(3):
            out.zero_()
            graph.replay()
            _sync()
            assert_close("peer-single-graph", out, ref)
    finally:
        torch.cuda.synchronize()
        assert lib.fsa_peer_free(region.value) == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("head_dim", [64, 128])
@pytest.mark.parametrize("kind", ["dense", "sparse", "gated"])
def test_transposed_and_untransposed_kernels_agree(kind, head_dim, dtype):
    """Up to 8 query heads per KV head run the transposed products (S^T = K Q^T, O^T = V^T P^T), more run the
    untransposed ones. The same 16 query heads (heads 8-15 repeat heads 0-7, so that every group below holds the same
    rows and votes alike) are decoded once as one group of 16 over one KV head and once as two groups of 8 over a
    duplicated KV head: both kernels must give the same outputs (elementwise 2e-2) and log-sum-exps and, with the
    threshold on, skip the same tiles. The groups of 8 are also checked against the eager oracle."""
    from flash_sparse_attn.ops.triton.flash_dec import attn_decode

    g = torch.Generator().manual_seed(11)
    b, sk, topk = 3, 3000, 512
    k = torch.randn(b, sk, 1, head_dim, generator=g)
    idx = torch.stack([torch.randperm(sk, generator=g)[:topk].sort().values for _ in range(b)]).to(torch.int32)
    # queries peaked on one of the gathered keys, so that the threshold skips tiles
    peak = torch.stack([k[i, int(idx[i, -5]), 0] for i in range(b)])                       # [b, d]
    q8 = peak[:, None, :] * 3 + torch.randn(b, 8, head_dim, generator=g) * 0.3
    q = torch.cat([q8, q8], dim=1).to(dtype)
    k = k.to(dtype)
    v = torch.randn(b, sk, 1, head_dim, generator=g).to(dtype)
    a8 = torch.randn(b, 8, generator=g)
    alpha = torch.cat([a8, a8], dim=1).to(dtype)
    delta = torch.randn(b, sk, 1, generator=g).to(dtype)
    n_tiles = (topk + 15) // 16

    def run(rep):  # the KV head is duplicated `rep` times, every copy serves 16 / rep query heads
        kk, vv = k.repeat_interleave(rep, dim=2), v.repeat_interleave(rep, dim=2)
        dd = delta.repeat_interleave(rep, dim=2).transpose(1, 2).contiguous()  # the launcher takes [B, Hkv, Sk]
        tmap = torch.zeros(b * rep * n_tiles, dtype=torch.uint8, device=DEV)
        kw = dict(gather_kv_indices=idx.to(DEV), num_splits=1)
        if kind == "sparse":
            kw.update(softmax_threshold=1.0, tile_map=tmap)
        elif kind == "gated":
            kw.update(alpha=alpha.to(DEV), delta=dd.to(DEV), softmax_threshold=-128.0, gate_threshold=-128.0)
        out, lse = attn_decode(kind, q.to(DEV), kk.to(DEV), vv.to(DEV), **kw)
        _sync()
        return out.float().cpu(), lse.cpu(), tmap.view(b, rep, n_tiles).cpu()

    out16, lse16, map16 = run(1)   # 16 query heads per KV head: untransposed
    out8, lse8, map8 = run(2)      # 8 per KV head: transposed
    assert torch.allclose(out8, out16, rtol=2e-2, atol=2e-2), float((out8 - out16).abs().max())
    assert torch.allclose(lse8, lse16, rtol=0, atol=2e-3)
    if kind == "sparse":
        assert int((map16 == 2).sum()) > 0, "the peaked inputs were meant to skip tiles"
        assert (map16 != 0).all() and (map8 != 0).all()
        assert torch.equal(map8[:, 0], map8[:, 1])
        assert float((map16[:, 0] == map8[:, 0]).float().mean()) >= 0.999
    ref = eager.gather_decode(q, k, v, idx, alpha=alpha if kind == "gated" else None,
                              delta=delta if kind == "gated" else None)
    assert_close("transposed-vs-oracle", out8.to(dtype), ref, rtol=3e-2, atol=3e-2)
