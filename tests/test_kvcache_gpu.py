"""KV-cache append (contiguous and paged, with device-side page allocation) and index localisation for a sharded
cache, through the C ABI, against plain torch indexing; then a decode step on the appended cache."""

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _sync():
    import flash_sparse_attn as fsa

    torch.cuda.synchronize()
    fsa.check_status()


def test_append_contiguous_cache():
    from flash_sparse_attn.utils.kvcache import append_kv

    g = torch.Generator().manual_seed(0)
    b, cap, hkv, d, t = 5, 300, 4, 128, 3
    kc = torch.randn(b, cap, hkv, d, generator=g).to(torch.bfloat16).to(DEV)
    vc = torch.randn(b, cap, hkv, d, generator=g).to(torch.bfloat16).to(DEV)
    kn = torch.randn(b, t, hkv, d, generator=g).to(torch.bfloat16).to(DEV)
    vn = torch.randn(b, t, hkv, d, generator=g).to(torch.bfloat16).to(DEV)
    used = torch.tensor([0, 7, 100, 296, 297], dtype=torch.int32, device=DEV)
    ref_k, ref_v = kc.clone(), vc.clone()
    for i, u in enumerate(used.tolist()):
        ref_k[i, u:u + t], ref_v[i, u:u + t] = kn[i], vn[i]
    append_kv(kn, vn, kc, vc, used)
    _sync()
    assert torch.equal(kc, ref_k) and torch.equal(vc, ref_v)
    assert used.tolist() == [3, 10, 103, 299, 300]


def test_append_paged_cache_allocates_pages_and_feeds_decode():
    import flash_sparse_attn as fsa
    from flash_sparse_attn.utils.kvcache import append_kv
    from oracle import eager

    g = torch.Generator().manual_seed(1)
    b, page, hq, hkv, d, max_pages, n_pages = 3, 64, 8, 2, 128, 6, 24
    kc = torch.zeros(n_pages, page, hkv, d, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    table = torch.full((b, max_pages), -1, dtype=torch.int32, device=DEV)
    free = torch.randperm(n_pages, generator=g).to(torch.int32).to(DEV)
    free_count = torch.tensor([n_pages], dtype=torch.int32, device=DEV)
    used = torch.zeros(b, dtype=torch.int32, device=DEV)
    # prefill of different lengths (one call per chunk), then single-token steps that cross page boundaries
    logical_k = [torch.zeros(0, hkv, d, dtype=torch.bfloat16) for _ in range(b)]
    logical_v = [torch.zeros(0, hkv, d, dtype=torch.bfloat16) for _ in range(b)]
    for t in (60, 3, 1, 1, 70, 1):
        kn = torch.randn(b, t, hkv, d, generator=g).to(torch.bfloat16)
        vn = torch.randn(b, t, hkv, d, generator=g).to(torch.bfloat16)
        append_kv(kn.to(DEV), vn.to(DEV), kc, vc, used, page_table=table, free_pages=free, free_count=free_count)
        for i in range(b):
            logical_k[i] = torch.cat([logical_k[i], kn[i]])
            logical_v[i] = torch.cat([logical_v[i], vn[i]])
    _sync()
    total = 136
    assert used.tolist() == [total] * b
    assert int(free_count.item()) == n_pages - b * 3          # three pages per sequence
    tab = table.cpu()
    assert (tab[:, :3] >= 0).all() and (tab[:, 3:] == -1).all()
    assert len(set(tab[:, :3].flatten().tolist())) == 3 * b    # no page handed out twice
    for i in range(b):
        got = kc[tab[i, :3].long().to(DEV)].reshape(-1, hkv, d)[:total].cpu()
        assert torch.equal(got, logical_k[i])
    q = torch.randn(b, hq, d, generator=g).to(torch.bfloat16)
    out = fsa.flash_sparse_attn_with_kvcache_func(q.to(DEV), kc, vc, page_table=table, seqused_k=used,
                                                  softmax_threshold=-128.0)
    _sync()
    ref = eager.decode(q, torch.stack(logical_k), torch.stack(logical_v))
    assert (out.float().cpu() - ref.float()).abs().max().item() < 2e-2


def test_append_reports_exhausted_free_list():
    import flash_sparse_attn as fsa
    from flash_sparse_attn.utils.kvcache import append_kv

    b, page, hkv, d = 2, 32, 1, 64
    kc = torch.zeros(1, page, hkv, d, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    table = torch.full((b, 2), -1, dtype=torch.int32, device=DEV)
    free = torch.zeros(1, dtype=torch.int32, device=DEV)
    free_count = torch.ones(1, dtype=torch.int32, device=DEV)
    used = torch.zeros(b, dtype=torch.int32, device=DEV)
    kn = torch.ones(b, 1, hkv, d, dtype=torch.bfloat16, device=DEV)
    append_kv(kn, kn, kc, vc, used, page_table=table, free_pages=free, free_count=free_count)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="device status 3"):
        fsa.check_status()
    assert int(free_count.item()) == 0 and int((table >= 0).sum()) == 1


def test_localize_indices_matches_host_arithmetic():
    from flash_sparse_attn.ops.triton import context_parallel as cp
    from flash_sparse_attn.utils.kvcache import localize_indices

    g = torch.Generator().manual_seed(2)
    rows, topk = 7, 333
    idx = torch.randint(-3, 5000, (rows, topk), generator=g).to(torch.int32)
    bounds = torch.tensor([[0, 5000], [1000, 2000], [4000, 4001], [0, 0], [2500, 5000], [17, 4999], [3000, 3100]],
                          dtype=torch.int32)
    local, count = localize_indices(idx.to(DEV), bounds.to(DEV))
    _sync()
    for r in range(rows):
        lo, hi = bounds[r].tolist()
        ref = cp.localize_indices(idx[r], lo, hi)
        kept = ref[ref >= 0]
        assert int(count[r]) == kept.numel()
        assert torch.equal(local[r, :kept.numel()].cpu(), kept)
        assert (local[r, kept.numel():] == -1).all()
