"""The gated, packed + quantised and paged top-k decode benchmark configurations at their FULL sizes:
size-independent properties (run-to-run equality, rows summing to one, linearity in V, the prefix property of a
causal mask) plus slices small enough for the eager oracle. Synthetic seeded inputs with the configurations'
shapes; tile skipping is switched off (threshold -128) where a slice is compared with the oracle, whose softmax
runs over the whole mask."""

import itertools

import pytest
import torch

from fixtures import assert_close
from oracle import eager

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ops():
    import flash_sparse_attn as fsa

    return fsa


def _randn(g, *shape, dtype=torch.bfloat16):
    return torch.randn(*shape, generator=g, device=DEV, dtype=dtype)


def test_gated_config_full_size():
    """B=4, S=8192, Hq=32, Hkv=8, D=128, per-KV-head windows from {512, 1024, 2048, 4096}, logsigmoid gate."""
    fsa = _ops()
    b, s, hq, hkv, d = 4, 8192, 32, 8, 128
    g = torch.Generator(device=DEV).manual_seed(0)
    q, k, v = _randn(g, b, s, hq, d), _randn(g, b, s, hkv, d), _randn(g, b, s, hkv, d)
    a, dl = _randn(g, b, s, hq), _randn(g, b, s, hkv)
    widths = torch.tensor([512, 1024, 2048, 4096])[torch.randint(0, 4, (hkv,), generator=torch.Generator().manual_seed(0))]
    ws = torch.stack([torch.zeros(hkv, dtype=torch.long), widths, torch.zeros(hkv, dtype=torch.long),
                      torch.zeros(hkv, dtype=torch.long)], dim=1).to(torch.int32)
    kw = dict(is_causal=True, window_sizes=ws.to(DEV), softmax_threshold=-128.0, gate_threshold=-128.0)
    out = fsa.flash_gated_attn_func(q, k, v, a, dl, **kw)
    again = fsa.flash_gated_attn_func(q, k, v, a, dl, **kw)
    ones = fsa.flash_gated_attn_func(q, k, torch.ones_like(v), a, dl, **kw)
    torch.cuda.synchronize()
    fsa.check_status()
    assert torch.equal(out, again)
    assert (ones.float() - 1.0).abs().max().item() < 1e-2
    # prefix property of the causal band: rows [r0, r1) only see keys < r1, so the eager oracle on that prefix with
    # the last r1 - r0 queries (bottom-right aligned) must reproduce them
    for bi, head, r0, r1 in ((0, 3, 0, 64), (2, 17, 4000, 4064), (3, 31, 8128, 8192)):
        kvh = head // (hq // hkv)
        ref = eager.forward(q[bi:bi + 1, r0:r1, head:head + 1].cpu(), k[bi:bi + 1, :r1, kvh:kvh + 1].cpu(),
                            v[bi:bi + 1, :r1, kvh:kvh + 1].cpu(), None, True, is_local=True,
                            window_sizes=ws[kvh:kvh + 1], alpha=a[bi:bi + 1, r0:r1, head:head + 1].cpu(),
                            delta=dl[bi:bi + 1, :r1, kvh:kvh + 1].cpu())
        assert_close(f"gated-full-b{bi}-h{head}-rows{r0}", out[bi:bi + 1, r0:r1, head:head + 1], ref)


def test_gated_config_full_size_backward():
    """Same configuration, backward: dq and dalpha of a 64-row block depend only on that block's rows and on the
    keys before its end, so the eager oracle on the causal prefix reproduces them; two runs agree in dk, dv, ddelta
    bit for bit (fixed accumulation order inside a CTA) and in dq to reduction noise."""
    fsa = _ops()
    b, s, hq, hkv, d = 4, 8192, 32, 8, 128
    g = torch.Generator(device=DEV).manual_seed(4)
    q, k, v = _randn(g, b, s, hq, d), _randn(g, b, s, hkv, d), _randn(g, b, s, hkv, d)
    a, dl, do = _randn(g, b, s, hq), _randn(g, b, s, hkv), _randn(g, b, s, hq, d)
    ws = torch.tensor([[0, w, 0, 0] for w in (512, 4096, 512, 4096, 1024, 4096, 1024, 2048)], dtype=torch.int32)
    kw = dict(is_causal=True, window_sizes=ws.to(DEV), softmax_threshold=-128.0, gate_threshold=-128.0)
    grads = []
    for _ in range(2):
        leaves = [t.detach().requires_grad_(True) for t in (q, k, v, a, dl)]
        fsa.flash_gated_attn_func(*leaves, **kw).backward(do)
        torch.cuda.synchronize()
        fsa.check_status()
        grads.append([t.grad for t in leaves])
    for i in (1, 2, 4):
        assert torch.equal(grads[0][i], grads[1][i])
    assert (grads[0][0].float() - grads[1][0].float()).abs().max().item() < 2e-2
    for bi, head, r0, r1 in ((1, 6, 0, 64), (3, 31, 8128, 8192)):
        kvh = head // (hq // hkv)
        ref = eager.backward(q[bi:bi + 1, r0:r1, head:head + 1].cpu(), k[bi:bi + 1, :r1, kvh:kvh + 1].cpu(),
                             v[bi:bi + 1, :r1, kvh:kvh + 1].cpu(), do[bi:bi + 1, r0:r1, head:head + 1].cpu(), None, True,
                             is_local=True, window_sizes=ws[kvh:kvh + 1], alpha=a[bi:bi + 1, r0:r1, head:head + 1].cpu(),
                             delta=dl[bi:bi + 1, :r1, kvh:kvh + 1].cpu())
        assert_close(f"gated-full-dq-b{bi}-h{head}", grads[0][0][bi:bi + 1, r0:r1, head:head + 1], ref[0], rtol=3e-2, atol=3e-2)
        assert_close(f"gated-full-da-b{bi}-h{head}", grads[0][3][bi:bi + 1, r0:r1, head:head + 1], ref[3], rtol=3e-2, atol=3e-2)


def test_varlen_quant_config_full_size():
    """16 packed sequences with lengths in [256, 4096], Hq=32, Hkv=8, D=128, FP8 inputs from `quantize_fp8`,
    split-KV on: two of the sequences against the eager oracle on the de-quantised tensors, run-to-run equality."""
    fsa = _ops()
    hq, hkv, d = 32, 8, 128
    lens = torch.randint(256, 4097, (16,), generator=torch.Generator().manual_seed(0)).tolist()
    cu = torch.tensor([0] + list(itertools.accumulate(lens)), dtype=torch.int32)
    total = cu[-1].item()
    g = torch.Generator(device=DEV).manual_seed(1)
    q, k, v = _randn(g, total, hq, d), _randn(g, total, hkv, d), _randn(g, total, hkv, d)
    from flash_sparse_attn.ops.triton.quant import quantize_fp8

    q8, k8, v8 = (quantize_fp8(t) for t in (q, k, v))
    kw = dict(is_causal=True, softmax_threshold=-128.0, is_quant=True, query_scale=q8[1], key_scale=k8[1],
              value_scale=v8[1], is_split_kv=True)
    cud = cu.to(DEV)
    out = fsa.flash_sparse_attn_varlen_func(q8[0], k8[0], v8[0], cud, cud, max(lens), max(lens), **kw)
    again = fsa.flash_sparse_attn_varlen_func(q8[0], k8[0], v8[0], cud, cud, max(lens), max(lens), **kw)
    torch.cuda.synchronize()
    fsa.check_status()
    assert out.dtype == torch.bfloat16 and torch.equal(out, again)
    deq = [(t.float() * sc.float()).to(torch.bfloat16) for t, sc in (q8, k8, v8)]
    shortest = min(range(16), key=lambda i: lens[i])
    for i in (shortest, 15):
        lo, hi = cu[i].item(), cu[i + 1].item()
        ref = eager.forward(deq[0][lo:hi, 4:6].unsqueeze(0).cpu(), deq[1][lo:hi, 1:2].unsqueeze(0).cpu(),
                            deq[2][lo:hi, 1:2].unsqueeze(0).cpu(), None, True)
        assert_close(f"varlen-quant-full-seq{i}", out[lo:hi, 4:6].unsqueeze(0), ref, rtol=1.5e-1, atol=1.5e-1)


def test_paged_topk_decode_config_full_size():
    """B=64 sequences with 4096..131072 cached tokens, Hq=64, Hkv=8, D=128, pages of 256 tokens behind a shuffled
    page table, 2048 gathered positions per sequence: every sequence of three KV heads against the eager oracle on
    the gathered rows, replay equality, V = 1 gives 1."""
    fsa = _ops()
    b, hq, hkv, d, page, topk = 64, 64, 8, 128, 256, 2048
    ctx = torch.randint(4096, 131073, (b,), generator=torch.Generator().manual_seed(0))
    pages_per = (ctx + page - 1) // page
    n_pages = int(pages_per.sum())
    max_pages = int(pages_per.max())
    g = torch.Generator(device=DEV).manual_seed(2)
    kc = torch.randn(n_pages, page, hkv, d, generator=g, device=DEV, dtype=torch.bfloat16)
    vc = torch.randn(n_pages, page, hkv, d, generator=g, device=DEV, dtype=torch.bfloat16)
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(3)).to(torch.int32)
    table = torch.zeros(b, max_pages, dtype=torch.int32)
    start = 0
    for i in range(b):
        n = int(pages_per[i])
        table[i, :n] = perm[start:start + n]
        start += n
    idx = torch.stack([torch.randperm(int(ctx[i]), generator=torch.Generator().manual_seed(100 + i))[:topk]
                       for i in range(b)]).to(torch.int32)
    q = _randn(g, b, hq, d)
    kw = dict(page_table=table.to(DEV), seqused_k=ctx.to(torch.int32).to(DEV), gather_kv_indices=idx.to(DEV))
    out = fsa.flash_sparse_attn_with_kvcache_func(q, kc, vc, **kw)
    again = fsa.flash_sparse_attn_with_kvcache_func(q, kc, vc, **kw)
    ones = fsa.flash_sparse_attn_with_kvcache_func(q, kc, torch.ones_like(vc), **kw)
    torch.cuda.synchronize()
    fsa.check_status()
    assert torch.equal(out, again)
    assert (ones.float() - 1.0).abs().max().item() < 1e-2
    # the gathered rows of every sequence, for three KV heads: logical position -> (page, row) on the host side
    rows = table.to(DEV).long().gather(1, (idx.to(DEV).long() // page)) * page + idx.to(DEV).long() % page  # [B, topk]
    group = hq // hkv
    for kvh in (0, 3, 7):
        ks = kc.view(n_pages * page, hkv, d)[rows.reshape(-1), kvh].view(b, topk, 1, d).cpu()
        vs = vc.view(n_pages * page, hkv, d)[rows.reshape(-1), kvh].view(b, topk, 1, d).cpu()
        ref = eager.decode(q[:, kvh * group:(kvh + 1) * group].cpu(), ks, vs)
        assert_close(f"paged-topk-full-kvh{kvh}", out[:, kvh * group:(kvh + 1) * group], ref, rtol=2.5e-2, atol=2.5e-2)
