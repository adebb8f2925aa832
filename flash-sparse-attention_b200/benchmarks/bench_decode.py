"""Decode benchmark on the paged top-k configuration: batch 64, context lengths uniform in
[4096, 131072], 64 query heads over 8 KV heads, head size 128, 256-token pages with a permuted page
table, top-k 2048 gathered positions per sequence (seeded synthetic data; the counterpart of the
reference's tests/benchmark_decode.py, which also times CUDA-graph replays).

Prints one JSON line per case: microseconds per step and algorithmic bytes / time. Algorithmic bytes of
a top-k step: B*Hkv*topk*D*2(K,V)*elem + B*topk*4 + 2*B*Hq*D*2; of a full-context step: sum(ctx)*Hkv*D*2*elem.

    python bench_decode.py [--case topk|full|all] [--dtype bf16|fp8|all] [--iters N] [--batch B]
"""

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import flash_sparse_attn as fsa  # noqa: E402

DEV = "cuda"
HQ, HKV, D, PAGE, TOPK = 64, 8, 128, 256, 2048


def build(batch, seed=0):
    g = torch.Generator().manual_seed(seed)
    ctx = torch.randint(4096, 131073, (batch,), generator=g)
    pages_per = (ctx + PAGE - 1) // PAGE
    n_pages = int(pages_per.sum())
    table = torch.zeros(batch, int(pages_per.max()), dtype=torch.int32)
    perm = torch.randperm(n_pages, generator=g).to(torch.int32)
    o = 0
    for b in range(batch):
        n = int(pages_per[b])
        table[b, :n] = perm[o:o + n]
        o += n
    idx = torch.stack([torch.randperm(int(ctx[b]), generator=g)[:TOPK].to(torch.int32) for b in range(batch)])
    return ctx, n_pages, table.to(DEV), idx.to(DEV), ctx.to(torch.int32).to(DEV)


def tensors(dtype, n_pages, batch):
    if dtype == "bf16":
        k = torch.randn(n_pages, PAGE, HKV, D, device=DEV, dtype=torch.bfloat16)
        v = torch.randn_like(k)
        q = torch.randn(batch, HQ, D, device=DEV, dtype=torch.bfloat16)
        return q, k, v, {}, 2
    mk = lambda *s: torch.randint(0, 120, s, device=DEV, dtype=torch.uint8).view(torch.float8_e4m3fn)  # noqa: E731
    sc = torch.full((1,), 0.01, device=DEV, dtype=torch.bfloat16)
    return (mk(batch, HQ, D), mk(n_pages, PAGE, HKV, D), mk(n_pages, PAGE, HKV, D),
            dict(is_quant=True, query_scale=sc, key_scale=sc, value_scale=sc), 1)


def time_graph(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="all", choices=["topk", "full", "all"])
    ap.add_argument("--dtype", default="all", choices=["bf16", "fp8", "all"])
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--batch", type=int, default=64)
    args = ap.parse_args()
    ctx, n_pages, table, idx, used = build(args.batch)
    for dtype in (["bf16", "fp8"] if args.dtype == "all" else [args.dtype]):
        q, k, v, kw, es = tensors(dtype, n_pages, args.batch)
        for case in (["topk", "full"] if args.case == "all" else [args.case]):
            if case == "topk":
                fn = lambda: fsa.flash_sparse_attn_with_kvcache_func(  # noqa: E731
                    q, k, v, page_table=table, gather_kv_indices=idx, seqused_k=used, **kw)
                nbytes = args.batch * HKV * TOPK * D * 2 * es + args.batch * TOPK * 4 + 2 * args.batch * HQ * D * 2
            else:
                fn = lambda: fsa.flash_sparse_attn_with_kvcache_func(  # noqa: E731
                    q, k, v, page_table=table, seqused_k=used, **kw)
                nbytes = int(ctx.sum()) * HKV * D * 2 * es
            us = time_graph(fn, args.iters if case == "topk" else max(3, args.iters // 10))
            fsa.check_status()
            print(json.dumps({"case": f"paged_{case}_decode", "dtype": dtype, "batch": args.batch, "us_per_step": us,
                              "algorithmic_mb": nbytes / 1e6, "tb_per_s": nbytes / us / 1e6,
                              "cache_gb": n_pages * PAGE * HKV * D * 2 * es / 1e9}), flush=True)
        del q, k, v


if __name__ == "__main__":
    main()
