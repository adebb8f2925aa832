"""Forward and decode at head sizes 128 / 192 / 256 (dense kinds, bf16): times with CUDA events.

    python benchmarks/bench_wide_heads.py [--seqlen 8192] [--iters 10]
"""

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import flash_sparse_attn as fsa  # noqa: E402


def bench(fn, iters, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seqlen", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--head-dims", type=int, nargs="+", default=[128, 192, 256])
    ap.add_argument("--no-decode", action="store_true")
    args = ap.parse_args()
    g = torch.Generator(device="cuda").manual_seed(0)
    mk = lambda *s: torch.randn(*s, device="cuda", dtype=torch.bfloat16, generator=g)  # noqa: E731
    for hd in args.head_dims:
        b, s, hq, hkv = 1, args.seqlen, 16, 4
        q, k, v = mk(b, s, hq, hd), mk(b, s, hkv, hd), mk(b, s, hkv, hd)
        with torch.no_grad():
            ms = bench(lambda: fsa.flash_dense_attn_func(q, k, v, is_causal=True), args.iters)
        flops = 4 * b * hq * hd * s * s / 2
        print(f"forward dense causal B{b} S{s} Hq{hq} Hkv{hkv} D{hd}: {ms:.3f} ms = {flops / ms / 1e9:.0f} TFLOP/s", flush=True)
        if args.no_decode:
            continue
        bb, sk = 64, 16384
        qd, kd, vd = mk(bb, 32, hd), mk(bb, sk, 4, hd), mk(bb, sk, 4, hd)
        ms = bench(lambda: fsa.flash_dense_attn_with_kvcache_func(qd, kd, vd), args.iters)
        nbytes = 2 * bb * sk * 4 * hd * 2
        print(f"decode dense B{bb} Sk{sk} Hq32 Hkv4 D{hd}: {ms * 1e3:.1f} us = {nbytes / ms / 1e9:.2f} TB/s", flush=True)
    fsa.check_status()


if __name__ == "__main__":
    main()
