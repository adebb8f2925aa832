"""Run ANOTHER installation of the `flash_sparse_attn` operator package (the upstream Triton back end) on the
seeded workloads of benchmarks/workloads.py and save its results and timings.

The upstream package and this repository's package share the import name, so this script runs in a process
of its own (started by tests/test_ref_triton_gpu.py or by hand) with the upstream installation directory put first
on sys.path; it never imports this repository's package.

    python tests/ref_triton_runner.py --ref-dir DIR --case c2|s16k|s16k_llm|c3|c4|c5 --out FILE.pt [--reps N]
                                      [--tile 128] [--autotune] [--no-bwd] [--small]

FILE.pt receives {"case", "results": {name: cpu tensor}, "ms": {...}, "error": str | None, "tile", "autotune"}.
"""

import argparse
import importlib.util
import os
import sys
import tempfile
import traceback

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def load_workloads():
    path = os.path.join(ROOT, "flash-sparse-attention_b200", "benchmarks", "workloads.py")
    spec = importlib.util.spec_from_file_location("fsa_workloads", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def time_ms(fn, reps):
    import torch

    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref-dir", required=True)
    ap.add_argument("--case", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--tile", type=int, default=128)
    ap.add_argument("--autotune", action="store_true")
    ap.add_argument("--no-bwd", action="store_true")
    ap.add_argument("--small", action="store_true", help="reduced batch (parity runs)")
    args = ap.parse_args()

    cfg_dir = tempfile.mkdtemp(prefix="fsa_ref_cfg_")
    os.environ.setdefault("FLASH_SPARSE_ATTENTION_LAUNCH_CONFIG_DIR", cfg_dir)
    os.environ.setdefault("TRITON_CACHE_DIR", os.path.join(cfg_dir, "triton"))
    sys.path.insert(0, os.path.abspath(args.ref_dir))
    import torch

    record = {"case": args.case, "results": {}, "ms": {}, "error": None, "tile": args.tile, "autotune": args.autotune}
    try:
        import flash_sparse_attn as ref

        assert os.path.abspath(ref.__file__).startswith(os.path.abspath(args.ref_dir)), ref.__file__
        wl = load_workloads()
        dev = "cuda"
        tune = dict(is_autotune=True) if args.autotune else dict(is_autotune=False, tile_mn=(args.tile, args.tile))
        res, ms = record["results"], record["ms"]

        def fwd_bwd(op, w, lead, grads):
            leaves = [t.detach().requires_grad_(True) for t in lead]
            kw = dict(w["kwargs"], **tune)
            out = op(*leaves, **kw)
            res["out"] = out.detach().cpu()
            if not args.no_bwd:
                out.backward(w["dout"])
                for n, t in zip(grads, leaves):
                    res[n] = t.grad.detach().cpu()
            torch.cuda.synchronize()
            with torch.no_grad():
                ms["fwd"] = time_ms(lambda: op(*lead, **kw), args.reps)
            if not args.no_bwd:
                def step():
                    for t in leaves:
                        t.grad = None
                    op(*leaves, **kw).backward(w["dout"])
                ms["fwd_bwd"] = time_ms(step, args.reps)

        if args.case == "c2":
            w = wl.c2(dev, batch=1 if args.small else 2)
            fwd_bwd(ref.flash_sparse_attn_func, w, (w["q"], w["k"], w["v"]), ("dq", "dk", "dv"))
        elif args.case in ("s16k", "s16k_llm"):
            w = wl.s16k(dev, data="iid" if args.case == "s16k" else "llm")
            fwd_bwd(ref.flash_sparse_attn_func, w, (w["q"], w["k"], w["v"]), ("dq", "dk", "dv"))
        elif args.case == "c3":
            w = wl.c3(dev, batch=1 if args.small else 4)
            fwd_bwd(ref.flash_gated_attn_func, w, (w["q"], w["k"], w["v"], w["alpha"], w["delta"]),
                    ("dq", "dk", "dv", "dalpha", "ddelta"))
        elif args.case == "c4":
            w = wl.c4(dev, n_seq=4 if args.small else 16)
            # bf16: upstream's FP8 (is_quant) path on packed sequences ended with "Triton Error [CUDA]: misaligned
            # address" on a B200 and is not run again
            fwd_bwd(ref.flash_sparse_attn_varlen_func, w, (w["q"], w["k"], w["v"]), ("dq", "dk", "dv"))
        elif args.case == "c5":
            w = wl.c5(dev, batch=8 if args.small else 64, paged=False)
            kw = dict(w["kwargs"], softmax_threshold=1.0)
            kw.pop("seqused_k")
            if args.autotune:
                kw["is_autotune"] = True
            else:
                kw["is_autotune"] = False
            op = ref.flash_sparse_attn_with_kvcache_func
            res["out"] = op(w["q"], w["k"], w["v"], **kw).cpu()
            torch.cuda.synchronize()
            ms["decode"] = time_ms(lambda: op(w["q"], w["k"], w["v"], **kw), max(args.reps, 10))
            g = torch.cuda.CUDAGraph()
            try:
                with torch.cuda.graph(g):
                    op(w["q"], w["k"], w["v"], **kw)
                ms["decode_graph"] = time_ms(g.replay, max(args.reps, 20))
            except Exception as e:  # noqa: BLE001
                ms["decode_graph_error"] = repr(e)[:200]
        else:
            raise ValueError(args.case)
    except Exception:  # noqa: BLE001
        record["error"] = traceback.format_exc()[-2000:]
    torch.save(record, args.out)
    print({"case": args.case, "ms": record["ms"], "error": record["error"]})


if __name__ == "__main__":
    main()
