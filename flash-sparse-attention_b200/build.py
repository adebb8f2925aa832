"""Build libfsa_b200.so (sm_100a only) in-tree with nvcc.

Usage: ``python build.py [--force] [--verbose]``. The library has no dependency on libcuda at link
time (the one driver entry point it needs is resolved at run time), so it loads on machines without
a GPU; compute calls then fail with an error code.
"""

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libfsa_b200.so")

SOURCES = [
    "fsa_api.cu",
    "fsa_aux.cu",
    "fsa_fwd_sm100.cu",
    "fsa_bwd_sm100.cu",
    "fsa_dec_sm100.cu",
    "fsa_static_scratch.cu",
    "fsa_quant.cu",
    "fsa_topk.cu",
    "fsa_kvcache.cu",
    "fsa_peer.cu",
]

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-O3",
    "-std=c++17",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
    "-Xptxas",
    "-v",
    "--expt-relaxed-constexpr",
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _newest_header():
    t = 0.0
    for root in (CSRC, os.path.join(HERE, "..", "include")):
        for f in os.listdir(root):
            if f.endswith((".h", ".cuh")):
                t = max(t, os.path.getmtime(os.path.join(root, f)))
    return t


def _compile(src, force, verbose):
    obj = os.path.join(OBJ, src.replace(".cu", ".o"))
    srcp = os.path.join(CSRC, src)
    if (
        not force
        and os.path.exists(obj)
        and os.path.getmtime(obj) >= max(os.path.getmtime(srcp), _newest_header())
    ):
        return obj, ""
    cmd = [_nvcc()] + NVCC_FLAGS + ["-c", srcp, "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    log = res.stdout + res.stderr
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{log}")
    with open(obj + ".log", "w") as f:
        f.write(log)
    if verbose:
        print(log)
    return obj, log


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    with ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as ex:
        results = list(ex.map(lambda s: _compile(s, force, verbose), SOURCES))
    objs = [o for o, _ in results]
    if (
        force
        or not os.path.exists(LIB)
        or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs)
    ):
        cmd = [_nvcc(), "-shared", "-o", LIB] + objs + ["-cudart", "static"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("link failed:\n" + res.stdout + res.stderr)
    return LIB


if __name__ == "__main__":
    lib = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(lib)
