"""Generate golden/schedule.npz from the REFERENCE's own integer schedule code.

Run once on a machine that has the reference repository checked out at REF (no GPU needed):

    python tests/golden/make_schedule_golden.py REF        (or set FSA_REFERENCE_DIR)

The reference's tile schedule is Triton device code (flash_sparse_attn/ops/triton/block_info.py). This script
runs those @triton.jit functions unchanged on the CPU with TRITON_INTERPRET=1: a small wrapper kernel calls one
function for one argument set and stores the integers it returns. Stored per function: the argument rows and the
result rows. Functions covered: get_n_block_min_max (:5-123), get_m_block_min_max (:126-224),
get_n_block_min_causal_local_mask (:227-246), get_n_block_min_before_local_mask (:249-271),
get_m_block_min_causal_local_mask (:274-296), get_m_block_max_before_local_mask (:299-318),
get_topk_n_block_min_max (:321-349); and the three composed schedules AttnFwdBlockScheduler.create
(scheduler.py:836-948), AttnBwdBlockScheduler.create (:994-1101), AttnDecBlockScheduler.create (:1147-1273), whose
bodies run unchanged on a plain namespace standing in for the config aggregate (the interpreter drops the
static methods of @aggregate classes, so the undecorated class is taken from the wrapper's closure, and the
constructor call that ends each `create` is replaced by a tuple of its nine arguments).
"""

import os
import random
import sys
import types

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np  # noqa: E402
import torch  # noqa: E402
import triton  # noqa: E402
import triton.language as tl  # noqa: E402

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FSA_REFERENCE_DIR", "reference")
sys.path.insert(0, REF)
from flash_sparse_attn.ops.triton import block_info as BI  # noqa: E402

from flash_sparse_attn.ops.triton import scheduler as SC  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def _create_of(aggregate):
    for cell in aggregate.__new__.__closure__:
        if isinstance(cell.cell_contents, type):
            return cell.cell_contents.__dict__["create"].__func__
    raise RuntimeError("undecorated class not found")


FWD_CREATE, BWD_CREATE, DEC_CREATE = (_create_of(c) for c in (SC.AttnFwdBlockScheduler, SC.AttnBwdBlockScheduler,
                                                              SC.AttnDecBlockScheduler))
SC.AttnFwdBlockScheduler = SC.AttnBwdBlockScheduler = SC.AttnDecBlockScheduler = lambda *nine: nine


@triton.jit
def k_fwd_create(out, sq, sk, m_block, split_idx, w_sink, w_left, w_right, w_near, NS: tl.constexpr, TN: tl.constexpr,
                 TM: tl.constexpr, CAUSAL: tl.constexpr, LOCAL: tl.constexpr, SPLIT: tl.constexpr, GPACK: tl.constexpr):
    cfg = types.SimpleNamespace(actual_seqlen_q=sq, actual_seqlen_k=sk, m_block=m_block, window_size_sink=w_sink,
                                window_size_left=w_left, window_size_right=w_right, window_size_near=w_near,
                                TILE_N=TN, TILE_M=TM, QHEAD_PER_KVHEAD_PACKGQA=GPACK)
    nine = FWD_CREATE(cfg, split_idx, NS, CAUSAL, LOCAL, SPLIT)
    for i in range(9):
        tl.store(out + i, nine[i])


@triton.jit
def k_bwd_create(out, sq, sk, n_block, split_idx, w_sink, w_left, w_right, w_near, NS: tl.constexpr, TN: tl.constexpr,
                 TM: tl.constexpr, CAUSAL: tl.constexpr, LOCAL: tl.constexpr, SPLIT: tl.constexpr):
    cfg = types.SimpleNamespace(actual_seqlen_q=sq, actual_seqlen_k=sk, n_block=n_block, window_size_sink=w_sink,
                                window_size_left=w_left, window_size_right=w_right, window_size_near=w_near,
                                TILE_N=TN, TILE_M=TM)
    nine = BWD_CREATE(cfg, split_idx, NS, CAUSAL, LOCAL, SPLIT)
    for i in range(9):
        tl.store(out + i, nine[i])


@triton.jit
def k_dec_create(out, sk, split_idx, w_sink, w_left, w_right, w_near, NS: tl.constexpr, TOPK: tl.constexpr,
                 TN: tl.constexpr, TM: tl.constexpr, LOCAL: tl.constexpr, GATHER: tl.constexpr, GPACK: tl.constexpr):
    cfg = types.SimpleNamespace(actual_seqlen_k=sk, window_size_sink=w_sink, window_size_left=w_left,
                                window_size_right=w_right, window_size_near=w_near, TILE_N=TN, TILE_M=TM,
                                QHEAD_PER_KVHEAD_PACKGQA=GPACK)
    nine = DEC_CREATE(cfg, split_idx, NS, TOPK, LOCAL, GATHER)
    for i in range(9):
        tl.store(out + i, nine[i])


@triton.jit
def k_n_block(out, sq, sk, m_block, split_idx, w_sink, w_left, w_right, w_near, NS: tl.constexpr, TN: tl.constexpr,
              TM: tl.constexpr, CAUSAL: tl.constexpr, LOCAL: tl.constexpr, SPLIT: tl.constexpr, GPACK: tl.constexpr):
    a, b, c, d, e, f = BI.get_n_block_min_max(sq, sk, m_block, split_idx, w_sink, w_left, w_right, w_near, NS, TN, TM,
                                              CAUSAL, LOCAL, SPLIT, GPACK)
    tl.store(out + 0, a)
    tl.store(out + 1, b)
    tl.store(out + 2, c)
    tl.store(out + 3, d)
    tl.store(out + 4, e)
    tl.store(out + 5, f)


@triton.jit
def k_m_block(out, sq, sk, n_block, split_idx, w_sink, w_left, w_right, w_near, NS: tl.constexpr, TN: tl.constexpr,
              TM: tl.constexpr, CAUSAL: tl.constexpr, LOCAL: tl.constexpr, SPLIT: tl.constexpr):
    a, b, c, d, e, f = BI.get_m_block_min_max(sq, sk, n_block, split_idx, w_sink, w_left, w_right, w_near, NS, TN, TM,
                                              CAUSAL, LOCAL, SPLIT)
    tl.store(out + 0, a)
    tl.store(out + 1, b)
    tl.store(out + 2, c)
    tl.store(out + 3, d)
    tl.store(out + 4, e)
    tl.store(out + 5, f)


@triton.jit
def k_edges_n(out, sq, sk, m_block, n_min, w_left, w_right, w_near, TN: tl.constexpr, TM: tl.constexpr,
              LOCAL: tl.constexpr, GPACK: tl.constexpr):
    a = BI.get_n_block_min_causal_local_mask(sq, sk, m_block, n_min, w_right, w_near, TN, TM, LOCAL, GPACK)
    b = BI.get_n_block_min_before_local_mask(sq, sk, m_block, n_min, w_left, w_right, w_near, TN, TM, LOCAL, GPACK)
    tl.store(out + 0, a)
    tl.store(out + 1, b)


@triton.jit
def k_edges_m(out, sq, sk, n_block, m_lim, w_left, w_right, w_near, TN: tl.constexpr, TM: tl.constexpr,
              CAUSAL: tl.constexpr, LOCAL: tl.constexpr):
    a = BI.get_m_block_min_causal_local_mask(sq, sk, n_block, m_lim, w_right, w_near, TN, TM, CAUSAL, LOCAL)
    b = BI.get_m_block_max_before_local_mask(sq, sk, n_block, m_lim, w_left, w_right, w_near, TN, TM, LOCAL)
    tl.store(out + 0, a)
    tl.store(out + 1, b)


@triton.jit
def k_topk(out, split_idx, NS: tl.constexpr, TOPK: tl.constexpr, TN: tl.constexpr):
    a, b, c, d, e, f = BI.get_topk_n_block_min_max(split_idx, NS, TOPK, TN)
    tl.store(out + 0, a)
    tl.store(out + 1, b)


def call(kernel, n_out, *args, **consts):
    out = torch.zeros(n_out, dtype=torch.int32)
    kernel[(1,)](out, *args, **consts)
    return out.tolist()


WINDOWS = [[0, 256, 0, 0], [0, 0, 0, 256], [0, 1024, 0, 0], [64, 94, 188, 256], [64, 94, 0, 256], [0, 300, 100, 200],
           [40, 100, 37, 77], [64, 448, 448, 1024], [128, 0, 0, 128], [0, 0, 0, 0]]
TILES = [(64, 64), (128, 128), (128, 64), (64, 128), (16, 64), (16, 256)]


def main():
    rnd = random.Random(20251125)
    fwd_a, fwd_r, bwd_a, bwd_r, en_a, en_r, em_a, em_r, tk_a, tk_r = ([] for _ in range(10))
    fwd_c, bwd_c, dec_a, dec_c = [], [], [], []

    def shape():
        kind = rnd.random()
        if kind < 0.15:
            return 1, rnd.choice([1, 63, 64, 300, 1024, 4097])  # one query position (decode)
        sk = rnd.choice([64, 128, 160, 300, 987, 1024, 1344, 4096, 5000])
        sq = sk if kind < 0.6 else rnd.randint(1, sk)
        return sq, sk

    for _ in range(420):
        sq, sk = shape()
        tm, tn = rnd.choice(TILES)
        local = rnd.random() < 0.6
        causal = rnd.random() < 0.6
        w = rnd.choice(WINDOWS) if local else [0, 0, 0, 0]
        ns = rnd.choice([1, 1, 2, 3, 4, 7])
        split = ns > 1 or rnd.random() < 0.2
        gpack = rnd.choice([1, 1, 1, 4, 8]) if tm >= 16 else 1
        if sq == 1:
            causal, gpack = False, rnd.choice([1, 4, 8, 16])
        m_blocks = -(-sq * gpack // tm)
        for mb in sorted({0, m_blocks - 1, rnd.randrange(m_blocks), rnd.randrange(m_blocks)}):
            for sp in sorted({0, ns - 1, rnd.randrange(ns)}):
                r = call(k_n_block, 6, sq, sk, mb, sp, *w, NS=ns, TN=tn, TM=tm, CAUSAL=causal, LOCAL=local,
                         SPLIT=split, GPACK=gpack)
                fwd_a.append([sq, sk, mb, sp, *w, ns, tn, tm, int(causal), int(local), int(split), gpack])
                fwd_r.append(r)
                fwd_c.append(call(k_fwd_create, 9, sq, sk, mb, sp, *w, NS=ns, TN=tn, TM=tm, CAUSAL=causal, LOCAL=local,
                                  SPLIT=split, GPACK=gpack))
                for n_min in sorted({r[0], r[2]}):
                    for loc in (False, True):
                        e = call(k_edges_n, 2, sq, sk, mb, n_min, w[1], w[2], w[3], TN=tn, TM=tm, LOCAL=loc, GPACK=gpack)
                        en_a.append([sq, sk, mb, n_min, w[1], w[2], w[3], tn, tm, int(loc), gpack])
                        en_r.append(e)
        if sq > 1:
            n_blocks = -(-sk // tn)
            for nb in sorted({0, n_blocks - 1, rnd.randrange(n_blocks), rnd.randrange(n_blocks)}):
                for sp in sorted({0, ns - 1, rnd.randrange(ns)}):
                    r = call(k_m_block, 6, sq, sk, nb, sp, *w, NS=ns, TN=tn, TM=tm, CAUSAL=causal, LOCAL=local,
                             SPLIT=split)
                    bwd_a.append([sq, sk, nb, sp, *w, ns, tn, tm, int(causal), int(local), int(split)])
                    bwd_r.append(r)
                    bwd_c.append(call(k_bwd_create, 9, sq, sk, nb, sp, *w, NS=ns, TN=tn, TM=tm, CAUSAL=causal,
                                      LOCAL=local, SPLIT=split))
                    for m_lim in sorted({r[0], r[1], r[2], r[3]}):
                        for cz, loc in ((False, False), (True, False), (False, True), (True, True)):
                            e = call(k_edges_m, 2, sq, sk, nb, m_lim, w[1], w[2], w[3], TN=tn, TM=tm, CAUSAL=cz, LOCAL=loc)
                            em_a.append([sq, sk, nb, m_lim, w[1], w[2], w[3], tn, tm, int(cz), int(loc)])
                            em_r.append(e)
    for topk in (1, 16, 63, 64, 100, 2048, 2049):
        for tn in (16, 64, 256):
            for ns in (1, 2, 3, 5, 8):
                for sp in range(ns):
                    tk_a.append([topk, sp, ns, tn])
                    tk_r.append(call(k_topk, 2, sp, NS=ns, TOPK=topk, TN=tn))
    for _ in range(160):
        sk = rnd.choice([1, 63, 64, 300, 1024, 1344, 4097, 20000])
        tn = rnd.choice([16, 64, 128, 256])
        local = rnd.random() < 0.6
        gather = rnd.random() < 0.3
        w = rnd.choice(WINDOWS) if local else [0, 0, 0, 0]
        ns = rnd.choice([1, 2, 3, 4, 7])
        topk = rnd.choice([16, 100, 2048]) if gather else 0
        gpack = rnd.choice([1, 4, 8, 16])
        for sp in range(ns):
            dec_a.append([sk, sp, *w, ns, topk, tn, 16, int(local), int(gather), gpack])
            dec_c.append(call(k_dec_create, 9, sk, sp, *w, NS=ns, TOPK=topk, TN=tn, TM=16, LOCAL=local, GATHER=gather,
                              GPACK=gpack))
    i32 = lambda x: np.asarray(x, dtype=np.int32)  # noqa: E731
    path = os.path.join(OUT, "schedule.npz")
    np.savez_compressed(path, fwd_args=i32(fwd_a), fwd_out=i32(fwd_r), bwd_args=i32(bwd_a), bwd_out=i32(bwd_r),
                        edges_n_args=i32(en_a), edges_n_out=i32(en_r), edges_m_args=i32(em_a), edges_m_out=i32(em_r),
                        topk_args=i32(tk_a), topk_out=i32(tk_r), fwd_create=i32(fwd_c), bwd_create=i32(bwd_c),
                        dec_args=i32(dec_a), dec_create=i32(dec_c))
    print(f"schedule: fwd {len(fwd_a)} bwd {len(bwd_a)} edges_n {len(en_a)} edges_m {len(em_a)} topk {len(tk_a)} dec {len(dec_a)} cases, "
          f"{os.path.getsize(path) / 1024:.0f} KiB")


if __name__ == "__main__":
    main()
