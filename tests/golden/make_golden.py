"""Generate the golden fixtures in this directory from the REFERENCE's own eager functions.

Run once, on a machine that has the reference repository checked out (read-only) at REF:

    python tests/golden/make_golden.py REF      (or set FSA_REFERENCE_DIR)

It imports the reference's tests/test_utils.py (eager fp32 oracles), tests/test_topk_gather_decode.py
(gathered-decode oracle) and flash_sparse_attn/ops/triton/utils.py (window / split heuristics), feeds
them seeded inputs and stores inputs + expected outputs as .npz (16-bit tensors as raw uint16).
The fixtures travel with the repository; the reference does not. Nothing here is needed at test time.
"""

import os
import sys

import numpy as np
import torch

REF = sys.argv[1] if len(sys.argv) > 1 and not sys.argv[1].startswith("--") else os.environ.get("FSA_REFERENCE_DIR", "reference")
sys.path.insert(0, os.path.join(REF, "tests"))
sys.path.insert(0, REF)

import test_utils as R  # noqa: E402  (reference tests/test_utils.py)
import test_topk_gather_decode as RT  # noqa: E402
from flash_sparse_attn.ops.triton import utils as RU  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))
DT = torch.bfloat16
CPU = torch.device("cpu")


def raw(t: torch.Tensor) -> np.ndarray:
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    return t.contiguous().numpy()


def save(name, **arrays):
    path = os.path.join(OUT, name + ".npz")
    np.savez_compressed(path, **{k: (raw(v) if isinstance(v, torch.Tensor) else np.asarray(v)) for k, v in arrays.items()})
    print(f"{name}: {os.path.getsize(path) / 1024:.0f} KiB")


def randn(*shape):
    return torch.randn(*shape, dtype=DT)


def lse_of(q, k, scale, is_causal, is_local, alpha=None, delta=None, logsig=True):
    s = R._reference_scores(q, k, scale, is_causal, is_local)
    if alpha is not None:
        a = alpha.transpose(1, 2).float()
        d = torch.repeat_interleave(delta.transpose(1, 2).float(), q.shape[2] // k.shape[2], dim=1)
        g = a.unsqueeze(-1) * d.unsqueeze(-2)
        s = s + (torch.nn.functional.logsigmoid(g) if logsig else g) * scale
    return torch.logsumexp(s, dim=-1)


def forward_cases():
    for name, sq, sk, causal in [("fwd_nc", 160, 160, False), ("fwd_causal", 160, 160, True),
                                 ("fwd_causal_sq_lt_sk", 96, 160, True)]:
        torch.manual_seed(1)
        q, k, v = randn(1, sq, 4, 64), randn(1, sk, 2, 64), randn(1, sk, 2, 64)
        a, d = randn(1, sq, 4), randn(1, sk, 2)
        scale = 64 ** -0.5
        save(name, q=q, k=k, v=v, alpha=a, delta=d, causal=causal,
             out_dense=R.reference_dense_forward(q, k, v, scale, causal),
             out_sparse=R.reference_sparse_forward(q, k, v, scale, causal),
             out_gated=R.reference_gated_forward(q, k, v, a, d, scale, causal, is_logsigmoid_gate=True),
             out_gated_lin=R.reference_gated_forward(q, k, v, a, d, scale, causal, is_logsigmoid_gate=False),
             lse_dense=lse_of(q, k, scale, causal, False),
             lse_gated=lse_of(q, k, scale, causal, False, a, d, True))


def local_case():
    # long enough for distinct per-head bands with the default near=1024 / sink=64
    torch.manual_seed(2)
    sq = sk = 1344
    q, k, v = randn(1, sq, 2, 64), randn(1, sk, 2, 64), randn(1, sk, 2, 64)
    scale = 64 ** -0.5
    ws = RU.window_sizes_heuristic(sk, 2, CPU)
    out = R.reference_sparse_forward(q, k, v, scale, True, is_local=True)
    # inputs are re-created from the seed at test time; a checksum guards the generator
    save("fwd_local", seed=2, shape=[1, sq, 2, 2, 64], window_sizes=ws, out=out,
         q_sum=q.float().sum().item(), k_sum=k.float().sum().item(), v_sum=v.float().sum().item(),
         lse=lse_of(q, k, scale, True, True))


def varlen_case():
    torch.manual_seed(3)
    lens = [64, 160, 96]
    cu = R.make_cu_seqlens(lens, CPU)
    t = sum(lens)
    q, k, v = randn(t, 4, 64), randn(t, 2, 64), randn(t, 2, 64)
    a, d = randn(t, 4), randn(t, 2)
    scale = 64 ** -0.5
    save("fwd_varlen", q=q, k=k, v=v, alpha=a, delta=d, cu_seqlens=cu,
         out_sparse=R._reference_varlen_forward("sparse", q, k, v, cu, cu, scale, True),
         out_gated=R._reference_varlen_forward("gated", q, k, v, cu, cu, scale, True, alpha=a, delta=d))


def decode_cases():
    torch.manual_seed(4)
    b, sk = 2, 200
    q, k, v = randn(b, 4, 64), randn(b, sk, 2, 64), randn(b, sk, 2, 64)
    a, d = randn(b, 4), randn(b, sk, 2)
    scale = 64 ** -0.5
    out_dense = R.reference_dense_forward(q.unsqueeze(1), k, v, scale, False).squeeze(1)
    out_gated = R.reference_gated_forward(q.unsqueeze(1), k, v, a.unsqueeze(1), d, scale, False).squeeze(1)
    lens = [200, 120]
    cu = R.make_cu_seqlens(lens, CPU)
    kp, vp = randn(sum(lens), 2, 64), randn(sum(lens), 2, 64)
    out_varlen = R._reference_varlen_decode("sparse", q, kp, vp, cu, scale)
    # gathered decode, with masked entries
    idx = RT._make_topk_indices([sk] * b, 64, CPU, include_invalid=True)
    k_top, v_top = RT._gather_topk_3d(k, idx), RT._gather_topk_3d(v, idx)
    out_gather = RT._reference_topk_decode("sparse", q, k_top, v_top, idx, scale)
    save("decode", q=q, k=k, v=v, alpha=a, delta=d, out_dense=out_dense, out_gated=out_gated, cu_seqlens=cu,
         k_packed=kp, v_packed=vp, out_varlen=out_varlen, gather_idx=idx, out_gather=out_gather)
    # local decode needs a long cache
    torch.manual_seed(5)
    sk = 1344
    q, k, v = randn(1, 2, 64), randn(1, sk, 2, 64), randn(1, sk, 2, 64)
    out = R.reference_sparse_forward(q.unsqueeze(1), k, v, scale, False, is_local=True).squeeze(1)
    save("decode_local", seed=5, shape=[1, sk, 2, 2, 64], out=out, q_sum=q.float().sum().item(),
         k_sum=k.float().sum().item(), v_sum=v.float().sum().item())


def backward_case():
    torch.manual_seed(6)
    sq = sk = 160
    q, k, v, do = randn(1, sq, 4, 64), randn(1, sk, 2, 64), randn(1, sk, 2, 64), randn(1, sq, 4, 64)
    a, d = randn(1, sq, 4), randn(1, sk, 2)
    scale = 64 ** -0.5
    res = {}
    for kind in ("dense", "gated"):
        leaves = [t.detach().float().requires_grad_(True) for t in ((q, k, v) if kind == "dense" else (q, k, v, a, d))]
        if kind == "dense":
            out = R.reference_dense_forward(*leaves, scale, True)
        else:
            out = R.reference_gated_forward(*leaves, scale, True, is_logsigmoid_gate=True)
        grads = torch.autograd.grad(out, leaves, do.float())
        for n, g in zip(("dq", "dk", "dv", "da", "dd"), grads):
            res[f"{n}_{kind}"] = g
    save("bwd_causal", q=q, k=k, v=v, dout=do, alpha=a, delta=d, **res)


def heuristics():
    rows = []
    for sk, hkv in [(160, 2), (1344, 2), (4096, 8), (8192, 8), (16384, 8), (131072, 8), (1024, 1), (3000, 4)]:
        rows.append([sk, hkv] + RU.window_sizes_heuristic(sk, hkv, CPU).flatten().tolist() + [0] * (32 - 4 * hkv))
    splits = []
    for sq, sk, sms, tm, tn, loc, hkv in [(4096, 4096, 148, 128, 128, False, 8), (4096, 4096, 148, 128, 128, True, 8),
                                         (1, 131072, 148, 16, 128, False, 8), (1, 131072, 148, 16, 256, True, 8),
                                         (8192, 8192, 148, 128, 128, True, 8), (256, 512, 148, 128, 128, False, 2),
                                         (16384, 16384, 148, 128, 128, False, 8), (64, 4096, 132, 64, 64, False, 4)]:
        splits.append([sq, sk, sms, tm, tn, int(loc), hkv, RU.num_splits_heuristic(sq, sk, sms, tm, tn, loc, hkv)])
    save("heuristics", windows=np.array(rows, dtype=np.int64), splits=np.array(splits, dtype=np.int64))


def topk_cases():
    """flash_sparse_attn/utils/mask.py:20-44 on rows WITHOUT equal scores (torch does not define which of
    several equal entries at the threshold it returns)."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("ref_mask", os.path.join(REF, "flash_sparse_attn", "utils", "mask.py"))
    ref_mask = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref_mask)
    g = torch.Generator().manual_seed(11)
    res = {}
    for name, shape, k, dt in [("a", (2, 3, 1000), 37, torch.float32), ("b", (1, 2, 4096), 512, torch.float32),
                               ("c", (2, 2, 200), 200, torch.float32), ("d", (1, 4, 250), 16, torch.bfloat16)]:
        n = shape[-1]
        rows = int(np.prod(shape[:-1]))
        if dt == torch.bfloat16:
            # distinct values that bf16 represents exactly
            base = torch.arange(n, dtype=torch.float32) - 100.0
        else:
            base = torch.randn(n * 4, generator=g).unique()[:n] * 3.0
        x = torch.stack([base[torch.randperm(n, generator=g)] for _ in range(rows)]).reshape(shape).to(dt)
        idx = ref_mask.topk_indices(x, k)
        res[f"{name}_scores"] = x
        res[f"{name}_k"] = torch.tensor(k)
        res[f"{name}_idx"] = idx
    save("topk", **res)


def padding_cases():
    """flash_sparse_attn/utils/padding.py:18-179: packing of right- and left-padded batches, with an
    `unused_mask`, and the three query-length branches of `upad_input`."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("ref_padding", os.path.join(REF, "flash_sparse_attn", "utils", "padding.py"))
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    g = torch.Generator().manual_seed(5)
    b, s = 3, 17
    res = {}
    for name, flip in (("right", False), ("left", True)):
        lens = torch.randint(1, s + 1, (b,), generator=g)
        mask = (torch.arange(s)[None] < lens[:, None]).to(torch.int32)
        if flip:
            mask = mask.flip(1)
        unused = ((torch.rand(b, s, generator=g) < 0.3) & (mask == 0)).to(torch.int32)
        x = torch.randn(b, s, 2, 4, generator=g)
        res[f"{name}_mask"], res[f"{name}_unused"], res[f"{name}_x"] = mask, unused, x
        for tag, um in (("", None), ("_u", unused)):
            packed, idx, cu, mx, used = ref.unpad_input(x, mask, um)
            res[f"{name}{tag}_packed"], res[f"{name}{tag}_idx"], res[f"{name}{tag}_cu"] = packed, idx, cu
            res[f"{name}{tag}_max"], res[f"{name}{tag}_used"] = torch.tensor(mx), used
        packed, idx, *_ = ref.unpad_input(x, mask)
        res[f"{name}_repadded"] = ref.pad_input(packed, idx, b, s)
        k = torch.randn(b, s + 2, 2, 4, generator=g)
        v = torch.randn(b, s + 2, 2, 4, generator=g)
        res[f"{name}_k"], res[f"{name}_v"] = k, v
        for ql in (s, 1, 5):
            q = torch.randn(b, ql, 2, 4, generator=g)
            qo, ko, vo, iq, (cq, ck), (mq, mk) = ref.upad_input(q, k, v, mask, ql, ref.unpad_input)
            pre = f"{name}_q{ql}"
            res[pre + "_q"], res[pre + "_qo"], res[pre + "_ko"], res[pre + "_vo"] = q, qo, ko, vo
            res[pre + "_iq"], res[pre + "_cq"], res[pre + "_ck"] = iq, cq, ck
            res[pre + "_mq"], res[pre + "_mk"] = torch.tensor(mq), torch.tensor(mk)
    save("padding", **res)


if __name__ == "__main__":
    torch.set_num_threads(8)
    topk_cases()
    padding_cases()
    if "--only-topk" in sys.argv or "--only-small" in sys.argv:
        sys.exit(0)
    forward_cases()
    local_case()
    varlen_case()
    decode_cases()
    backward_case()
    heuristics()
