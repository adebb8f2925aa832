"""The C-ABI library loads without a GPU and exports every symbol include/*.h declares."""

import ctypes
import glob
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    names = set()
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = open(h).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        for m in re.finditer(r"\b(fsa_[a-z0-9_]+)\s*\(", text):
            names.add(m.group(1))
    return names


def test_library_exports_declared_symbols():
    from flash_sparse_attn import _lib

    lib = _lib.load()
    names = _declared_symbols()
    assert {"fsa_fwd", "fsa_abi_version", "fsa_status_string", "fsa_quantize_fp8", "fsa_fp8_widen"} <= names
    for n in sorted(names):
        assert hasattr(lib, n), f"libfsa_b200.so does not export {n}"
    assert lib.fsa_abi_version() == _lib.ABI_VERSION
    assert b"ok" == lib.fsa_status_string(0)
    assert b"unsupported" in lib.fsa_status_string(-2)


def test_struct_layout_matches_header():
    """Field order of the ctypes mirror equals the field order of the C struct."""
    from flash_sparse_attn import _lib

    text = open(os.path.join(ROOT, "include", "fsa_b200.h")).read()
    for cname, cls in (("FsaFwdArgs", _lib.FsaFwdArgs), ("FsaBwdArgs", _lib.FsaBwdArgs),
                       ("FsaDecArgs", _lib.FsaDecArgs), ("FsaKvAppendArgs", _lib.FsaKvAppendArgs)):
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (cname, cname), text, flags=re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        fields = []
        for stmt in body.split(";"):
            stmt = stmt.strip()
            if not stmt:
                continue
            decl = stmt.split(",")
            for i, part in enumerate(decl):
                fields.append(re.findall(r"[A-Za-z_][A-Za-z0-9_]*", part)[-1])
        assert fields == [f[0] for f in cls._fields_], cname


def test_compute_without_gpu_fails_loudly():
    """No CPU fallback: calling an operator on CPU tensors raises instead of computing."""
    import pytest
    import torch

    from flash_sparse_attn import flash_dense_attn_func

    q = torch.zeros(1, 8, 1, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        flash_dense_attn_func(q, q, q)


def test_function_aliases_and_status_word_on_cpu():
    """The reference's autograd Function names resolve, and a non-zero status word makes check_status raise once
    (it resets the word, so the next call passes)."""
    import pytest
    import torch

    from flash_sparse_attn import _lib
    from flash_sparse_attn.ops.triton import interface

    for name in ("FlashDenseAttnFunc", "FlashDenseAttnVarlenFunc", "FlashSparseAttnFunc", "FlashSparseAttnVarlenFunc",
                 "FlashGatedAttnFunc", "FlashGatedAttnVarlenFunc"):
        assert callable(getattr(interface, name).apply)
    fake = torch.ones(1, dtype=torch.int32)
    _lib._status_words[("cpu", 0)] = fake
    try:
        with pytest.raises(RuntimeError, match="device status 1"):
            _lib.check_status()
        assert int(fake.item()) == 0
        _lib.check_status()
    finally:
        del _lib._status_words[("cpu", 0)]


def test_workspace_sizes_from_the_library():
    """Host arithmetic behind fsa_*_workspace_bytes (no GPU needed)."""
    from flash_sparse_attn import _lib

    lib = _lib.load()
    a = _lib.FsaBwdArgs()
    a.batch, a.seqlen_q, a.seqlen_k, a.heads_q, a.heads_kv, a.head_dim = 2, 300, 500, 8, 2, 96
    a.kind, a.dtype, a.num_splits, a.flags = _lib.KIND_GATED, _lib.DT_BF16, 3, _lib.F_SPLIT | _lib.F_DETERMINISTIC
    a.delta_numel = 2 * 2 * 500
    w = _lib.FsaBwdWorkspace()
    assert lib.fsa_bwd_workspace_bytes(ctypes.byref(a), ctypes.byref(w)) == 0
    rows = 2 * 384
    assert w.lse2_ws == w.dpsum_ws == w.da_accum == 4 * 8 * rows
    assert w.dq_accum == 4 * 8 * rows * 128 and w.alpha_ws == 2 * 8 * rows
    assert w.dk_partial == w.dv_partial == 4 * 3 * 2 * 500 * 2 * 96
    assert w.dd_partial == 4 * 3 * 2000 and w.dq_order == 2 * 2 * 2 * 4 * 3 and w.dq_turn == 4 * 2 * 8 * 3
    f = _lib.FsaFwdArgs()
    f.batch, f.seqlen_q, f.seqlen_k, f.heads_q, f.heads_kv, f.head_dim = 2, 300, 500, 8, 2, 96
    f.kind, f.num_splits, f.flags = _lib.KIND_SPARSE, 4, _lib.F_SPLIT
    fw = _lib.FsaFwdWorkspace()
    assert lib.fsa_fwd_workspace_bytes(ctypes.byref(f), ctypes.byref(fw)) == 0
    assert fw.out_partial == 4 * 4 * 600 * 8 * 96 and fw.lse_partial == 4 * 4 * 600 * 8 and fw.gate_ws == 0
    d = _lib.FsaDecArgs()
    d.batch, d.heads_q, d.head_dim, d.num_splits = 5, 16, 128, 1
    dw = _lib.FsaDecWorkspace()
    assert lib.fsa_decode_workspace_bytes(ctypes.byref(d), ctypes.byref(dw)) == 0 and dw.out_partial == 0
    d.partial_only = 1
    assert lib.fsa_decode_workspace_bytes(ctypes.byref(d), ctypes.byref(dw)) == 0
    assert dw.out_partial == 4 * 5 * 16 * 128 and dw.lse_partial == 4 * 5 * 16
