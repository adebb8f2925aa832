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
                       ("FsaDecArgs", _lib.FsaDecArgs)):
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
