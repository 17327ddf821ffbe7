"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "nncase_b200.h")).read()
    return sorted(set(re.findall(r"NNCB_API\s+[\w\s\*]+?\b(nncb_\w+)\s*\(", text)))


def test_header_declares_symbols():
    names = _declared()
    assert len(names) >= 30 and "nncb_qconv2d_run" in names and "nncb_quantize" in names


def test_library_exports_every_declared_symbol():
    from nncase_b200 import lib as L
    lib = L.load()
    for name in _declared():
        assert hasattr(lib, name), name
    assert set(_declared()) == set(L.SIGNATURES), "ctypes binding and header disagree"
    assert b"sm_100a" in lib.nncb_version()


def test_no_gpu_means_loud_failure():
    """Without a device the library reports an error instead of computing anywhere else."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from nncase_b200 import lib as L
    lib = L.load()
    h = ctypes.c_void_p()
    rc = lib.nncb_context_create(0, None, ctypes.byref(h))
    assert rc < 0
    assert lib.nncb_last_error()
    from nncase_b200.kernels import Context
    with pytest.raises(L.NncbError):
        Context(0)


def test_product_does_not_import_oracle():
    """Nothing under the package imports, links or loads the CPU oracles."""
    pkg = os.path.join(ROOT, "nncase_b200")
    pat = re.compile(r"^\s*(from|import)\s+oracle\b|libqoracle|libnncase_ref|oracle[/.](qoracle|ref|program|attention)\.py",
                     re.M)
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h", "Makefile")):
                src = open(os.path.join(dirpath, f), errors="ignore").read()
                assert not pat.search(src), os.path.join(dirpath, f)
