"""The C-ABI library loads without a GPU and exports every function the header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    names = []
    for f in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if f.endswith(".h"):
            text = open(os.path.join(ROOT, "include", f)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names += re.findall(r"\b(cxg_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    import cxgnncomp_backend  # builds nothing: the library must already be there
    lib = ctypes.CDLL(os.path.abspath(cxgnncomp_backend._LIB_PATH))
    names = declared_functions()
    assert len(names) >= 5
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/ but not exported"


def test_argument_checks_without_gpu():
    import cxgnncomp_backend as be
    # NULL descriptor and bad sizes are refused before any CUDA call is made
    assert be._lib.cxg_spmm_csr(None, None, 0, None) == -2
    need = ctypes.c_size_t(0)
    assert be._spmm_ws(10, 100, 0, 1, 0, ctypes.byref(need)) == -1
    assert b"bad sizes" in be._lib.cxg_last_error_string()
    assert be._spmm_ws(1000, 100000, 128, 1, 0, ctypes.byref(need)) == 0 and need.value > 0
    assert be._lib.cxg_abi_version() >= 1


def test_cpu_tensors_are_refused():
    import torch
    import cxgnncomp_backend as be
    import pytest
    ptr = torch.tensor([0, 1, 2]); idx = torch.tensor([0, 1]); x = torch.randn(2, 4)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        be.sage_sum_forward(x, ptr, idx, 2)
