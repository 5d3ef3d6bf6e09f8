"""The shared library loads without a GPU and exports every entry point the header declares."""

import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_entries():
    text = open(os.path.join(ROOT, "include", "linquant_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lq_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from linquant_b200 import build

    lib = ctypes.CDLL(build.build())
    names = declared_entries()
    assert len(names) >= 25, names
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared in include/linquant_b200.h but not exported: {missing}"
    lib.lq_version.restype = ctypes.c_int
    assert lib.lq_version() >= 100


def test_host_side_validation_needs_no_gpu():
    from linquant_b200 import _cabi

    L = _cabi.lib()
    p = _cabi.ZooProblem()
    p.B, p.T, p.H, p.K, p.V, p.chunk = 1, 100, 2, 64, 64, 64
    L.lq_simple_gla_fwd.argtypes = [ctypes.POINTER(_cabi.ZooProblem), ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]
    assert L.lq_simple_gla_fwd(ctypes.byref(p), None, 0, None) == 2  # LQ_ERR_SHAPE: T % chunk != 0
    assert b"multiple of the chunk size" in L.lq_last_error_string()
    p.T, p.K = 128, 96
    assert L.lq_simple_gla_fwd(ctypes.byref(p), None, 0, None) == 4  # LQ_ERR_UNSUPPORTED
    p.K = 64
    assert L.lq_simple_gla_fwd(ctypes.byref(p), None, 0, None) == 1  # LQ_ERR_NULL: no tensors given
    assert L.lq_zoo_workspace_bytes(ctypes.byref(p), 0) > 0


def test_cuda_ops_refuse_cpu_tensors():
    import pytest
    import torch

    from linquant_b200 import _cabi
    from linquant_b200.kernels.zoo import chunk_simple_gla_int8

    x = torch.zeros(1, 64, 1, 64, dtype=torch.float16)
    with pytest.raises(_cabi.LinQuantError):
        chunk_simple_gla_int8(x, x, x, None, {})


def test_ctypes_layouts_match_the_compiled_structs():
    """The ctypes mirrors of the three descriptor structs have the size the library was compiled with."""
    from linquant_b200 import _cabi
    from linquant_b200.kernels.mamba2 import _ssd

    L = _cabi.lib()
    L.lq_struct_bytes.restype = ctypes.c_ulonglong
    L.lq_struct_bytes.argtypes = [ctypes.c_int]
    assert L.lq_struct_bytes(0) == ctypes.sizeof(_cabi.ZooProblem)
    assert L.lq_struct_bytes(1) == ctypes.sizeof(_ssd.SsdProblem)
    assert L.lq_struct_bytes(2) == ctypes.sizeof(_cabi.ZooWorkspace)
