"""CPU checks of the boundary: the library builds/loads and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = []
    inc = os.path.join(ROOT, "include")
    for fn in os.listdir(inc):
        if fn.endswith(".h"):
            text = open(os.path.join(inc, fn)).read()
            names += re.findall(r"VIG_API\s+[\w\s\*]+?\b(vig_\w+)\s*\(", text)
    return sorted(set(names))


def test_header_declares_the_path():
    names = declared_symbols()
    for required in ("vig_bigla_fwd", "vig_bigla_workspace_bytes", "vig_dwconv3x3_fwd", "vig_gate_inject_fwd",
                     "vig_add_rmsnorm_fwd", "vig_swiglu_fwd", "vig_version", "vig_strerror", "vig_linear_bias_fwd",
                     "vig_linear_bias_supported"):
        assert required in names


def test_library_exports_every_declared_symbol():
    from vig_b200 import build
    lib = ctypes.CDLL(build.build())
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
    assert lib.vig_version() >= 100
    lib.vig_strerror.restype = ctypes.c_char_p
    assert lib.vig_strerror(0) == b"ok"
    assert b"NULL" in lib.vig_strerror(-1)


def test_python_binding_covers_the_header():
    from vig_b200 import _lib
    assert set(declared_symbols()) <= set(_lib._SIGNATURES)


def test_workspace_query_and_argument_rejection_need_no_gpu():
    from vig_b200 import _lib
    L = _lib.lib()
    assert L.vig_bigla_workspace_bytes(2, 3, 196, 64, 64, 0, 0) > 0
    assert L.vig_bigla_workspace_bytes(2, 3, 196, 48, 64, 0, 0) == 0          # unsupported dk
    # rejected before any CUDA call: unsupported head dim, bad dtype, bad direction mask
    args = [None] * 6 + [1, 1, 8, 48, 64, 0] + [None] * 6 + [-1.0, 1.0, 0.0, float("nan")] + [None] * 6 + [3, 0, None, 0, None, None]
    assert L.vig_bigla_fwd(*args) == -2
    args[11] = 7; args[9] = 64
    assert L.vig_bigla_fwd(*args) == -3
    args[11] = 0; args[28] = 0
    assert L.vig_bigla_fwd(*args) == -6


def test_ops_refuse_cpu_tensors():
    import torch
    import vig_b200
    x = torch.zeros(1, 1, 4, 64)
    with pytest.raises(RuntimeError):
        vig_b200.bi_gla(x, x, x, x, x)
    with pytest.raises(RuntimeError):
        vig_b200.add_rmsnorm(torch.zeros(2, 64), torch.ones(64))
