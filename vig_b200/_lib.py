"""ctypes binding of ``libvig_b200.so`` (the C ABI declared in ``include/vig_b200.h``).

There is no fallback: if the library is missing or a call is rejected, a ``RuntimeError`` is raised.
"""
import ctypes
import os
from ctypes import c_float, c_int, c_int32, c_int64, c_size_t, c_void_p, POINTER

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("VIG_B200_LIB") or os.path.join(_HERE, "libvig_b200.so")

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
IMPL_AUTO, IMPL_SIMT, IMPL_TC, IMPL_TC_SINGLE, IMPL_TC_SPLIT, IMPL_TC_WAVE = 0, 1, 2, 3, 4, 5

_lib = None

_P64 = POINTER(c_int64)
_SIGNATURES = {
    "vig_version": (c_int, []),
    "vig_strerror": (ctypes.c_char_p, [c_int]),
    "vig_bigla_workspace_bytes": (c_size_t, [c_int] * 7),
    "vig_bigla_fwd": (c_int, [c_void_p] * 6 + [c_int] * 6 + [_P64] * 6 + [c_float] * 4 + [c_void_p] * 6 +
                      [c_int, c_int, c_void_p, c_size_t, c_void_p, c_void_p]),
    "vig_bigla_bwd_workspace_bytes": (c_size_t, [c_int] * 5),
    "vig_bigla_bwd": (c_int, [c_void_p] * 11 + [c_int] * 6 + [_P64] * 6 + [c_float, c_float, c_int, c_void_p, c_size_t, c_void_p]),
    "vig_bigla_noalloc_scratch_bytes": (c_size_t, []),
    "vig_bigla_fwd_noalloc": (c_int, [c_void_p] * 6 + [c_int] * 6 + [_P64] * 6 + [c_float] * 4 + [c_int, c_void_p, c_void_p]),
    "vig_dwconv3x3_fwd": (c_int, [c_void_p] * 4 + [c_int] * 6 + [c_void_p] * 2),
    "vig_dwconv3x3_halo_fwd": (c_int, [c_void_p] * 6 + [c_int] * 6 + [c_void_p]),
    "vig_gate_inject_fwd": (c_int, [c_void_p, _P64] + [c_void_p] * 5 + [c_int64] * 3 + [c_int] * 4 + [c_float, c_int, c_int, c_void_p]),
    "vig_add_rmsnorm_fwd": (c_int, [c_void_p] * 5 + [c_int64, c_int, c_float, c_int, c_void_p]),
    "vig_layernorm_act_fwd": (c_int, [c_void_p] * 5 + [c_int64, c_int, c_float, c_int, c_int, c_void_p]),
    "vig_linear_bias_supported": (c_int, [c_int64, c_int, c_int, c_int]),
    "vig_linear_bias_fwd": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_int, c_void_p, c_void_p]),
    "vig_linear_swiglu_supported": (c_int, [c_int64, c_int, c_int, c_int]),
    "vig_linear_swiglu_preferred": (c_int, [c_int64, c_int, c_int, c_int]),
    "vig_linear_swiglu_fwd": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_int, c_void_p, c_void_p]),
    "vig_linear_add_rmsnorm_supported": (c_int, [c_int64, c_int, c_int, c_int]),
    "vig_linear_add_rmsnorm_fwd": (c_int, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_float, c_int, c_void_p, c_void_p]),
    "vig_layernorm_act_add_fwd": (c_int, [c_void_p] * 5 + [c_int64, c_void_p, c_int64, c_int, c_float, c_int, c_int, c_void_p]),
    "vig_layernorm_act_add_rmsnorm_fwd": (c_int, [c_void_p] * 5 + [c_int64, c_void_p, c_void_p, c_float, c_void_p, c_int64, c_int, c_float, c_int, c_int, c_void_p]),
    "vig_stem_unfold_fwd": (c_int, [c_void_p, c_void_p] + [c_int] * 6 + [c_void_p]),
    "vig_stem_fold_fwd": (c_int, [c_void_p, c_void_p] + [c_int] * 5 + [c_void_p]),
    "vig_stem_conv_ln_supported": (c_int, [c_int] * 6),
    "vig_stem_conv_ln_fwd": (c_int, [c_void_p] * 6 + [c_int] * 5 + [c_float, c_int, c_int, c_void_p, c_void_p]),
    "vig_swiglu_fwd": (c_int, [c_void_p] * 3 + [c_int64, c_int, c_int64, c_int64, c_int, c_void_p]),
}
EXPORTS = tuple(_SIGNATURES)


def lib():
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m vig_b200.build` "
                               "(there is no CPU or PyTorch fallback)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name, None)
            if fn is None:
                continue        # optional entry points are checked where they are used
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def register(name, restype, argtypes):
    """Declare the signature of an additional entry point."""
    _SIGNATURES[name] = (restype, argtypes)
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.restype, fn.argtypes = restype, argtypes


def check(status, what):
    if status != 0:
        msg = lib().vig_strerror(int(status)).decode()
        raise RuntimeError(f"{what} failed with status {status}: {msg}")


def ptr(t):
    return None if t is None else c_void_p(t.data_ptr())


def stream_ptr():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def dtype_code(t):
    try:
        return DTYPE_CODE[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}; expected float32, bfloat16 or float16") from None


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("vig_b200 kernels need CUDA tensors; there is no CPU path")


def strides3(t):
    """(b, h, l) element strides of a [B,H,L,d] view whose last dimension is contiguous."""
    if t.stride(-1) != 1 and t.shape[-1] != 1:
        raise ValueError("last dimension must be contiguous")
    return (c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))
