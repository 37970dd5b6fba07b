"""ctypes binding of libtpf_b200.so (C ABI declared in include/tpf_b200.h).

The library is the only route from the Python operators to the device; there
is no fallback.  A missing library raises at first use with the build command.
"""
from __future__ import annotations

import ctypes
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtpf_b200.so")

_P = ctypes.c_void_p
_I = ctypes.c_int64
_i = ctypes.c_int
_f = ctypes.c_float
_PI = ctypes.POINTER(ctypes.c_int64)

# name -> argtypes; every function returns int (0 = ok) unless listed in _RESTYPES.
SIGNATURES = {
    "tpf_version": [],
    "tpf_last_error_string": [],
    "tpf_device_status": [ctypes.POINTER(ctypes.c_int)],
    "tpf_bmm_bf16": [_P, _I, _I, _i, _P, _I, _I, _i, _P, _I, _I, _i, _I, _I, _I, _I, _I, _i, _P],
    "tpf_attn_fwd": [_P, _P, _P, _PI, _PI, _PI, _P, _I, _P, _I, _I, _P, _P, _I, _I, _I, _I, _I, _f, _P],
    "tpf_attn_bwd_workspace_bytes": [_I, _I, _I, _I, _I, _I],
    "tpf_launch_count": [],
    "tpf_selftest_bounded_wait": [_P, _P],
    "tpf_attn_bwd_stages": [_P, _P, _P, _P, _PI, _PI, _PI, _P, _P, _P, _I, _P, _I, _I, _P, _P, _P, _P, _P, _P, _I,
                            _I, _I, _I, _I, _I, _f, _i, _P],
    "tpf_attn_bwd_static_scratch_capacity": [],
    "tpf_attn_bwd_static_scratch": [_P, _P, _P, _P, _PI, _PI, _PI, _P, _P, _P, _I, _P, _I, _I, _P, _P, _P, _P, _P,
                                    _I, _I, _I, _I, _I, _f, _P],
    "tpf_attn_bwd": [_P, _P, _P, _P, _PI, _PI, _PI, _P, _P, _P, _I, _P, _I, _I, _P, _P, _P, _P, _P, _P, _I,
                     _I, _I, _I, _I, _I, _f, _P],
    "tpf_trimul_fwd_workspace_bytes": [_I, _I, _I],
    "tpf_trimul_bwd_workspace_bytes": [_I, _I, _I],
    "tpf_trimul_bwd_stages_workspace_bytes": [_I, _I, _I],
    "tpf_trimul_fwd_stages": [_P] * 10 + [_i, _I, _I, _I] + [_P] * 12 + [_I, _I, _i, _P],
    "tpf_trimul_bwd_stages": [_P] * 9 + [_i, _I, _I, _I] + [_P] * 21 + [_I, _I, _i, _P, _P, _P, _P],
    "tpf_trimul_fwd": [_P] * 10 + [_i, _I, _I, _I] + [_P] * 12 + [_I, _P],
    "tpf_trimul_bwd": [_P] * 9 + [_i, _I, _I, _I] + [_P] * 21 + [_I, _P],
}
_RESTYPES = {"tpf_trimul_fwd_workspace_bytes": ctypes.c_int64, "tpf_trimul_bwd_workspace_bytes": ctypes.c_int64,
             "tpf_trimul_bwd_stages_workspace_bytes": ctypes.c_int64,
             "tpf_attn_bwd_workspace_bytes": ctypes.c_int64,
             "tpf_attn_bwd_static_scratch_capacity": ctypes.c_int64, "tpf_launch_count": ctypes.c_int64,
             "tpf_version": ctypes.c_char_p, "tpf_last_error_string": ctypes.c_char_p}

ERROR_NAMES = {1: "invalid argument", 2: "unsupported", 3: "CUDA error", 4: "workspace", 5: "device status"}

_lock = threading.Lock()
_lib = None


class TpfError(RuntimeError):
    """A C-ABI call returned a non-zero code."""

    def __init__(self, name, code, message):
        super().__init__(f"{name} failed [{ERROR_NAMES.get(code, code)}]: {message}")
        self.code = code


def load():
    """Load the shared library (once) and attach signatures."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m openfold3_triangle_kernel_b200.build` "
                "(nvcc, sm_100a).  There is no CPU or PyTorch fallback for these operators.")
        lib = ctypes.CDLL(LIB_PATH)
        for name, argtypes in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = _RESTYPES.get(name, ctypes.c_int)
        _lib = lib
    return _lib


def call(name, *args):
    """Call an int-returning entry point; raise TpfError on a non-zero code."""
    lib = load()
    rc = getattr(lib, name)(*args)
    if rc != 0:
        msg = lib.tpf_last_error_string().decode("utf-8", "replace")
        if rc in (1, 2):
            raise ValueError(f"{name}: {msg}")
        raise TpfError(name, rc, msg)


def device_status():
    """Synchronise nothing; read-and-clear the device status words (0 = healthy)."""
    st = ctypes.c_int(0)
    call("tpf_device_status", ctypes.byref(st))
    return st.value


def version():
    return load().tpf_version().decode()


def ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


def i64_array(values):
    return (ctypes.c_int64 * len(values))(*[int(v) for v in values])


def current_stream():
    import torch
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
