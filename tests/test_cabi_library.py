"""The C-ABI shared library loads without a GPU and exports every symbol that
include/tpf_b200.h declares; argument validation works without touching a device."""
import ctypes
import os
import re

import pytest

from openfold3_triangle_kernel_b200 import _cabi as C

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "tpf_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tpf_[a-z0-9_]+)\s*\(", text)))


def test_library_exists_and_loads():
    lib = C.load()
    assert C.version().startswith("tpf_b200")
    assert lib.tpf_last_error_string() is not None


def test_every_declared_symbol_is_exported():
    lib = ctypes.CDLL(C.LIB_PATH)
    names = _declared_symbols()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), n


def test_python_signature_table_matches_header():
    assert sorted(C.SIGNATURES) == _declared_symbols()


def test_argument_validation_needs_no_device():
    null = ctypes.c_void_p(0)
    with pytest.raises(ValueError, match="null pointer"):
        C.call("tpf_bmm_bf16", null, 8, 8, 0, null, 8, 8, 0, null, 8, 8, 0, 8, 8, 8, 1, 0, 128, null)
    one = ctypes.c_void_p(256)
    with pytest.raises(ValueError, match="multiples of 8"):
        C.call("tpf_bmm_bf16", one, 7, 8, 0, one, 8, 8, 0, one, 8, 8, 0, 8, 8, 8, 1, 0, 128, null)
    st = C.i64_array([1, 1, 1, 1])
    with pytest.raises(ValueError, match="head dim"):
        C.call("tpf_attn_fwd", one, one, one, st, st, st, one, 8, one, 8, 1, one, one, 1, 1, 1, 8, 24, 1.0, null)
    with pytest.raises(ValueError, match="bias row pitch"):
        C.call("tpf_attn_fwd", one, one, one, st, st, st, one, 8, one, 7, 1, one, one, 1, 1, 1, 7, 32, 1.0, null)
    # pointers that the kernels access with 16-byte vectors must be 16-byte aligned
    mis = ctypes.c_void_p(264)
    with pytest.raises(ValueError, match="out must be 16-byte aligned"):
        C.call("tpf_attn_fwd", one, one, one, st, st, st, one, 8, one, 8, 1, mis, one, 1, 1, 1, 8, 32, 1.0, null)
    bwd = lambda dq, dbias, stages: C.call(  # noqa: E731
        "tpf_attn_bwd_stages", one, one, one, one, st, st, st, one, one, one, 8, one, 8, 1, dq, one, one, dbias, one,
        null, 0, 1, 1, 1, 8, 32, 1.0, stages, null)
    with pytest.raises(ValueError, match="dq must be 16-byte aligned"):
        bwd(mis, one, 2)
    with pytest.raises(ValueError, match="dbias must be 16-byte aligned"):
        bwd(one, mis, 4)
    args = [one] * 10 + [0, 1, 12, 128] + [one] * 12 + [1 << 20, null]
    with pytest.raises(ValueError, match="multiple of 8"):
        C.call("tpf_trimul_fwd", *args)
    args = [one] * 10 + [0, 1, 16, 48] + [one] * 12 + [1 << 20, null]
    with pytest.raises(ValueError, match="not in"):
        C.call("tpf_trimul_fwd", *args)
    args = [one] * 10 + [2, 1, 16, 64] + [one] * 12 + [1 << 20, null]
    with pytest.raises(ValueError, match="direction"):
        C.call("tpf_trimul_fwd", *args)


def test_workspace_queries():
    lib = C.load()
    # N = 384, D = 32: dQ/dK/dV of a plane stay on chip -> only dBias chunk planes
    ws = lib.tpf_attn_bwd_workspace_bytes(1, 384, 4, 384, 32, 1)
    assert ws > 0 and ws % 256 == 0
    # a single key strip and a machine-filling dBias grid need nothing
    assert lib.tpf_attn_bwd_workspace_bytes(1, 4, 4, 128, 64, 2) >= 0
    assert lib.tpf_attn_bwd_workspace_bytes(0, 4, 4, 128, 64, 1) == 0
    assert lib.tpf_trimul_fwd_workspace_bytes(1, 384, 128) >= 12 * 128 * 128 * 2
    assert lib.tpf_trimul_bwd_workspace_bytes(1, 384, 128) > 384 * 384 * 128 * 2 * 10
    assert lib.tpf_trimul_bwd_workspace_bytes(1, 384, 100) == 0
