"""The C-ABI library loads on a machine without a GPU and exports every entry point that
include/*.h declares.  No compute call is made here."""
import ctypes
import glob
import os
import re

import pytest

from conftest import ROOT


def declared_symbols():
    names = set()
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = re.sub(r"/\*.*?\*/", "", open(h).read(), flags=re.S)
        names.update(re.findall(r"\b(ap_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


@pytest.fixture(scope="module")
def lib():
    import any_precision_ext
    if not os.path.exists(any_precision_ext.library_path()):
        import importlib.util
        spec = importlib.util.spec_from_file_location("_ap_build", os.path.join(ROOT, "any-precision-llm_b200", "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build()
    return any_precision_ext.load_library()


def test_header_declares_the_operator_entry_points():
    syms = declared_symbols()
    for need in ("ap_matmul_kbit", "ap_dequant_kbit", "ap_strerror", "ap_version"):
        assert need in syms


def test_every_declared_symbol_is_exported(lib):
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"


def test_version_and_error_strings(lib):
    assert lib.ap_version() >= 1
    assert lib.ap_strerror(0) == b"ok"
    for code in range(-6, 0):
        assert lib.ap_strerror(code) not in (b"", b"unknown error code")
    assert lib.ap_strerror(-99) == b"unknown error code"


def test_argument_checks_return_codes_without_touching_a_gpu(lib):
    # Null pointers and bad shapes are rejected before any CUDA call.
    assert lib.ap_dequant_kbit(None, 0, None, None, 4, 32, 3, None) == -1
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.cast(buf, ctypes.c_void_p)
    aligned = (p.value + 15) & ~15
    assert lib.ap_dequant_kbit(aligned, 4, aligned, aligned, 4, 32, 9, None) == -2     # w_bits
    assert lib.ap_dequant_kbit(aligned, 4, aligned, aligned, 4, 48, 3, None) == -3     # K % 32
    assert lib.ap_dequant_kbit(aligned, 3, aligned, aligned, 4, 32, 3, None) == -3     # plane stride too small
    assert lib.ap_dequant_kbit(aligned, 4, aligned, aligned + 2, 4, 32, 3, None) == -4  # out alignment
    assert lib.ap_matmul_kbit(None, aligned, 4, aligned, aligned, 1, 4, 32, 3, None) == -1
    assert lib.ap_matmul_kbit(aligned, aligned, 4, aligned, aligned, 0, 4, 32, 3, None) == -3


def test_split_k_and_all_reduce_entry_points_check_their_arguments(lib):
    """The newer entry points reject bad arguments before any CUDA call, like the two operators."""
    vp, i, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
    lib.ap_gemm_kbit_splits.restype = i
    lib.ap_gemm_kbit_workspace_bytes.restype = sz
    lib.ap_comm_buffer_bytes.restype = sz
    lib.ap_comm_buffer_bytes.argtypes = [sz]
    lib.ap_allreduce_oneshot.restype = i
    lib.ap_allreduce_oneshot.argtypes = [vp, vp, i, ctypes.POINTER(vp), i, i, sz, vp, vp]
    # split counts: none for shapes the TMA variants do not take or above 256 tokens; several for few row blocks
    assert lib.ap_gemm_kbit_splits(64, 4096, 4096 + 128) == 1
    assert lib.ap_gemm_kbit_splits(512, 4096, 4096) == 1
    assert 2 <= lib.ap_gemm_kbit_splits(64, 4096, 4096) <= 8
    assert lib.ap_gemm_kbit_splits(64, 28672, 8192) == 1
    assert lib.ap_gemm_kbit_workspace_bytes(64, 4096, 1) == 0
    assert lib.ap_gemm_kbit_workspace_bytes(64, 4096, 4) == 64 * 1024 + 4 * 64 * 4096 * 4
    # communication buffer: header + two generations of eight inbox slots
    assert lib.ap_comm_buffer_bytes(1000) == 20480 + 2 * 8 * 2 * 1024      # half of every inbox line is sequence numbers
    buf = ctypes.create_string_buffer(8192)
    base = (ctypes.cast(buf, vp).value + 255) & ~255
    table = (vp * 2)(base, base)
    assert lib.ap_allreduce_oneshot(None, base, 64, table, 0, 2, 4096, None, None) == -1
    assert lib.ap_allreduce_oneshot(base, base, 60, table, 0, 2, 4096, None, None) == -3      # count % 8
    assert lib.ap_allreduce_oneshot(base, base, 64, table, 2, 2, 4096, None, None) == -3      # rank out of range
    assert lib.ap_allreduce_oneshot(base, base, 64, table, 0, 9, 4096, None, None) == -3      # more than 8 ranks
    assert lib.ap_allreduce_oneshot(base, base, 4096, table, 0, 2, 4096, None, None) == -3    # payload above the stated maximum
    assert lib.ap_allreduce_oneshot(base + 2, base, 64, table, 0, 2, 4096, None, None) == -4  # alignment
