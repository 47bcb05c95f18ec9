"""The split-K GEMV entry point that brings its own scratch (ap_matmul_kbit_splitk_noalloc).

Some callers of this library may not allocate device memory at the point where they call it: a
serving loop whose memory pool is frozen, a host framework that owns the device heap, a plugin
that receives nothing but its operands.  For them the library carries a fixed 2 MiB scratch area.
The test drives the entry point straight through the C ABI with ctypes, twice in a row on each
case (the second call finds the first call's leftovers in the shared area), and compares with the
workspace variant of the same kernel, which the other tests already hold against the oracle.

Named so that pytest collects it last: a run that stops at the first failure has then already
been through every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

# same tolerances as tests/test_gpu_parity.py
MAX_REL = 1e-2
REL_FLOOR = 0.05
MEAN_ABS = 1e-3


@pytest.fixture(scope="module")
def lib():
    import any_precision_ext
    lib = any_precision_ext.load_library()
    vp, i, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
    lib.ap_matmul_kbit_splitk_noalloc.restype = i
    lib.ap_matmul_kbit_splitk_noalloc.argtypes = [vp, vp, i64, vp, vp, i, i, i, i, i, vp]
    lib.ap_builtin_scratch_bytes.restype = ctypes.c_size_t
    assert torch.cuda.is_available(), "this test needs a CUDA device"
    return lib


def _operands(N, K, M, w, seed):
    from anyprec_b200 import packing
    gen = torch.Generator(device="cuda").manual_seed(seed)
    q = packing.random_qweight(8, N, K, device="cuda", generator=gen)
    lut = packing.random_lut(N, w, device="cuda", generator=gen)
    x = torch.randn((M, K), device="cuda", generator=gen).to(torch.float16)
    return x, q, lut


def _close(y, ref):
    y, ref = y.double().cpu().numpy(), ref.double().cpu().numpy()
    err = np.abs(y - ref)
    denom = np.maximum(np.abs(ref), REL_FLOOR * np.abs(ref).max())
    assert (err / denom).max() <= MAX_REL
    assert err.mean() <= MEAN_ABS


@pytest.mark.parametrize("N,K,M,w,splits", [(128, 8192, 1, 4, 8), (1024, 4096, 3, 8, 4), (64, 11008, 8, 3, 5),
                                             (256, 2048, 1, 6, 2), (512, 3584, 12, 5, 3)])
def test_noalloc_matches_workspace_variant_twice(lib, N, K, M, w, splits):
    import any_precision_ext as ext
    x, q, lut = _operands(N, K, M, w, seed=N + K + w)
    want = ext.matmul_kbit(x, q, lut, w, splits=splits)            # workspace variant (ap_matmul_kbit_splitk)
    unsplit = ext.matmul_kbit(x, q, lut, w, splits=1)
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):
        out = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
        rc = lib.ap_matmul_kbit_splitk_noalloc(x.data_ptr(), q.data_ptr(), q.stride(0), lut.data_ptr(), out.data_ptr(),
                                               M, N, K, w, splits, stream)
        assert rc == 0, lib.ap_strerror(rc)
        torch.cuda.synchronize()
        assert not torch.isnan(out).any(), f"call {call}: some outputs were never written"
        # the splits are summed in a fixed order, so the two variants agree to the last bit
        assert torch.equal(out, want), f"call {call}"
        _close(out, unsplit)


def test_noalloc_refuses_what_does_not_fit(lib):
    cap = lib.ap_builtin_scratch_bytes()
    assert cap == 2 * 1024 * 1024
    N, K, M, w = 70000 // 16 * 16, 8192, 1, 3                      # 8 splits x 69 984 floats > 2 MiB
    x, q, lut = _operands(N, K, M, w, seed=1)
    out = torch.zeros((M, N), dtype=torch.float16, device="cuda")
    rc = lib.ap_matmul_kbit_splitk_noalloc(x.data_ptr(), q.data_ptr(), q.stride(0), lut.data_ptr(), out.data_ptr(),
                                           M, N, K, w, 8, None)
    assert rc == -8
    assert b"scratch" in lib.ap_strerror(rc)
    # one split needs no scratch at all and is always accepted
    rc = lib.ap_matmul_kbit_splitk_noalloc(x.data_ptr(), q.data_ptr(), q.stride(0), lut.data_ptr(), out.data_ptr(),
                                           M, N, K, w, 1, None)
    assert rc == 0
    # a request for more ranges than the row has 1024-weight groups is judged by what will run: K = 128
    # has one group, so nothing is split and nothing is refused
    x2, q2, lut2 = _operands(N, 128, M, w, seed=2)
    rc = lib.ap_matmul_kbit_splitk_noalloc(x2.data_ptr(), q2.data_ptr(), q2.stride(0), lut2.data_ptr(), out.data_ptr(),
                                           M, N, 128, w, 8, None)
    assert rc == 0
    torch.cuda.synchronize()


def test_noalloc_scratch_serves_changing_shapes(lib):
    """Calls of different shapes share the one area: the ticket counters of a layer with many rows
    must not lie where an earlier layer with few rows left partial sums."""
    import any_precision_ext as ext
    stream = torch.cuda.current_stream().cuda_stream
    for N, K, M, w, splits in [(256, 4096, 8, 4, 4), (4096, 2048, 1, 3, 2), (512, 8192, 8, 8, 8), (8192, 1024, 2, 5, 1 + 1),
                               (2048, 4096, 1, 6, 2)]:
        x, q, lut = _operands(N, K, M, w, seed=3 * N + K)
        want = ext.matmul_kbit(x, q, lut, w, splits=splits)
        out = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
        rc = lib.ap_matmul_kbit_splitk_noalloc(x.data_ptr(), q.data_ptr(), q.stride(0), lut.data_ptr(), out.data_ptr(),
                                               M, N, K, w, splits, stream)
        assert rc == 0, lib.ap_strerror(rc)
        torch.cuda.synchronize()
        assert torch.equal(out, want), (N, K, M, w, splits)
        _close(out, ext.matmul_kbit(x, q, lut, w, splits=1))
