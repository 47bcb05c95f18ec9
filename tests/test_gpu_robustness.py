"""Stand-ins for a memory checker (none can be run on the GPUs these tests use) and regression
tests for hazards found by review:

* guard bands: every operator writes into the middle of a larger buffer whose margins hold NaN
  patterns; the margins must come back untouched and the payload fully written;
* a table entry that is Inf or NaN must not leak into rows through the zero-padded lanes of a short
  last group (K % 1024 != 0);
* the fused prefill kernel's hand-over between its warps, repeated many times on the one-block
  shapes where a race would show;
* a CUDA graph that captured a split-K call keeps working after the module's scratch buffer has
  been replaced by a larger one.
"""
import numpy as np
import pytest
import torch

from conftest import make_layer
from oracle import oracle

pytestmark = pytest.mark.gpu

MAX_REL = 1e-2
REL_FLOOR = 0.05
MEAN_ABS = 1e-3
GUARD = 256          # halfs of margin on either side


@pytest.fixture(scope="module")
def ext():
    import any_precision_ext
    any_precision_ext.load_library()
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    return any_precision_ext


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def close(y, ref):
    y, ref = np.asarray(y, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    err = np.abs(y - ref)
    denom = np.maximum(np.abs(ref), REL_FLOOR * np.abs(ref).max())
    assert (err / denom).max() <= MAX_REL, f"max rel err {(err / denom).max():.3e}"
    assert err.mean() <= MEAN_ABS


def guarded(shape):
    """A NaN-filled flat buffer and a contiguous view of `shape` in its middle (16-byte aligned)."""
    n = int(np.prod(shape))
    flat = torch.full((n + 2 * GUARD,), float("nan"), dtype=torch.float16, device="cuda")
    return flat, flat[GUARD:GUARD + n].view(*shape)


def check_guards(flat, n, what):
    assert torch.isnan(flat[:GUARD]).all(), f"{what}: wrote before the output"
    assert torch.isnan(flat[GUARD + n:]).all(), f"{what}: wrote past the output"
    assert not torch.isnan(flat[GUARD:GUARD + n]).any(), f"{what}: left part of the output unwritten"


@pytest.mark.parametrize("N", [4, 16, 48])
@pytest.mark.parametrize("K", [32, 1024, 1056, 11008])
def test_guard_bands_decode_and_dequant(ext, N, K):
    codes, luts = make_layer(N, K, seed=N * 13 + K)
    qn = oracle.pack(codes)
    q = dev(qn)
    rng = np.random.default_rng(N + K)
    for w in range(3, 9):
        lut = dev(luts[w])
        flat, W = guarded((N, K))
        ext.dequant_kbit(q, lut, w, out=W)
        torch.cuda.synchronize()
        check_guards(flat, N * K, f"dequant N={N} K={K} w={w}")
        assert np.array_equal(W.cpu().numpy().view(np.uint16), oracle.c_dequant(qn, luts[w], w).view(np.uint16))
        for M in range(1, 9):
            xn = rng.normal(size=(M, K)).astype(np.float16)
            flat, y = guarded((M, N))
            ext.matmul_kbit(dev(xn), q, lut, w, out=y)
            torch.cuda.synchronize()
            check_guards(flat, M * N, f"matmul N={N} K={K} w={w} M={M}")
            if M in (1, 5, 8):
                close(y.cpu().numpy(), oracle.c_matmul(xn, qn, luts[w], w))


@pytest.mark.parametrize("N,K,M", [(128, 1024, 9), (128, 2304, 100), (256, 1152, 70), (128, 11008, 130)])
def test_guard_bands_fused_prefill(ext, N, K, M):
    """Token counts that are not a multiple of the kernel's token block, with and without split-K."""
    codes, luts = make_layer(N, K, seed=N + K + M)
    qn = oracle.pack(codes)
    q = dev(qn)
    xn = np.random.default_rng(M).normal(size=(M, K)).astype(np.float16)
    x = dev(xn)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for w in (3, 4, 6, 8):
        ref = oracle.c_matmul(xn, qn, luts[w], w)
        for splits in (1, 2):
            if splits > 1 and K % 256:
                continue
            flat, y = guarded((M, N))
            ext.gemm_kbit(x, q, dev(luts[w]), w, out=y, status=status, splits=splits)
            torch.cuda.synchronize()
            check_guards(flat, M * N, f"gemm N={N} K={K} M={M} w={w} splits={splits}")
            close(y.cpu().numpy(), ref)
    assert int(status.item()) == 0


@pytest.mark.parametrize("K", [1152, 11008, 3584, 1056])
@pytest.mark.parametrize("bad", [float("inf"), float("nan")])
def test_non_finite_table_entry_stays_in_its_own_products(ext, K, bad):
    """Entry 0 of every row's table is Inf/NaN and no weight uses code 0: the result must be
    finite and right.  Lanes past the end of a short last group used to multiply entry 0 by zero."""
    N = 32
    rng = np.random.default_rng(K)
    for w in (3, 4, 5, 8):
        hi = (1 << w)
        codes_w = rng.integers(1, hi, size=(N, K), dtype=np.uint8)               # never code 0 at this precision
        codes = (codes_w.astype(np.uint16) << (8 - w)).astype(np.uint8)          # parent codes whose top w bits are codes_w
        qn = oracle.pack(codes)
        lut = np.sort(rng.normal(0, 0.02, size=(N, hi)).astype(np.float32), axis=1).astype(np.float16)
        good = lut.copy()
        lut[:, 0] = bad
        for M in (1, 2, 8):
            xn = rng.normal(size=(M, K)).astype(np.float16)
            y = ext.matmul_kbit(dev(xn), dev(qn), dev(lut), w).cpu().numpy()
            assert np.isfinite(y).all(), f"K={K} w={w} M={M}: {np.count_nonzero(~np.isfinite(y))} non-finite outputs"
            close(y, oracle.c_matmul(xn, qn, good, w))


@pytest.mark.parametrize("N,K,M", [(128, 2048, 64), (128, 2048, 100), (128, 11008, 64), (128, 11008, 100)])
def test_fused_prefill_hand_over_many_times(ext, N, K, M):
    """One thread block, eight or 43 super-tiles: the shape on which a hand-over race between the
    producer warps and the two MMA-issuing warps showed once.  Fifty launches per case, each compared
    with the oracle; the status word (set when a bounded wait runs out) must stay 0."""
    codes, luts = make_layer(N, K, seed=N + K + M)
    qn = oracle.pack(codes)
    q = dev(qn)
    xn = np.random.default_rng(M).normal(size=(M, K)).astype(np.float16)
    x = dev(xn)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for w in (3, 4, 8):
        lut = dev(luts[w])
        ref = oracle.c_matmul(xn, qn, luts[w], w)
        for splits in (1, 2):
            first = None
            for it in range(50):
                y = ext.gemm_kbit(x, q, lut, w, status=status, splits=splits)
                if first is None:
                    first = y.clone()
                    close(first.cpu().numpy(), ref)
                else:
                    assert torch.equal(y, first), f"w={w} splits={splits}: launch {it} differs from launch 0"
            assert int(status.item()) == 0, f"w={w} splits={splits}: a bounded wait ran out"


def test_graph_survives_scratch_regrow(ext):
    """A graph captured with a split-K call holds the scratch buffer's address.  When a later call needs a
    larger scratch the module replaces it but keeps the old one alive; the replayed graph must still
    write the right result while other tensors are allocated and filled meanwhile."""
    from anyprec_b200 import packing
    gen = torch.Generator(device="cuda").manual_seed(3)
    N, K = 256, 8192
    q = packing.random_qweight(8, N, K, device="cuda", generator=gen)
    lut = packing.random_lut(N, 4, device="cuda", generator=gen)
    x = torch.randn((1, K), device="cuda", generator=gen).to(torch.float16)
    want = ext.matmul_kbit(x, q, lut, 4, splits=1)
    stream = torch.cuda.Stream()
    out = torch.empty((1, N), dtype=torch.float16, device="cuda")
    with torch.cuda.stream(stream):
        ext.matmul_kbit(x, q, lut, 4, out=out, splits=8)                         # creates this stream's scratch
        torch.cuda.synchronize()
        before = ext._workspaces[(torch.cuda.current_device(), stream.cuda_stream)]
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            ext.matmul_kbit(x, q, lut, 4, out=out, splits=8)
        # force a regrow on the same stream: far more partial sums than the scratch holds
        big_n = 65536
        qb = packing.random_qweight(3, big_n, 2048, device="cuda", generator=gen)
        lb = packing.random_lut(big_n, 3, device="cuda", generator=gen)
        xb = torch.randn((8, 2048), device="cuda", generator=gen).to(torch.float16)
        need = ext.load_library().ap_matmul_kbit_workspace_bytes(8, big_n, 8)
        assert need > before.numel()
        ext.matmul_kbit(xb, qb, lb, 3, splits=8)
        after = ext._workspaces[(torch.cuda.current_device(), stream.cuda_stream)]
        assert after.data_ptr() != before.data_ptr() and after.numel() >= need
    torch.cuda.synchronize()
    del before
    junk = [torch.full((1 << 20,), 7, dtype=torch.int32, device="cuda") for _ in range(16)]   # would land in a freed scratch
    for _ in range(3):
        out.fill_(float("nan"))
        g.replay()
        torch.cuda.synchronize()
        assert torch.allclose(out.float(), want.float(), rtol=2e-3, atol=2e-3)
    assert all(int(j[0]) == 7 and int(j[-1]) == 7 for j in junk)
    assert ext.reserve_workspace(nbytes=1 << 20) >= 1 << 20
