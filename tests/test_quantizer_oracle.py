"""The seed + upscale oracle (oracle/seed_upscale.py) against the fixtures that the reference's own
``_seed_and_upscale_layer`` produced (tests/golden/make_quantizer_fixture.py: the reference routine run
unmodified, with the oracle's two k-means primitives standing in for the package the reference imports
them from), and its own invariants."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import oracle
from oracle import seed_upscale as su

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
FIXTURES = sorted(glob.glob(os.path.join(GOLDEN, "quantizer_*.npz")))


def fixture_layers():
    for path in FIXTURES:
        g = np.load(path)
        for i in range(int(g["modules"])):
            yield os.path.basename(path), g, i


def test_fixtures_present():
    assert len(FIXTURES) == 3


@pytest.mark.parametrize("blocked", [False, True])
def test_rows_equal_the_reference_routine(blocked):
    """Codes and fp32 tables of every level, bit for bit; with the reference's left-to-right prefix sums and
    with the CUDA kernel's blocked order."""
    for name, g, i in fixture_layers():
        sb, pb = int(g["seed_bit"]), int(g["parent_bit"])
        w, s = g[f"weight{i}"], g[f"sens{i}"]
        for r in range(w.shape[0]):
            luts, codes = su.seed_and_upscale_row(w[r], s[r], sb, pb, blocked=blocked)
            assert np.array_equal(codes, g[f"codes{i}"][r]), (name, i, r)
            for j, b in enumerate(range(sb, pb + 1)):
                assert np.array_equal(luts[j], g[f"lut{i}_{b}_f32"][r]), (name, i, r, b)


def test_layer_output_packs_to_what_the_reference_packer_made():
    """fp16 tables equal the ones the reference's saver + packer stored, and this repo's packer turns the codes
    into the reference packer's ``qweight``."""
    from anyprec_b200 import packing
    for name, g, i in fixture_layers():
        sb, pb = int(g["seed_bit"]), int(g["parent_bit"])
        luts, codes = su.seed_and_upscale_layer(g[f"weight{i}"], g[f"sens{i}"], sb, pb)
        for b in range(sb, pb + 1):
            assert np.array_equal(luts[b].view(np.uint16), g[f"lut{i}_{b}"].view(np.uint16)), (name, i, b)
        assert np.array_equal(oracle.pack(codes, parent_bits=pb), g[f"qweight{i}"])
        assert np.array_equal(packing.pack_codes(torch.from_numpy(codes), pb).numpy(), g[f"qweight{i}"])


def tie_heavy_row(rng, K):
    x = rng.normal(0.0, 0.02, size=K).astype(np.float16).astype(np.float32)     # a checkpoint's values repeat
    x[rng.random(K) < 0.02] = 0.0
    x[rng.random(K) < 0.01] = -0.0
    return x, (rng.normal(size=K) ** 2).astype(np.float32)


@pytest.mark.parametrize("K", [64, 1000, 4096])
def test_invariants_on_rows_with_repeated_values(K):
    rng = np.random.default_rng(K)
    x, s = tie_heavy_row(rng, K)
    luts, codes = su.seed_and_upscale_row(x, s, 3, 8)
    l2, c2 = su.seed_and_upscale_row(x, s, 3, 8, blocked=True)
    assert np.array_equal(codes, c2) and all(np.array_equal(a, b) for a, b in zip(luts, l2))
    prev = None
    for j, b in enumerate(range(3, 9)):
        t = luts[j]
        assert t.shape == (1 << b,) and np.all(np.diff(t) >= 0)                   # ascending tables
        deq = t[codes >> (8 - b)]
        err = float((s.astype(np.float64) * (x != 0) * (x - deq.astype(np.float64)) ** 2).sum())
        assert prev is None or err <= prev * (1 + 1e-9)                            # every bit helps
        prev = err
        if j:                                                                       # children bracket nothing outside the row
            assert t.min() >= x.min() and t.max() <= x.max()
    # equal values share a code at the seed level (a border never falls inside a run of equal values there)
    order = np.argsort(x + np.float32(0), kind="stable")
    sx, sc = (x + np.float32(0))[order], (codes >> 5)[order]
    assert np.all(np.diff(sc.astype(int)) >= 0)
    same = sx[1:] == sx[:-1]
    assert np.all(sc[1:][same] == sc[:-1][same])


def test_degenerate_rows():
    # one value; all zeros (no sample weight anywhere: treated as unweighted); fewer values than clusters
    for x in (np.full(40, 0.25, np.float32), np.zeros(64, np.float32), np.array([0.1, -0.2, 0.3], np.float32)):
        s = np.ones_like(x)
        luts, codes = su.seed_and_upscale_row(x, s, 3, 8)
        deq = luts[-1][codes]
        assert np.array_equal(deq, x + np.float32(0)), (x[:4], deq[:4])
    # zero sensitivity everywhere: plain (unweighted) k-means, still a valid quantisation
    rng = np.random.default_rng(3)
    x = rng.normal(size=300).astype(np.float32)
    luts, codes = su.seed_and_upscale_row(x, np.zeros(300, np.float32), 3, 8)
    assert np.abs(luts[-1][codes] - x).max() < 0.2


def test_two_cluster_split_is_a_lloyd_fixed_point():
    rng = np.random.default_rng(11)
    for n in (2, 3, 7, 100, 1001):
        x = np.sort(rng.normal(size=n).astype(np.float32))
        w = (rng.normal(size=n) ** 2).astype(np.float64)
        wp, wxp = np.cumsum(w), np.cumsum(w * x.astype(np.float64))
        c, b = su.kmeans_two_cluster(x, wp, wxp, 0, n)
        d = int(b[1])
        assert 1 <= d <= n - 1 and c[0] <= c[1]
        mid = (c[0] + c[1]) / 2
        assert x[d - 1] <= mid < x[d] or n == 2
