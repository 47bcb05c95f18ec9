"""Generate ``tests/golden/quantizer_*.npz`` by running the reference project's own seed + upscale code.

Run on a machine that has the reference tree:

    python tests/golden/make_quantizer_fixture.py --ref /path/to/any-precision-llm

What is run, unmodified and loaded from where it lies: ``any_precision/quantization/quantize.py`` —
its ``_seed_and_upscale_layer`` (quantize.py:85-187, with ``_upscale_group`` and ``_increment_group``)
is compiled by numba and fed seeded synthetic layers.  The package it imports for its two k-means
primitives, ``flash1dkmeans``, is not part of the reference tree and not installed; a stand-in module of
that name is registered first, whose ``numba_kmeans_1d_k_cluster`` and ``numba_kmeans_1d_two_cluster``
are ``oracle/seed_upscale.py``'s ``kmeans_k_cluster`` and ``kmeans_two_cluster`` handed to ``numba.njit``
(same source, same argument names as the reference's call sites at quantize.py:56-62 and :145-155).
The fixture therefore pins everything the reference does around those two calls — masking, sorting,
prefix sums, fp32 casts, border bookkeeping, empty clusters, labels, un-sorting — and the test that reads
it checks the oracle's row routine against it.

The reference's file layout for a quantised layer (``weights/l0.pt``, ``lut_{b}/l0.pt``,
quantize.py:200-218) is then written from the result and packed by the reference's
``pack.py::_process_layer_data``; the packed ``qweight`` is stored too.
"""
from __future__ import annotations

import argparse
import importlib.util
import os
import sys
import tempfile
import types

os.environ.setdefault("NUMBA_CACHE_DIR", tempfile.mkdtemp(prefix="numba_cache_"))
os.environ["PYTHONDONTWRITEBYTECODE"] = "1"
sys.dont_write_bytecode = True

import numba
import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import seed_upscale as su  # noqa: E402

# (name, [(N, K), ...] modules of the layer, seed_bit, parent_bit)
CASES = [
    ("s3p8", [(12, 512), (8, 1056)], 3, 8),
    ("s4p6", [(6, 96), (5, 2048)], 4, 6),
    ("s3p3", [(4, 256)], 3, 3),
]
SEED = 20250314


def _rebind(fn, env):
    """``fn`` with its module-level names looked up in ``env`` (so that jitted helpers are found)."""
    g = dict(fn.__globals__)
    g.update(env)
    return types.FunctionType(fn.__code__, g, fn.__name__, fn.__defaults__, fn.__closure__)


def install_kmeans_stand_in():
    env = {"_range_sum": numba.njit(su._range_sum), "_count_le": numba.njit(su._count_le)}
    k_cluster = numba.njit(_rebind(su.kmeans_k_cluster, env))
    two_cluster = numba.njit(_rebind(su.kmeans_two_cluster, env))

    @numba.njit
    def numba_kmeans_1d_k_cluster(sorted_X, n_clusters, max_iter, weights_prefix_sum, weighted_X_prefix_sum,
                                  weighted_X_squared_prefix_sum, start_idx, stop_idx, random_state=None):
        return k_cluster(sorted_X, n_clusters, max_iter, weights_prefix_sum, weighted_X_prefix_sum, start_idx, stop_idx)

    @numba.njit
    def numba_kmeans_1d_two_cluster(sorted_X, weights_prefix_sum, weighted_X_prefix_sum, start_idx, stop_idx):
        return two_cluster(sorted_X, weights_prefix_sum, weighted_X_prefix_sum, start_idx, stop_idx)

    mod = types.ModuleType("flash1dkmeans")
    mod.numba_kmeans_1d_k_cluster = numba_kmeans_1d_k_cluster
    mod.numba_kmeans_1d_two_cluster = numba_kmeans_1d_two_cluster
    sys.modules["flash1dkmeans"] = mod


def load_by_path(ref_root, rel, name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(ref_root, rel))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def make_layer(rng, shapes):
    """fp32 N(0, 0.02) weights with exact zeros, squared-normal sensitivities, one row without any
    sensitivity.  Apart from the zeros (which carry no sample weight) no value occurs twice in a row: the
    reference sorts with numba's ``np.argsort``, which leaves the order of equal values to its
    implementation, and that order decides how the sample weights of equal values fall on the two sides of
    a split.  Rows with repeated values are covered by the tests that compare the CUDA kernel with the
    oracle (both keep equal values in their original order)."""
    weights, sens = [], []
    for N, K in shapes:
        w = rng.normal(0.0, 0.02, size=(N, K)).astype(np.float32)
        for r in range(N):
            assert len(np.unique(w[r])) == K
        w[rng.random(size=(N, K)) < 0.01] = 0.0
        s = (rng.normal(size=(N, K)) ** 2).astype(np.float32)
        s[0] = 0.0
        weights.append(w)
        sens.append(s)
    return weights, sens


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="root of the reference tree")
    args = ap.parse_args()
    install_kmeans_stand_in()
    refq = load_by_path(args.ref, "any_precision/quantization/quantize.py", "_ref_quantize")
    refpack = load_by_path(args.ref, "any_precision/quantization/pack.py", "_ref_pack")
    rng = np.random.default_rng(SEED)
    for name, shapes, seed_bit, parent_bit in CASES:
        weights, sens = make_layer(rng, shapes)
        luts_by_module, codes_by_module = refq._seed_and_upscale_layer(
            numba.typed.List(sens), numba.typed.List(weights), seed_bit, parent_bit, 1)
        out = {"seed_bit": seed_bit, "parent_bit": parent_bit, "modules": len(shapes)}
        names = [f"m{i}" for i in range(len(shapes))]
        with tempfile.TemporaryDirectory() as d:
            # the reference's own saver: fp16 tables, uint8 codes, one file per layer (quantize.py:200-218)
            refq._save_results(d, seed_bit, parent_bit, names, luts_by_module, codes_by_module, 0)
            _, packed = refpack._process_layer_data((0, d, "model", "layers", names, parent_bit, seed_bit))
        for i, nm in enumerate(names):
            out[f"weight{i}"] = weights[i]
            out[f"sens{i}"] = sens[i]
            out[f"codes{i}"] = np.asarray(codes_by_module[i]).astype(np.uint8)[:, 0, :]
            for j, b in enumerate(range(seed_bit, parent_bit + 1)):
                out[f"lut{i}_{b}_f32"] = np.asarray(luts_by_module[i][j])[:, 0, :].astype(np.float32)
                out[f"lut{i}_{b}"] = packed[f"model.layers.0.{nm}.lut{b}"]
            out[f"qweight{i}"] = packed[f"model.layers.0.{nm}.qweight"]
        path = os.path.join(HERE, f"quantizer_{name}.npz")
        np.savez_compressed(path, **out)
        print(f"wrote {path} ({os.path.getsize(path) / 1024:.1f} KB)")


if __name__ == "__main__":
    main()
