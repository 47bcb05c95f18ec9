"""Generate the committed golden vectors by running the reference project's own code.

Run on a machine that has the reference tree:

    python tests/golden/make_golden.py [--ref /path/to/any-precision-llm]

What is run, unmodified and loaded from where it lies:

* the reference packer ``any_precision/quantization/pack.py`` — its
  ``_process_layer_data`` (pack.py:79-114) is fed a layer directory laid out the way
  the reference quantizer writes it (``weights/l0.pt``, ``lut_{b}/l0.pt``) and returns
  the ``qweight`` bitplanes and ``lut{b}`` tables of the packed checkpoint;
* the reference kernel source ``any_precision/modules/kernels/dequant.cuh`` compiled
  for the host by ``oracle/Makefile`` (``oracle/_ref/libref_dequant.so``) — its
  ``dequant_kbit_store<w>`` produces the dequantised fp16 weights.

Each case is written to ``tests/golden/case_*.npz`` with the input codes, the LUTs,
the reference's qweight, and for every w in 3..8 the reference's dequantised weights
(full arrays for small cases, SHA-256 digests for all).  Inputs are seeded synthetic
data: uniform uint8 codes and per-row sorted N(0, 0.02) fp16 centroids.
"""
from __future__ import annotations

import argparse
import hashlib
import importlib.util
import os
import sys
import tempfile

os.environ.setdefault("NUMBA_CACHE_DIR", tempfile.mkdtemp(prefix="numba_cache_"))
os.environ["PYTHONDONTWRITEBYTECODE"] = "1"
sys.dont_write_bytecode = True

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

# (name, N, K, store_full_dequant)
CASES = [
    ("k32", 4, 32, True),            # one word per row: the tail rule with E = 1
    ("k64", 4, 64, True),            # E = 2
    ("k1024", 8, 1024, True),        # exactly one full group
    ("k1056", 4, 1056, True),        # full group + tail of one word
    ("k2048", 4, 2048, False),
    ("k3584", 4, 3584, False),       # 3 full groups + tail E = 16 (an 8-way shard of 28672)
    ("k4096", 16, 4096, False),      # the 4096 x 4096 layer's row length
    ("k11008", 4, 11008, False),     # 10 full groups + tail E = 24
]
SEED = 20240229
PARENT, SEEDP = 8, 3


def load_reference_packer(ref_root: str):
    path = os.path.join(ref_root, "any_precision", "quantization", "pack.py")
    spec = importlib.util.spec_from_file_location("_ref_pack", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def make_inputs(rng: np.random.Generator, N: int, K: int):
    codes = rng.integers(0, 256, size=(N, K), dtype=np.uint8)
    luts = {}
    for b in range(SEEDP, PARENT + 1):
        cent = np.sort(rng.normal(0.0, 0.02, size=(N, 1 << b)).astype(np.float32), axis=1)
        luts[b] = cent.astype(np.float16)
    return codes, luts


def run_reference_packer(refpack, codes: np.ndarray, luts: dict) -> dict:
    """Lay the inputs out as the reference quantizer does and call its packer."""
    N, K = codes.shape
    with tempfile.TemporaryDirectory() as d:
        os.makedirs(os.path.join(d, "weights"))
        torch.save({"proj": codes.reshape(N, 1, K)}, os.path.join(d, "weights", "l0.pt"))
        for b, lut in luts.items():
            os.makedirs(os.path.join(d, f"lut_{b}"))
            torch.save({"proj": lut.reshape(N, 1, 1 << b)}, os.path.join(d, f"lut_{b}", "l0.pt"))
        _, data = refpack._process_layer_data((0, d, "model", "layers", ["proj"], PARENT, SEEDP))
    return data


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="root of a checkout of the reference project (SNU-ARC/any-precision-llm)")
    args = ap.parse_args()

    from oracle import oracle

    os.environ["REF_ROOT"] = args.ref
    oracle.build()
    if oracle.reflib() is None:
        raise SystemExit("oracle/_ref/libref_dequant.so missing: run `make -C oracle ref` first")
    refpack = load_reference_packer(args.ref)
    rng = np.random.default_rng(SEED)

    for name, N, K, full in CASES:
        codes, luts = make_inputs(rng, N, K)
        data = run_reference_packer(refpack, codes, luts)
        qweight = np.asarray(data["model.layers.0.proj.qweight"])
        assert qweight.dtype == np.int32 and qweight.shape == (PARENT, N, K // 32)
        out = {"codes": codes, "qweight": qweight}
        for b in range(SEEDP, PARENT + 1):
            lut = np.asarray(data[f"model.layers.0.proj.lut{b}"])
            assert lut.dtype == np.float16 and np.array_equal(lut, luts[b])
            out[f"lut{b}"] = lut
            w = oracle.ref_dequant(qweight, lut, b)
            out[f"sha256_w{b}"] = np.frombuffer(hashlib.sha256(w.tobytes()).digest(), dtype=np.uint8)
            if full:
                out[f"dequant_w{b}"] = w
        path = os.path.join(HERE, f"case_{name}.npz")
        np.savez_compressed(path, **out)
        print(f"{name}: N={N} K={K} -> {os.path.getsize(path)} bytes")

    # Single-bit known answers: one weight with parent code 0x80 (only plane 0 set).
    # The reference packer says which (word, bit) that weight lands in.
    kat = {}
    for K in (32, 1024, 1056, 11008):
        pos = []
        ks = sorted({0, 1, 7, 8, 31, K // 2 + 3, K - 9, K - 1})
        for k in ks:
            codes = np.zeros((4, K), dtype=np.uint8)
            codes[1, k] = 0x80
            luts = {b: np.zeros((4, 1 << b), dtype=np.float16) for b in range(SEEDP, PARENT + 1)}
            q = np.asarray(run_reference_packer(refpack, codes, luts)["model.layers.0.proj.qweight"]).view(np.uint32)
            assert np.count_nonzero(q) == 1
            p, n, wd = [int(v[0]) for v in np.nonzero(q)]
            bit = int(q[p, n, wd]).bit_length() - 1
            assert p == 0 and n == 1
            pos.append((k, wd, bit))
        kat[f"K{K}"] = np.asarray(pos, dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "single_bit_positions.npz"), **kat)
    print("single_bit_positions.npz written")


if __name__ == "__main__":
    main()
