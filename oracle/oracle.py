"""CPU oracle for the any-precision bitplane serving path.  TEST INFRASTRUCTURE ONLY.

A numpy restatement of what the reference project (SNU-ARC/any-precision-llm) computes
on its bitplane operands, plus ctypes access to the same restatement in C
(``anyprec_oracle.c``) and, where it has been built, to the reference's own
``dequant.cuh`` compiled for the host (``_ref/libref_dequant.so``).

The shipped CUDA library and its Python front end never import this module; it exists
to check them and to time the CPU baseline.

Parity status: the reference has no tests or golden vectors for this path.  The oracle
is pinned against outputs of the reference's own packer and dequantisation kernel source
run on the build machine (``tests/golden/make_golden.py`` made the committed vectors).

Citations are paths inside the reference project.

* ``qweight`` int32 ``[P, N, K/32]``, plane 0 = MSB of the parent code
  (any_precision/quantization/pack.py:90-96).
* byte permutation inside a row (pack.py:12-76; read back by
  any_precision/modules/kernels/matmul.cuh:73-76,86,95-125 and dequant.cuh:207-240):
  word ``t`` of a group of ``E`` words (E = 32, or (K % 1024)/32 for the last, partial
  group), byte ``j`` from the most significant, bit ``e`` from that byte's MSB, holds the
  plane bit of weight ``k = base + 8*E*j + 8*t + e``.
* ``c_w = c_P >> (P - w)`` and ``W_w[n, k] = lut_w[n, c_w[n, k]]``
  (any_precision/evaluate/eval.py:104-105, dequant.cuh:226-240).
* ``y = x @ W_w.T`` (matmul.cuh:117-131), here in fp32/fp64 rather than the reference's
  fp16 accumulation.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from functools import lru_cache

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))


# --------------------------------------------------------------------------- numpy
@lru_cache(maxsize=64)
def element_map(K: int) -> np.ndarray:
    """``kmap[word, j, e]`` = weight index k held by byte ``j`` (MSB first), bit ``e``
    (MSB first) of int32 word ``word`` of a row.  Follows pack.py:12-76."""
    if K % 32 != 0:
        raise ValueError("K must be a multiple of 32")
    words = K // 32
    full = K // 1024
    tail_e = (K % 1024) // 32
    kmap = np.empty((words, 4, 8), dtype=np.int64)
    j = np.arange(4).reshape(1, 4, 1)
    e = np.arange(8).reshape(1, 1, 8)
    for g in range(full):
        t = np.arange(32).reshape(32, 1, 1)
        kmap[g * 32:(g + 1) * 32] = g * 1024 + 256 * j + 8 * t + e
    if tail_e:
        t = np.arange(tail_e).reshape(tail_e, 1, 1)
        kmap[full * 32:] = full * 1024 + 8 * tail_e * j + 8 * t + e
    return kmap


def pack(codes: np.ndarray, parent_bits: int = 8) -> np.ndarray:
    """uint8 codes ``[N, K]`` -> int32 ``[P, N, K/32]`` (pack.py:90-99 then :12-76)."""
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    N, K = codes.shape
    kmap = element_map(K)                       # [words, 4, 8]
    gathered = codes[:, kmap.reshape(-1)]        # [N, words*32], MSB-first bit order
    out = np.empty((parent_bits, N, K // 32), dtype=np.uint32)
    for p in range(parent_bits):
        bits = (gathered >> (parent_bits - 1 - p)) & 1
        by = np.packbits(bits.astype(np.uint8), axis=1, bitorder="big")   # [N, words*4]
        out[p] = np.ascontiguousarray(by).reshape(N, K // 32, 4).view(">u4").reshape(N, K // 32)
    return out.view(np.int32)


def unpack(qweight: np.ndarray, w_bits: int) -> np.ndarray:
    """int32 ``[>=w, N, K/32]`` -> w-bit codes uint8 ``[N, K]`` from planes ``0..w-1``."""
    q = np.ascontiguousarray(qweight[:w_bits]).view(np.uint32)
    _, N, words = q.shape
    K = words * 32
    kmap = element_map(K).reshape(-1)
    codes = np.zeros((N, K), dtype=np.uint8)
    for p in range(w_bits):
        by = q[p].astype(">u4").view(np.uint8).reshape(N, words * 4)
        bits = np.unpackbits(by, axis=1, bitorder="big")                   # [N, K] permuted
        plane = np.empty_like(bits)
        plane[:, kmap] = bits
        codes |= (plane << (w_bits - 1 - p)).astype(np.uint8)
    return codes


def dequant(qweight: np.ndarray, lut: np.ndarray, w_bits: int) -> np.ndarray:
    """fp16 ``[N, K]``: ``lut[n, c_w[n, k]]`` (eval.py:104-105)."""
    codes = unpack(qweight, w_bits)
    lut = np.asarray(lut)
    assert lut.shape == (codes.shape[0], 1 << w_bits), lut.shape
    return np.take_along_axis(lut, codes.astype(np.int64), axis=1)


def matmul(x: np.ndarray, qweight: np.ndarray, lut: np.ndarray, w_bits: int) -> np.ndarray:
    """fp32 ``x @ W_w.T`` with fp64 accumulation; x ``[..., K]`` fp16."""
    W = dequant(qweight, lut, w_bits).astype(np.float64)
    x2 = np.asarray(x).astype(np.float64).reshape(-1, W.shape[1])
    y = x2 @ W.T
    return y.astype(np.float32).reshape(*np.asarray(x).shape[:-1], W.shape[0])


def algorithmic_bytes_gemv(M: int, N: int, K: int, w_bits: int) -> int:
    """planes + that precision's LUT + activations in + out."""
    return N * K * w_bits // 8 + N * (1 << w_bits) * 2 + M * K * 2 + M * N * 2


# --------------------------------------------------------------------------- C oracle
def reference_root():
    """Where a checkout of the reference project lies, or None: the ``REF_ROOT`` environment variable,
    else a directory named ``reference`` beside this repository."""
    cand = os.environ.get("REF_ROOT") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    return cand if os.path.isdir(os.path.join(cand, "any_precision", "modules", "kernels")) else None


def build(force: bool = False) -> None:
    """Compile ``liboracle.so`` (and ``_ref/`` when the reference tree is present)."""
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "anyprec_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "liboracle.so"], check=True, capture_output=True)
    ref = reference_root()
    if ref is None:
        return                      # the checkers built from the reference's sources travel prebuilt
    ref_so = os.path.join(_HERE, "_ref", "libref_dequant.so")
    if force or not os.path.exists(ref_so):
        subprocess.run(["make", "-C", _HERE, f"REF_ROOT={ref}", "ref"], check=True, capture_output=True)
    shim = os.path.join(_HERE, "ref_cuda_shim.cu")
    cuda_so = os.path.join(_HERE, "_ref", "libref_cuda.so")
    if force or not os.path.exists(cuda_so) or os.path.getmtime(cuda_so) < os.path.getmtime(shim):
        subprocess.run(["make", "-C", _HERE, f"REF_ROOT={ref}", "refcuda"], check=True, capture_output=True)


def usable_cpus() -> int:
    """CPUs this process may really use: the affinity mask, cut down to the cgroup CPU quota
    when there is one.  A container can see every core of a large host while its quota allows
    far fewer; an OpenMP team sized for the visible cores then spends its quota spinning."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    try:
        with open("/sys/fs/cgroup/cpu.max") as f:
            quota, period = f.read().split()[:2]
        if quota != "max":
            n = min(n, max(1, int(int(quota) / int(period))))
    except (OSError, ValueError):
        try:
            with open("/sys/fs/cgroup/cpu/cpu.cfs_quota_us") as f:
                quota = int(f.read())
            with open("/sys/fs/cgroup/cpu/cpu.cfs_period_us") as f:
                period = int(f.read())
            if quota > 0:
                n = min(n, max(1, quota // period))
        except (OSError, ValueError):
            pass
    return max(1, n)


@lru_cache(maxsize=1)
def clib() -> ctypes.CDLL:
    build()
    lib = ctypes.CDLL(os.path.join(_HERE, "liboracle.so"))
    lib.ap_oracle_set_threads.argtypes = [ctypes.c_int]
    lib.ap_oracle_set_threads(min(8, usable_cpus()))    # checks are small; a big team only adds overhead
    i, i64, p = ctypes.c_int, ctypes.c_int64, ctypes.c_void_p
    lib.ap_oracle_pack.argtypes = [p, i, i, i, p]
    lib.ap_oracle_unpack.argtypes = [p, i64, i, i, i, p]
    lib.ap_oracle_dequant.argtypes = [p, i64, p, i, i, i, p]
    lib.ap_oracle_matmul.argtypes = [p, p, i64, p, i, i, i, i, p]
    lib.ap_oracle_set_threads.argtypes = [i]
    return lib


def _ptr(a: np.ndarray) -> int:
    return a.ctypes.data


def c_pack(codes: np.ndarray, parent_bits: int = 8) -> np.ndarray:
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    N, K = codes.shape
    out = np.empty((parent_bits, N, K // 32), dtype=np.int32)
    rc = clib().ap_oracle_pack(_ptr(codes), N, K, parent_bits, _ptr(out))
    assert rc == 0
    return out


def c_unpack(qweight: np.ndarray, w_bits: int) -> np.ndarray:
    q = np.ascontiguousarray(qweight, dtype=np.int32)
    _, N, words = q.shape
    out = np.empty((N, words * 32), dtype=np.uint8)
    rc = clib().ap_oracle_unpack(_ptr(q), N * words, N, words * 32, w_bits, _ptr(out))
    assert rc == 0
    return out


def c_dequant(qweight: np.ndarray, lut: np.ndarray, w_bits: int) -> np.ndarray:
    q = np.ascontiguousarray(qweight, dtype=np.int32)
    lut = np.ascontiguousarray(lut, dtype=np.float16)
    _, N, words = q.shape
    out = np.empty((N, words * 32), dtype=np.float16)
    rc = clib().ap_oracle_dequant(_ptr(q), N * words, _ptr(lut), N, words * 32, w_bits, _ptr(out))
    assert rc == 0
    return out


def c_matmul(x: np.ndarray, qweight: np.ndarray, lut: np.ndarray, w_bits: int,
             threads: int | None = None) -> np.ndarray:
    q = np.ascontiguousarray(qweight, dtype=np.int32)
    lut = np.ascontiguousarray(lut, dtype=np.float16)
    x = np.ascontiguousarray(x, dtype=np.float16)
    _, N, words = q.shape
    K = words * 32
    M = x.size // K
    out = np.empty((M, N), dtype=np.float32)
    if threads:
        clib().ap_oracle_set_threads(threads)
    rc = clib().ap_oracle_matmul(_ptr(x), _ptr(q), N * words, _ptr(lut), M, N, K, w_bits, _ptr(out))
    assert rc == 0
    return out.reshape(*x.shape[:-1], N)


def c_threads() -> int:
    return clib().ap_oracle_max_threads()


def c_set_threads(n: int) -> None:
    clib().ap_oracle_set_threads(int(n))


# --------------------------------------------------------------------------- reference kernel on the host
@lru_cache(maxsize=1)
def reflib():
    """The reference's dequant.cuh compiled for the host, or None if it was never built."""
    path = os.path.join(_HERE, "_ref", "libref_dequant.so")
    if not os.path.exists(path):
        try:
            build()
        except Exception:
            return None
    if not os.path.exists(path):
        return None
    lib = ctypes.CDLL(path)
    i, p = ctypes.c_int, ctypes.c_void_p
    lib.ref_dequant_kbit.argtypes = [p, p, p, i, i, i]
    lib.ref_transpose_word.argtypes = [p, i, p]
    return lib


def ref_dequant(qweight: np.ndarray, lut: np.ndarray, w_bits: int) -> np.ndarray:
    """dequant_kbit_store<w_bits> of the reference (dequant.cuh:177-242) run on the CPU.
    Needs a contiguous qweight whose plane stride is N*K/32 and N % 4 == 0
    (kernels/main.cu:82)."""
    lib = reflib()
    if lib is None:
        raise RuntimeError("oracle/_ref/libref_dequant.so has not been built")
    q = np.ascontiguousarray(qweight, dtype=np.int32)
    lut = np.ascontiguousarray(lut, dtype=np.float16)
    _, N, words = q.shape
    out = np.zeros((N, words * 32), dtype=np.float16)
    rc = lib.ref_dequant_kbit(_ptr(q), _ptr(lut), _ptr(out), N, words * 32, w_bits)
    assert rc == 0
    return out
