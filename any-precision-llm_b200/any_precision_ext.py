"""Drop-in replacement for the reference project's ``any_precision_ext`` extension module.

The reference builds ``any_precision_ext`` from ``any_precision/modules/kernels/main.cu`` with
pybind11/libtorch and exports ``matmul_kbit(in, qweight, lut, w_bits)`` and
``dequant_kbit(qweight, lut, w_bits)`` (main.cu:60-148); ``AnyPrecisionLinear`` imports exactly
those two names (any_precision/modules/AnyPrecisionLinear.py:4-7).  This module exports the same
two callables with the same positional signatures and return conventions, bound with ctypes to
the C ABI of ``lib/libanyprec_sm100.so`` (``include/anyprec_b200.h``).

Differences from the reference, all on the safe side:

* kernels are enqueued on torch's *current* stream (the reference uses the legacy default
  stream, main.cu:83,134), so calls can be captured in CUDA graphs;
* argument errors raise ``ValueError``/``TypeError`` and CUDA launch errors raise
  ``RuntimeError``; the reference uses ``assert`` and ``exit()`` (main.cu:5-12,68-70,108-111);
* ``matmul_kbit`` accepts any number of rows (the reference asserts ``M <= 8``), accumulates in
  fp32 (the reference accumulates in fp16, matmul.cuh:120-130) and takes an optional ``out=``;
* ``qweight`` may be a row slice ``full[:, n0:n1, :]`` of a larger tensor (no copy is made).

There is no CPU path: without the compiled library, or with tensors that are not on a CUDA
device, every call raises.
"""
from __future__ import annotations

import ctypes
import os

import torch

import warnings

__all__ = ["matmul_kbit", "dequant_kbit", "gemm_kbit", "gemm_kbit_supported", "take_wait_expired", "library_path",
           "load_library", "reserve_workspace"]

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "lib", "libanyprec_sm100.so")
_lib = None


def library_path() -> str:
    return _LIB_PATH


def load_library() -> ctypes.CDLL:
    """Load ``libanyprec_sm100.so`` (once) and declare its entry points."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise ModuleNotFoundError(
            f"{_LIB_PATH} is missing: build it with `python any-precision-llm_b200/build.py` "
            "(needs nvcc; there is no CPU fallback)")
    lib = ctypes.CDLL(_LIB_PATH)
    vp, i, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
    lib.ap_version.restype = i
    lib.ap_strerror.restype = ctypes.c_char_p
    lib.ap_strerror.argtypes = [i]
    lib.ap_last_cuda_error.restype = ctypes.c_char_p
    lib.ap_take_wait_expired.restype = i
    lib.ap_take_wait_expired.argtypes = []
    lib.ap_dequant_kbit.restype = i
    lib.ap_dequant_kbit.argtypes = [vp, i64, vp, vp, i, i, i, vp]
    lib.ap_matmul_kbit.restype = i
    lib.ap_matmul_kbit.argtypes = [vp, vp, i64, vp, vp, i, i, i, i, vp]
    lib.ap_matmul_kbit_workspace_bytes.restype = ctypes.c_size_t
    lib.ap_matmul_kbit_workspace_bytes.argtypes = [i, i, i]
    lib.ap_matmul_kbit_splitk.restype = i
    lib.ap_matmul_kbit_splitk.argtypes = [vp, vp, i64, vp, vp, i, i, i, i, i, vp, ctypes.c_size_t, vp]
    lib.ap_matmul_kbit_gated.restype = i
    lib.ap_matmul_kbit_gated.argtypes = [vp, vp, i64, vp, vp, i, i, i, i, i, vp, ctypes.c_size_t, vp]
    lib.ap_matmul_kbit_prenorm.restype = i
    lib.ap_matmul_kbit_prenorm.argtypes = [vp, vp, i64, vp, vp, i, i, i, i, i, vp, ctypes.c_size_t, i, vp, i, i, ctypes.c_float, vp]
    lib.ap_matmul_kbit_push.restype = i
    lib.ap_matmul_kbit_push.argtypes = [vp, vp, i64, vp, i, i, i, i, i, vp, ctypes.c_size_t, ctypes.POINTER(vp), i, i,
                                        ctypes.c_size_t, vp]
    lib.ap_matmul_kbit_residual.restype = i
    lib.ap_matmul_kbit_residual.argtypes = [vp, vp, i64, vp, vp, i, i, i, i, i, vp, ctypes.c_size_t, vp, vp, vp, vp]
    lib.ap_silu_mul.restype = i
    lib.ap_silu_mul.argtypes = [vp, vp, i, i, i, vp]
    lib.ap_gemm_kbit.restype = i
    lib.ap_gemm_kbit.argtypes = [vp, vp, i64, vp, vp, i, i, i, i, vp, vp]
    lib.ap_gemm_kbit_splits.restype = i
    lib.ap_gemm_kbit_splits.argtypes = [i, i, i]
    lib.ap_gemm_kbit_workspace_bytes.restype = ctypes.c_size_t
    lib.ap_gemm_kbit_workspace_bytes.argtypes = [i, i, i]
    lib.ap_gemm_kbit_splitk.restype = i
    lib.ap_gemm_kbit_splitk.argtypes = [vp, vp, i64, vp, vp, i, i, i, i, vp, i, vp, ctypes.c_size_t, vp]
    _lib = lib
    return lib


class _NoGuard:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NO_GUARD = _NoGuard()


_get_device = getattr(torch._C, "_cuda_getDevice", None) or torch.cuda.current_device
_get_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _on_device(device: torch.device):
    """Device guard that costs nothing in the common case (operands on the current device)."""
    if device.index is None or device.index == _get_device():
        return _NO_GUARD
    return torch.cuda.device(device)


def _current_stream(device: torch.device) -> int:
    """Raw handle of torch's current stream on ``device`` (the launch stream of every call here)."""
    if _get_raw_stream is not None:
        return _get_raw_stream(device.index if device.index is not None else _get_device())
    return torch.cuda.current_stream(device).cuda_stream


def _raise(lib, rc: int, what: str):
    msg = lib.ap_strerror(rc).decode()
    if rc == -5:
        raise RuntimeError(f"{what}: {msg}: {lib.ap_last_cuda_error().decode()}")
    raise ValueError(f"{what}: {msg}")


def _check_operands(qweight: torch.Tensor, lut: torch.Tensor, w_bits: int):
    # One shape and one stride query per tensor: this runs on every call, and each query of a tensor's
    # metadata costs a few hundred nanoseconds of host time.
    if not isinstance(w_bits, int) or not 3 <= w_bits <= 8:
        raise ValueError(f"w_bits must be an integer in [3, 8], got {w_bits!r}")
    qshape = qweight.shape
    if qweight.dtype != torch.int32 or len(qshape) != 3:
        raise TypeError("qweight must be an int32 tensor of shape [planes, N, K/32]")
    lshape = lut.shape
    if lut.dtype != torch.float16 or len(lshape) != 2:
        raise TypeError("lut must be a float16 tensor of shape [N, 2**w_bits]")
    if not qweight.is_cuda or lut.device != qweight.device:
        raise ValueError("qweight and lut must live on the same CUDA device (there is no CPU path)")
    planes, N, words = qshape
    if planes < w_bits:
        raise ValueError(f"qweight holds {planes} planes, fewer than w_bits={w_bits}")
    if lshape[0] != N or lshape[1] != (1 << w_bits):
        raise ValueError(f"lut has shape {tuple(lshape)}, expected {(N, 1 << w_bits)}")
    if not lut.is_contiguous():
        raise ValueError("lut must be contiguous")
    if words == 0 or N == 0:
        raise ValueError("empty qweight")
    # rows contiguous, words contiguous; the plane stride may exceed N*words (row slice)
    s0, s1, s2 = qweight.stride()
    if s2 != 1 or s1 != words or (planes > 1 and s0 < N * words):
        raise ValueError("qweight rows must be contiguous (a row slice of a contiguous tensor is fine)")
    plane_stride = s0 if planes > 1 else N * words
    return N, words * 32, plane_stride


def dequant_kbit(qweight: torch.Tensor, lut: torch.Tensor, w_bits: int, *, out: torch.Tensor | None = None):
    """fp16 ``[N, K]`` weight at precision ``w_bits``: ``lut[n, code >> (planes - w_bits)]``.

    Same call as the reference's ``dequant_kbit`` (kernels/main.cu:60-91); bit-exact with it.
    """
    N, K, plane_stride = _check_operands(qweight, lut, w_bits)
    lib = load_library()
    if out is None:
        out = torch.empty((N, K), dtype=torch.float16, device=qweight.device)
    elif out.shape != (N, K) or out.dtype != torch.float16 or not out.is_contiguous() or out.device != qweight.device:
        raise ValueError("out must be a contiguous float16 [N, K] tensor on the operands' device")
    with _on_device(qweight.device):
        stream = _current_stream(qweight.device)
        rc = lib.ap_dequant_kbit(qweight.data_ptr(), plane_stride, lut.data_ptr(), out.data_ptr(), N, K, w_bits, stream)
    if rc != 0:
        _raise(lib, rc, "dequant_kbit")
    return out


_workspaces: dict = {}     # (device index, stream) -> uint8 tensor whose ticket area is zero between calls
_sm_counts: dict = {}
_split_choice: dict = {}


def take_wait_expired() -> bool:
    """Synchronise the current device and say whether a decode kernel gave up one of its bounded
    waits since the last call (its output is then invalid).  A diagnostic, not for the serving loop."""
    lib = load_library()
    rc = lib.ap_take_wait_expired()
    if rc < 0:
        _raise(lib, rc, "take_wait_expired")
    return bool(rc)


def _pick_splits(device: torch.device, N: int, K: int) -> int:
    """How many ranges to cut K into: enough thread blocks (one per 16 rows and range) to give every
    SM about two, never more ranges than 1024-weight groups, at most 8."""
    key = (device.index, N, K)
    hit = _split_choice.get(key)
    if hit is not None:
        return hit
    _split_choice[key] = choice = _pick_splits_uncached(device, N, K)
    return choice


def _pick_splits_uncached(device: torch.device, N: int, K: int) -> int:
    if N % 16 or K % 128:
        return 1
    sms = _sm_counts.get(device.index)
    if sms is None:
        sms = _sm_counts[device.index] = torch.cuda.get_device_properties(device).multi_processor_count
    tiles = N // 16
    if tiles >= 2 * sms:
        return 1
    return max(1, min(8, (K + 1023) // 1024, (2 * sms) // tiles))


def _workspace(lib, device: torch.device, stream: int, M: int, N: int, splits: int):
    return _workspace_bytes(device, stream, lib.ap_matmul_kbit_workspace_bytes(M, N, splits))


_retired_workspaces: list = []     # superseded scratch tensors: captured graphs may still hold their addresses
_warned_unsplit = False
_MIN_WORKSPACE = 8 << 20            # covers 8 rows x 8 ranges x 28672 output rows (7.1 MB) without regrowing


def _workspace_bytes(device: torch.device, stream: int, need: int):
    """The split-K scratch of (device, stream), grown to ``need`` bytes; its ticket area is zero between
    calls.  None during a graph capture that would have to allocate (the caller then runs unsplit, and
    a warning says so once: call ``reserve_workspace`` before capturing).  A scratch tensor that was
    handed out is never freed: a CUDA graph captured earlier holds its address as partial-sum and
    ticket area, so when a larger one replaces it the old one is kept alive beside it."""
    global _warned_unsplit
    key = (device.index, stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < need:
        if torch.cuda.is_current_stream_capturing():
            if not _warned_unsplit:
                _warned_unsplit = True
                warnings.warn("any_precision_ext: the split-K scratch of this stream would have to grow during a CUDA "
                              f"graph capture ({need} bytes needed); this call runs without split-K (slower on layers "
                              "with few rows).  Call any_precision_ext.reserve_workspace(device, nbytes) on the "
                              "capturing stream before the capture.", RuntimeWarning, stacklevel=3)
            return None                      # no allocation inside a graph capture: run unsplit
        if ws is not None:
            _retired_workspaces.append(ws)
        ws = torch.zeros(max(need, _MIN_WORKSPACE), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def reserve_workspace(device=None, nbytes: int = _MIN_WORKSPACE) -> int:
    """Make sure the split-K scratch of torch's current stream on ``device`` holds at least ``nbytes``
    (default 8 MiB), so that later calls on that stream, inside a CUDA graph capture included, never
    have to grow it.  ``ap_matmul_kbit_workspace_bytes(M, N, splits)`` / ``ap_gemm_kbit_workspace_bytes``
    of the C ABI give the need of a call.  Returns the size now reserved."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    with torch.cuda.device(device):
        ws = _workspace_bytes(device, _current_stream(device), int(nbytes))
    if ws is None:
        raise RuntimeError("reserve_workspace cannot allocate while the stream is being captured")
    return ws.numel()


def matmul_kbit(x: torch.Tensor, qweight: torch.Tensor, lut: torch.Tensor, w_bits: int, *,
                out: torch.Tensor | None = None, splits: int | None = None, gated: bool = False,
                prenorm=None, residual=None, push=None):
    """``x @ W_w.T`` for fp16 ``x[..., K]``; returns fp16 ``[..., N]``.

    Same call as the reference's ``matmul_kbit`` (kernels/main.cu:93-143).  ``splits`` (default:
    chosen from the shape) cuts K into ranges taken by different thread blocks, for layers with too
    few rows to fill the GPU; the scratch it needs is kept per device and stream by this module.
    ``gated=True`` (no counterpart in the reference): the operand holds a gated MLP's gate and up
    projections stacked tile by tile (``packing.interleave_gate_up``) and the result is
    ``silu(gate) * up`` of shape ``[..., N / 2]``; at most eight rows, fast-kernel shapes only.
    ``residual=(h, norm_weight, ssq)`` and ``prenorm=(ssq, width, eps)`` (no counterpart either) fold a
    pre-norm decoder's residual add and RMSNorm into a pair of products: the first adds its result to
    ``h`` in place, returns ``h * norm_weight`` and leaves per-tile sums of squares in ``ssq`` (fp32
    ``[rows, N / 16]``); the second takes that as ``x`` and scales its result by
    ``rsqrt(sum(ssq) / width + eps)`` (``ap_matmul_kbit_residual`` / ``ap_matmul_kbit_prenorm``; a
    fourth entry of ``prenorm`` gives the number of partial sums per row when another kernel wrote them).
    ``push=comm.OneShotAllReduce(...).push_target`` (tensor parallelism): the product is a row-parallel
    layer's partial result and goes straight into the all-reduce inboxes of all ranks instead of a tensor
    (``ap_matmul_kbit_push``; returns None; ``OneShotAllReduce.collect`` must follow).
    """
    N, K, plane_stride = _check_operands(qweight, lut, w_bits)
    if x.dtype != torch.float16:
        raise TypeError("x must be float16")
    if x.device != qweight.device:
        raise ValueError("x must be on the same CUDA device as qweight")
    xshape = x.shape
    if len(xshape) < 1 or xshape[-1] != K:
        raise ValueError(f"x has last dimension {xshape[-1] if len(xshape) else None}, expected K={K}")
    lead = xshape[:-1]
    if len(xshape) == 2 and x.is_contiguous():
        x2, M = x, xshape[0]
    else:
        x2 = x.reshape(-1, K).contiguous()
        M = x2.shape[0]
    if M == 0:
        return torch.empty((*lead, N), dtype=torch.float16, device=x.device)
    lib = load_library()
    if push is not None:
        if gated or prenorm is not None or residual is not None or out is not None or M > 8 or N % 16:
            raise ValueError("push= goes with a plain product of at most eight rows and N % 16 == 0")
        table, rank, world, max_payload = push
        with _on_device(x.device):
            stream = _current_stream(qweight.device)
            if splits is None:
                splits = _pick_splits(x.device, N, K)
            ws = _workspace(lib, x.device, stream, M, N, splits) if splits > 1 else None
            rc = lib.ap_matmul_kbit_push(x2.data_ptr(), qweight.data_ptr(), plane_stride, lut.data_ptr(), M, N, K, w_bits,
                                         splits if ws is not None else 1, ws.data_ptr() if ws is not None else None,
                                         ws.numel() if ws is not None else 0, table, rank, world, max_payload, stream)
        if rc != 0:
            _raise(lib, rc, "matmul_kbit")
        return None
    n_out = N // 2 if gated else N
    if gated and (N % 16 or M > 8):
        raise ValueError("gated=True needs a row count that is a multiple of 16 and at most eight activation rows")
    if out is None:
        out = torch.empty((*lead, n_out), dtype=torch.float16, device=x.device)
    elif tuple(out.shape) != (*lead, n_out) or out.dtype != torch.float16 or not out.is_contiguous() \
            or out.device != x.device:
        raise ValueError("out must be a contiguous float16 [..., N] tensor on the operands' device")
    with _on_device(x.device):
        stream = _current_stream(qweight.device)
        if splits is None:
            splits = _pick_splits(x.device, N, K)
        ws = _workspace(lib, x.device, stream, M, N, splits) if splits > 1 else None
        wsp, wsn, nsp = (ws.data_ptr(), ws.numel(), splits) if ws is not None else (None, 0, 1)
        if residual is not None:
            h, norm_w, ssq = residual
            if gated or prenorm is not None or h.shape != out.shape or h.dtype != torch.float16 or not h.is_contiguous() \
                    or norm_w.dtype != torch.float16 or norm_w.numel() != N or ssq.dtype != torch.float32 \
                    or ssq.numel() < M * (N // 16) or N % 16 or M > 8:
                raise ValueError("residual=(h [..., N] fp16, norm_weight [N] fp16, ssq fp32 [rows * N / 16]), at most eight rows")
            rc = lib.ap_matmul_kbit_residual(x2.data_ptr(), qweight.data_ptr(), plane_stride, lut.data_ptr(), out.data_ptr(),
                                             M, N, K, w_bits, nsp, wsp, wsn, h.data_ptr(), norm_w.data_ptr(), ssq.data_ptr(), stream)
        elif prenorm is not None:
            ssq, width, eps = prenorm[:3]
            blocks = prenorm[3] if len(prenorm) > 3 else width // 16       # entries per row: one per 16-row tile of the writer
            if ssq.dtype != torch.float32 or blocks < 1 or ssq.numel() < M * blocks:
                raise ValueError("prenorm=(ssq fp32 [rows * blocks], width, eps[, blocks = width / 16])")
            rc = lib.ap_matmul_kbit_prenorm(x2.data_ptr(), qweight.data_ptr(), plane_stride, lut.data_ptr(), out.data_ptr(),
                                            M, N, K, w_bits, nsp, wsp, wsn, 1 if gated else 0, ssq.data_ptr(), blocks,
                                            width, eps, stream)
        elif gated:
            rc = lib.ap_matmul_kbit_gated(x2.data_ptr(), qweight.data_ptr(), plane_stride, lut.data_ptr(), out.data_ptr(),
                                          M, N, K, w_bits, splits if ws is not None else 1,
                                          ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0, stream)
        elif ws is None:
            rc = lib.ap_matmul_kbit(x2.data_ptr(), qweight.data_ptr(), plane_stride, lut.data_ptr(), out.data_ptr(),
                                    M, N, K, w_bits, stream)
        else:
            rc = lib.ap_matmul_kbit_splitk(x2.data_ptr(), qweight.data_ptr(), plane_stride, lut.data_ptr(),
                                           out.data_ptr(), M, N, K, w_bits, splits, ws.data_ptr(), ws.numel(), stream)
    if rc != 0:
        _raise(lib, rc, "matmul_kbit")
    return out


def gated_supported(x: torch.Tensor, qweight: torch.Tensor, lut: torch.Tensor) -> bool:
    """Whether ``matmul_kbit(..., gated=True)`` takes these operands: up to eight rows, ``K % 128 == 0``,
    ``N % 16 == 0``, 16-byte aligned ``x``, ``qweight`` and ``lut``, the TMA loader not switched off."""
    rows = x.numel() // x.shape[-1]
    K = qweight.shape[2] * 32
    return (rows <= 8 and K % 128 == 0 and qweight.shape[1] % 16 == 0 and qweight.stride(0) % 4 == 0 and
            (x.data_ptr() | qweight.data_ptr() | lut.data_ptr()) % 16 == 0 and
            not os.environ.get("AP_GEMV_LOADER", "").startswith("c"))


def silu_mul(gate_up: torch.Tensor, *, tiled: bool = False, out: torch.Tensor | None = None):
    """``silu(gate) * up`` for fp16 ``gate_up[..., 2 F]`` holding ``gate | up`` side by side or
    (``tiled``) tile by tile as ``matmul_kbit`` returns them for a ``packing.interleave_gate_up`` operand.
    No counterpart in the reference (it leaves this to the framework's MLP)."""
    if gate_up.dtype != torch.float16 or not gate_up.is_cuda or not gate_up.is_contiguous() or gate_up.shape[-1] % 2:
        raise ValueError("gate_up must be a contiguous float16 CUDA tensor with an even last dimension")
    F = gate_up.shape[-1] // 2
    rows = gate_up.numel() // (2 * F)
    if out is None:
        out = torch.empty((*gate_up.shape[:-1], F), dtype=torch.float16, device=gate_up.device)
    elif out.numel() != rows * F or out.dtype != torch.float16 or not out.is_contiguous() or out.device != gate_up.device:
        raise ValueError("out must be a contiguous float16 [..., F] tensor on the operand's device")
    lib = load_library()
    with _on_device(gate_up.device):
        rc = lib.ap_silu_mul(gate_up.data_ptr(), out.data_ptr(), rows, F, 1 if tiled else 0, _current_stream(gate_up.device))
    if rc != 0:
        _raise(lib, rc, "silu_mul")
    return out


def gemm_kbit_supported(x: torch.Tensor, qweight: torch.Tensor) -> bool:
    """Whether ``gemm_kbit`` takes these operands (N % 128 == 0, K % 128 == 0, aligned pointers)."""
    if qweight.dim() != 3 or x.dim() < 1:
        return False
    _, N, words = qweight.shape
    return N % 128 == 0 and words % 4 == 0 and x.data_ptr() % 16 == 0 and qweight.data_ptr() % 16 == 0 \
        and (qweight.stride(0) % 4 == 0 or qweight.shape[0] == 1)


def gemm_kbit(x: torch.Tensor, qweight: torch.Tensor, lut: torch.Tensor, w_bits: int, *,
              out: torch.Tensor | None = None, status: torch.Tensor | None = None, splits: int | None = None):
    """Prefill product ``x @ W_w.T`` with the weight dequantised inside the kernel and multiplied
    on the tensor cores (fp32 accumulation); fp16 ``[..., N]``.

    No counterpart in the reference, which materialises the fp16 weight with ``dequant_kbit`` and
    calls ``torch.matmul`` (any_precision/modules/AnyPrecisionLinear.py:60-62).  Raises
    ``ValueError`` for shapes the kernel does not take (see ``gemm_kbit_supported``).  ``status``
    is an optional int32 device tensor of one element that the kernel sets to 1 if an internal
    bounded wait expired.
    """
    N, K, plane_stride = _check_operands(qweight, lut, w_bits)
    if x.dtype != torch.float16 or x.device != qweight.device:
        raise TypeError("x must be float16 on the same CUDA device as qweight")
    if x.dim() < 1 or x.shape[-1] != K:
        raise ValueError(f"x has last dimension {x.shape[-1] if x.dim() else None}, expected K={K}")
    lead = x.shape[:-1]
    x2 = x.reshape(-1, K)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    M = x2.shape[0]
    if M == 0:
        return torch.empty((*lead, N), dtype=torch.float16, device=x.device)
    lib = load_library()
    if out is None:
        out = torch.empty((*lead, N), dtype=torch.float16, device=x.device)
    elif tuple(out.shape) != (*lead, N) or out.dtype != torch.float16 or not out.is_contiguous() \
            or out.device != x.device:
        raise ValueError("out must be a contiguous float16 [..., N] tensor on the operands' device")
    if status is not None and (status.dtype != torch.int32 or status.numel() != 1 or status.device != x.device):
        raise ValueError("status must be a one-element int32 tensor on the operands' device")
    with _on_device(x.device):
        stream = _current_stream(qweight.device)
        if splits is None:
            splits = lib.ap_gemm_kbit_splits(M, N, K)
        ws = None
        if splits > 1 and K % 256 == 0:
            ws = _workspace_bytes(x.device, stream, lib.ap_gemm_kbit_workspace_bytes(M, N, splits))
        st = status.data_ptr() if status is not None else None
        if ws is None:
            rc = lib.ap_gemm_kbit(x2.data_ptr(), qweight.data_ptr(), plane_stride, lut.data_ptr(), out.data_ptr(),
                                  M, N, K, w_bits, st, stream)
        else:
            rc = lib.ap_gemm_kbit_splitk(x2.data_ptr(), qweight.data_ptr(), plane_stride, lut.data_ptr(), out.data_ptr(),
                                         M, N, K, w_bits, st, splits, ws.data_ptr(), ws.numel(), stream)
    if rc != 0:
        _raise(lib, rc, "gemm_kbit")
    return out
