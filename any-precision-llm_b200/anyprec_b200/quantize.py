"""Seed + incremental-upscale quantisation on the GPU.

The reference quantises a model layer by layer on the CPU: ``seed_and_upscale`` (any_precision/
quantization/quantize.py:250-324) loads a layer's weights and sensitivities, runs the numba routine
``_seed_and_upscale_layer`` (:85-187) over the rows and saves, per layer, ``weights/l{L}.pt`` (a dict
module name -> uint8 codes ``[N, group_count, K / group_count]``) and ``lut_{b}/l{L}.pt`` (a dict module name ->
fp16 tables ``[N, group_count, 2**b]``) for ``b = seed .. parent`` (:200-218), which its packer then reads
(pack.py:79-114).  Here the row routine is one CUDA kernel (``ap_seed_upscale``, one thread block per
row); the file layout is kept, so the reference's packer, or ``packing.pack_codes``, takes the result.

``group_count`` other than 1 is not supported (the reference's packer refuses it too, pack.py:126-127).
The seed k-means starts deterministically (the reference's starts from a random draw), so two runs give
the same model.
"""
from __future__ import annotations

import ctypes
import os

import torch

import any_precision_ext as _ext

from . import packing
from .modules.AnyPrecisionLinear import AnyPrecisionLinear

__all__ = ["seed_and_upscale_layer", "quantize_linear", "save_layer", "MAX_ITER"]

MAX_ITER = 50            # Lloyd assignments of the seed k-means (quantize.py:148)


def _lib():
    lib = _ext.load_library()
    if not getattr(lib, "_quantize_ready", False):
        vp, i = ctypes.c_void_p, ctypes.c_int
        lib.ap_seed_upscale_workspace_bytes.restype = ctypes.c_size_t
        lib.ap_seed_upscale_workspace_bytes.argtypes = [i, i]
        lib.ap_seed_upscale.restype = i
        lib.ap_seed_upscale.argtypes = [vp, vp, i, i, i, i, i, vp, vp, vp, ctypes.c_size_t, vp]
        lib._quantize_ready = True
    return lib


def seed_and_upscale_layer(weight: torch.Tensor, sensitivity: torch.Tensor, seed_precision: int = 3,
                           parent_precision: int = 8, max_iter: int = MAX_ITER, blocks: int | None = None):
    """``(luts, codes)`` for one linear layer: ``luts[b]`` is the fp16 table ``[N, 2**b]`` for
    ``b = seed_precision .. parent_precision`` and ``codes`` the uint8 parent codes ``[N, K]`` whose top ``b``
    bits index ``luts[b]``.  ``weight`` and ``sensitivity`` are CUDA tensors ``[N, K]`` (any float dtype; they
    are read as fp32, as the reference converts them, quantize.py:192-194); ``K`` up to 32768."""
    if weight.dim() != 2 or weight.shape != sensitivity.shape:
        raise ValueError("weight and sensitivity must be [N, K] tensors of the same shape")
    if not weight.is_cuda or sensitivity.device != weight.device:
        raise ValueError("weight and sensitivity must live on the same CUDA device (there is no CPU path)")
    if not 1 <= seed_precision <= parent_precision <= 8:
        raise ValueError("need 1 <= seed_precision <= parent_precision <= 8")
    N, K = weight.shape
    if K > 32768:
        raise ValueError("rows longer than 32768 weights are not supported")
    dev = weight.device
    w = weight.to(torch.float32).contiguous()
    s = sensitivity.to(torch.float32).contiguous()
    lib = _lib()
    if blocks is None:
        blocks = min(N, 4 * torch.cuda.get_device_properties(dev).multi_processor_count)
    entries = sum(1 << b for b in range(seed_precision, parent_precision + 1))
    codes = torch.empty((N, K), dtype=torch.uint8, device=dev)
    luts = torch.empty(N * entries, dtype=torch.float16, device=dev)
    work = torch.empty(lib.ap_seed_upscale_workspace_bytes(K, blocks), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        rc = lib.ap_seed_upscale(w.data_ptr(), s.data_ptr(), N, K, seed_precision, parent_precision, max_iter,
                                 codes.data_ptr(), luts.data_ptr(), work.data_ptr(), work.numel(),
                                 torch.cuda.current_stream(dev).cuda_stream)
    if rc != 0:
        raise RuntimeError(f"ap_seed_upscale: {lib.ap_strerror(rc).decode()}")
    out, off = {}, 0
    for b in range(seed_precision, parent_precision + 1):
        out[b] = luts[off:off + N * (1 << b)].view(N, 1 << b)
        off += N * (1 << b)
    return out, codes


def quantize_linear(weight: torch.Tensor, sensitivity: torch.Tensor, seed_precision: int = 3, parent_precision: int = 8,
                    bias: torch.Tensor | None = None, precisions=None) -> AnyPrecisionLinear:
    """Quantise one layer and pack it: an ``AnyPrecisionLinear`` ready to run (``K % 32 == 0``)."""
    luts, codes = seed_and_upscale_layer(weight, sensitivity, seed_precision, parent_precision)
    N, K = codes.shape
    supported = list(range(seed_precision, parent_precision + 1))
    layer = AnyPrecisionLinear(K, N, supported, bias=bias is not None, precisions=precisions, device="meta")
    layer.qweight = packing.pack_codes(codes, parent_precision)
    for b in supported:
        setattr(layer, f"lut{b}", luts[b].contiguous())
    if bias is not None:
        layer.bias = bias.to(weight.device, torch.float16)
    layer.prune_precisions()
    return layer


def save_layer(output_folder: str, layer_index: int, module_names, luts_by_module, codes_by_module,
               seed_precision: int, parent_precision: int):
    """Write one layer's results where and how the reference's quantiser does (quantize.py:200-218): numpy
    arrays in dicts keyed by module name, tables as fp16 ``[N, 1, 2**b]``, codes as uint8 ``[N, 1, K]``."""
    for b in range(seed_precision, parent_precision + 1):
        path = os.path.join(output_folder, f"lut_{b}", f"l{layer_index}.pt")
        os.makedirs(os.path.dirname(path), exist_ok=True)
        torch.save({name: luts[b].detach().cpu().numpy()[:, None, :] for name, luts in zip(module_names, luts_by_module)}, path)
    path = os.path.join(output_folder, "weights", f"l{layer_index}.pt")
    os.makedirs(os.path.dirname(path), exist_ok=True)
    torch.save({name: codes.detach().cpu().numpy()[:, None, :] for name, codes in zip(module_names, codes_by_module)}, path)
