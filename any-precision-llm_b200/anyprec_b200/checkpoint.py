"""Reading packed any-precision checkpoints as the reference project writes them.

The reference's packer stores a model as ``pytorch_model.bin`` (one ``torch.save``d state dict,
any_precision/quantization/pack.py:175) beside the model's ``config.json``, to which it adds
``anyprec = {seed_precision, parent_precision, group_count, arch_config}`` (pack.py:165-171).  In the
state dict every quantised linear ``{model_name}.{layers_name}.{L}.{module}`` has lost its
``.weight`` and carries ``.qweight`` (int32 ``[parent_precision, N, K/32]``) and ``.lut{b}`` (fp16
``[N, 2**b]``) for ``b = seed .. parent`` (pack.py:101-112); everything else (embeddings, norms,
``lm_head``) is the original tensor.

The reference loads such a directory by building an empty Hugging Face model, swapping its linears
and calling ``accelerate.load_checkpoint_and_dispatch`` (any_precision/modules/
AnyPrecisionForCausalLM.py:54-86,141-162).  Here the directory is read directly: no ``accelerate``,
no model class needed to get at the layers.
"""
from __future__ import annotations

import json
import os
import re

import torch

from .modules.AnyPrecisionLinear import AnyPrecisionLinear

__all__ = ["read_packed", "quantized_linear_names", "build_linear", "load_linears"]


def read_packed(path: str):
    """``(config, state_dict)`` of a packed checkpoint directory: ``config`` is the parsed
    ``config.json`` (a dict with an ``anyprec`` entry), ``state_dict`` maps names to CPU tensors."""
    cfg_path = os.path.join(path, "config.json")
    bin_path = os.path.join(path, "pytorch_model.bin")
    if not os.path.exists(cfg_path) or not os.path.exists(bin_path):
        raise FileNotFoundError(f"{path}: expected config.json and pytorch_model.bin (a packed any-precision checkpoint)")
    with open(cfg_path) as f:
        config = json.load(f)
    ap = config.get("anyprec")
    if not isinstance(ap, dict) or not {"seed_precision", "parent_precision", "arch_config"} <= set(ap):
        raise ValueError(f"{cfg_path}: no 'anyprec' entry with seed_precision, parent_precision and arch_config")
    if ap.get("group_count", 1) != 1:
        raise ValueError("only group_count == 1 is a supported packing (one table per output row)")
    state_dict = torch.load(bin_path, map_location="cpu", weights_only=True)
    return config, state_dict


def quantized_linear_names(config: dict, state_dict: dict):
    """Dotted names of the quantised linears, in layer order then in ``arch_config.module_names`` order."""
    arch = config["anyprec"]["arch_config"]
    prefix = f"{arch['model_name']}.{arch['layers_name']}."
    pat = re.compile(re.escape(prefix) + r"(\d+)\.(.+)\.qweight$")
    found = {}
    for key in state_dict:
        m = pat.match(key)
        if m:
            found[(int(m.group(1)), m.group(2))] = key[:-len(".qweight")]
    order = {name: i for i, name in enumerate(arch["module_names"])}
    unknown = sorted({mod for _, mod in found} - set(order))
    if unknown:
        raise ValueError(f"checkpoint holds quantised modules that arch_config does not name: {unknown}")
    return [found[k] for k in sorted(found, key=lambda k: (k[0], order[k[1]]))]


def build_linear(name: str, config: dict, state_dict: dict, precisions=None, device=None) -> AnyPrecisionLinear:
    """One ``AnyPrecisionLinear`` with the buffers of ``name`` loaded (``load_state_dict`` by buffer
    name, as the reference's loader does) and pruned to ``precisions`` (default: every supported one)."""
    ap = config["anyprec"]
    supported = list(range(int(ap["seed_precision"]), int(ap["parent_precision"]) + 1))
    precisions = supported if precisions is None else sorted(precisions)
    if len(set(precisions)) != len(precisions) or any(p not in supported for p in precisions):
        raise ValueError(f"precisions {precisions} must be distinct members of {supported}")
    q = state_dict[name + ".qweight"]
    if q.dtype != torch.int32 or q.dim() != 3 or q.shape[0] != supported[-1]:
        raise ValueError(f"{name}.qweight: expected int32 [{supported[-1]}, N, K/32], got {q.dtype} {tuple(q.shape)}")
    N, K = q.shape[1], q.shape[2] * 32
    bias = state_dict.get(name + ".bias")
    layer = AnyPrecisionLinear(K, N, supported, bias=bias is not None, precisions=list(precisions), device="cpu")
    own = {"qweight": q}
    for b in supported:
        lut = state_dict.get(f"{name}.lut{b}")
        if lut is None or tuple(lut.shape) != (N, 1 << b):
            raise ValueError(f"{name}.lut{b}: missing or not [{N}, {1 << b}]")
        own[f"lut{b}"] = lut.to(torch.float16)
    if bias is not None:
        own["bias"] = bias.to(torch.float16)
    layer.load_state_dict(own, strict=True)
    layer.prune_precisions()
    if device is not None:
        layer = layer.to(device)
        layer.qweight = layer.qweight.contiguous()
    return layer


def load_linears(path: str, precisions=None, device=None):
    """``(config, {dotted name: AnyPrecisionLinear}, rest)`` for a packed checkpoint directory; ``rest``
    is the state dict without the quantised linears' tensors (embeddings, norms, ``lm_head``)."""
    config, state_dict = read_packed(path)
    names = quantized_linear_names(config, state_dict)
    layers = {name: build_linear(name, config, state_dict, precisions, device) for name in names}
    taken = {k for name in names for k in state_dict if k.startswith(name + ".")}
    rest = {k: v for k, v in state_dict.items() if k not in taken}
    return config, layers, rest
