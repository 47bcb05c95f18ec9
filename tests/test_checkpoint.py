"""The packed-checkpoint loader against a checkpoint written by the reference's own packer
(tests/golden/tiny_llama_packed, made by tests/golden/make_tiny_checkpoint.py), on the CPU.

Also the drop-in claim from the other side: the reference's own ``AnyPrecisionLinear`` class, loaded
from its file where a checkout of the reference is at hand, constructs on top of this repository's
``any_precision_ext`` and agrees with the mirror class in constructor arguments, buffer names and
shapes, so that the same state dict loads into both."""
import importlib.util
import os
import sys

import numpy as np
import pytest
import torch

from conftest import GOLDEN_DIR
from oracle import oracle

CKPT = os.path.join(GOLDEN_DIR, "tiny_llama_packed")
MODULES = ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
           "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj"]


def test_reads_config_and_state_dict():
    from anyprec_b200 import checkpoint
    config, sd = checkpoint.read_packed(CKPT)
    ap = config["anyprec"]
    assert (ap["seed_precision"], ap["parent_precision"], ap["group_count"]) == (3, 5, 1)
    assert ap["arch_config"]["module_names"] == MODULES
    names = checkpoint.quantized_linear_names(config, sd)
    assert names == [f"model.layers.{L}.{m}" for L in range(2) for m in MODULES]
    for n in names:
        assert n + ".weight" not in sd                      # the packer drops the fp16 weight
        assert sd[n + ".qweight"].dtype == torch.int32 and sd[n + ".qweight"].shape[0] == 5
        for b in (3, 4, 5):
            assert sd[f"{n}.lut{b}"].dtype == torch.float16


def test_loaded_layers_match_what_went_into_the_packer():
    from anyprec_b200 import checkpoint
    config, layers, rest = checkpoint.load_linears(CKPT)
    assert len(layers) == 14
    assert set(rest) == {"lm_head.weight", "model.embed_tokens.weight", "model.norm.weight"} | {
        f"model.layers.{L}.{n}.weight" for L in range(2) for n in ("input_layernorm", "post_attention_layernorm")}
    with np.load(os.path.join(CKPT, "inputs.npz")) as z:
        for key in z.files:                                  # codes.{L}.{module}
            _, L, module = key.split(".", 2)
            layer = layers[f"model.layers.{L}.{module}"]
            codes = z[key]
            assert (layer.out_features, layer.in_features) == codes.shape
            assert layer.supported_bits == [3, 4, 5] and layer.precisions == [3, 4, 5] and layer.precision == 5
            q = layer.qweight.numpy()
            assert np.array_equal(q, oracle.pack(codes, parent_bits=5))
            assert np.array_equal(oracle.unpack(q, 5), codes)
            for b in (3, 4, 5):
                lut = getattr(layer, f"lut{b}").numpy()
                assert lut.shape == (codes.shape[0], 1 << b) and np.all(np.diff(lut.astype(np.float32), axis=1) >= 0)


def test_precisions_argument_prunes_planes_and_tables():
    from anyprec_b200 import checkpoint
    _, layers, _ = checkpoint.load_linears(CKPT, precisions=[4, 3])
    layer = layers["model.layers.1.mlp.down_proj"]
    assert layer.precisions == [3, 4] and layer.precision == 4
    assert layer.qweight.shape == (4, 128, 8)                # planes 0..3 of five
    assert hasattr(layer, "lut3") and hasattr(layer, "lut4") and not hasattr(layer, "lut5")
    with pytest.raises(RuntimeError):
        layer.set_precision(5)
    with pytest.raises(ValueError):
        checkpoint.load_linears(CKPT, precisions=[2])
    with pytest.raises(FileNotFoundError):
        checkpoint.read_packed(GOLDEN_DIR)


def test_reference_module_class_runs_on_this_extension():
    ref = oracle.reference_root()
    if ref is None:
        pytest.skip("no checkout of the reference project here")
    import any_precision_ext                                  # noqa: F401  (this repository's, first on sys.path)
    assert os.path.dirname(any_precision_ext.__file__).endswith("any-precision-llm_b200")
    path = os.path.join(ref, "any_precision", "modules", "AnyPrecisionLinear.py")
    spec = importlib.util.spec_from_file_location("_ref_ap_linear", path)
    mod = importlib.util.module_from_spec(spec)
    sys.dont_write_bytecode = True
    spec.loader.exec_module(mod)
    assert mod.matmul_kbit is any_precision_ext.matmul_kbit and mod.dequant_kbit is any_precision_ext.dequant_kbit
    from anyprec_b200 import AnyPrecisionLinear, checkpoint
    theirs = mod.AnyPrecisionLinear(128, 256, [3, 4, 5], bias=False, precisions=[3, 5], dtype=torch.float16)
    ours = AnyPrecisionLinear(128, 256, [3, 4, 5], bias=False, precisions=[3, 5])
    a, b = theirs.state_dict(), ours.state_dict()
    assert list(a) == list(b) == ["qweight", "lut3", "lut4", "lut5"]
    assert all(a[k].shape == b[k].shape and a[k].dtype == b[k].dtype for k in a)
    assert theirs.extra_repr() == ours.extra_repr()
    # the same checkpoint entries load into both classes
    _, sd = checkpoint.read_packed(CKPT)
    own = {k: sd[f"model.layers.0.mlp.gate_proj.{k}"] for k in a}
    theirs.load_state_dict(own)
    ours.load_state_dict(own)
    theirs.prune_precisions()
    ours.prune_precisions()
    assert list(theirs.state_dict()) == list(ours.state_dict()) == ["qweight", "lut3", "lut5"]
    assert torch.equal(theirs.qweight, ours.qweight)
