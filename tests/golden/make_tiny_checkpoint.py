"""Write the committed tiny packed checkpoint by running the reference project's own packer.

    python tests/golden/make_tiny_checkpoint.py --ref /path/to/any-precision-llm

A two-layer Llama-shaped model (hidden 128, 4 heads / 2 KV heads of 32, FFN 256, vocabulary 96),
parent precision 5, seed precision 3, is laid out on disk the way the reference quantizer leaves
a model for its packer (``weights/l{L}.pt`` with uint8 codes ``[N, 1, K]`` per module,
``lut_{b}/l{L}.pt`` with fp16 tables ``[N, 1, 2**b]``), and the reference's
``_process_layer_data`` (any_precision/quantization/pack.py:79-114), loaded from where it lies,
turns every layer into ``{model}.{layers}.{L}.{module}.qweight`` / ``.lut{b}`` entries.  The state
dict (plus fp16 embeddings, norms and ``lm_head``) is saved as ``pytorch_model.bin`` and the model
configuration with its ``anyprec`` entry as ``config.json``, which is what the reference's
``pack`` writes (pack.py:165-177).  ``inputs.npz`` keeps the codes of two of the layers that went in, for spot checks.

Inputs are seeded synthetic data (uniform codes, sorted N(0, 0.05) tables); nothing is taken from
any pretrained model.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import sys
import tempfile

os.environ.setdefault("NUMBA_CACHE_DIR", tempfile.mkdtemp(prefix="numba_cache_"))
os.environ["PYTHONDONTWRITEBYTECODE"] = "1"
sys.dont_write_bytecode = True

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "tiny_llama_packed")

HIDDEN, HEADS, KV_HEADS, HEAD_DIM, FFN, LAYERS, VOCAB = 128, 4, 2, 32, 256, 2, 96
PARENT, SEEDP = 5, 3
MODULES = ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
           "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj"]
SHAPES = {"self_attn.q_proj": (HEADS * HEAD_DIM, HIDDEN), "self_attn.k_proj": (KV_HEADS * HEAD_DIM, HIDDEN),
          "self_attn.v_proj": (KV_HEADS * HEAD_DIM, HIDDEN), "self_attn.o_proj": (HIDDEN, HEADS * HEAD_DIM),
          "mlp.gate_proj": (FFN, HIDDEN), "mlp.up_proj": (FFN, HIDDEN), "mlp.down_proj": (HIDDEN, FFN)}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="root of a checkout of the reference project")
    args = ap.parse_args()
    path = os.path.join(args.ref, "any_precision", "quantization", "pack.py")
    spec = importlib.util.spec_from_file_location("_ref_pack", path)
    refpack = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(refpack)

    rng = np.random.default_rng(5150)
    state, inputs = {}, {}
    with tempfile.TemporaryDirectory() as d:
        os.makedirs(os.path.join(d, "weights"))
        for b in range(SEEDP, PARENT + 1):
            os.makedirs(os.path.join(d, f"lut_{b}"))
        for L in range(LAYERS):
            weights, luts = {}, {b: {} for b in range(SEEDP, PARENT + 1)}
            for name in MODULES:
                N, K = SHAPES[name]
                codes = rng.integers(0, 1 << PARENT, size=(N, K), dtype=np.uint8)
                weights[name] = codes.reshape(N, 1, K)
                if L == 0 and name in ("self_attn.q_proj", "mlp.down_proj"):
                    inputs[f"codes.{L}.{name}"] = codes                      # spot checks of the packer's output
                for b in range(SEEDP, PARENT + 1):
                    cent = np.sort(rng.normal(0.0, 0.05, size=(N, 1 << b)).astype(np.float32), axis=1).astype(np.float16)
                    luts[b][name] = cent.reshape(N, 1, 1 << b)
            torch.save(weights, os.path.join(d, "weights", f"l{L}.pt"))
            for b in luts:
                torch.save(luts[b], os.path.join(d, f"lut_{b}", f"l{L}.pt"))
        for L in range(LAYERS):
            idx, data = refpack._process_layer_data((L, d, "model", "layers", MODULES, PARENT, SEEDP))
            assert idx == L
            for key, value in data.items():
                state[key] = torch.from_numpy(np.asarray(value))          # as pack.py:160
    g = torch.Generator().manual_seed(99)
    state["model.embed_tokens.weight"] = (torch.randn((VOCAB, HIDDEN), generator=g) * 0.5).half()
    state["lm_head.weight"] = (torch.randn((VOCAB, HIDDEN), generator=g) * 0.1).half()
    state["model.norm.weight"] = (1.0 + 0.1 * torch.randn(HIDDEN, generator=g)).half()
    for L in range(LAYERS):
        state[f"model.layers.{L}.input_layernorm.weight"] = (1.0 + 0.1 * torch.randn(HIDDEN, generator=g)).half()
        state[f"model.layers.{L}.post_attention_layernorm.weight"] = (1.0 + 0.1 * torch.randn(HIDDEN, generator=g)).half()
    config = {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": HIDDEN,
        "intermediate_size": FFN, "num_attention_heads": HEADS, "num_key_value_heads": KV_HEADS,
        "num_hidden_layers": LAYERS, "vocab_size": VOCAB, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
        "max_position_embeddings": 256, "hidden_act": "silu", "tie_word_embeddings": False, "torch_dtype": "float16",
        "anyprec": {"seed_precision": SEEDP, "parent_precision": PARENT, "group_count": 1,
                    "arch_config": {"model_name": "model", "layers_name": "layers", "module_names": MODULES}},
    }
    os.makedirs(OUT, exist_ok=True)
    torch.save(state, os.path.join(OUT, "pytorch_model.bin"))
    with open(os.path.join(OUT, "config.json"), "w") as f:
        json.dump(config, f, indent=1)
    np.savez_compressed(os.path.join(OUT, "inputs.npz"), **inputs)
    for fn in sorted(os.listdir(OUT)):
        print(fn, os.path.getsize(os.path.join(OUT, fn)))


if __name__ == "__main__":
    main()
