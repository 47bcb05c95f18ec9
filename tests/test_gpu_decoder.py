"""The packed-checkpoint loader and the minimal decoder on a GPU, against the CPU oracle and an fp32
restatement of a Llama forward pass over the oracle's dequantised weights.

The checkpoint (tests/golden/tiny_llama_packed) was written by the reference's own packer; nothing here
reads the reference tree."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN_DIR
from oracle import oracle

pytestmark = pytest.mark.gpu

CKPT = os.path.join(GOLDEN_DIR, "tiny_llama_packed")
MAX_REL = 1e-2
REL_FLOOR = 0.05
MEAN_ABS = 1e-3


def close(y, ref, max_rel=MAX_REL, mean_abs=MEAN_ABS):
    y, ref = np.asarray(y, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    err = np.abs(y - ref)
    denom = np.maximum(np.abs(ref), REL_FLOOR * np.abs(ref).max())
    assert (err / denom).max() <= max_rel, f"max rel err {(err / denom).max():.3e}"
    assert err.mean() <= mean_abs * max(1.0, np.abs(ref).max()), f"mean abs err {err.mean():.3e}"


def test_loaded_layers_forward_at_every_precision():
    from anyprec_b200 import checkpoint
    config, layers, _ = checkpoint.load_linears(CKPT, device="cuda")
    _, sd = checkpoint.read_packed(CKPT)
    rng = np.random.default_rng(0)
    for name, layer in layers.items():
        qn = sd[name + ".qweight"].numpy()
        for rows in (1, 3, 24):
            xn = rng.normal(size=(rows, layer.in_features)).astype(np.float16)
            x = torch.from_numpy(xn).cuda()
            for w in (3, 4, 5):
                lut = sd[f"{name}.lut{w}"].numpy()
                y = layer(x, precision=w).cpu().numpy()
                close(y, oracle.c_matmul(xn, qn, lut, w))


def reference_forward(sd, config, ids, w):
    """Plain fp32 Llama forward over the oracle's dequantised weights: logits [T, vocab] for one sequence."""
    H, KV = config["num_attention_heads"], config["num_key_value_heads"]
    hidden = config["hidden_size"]
    D = hidden // H
    eps, theta = config["rms_norm_eps"], config["rope_theta"]

    def W(name):
        return torch.from_numpy(oracle.c_dequant(sd[name + ".qweight"].numpy(), sd[f"{name}.lut{w}"].numpy(), w).astype(np.float32))

    def norm(x, g):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * g.float()

    T = len(ids)
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.float64) / D))
    ang = torch.arange(T, dtype=torch.float64)[:, None] * inv[None, :]
    cos, sin = ang.cos().float(), ang.sin().float()

    def rope(x):                                             # [T, heads, D]
        a, b = x[..., :D // 2], x[..., D // 2:]
        return torch.cat([a * cos[:, None] - b * sin[:, None], b * cos[:, None] + a * sin[:, None]], dim=-1)

    h = sd["model.embed_tokens.weight"].float()[ids]
    for L in range(config["num_hidden_layers"]):
        p = f"model.layers.{L}."
        y = norm(h, sd[p + "input_layernorm.weight"])
        q = rope((y @ W(p + "self_attn.q_proj").T).view(T, H, D))
        k = rope((y @ W(p + "self_attn.k_proj").T).view(T, KV, D))
        v = (y @ W(p + "self_attn.v_proj").T).view(T, KV, D)
        k, v = k.repeat_interleave(H // KV, dim=1), v.repeat_interleave(H // KV, dim=1)
        att = torch.einsum("thd,shd->hts", q, k) / D ** 0.5
        att = att.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf")).softmax(-1)
        o = torch.einsum("hts,shd->thd", att, v).reshape(T, H * D)
        h = h + o @ W(p + "self_attn.o_proj").T
        y = norm(h, sd[p + "post_attention_layernorm.weight"])
        g, u = y @ W(p + "mlp.gate_proj").T, y @ W(p + "mlp.up_proj").T
        h = h + (torch.nn.functional.silu(g) * u) @ W(p + "mlp.down_proj").T
    return norm(h, sd["model.norm.weight"]) @ sd["lm_head.weight"].float().T


@pytest.mark.parametrize("batch", [1, 2])
def test_decoder_prefill_and_decode_against_fp32_forward(batch):
    from anyprec_b200 import checkpoint
    from anyprec_b200.decoder import AnyPrecisionLlama
    config, sd = checkpoint.read_packed(CKPT)
    model = AnyPrecisionLlama.from_packed(CKPT, device="cuda", batch=batch, max_seq=64 if batch == 1 else 192)
    assert model.precisions == [3, 4, 5] and model.spec.kv_heads == 2
    gen = torch.Generator().manual_seed(batch)
    ids = torch.randint(0, config["vocab_size"], (batch, 20), generator=gen)
    for w in (3, 5):
        model.set_precision(w)
        logits = model.prefill(ids).float().cpu()
        for b in range(batch):
            ref = reference_forward(sd, config, ids[b].tolist(), w)
            close(logits[b].numpy(), ref[-1].numpy(), max_rel=3e-2, mean_abs=5e-3)
        # three decode steps (eager), each compared with a full fp32 forward of the grown sequence
        seqs = [ids[b].tolist() for b in range(batch)]
        model.tok.copy_(logits.argmax(-1).cuda())
        for _ in range(3):
            toks = model.tok.cpu().tolist()
            for b in range(batch):
                seqs[b].append(toks[b])
            model._decode_step()
            y = (model.y.float() @ model.lm_head.float().T).cpu()
            for b in range(batch):
                ref = reference_forward(sd, config, seqs[b], w)
                close(y[b].numpy(), ref[-1].numpy(), max_rel=3e-2, mean_abs=5e-3)
    assert model.precision == 5


def test_generate_graph_replay_equals_eager_and_restores_precision():
    from anyprec_b200.decoder import AnyPrecisionLlama
    model = AnyPrecisionLlama.from_packed(CKPT, device="cuda", batch=1, max_seq=256)
    assert model.attn_splits == 4                        # the cached positions of a head are cut over four blocks
    ids = torch.randint(0, model.spec.vocab, (1, 12), generator=torch.Generator().manual_seed(3))
    model.set_precision(4)
    for w in (3, 5):
        eager = model.generate(ids, 24, precision=w, use_graph=False)
        graph = model.generate(ids, 24, precision=w, use_graph=True)
        again = model.generate(ids, 24, precision=w, use_graph=True)          # second call replays the cached graph
        assert eager.shape == (1, 36) and torch.equal(eager[:, :12].cpu(), ids)
        assert torch.equal(eager, graph) and torch.equal(graph, again)
        assert model.precision == 4
    with pytest.raises(RuntimeError):
        model.generate(ids, 4, precision=7)
    with pytest.raises(ValueError):
        model.generate(ids, 300)


def test_random_init_llama_shapes_run():
    """The benchmark's construction path on a cut-down model: random planes and tables, fused q+k+v and
    gate+up, every precision 3..8, batch 2."""
    from anyprec_b200.decoder import AnyPrecisionLlama, LlamaSpec
    spec = LlamaSpec(hidden=512, heads=4, kv_heads=4, ffn=1408, layers=2, vocab=1000)
    model = AnyPrecisionLlama.random_init(spec, "cuda", seed=1, batch=2, max_seq=80)
    ids = torch.randint(0, spec.vocab, (2, 40), generator=torch.Generator().manual_seed(1))
    for w in (3, 6, 8):
        out = model.generate(ids, 16, precision=w)
        assert out.shape == (2, 56) and int(out.max()) < spec.vocab
    import any_precision_ext as ext
    assert not ext.take_wait_expired()
