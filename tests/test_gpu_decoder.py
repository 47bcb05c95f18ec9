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


@pytest.mark.parametrize("fold", [True, False])
@pytest.mark.parametrize("batch", [1, 2])
def test_decoder_prefill_and_decode_against_fp32_forward(batch, fold):
    """`fold`: the decode step with every residual add + RMSNorm folded into the products around it (five
    launches per layer), or with the norms as launches of their own."""
    from anyprec_b200 import checkpoint
    from anyprec_b200.decoder import AnyPrecisionLlama
    config, sd = checkpoint.read_packed(CKPT)
    model = AnyPrecisionLlama.from_packed(CKPT, device="cuda", batch=batch, max_seq=64 if batch == 1 else 192)
    model.fold_norms = fold
    assert model._folded_norms()
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
            y = model.last_logits().cpu()
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
        model.fold_norms = False                                               # the unfolded step picks the same tokens
        model._graphs.clear()
        assert torch.equal(model.generate(ids, 24, precision=w, use_graph=True), eager)
        model.fold_norms = True
        model._graphs.clear()
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


@pytest.mark.parametrize("heads,kv_heads,D,splits", [(8, 8, 128, 1), (8, 2, 128, 4), (4, 1, 64, 3), (2, 2, 32, 2), (2, 1, 256, 5)])
def test_attention_with_rotation_inside_equals_the_two_separate_kernels(heads, kv_heads, D, splits):
    """ap_decode_attention_rope against ap_rope_cache followed by ap_decode_attention: outputs and both caches
    bit for bit, at positions that put the new token first, inside and at the end of a split, and out of range."""
    from anyprec_b200.decoder import _ops
    lib = _ops()
    B, max_seq = 3, 300
    g = torch.Generator(device="cuda").manual_seed(heads * 100 + D)
    width = (heads + 2 * kv_heads) * D
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, dtype=torch.float64) / D))
    ang = torch.arange(max_seq, dtype=torch.float64)[:, None] * inv[None, :]
    cos_sin = torch.cat([ang.cos(), ang.sin()], dim=1).float().cuda().contiguous()
    scratch_bytes = lib.ap_decode_attention_scratch_bytes(B, heads, D, splits)
    stream = torch.cuda.current_stream().cuda_stream
    for positions in ([0, 1, 2], [255, 256, 299], [17, 128, 64], [300, -1, 5]):
        pos = torch.tensor(positions, dtype=torch.int32, device="cuda")
        qkv = torch.randn((B, width), device="cuda", generator=g).half()
        k0 = torch.randn((B, kv_heads, max_seq, D), device="cuda", generator=g).half()
        v0 = torch.randn((B, kv_heads, max_seq, D), device="cuda", generator=g).half()
        results = []
        for fused in (False, True):
            q, k, v = qkv.clone(), k0.clone(), v0.clone()
            out = torch.zeros((B, heads * D), dtype=torch.float16, device="cuda")
            scratch = torch.zeros(max(scratch_bytes, 16), dtype=torch.uint8, device="cuda")
            sp = scratch.data_ptr() if splits > 1 else None
            if fused:
                rc = lib.ap_decode_attention_rope(q.data_ptr(), width, cos_sin.data_ptr(), k.data_ptr(), v.data_ptr(), pos.data_ptr(),
                                                  out.data_ptr(), B, heads, kv_heads, D, max_seq, D ** -0.5, splits, sp, stream)
                assert rc == 0 and torch.equal(q, qkv)                  # the raw row is left alone
            else:
                assert lib.ap_rope_cache(q.data_ptr(), cos_sin.data_ptr(), pos.data_ptr(), k.data_ptr(), v.data_ptr(), B, 1, heads,
                                         kv_heads, D, max_seq, stream) == 0
                assert lib.ap_decode_attention(q.data_ptr(), width, k.data_ptr(), v.data_ptr(), pos.data_ptr(), out.data_ptr(), B,
                                               heads, kv_heads, D, max_seq, D ** -0.5, splits, sp, stream) == 0
            torch.cuda.synchronize()
            assert int(scratch[: B * heads * 4].view(torch.int32).abs().sum()) == 0 or splits == 1
            results.append((out, k, v))
        (o1, k1, v1), (o2, k2, v2) = results
        valid = [b for b, p in enumerate(positions) if 0 <= p < max_seq]
        assert torch.equal(k1, k2) and torch.equal(v1, v2), positions
        assert torch.equal(o1[valid], o2[valid]), positions
        # and the caches did change exactly at the new positions
        for b, p in enumerate(positions):
            if 0 <= p < max_seq:
                assert not torch.equal(k2[b, :, p], k0[b, :, p]) and torch.equal(v2[b, :, p], qkv[b, (heads + kv_heads) * D:].view(kv_heads, D))
        for b, p in enumerate(positions):                   # the earlier positions are untouched
            q0 = min(max(p, 0), max_seq)
            assert torch.equal(k2[b, :, :q0], k0[b, :, :q0]) and torch.equal(v2[b, :, :q0], v0[b, :, :q0])
