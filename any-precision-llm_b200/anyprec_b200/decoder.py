"""A minimal Llama-style decoder over ``AnyPrecisionLinear`` layers, for decode-rate measurements
and for running packed checkpoints without Hugging Face ``transformers`` or ``accelerate``.

The reference wraps the stock Hugging Face model and swaps its linears
(any_precision/modules/AnyPrecisionForCausalLM.py:29-86); precision is selected per call with
``forward(..., precision=)`` / ``generate(..., precision=)`` (:88-111) or ``set_precision`` (:171-174),
and its ``fuse_layers`` is a stub (:186-190).  This class keeps that calling convention
(``set_precision``, ``generate(input_ids, max_new_tokens, precision=)``) and does the fusion the
reference leaves open:

* q, k and v are one ``AnyPrecisionLinear`` (rows stacked, ``AnyPrecisionLinear.fuse``), gate and up
  another (rows stacked tile by tile, ``AnyPrecisionLinear.fuse_gated``), so a decoder layer issues four
  any-precision launches;
* residual add + RMSNorm and rotary embedding + KV-cache write are one small kernel each
  (``ap_add_rmsnorm``, ``ap_rope_cache``); SiLU * up is the epilogue of the gate+up launch in a decode
  step (``ap_matmul_kbit_gated``) and one small kernel (``ap_silu_mul``) after the prompt's GEMM;
* a decode step reads its position from device memory, so one CUDA graph per precision is captured
  once and replayed for every generated token.

Attention over the static KV cache is ``ap_decode_attention_rope`` for a decode step (one query per sequence,
grouped-query heads, fp32 softmax; it rotates q and k and stores the new k and v itself) and ``torch.nn.functional.scaled_dot_product_attention`` for the
prompt; ``lm_head`` and the embeddings stay fp16, as in the reference (only the modules its
architecture files name are quantised, any_precision/analyzer/architectures/llama.yaml:5-12).
Greedy sampling only; batch size fixed at construction.
"""
from __future__ import annotations

import ctypes
import dataclasses
import math

import torch
import torch.nn.functional as F

import any_precision_ext as _ext

from .modules.AnyPrecisionLinear import AnyPrecisionLinear

__all__ = ["LlamaSpec", "AnyPrecisionLlama"]


@dataclasses.dataclass
class LlamaSpec:
    hidden: int
    heads: int
    kv_heads: int
    ffn: int
    layers: int
    vocab: int
    head_dim: int = 0
    rms_eps: float = 1e-5
    rope_theta: float = 10000.0

    def __post_init__(self):
        if not self.head_dim:
            self.head_dim = self.hidden // self.heads

    @classmethod
    def llama2_7b(cls):
        return cls(hidden=4096, heads=32, kv_heads=32, ffn=11008, layers=32, vocab=32000)

    @classmethod
    def llama2_70b(cls):
        return cls(hidden=8192, heads=64, kv_heads=8, ffn=28672, layers=80, vocab=32000)

    @classmethod
    def from_hf_config(cls, cfg: dict):
        return cls(hidden=cfg["hidden_size"], heads=cfg["num_attention_heads"],
                   kv_heads=cfg.get("num_key_value_heads", cfg["num_attention_heads"]), ffn=cfg["intermediate_size"],
                   layers=cfg["num_hidden_layers"], vocab=cfg["vocab_size"], head_dim=cfg.get("head_dim", 0) or 0,
                   rms_eps=cfg.get("rms_norm_eps", 1e-5), rope_theta=cfg.get("rope_theta", 10000.0))


def _ops():
    lib = _ext.load_library()
    if getattr(lib, "_decoder_ready", False):
        return lib
    vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.ap_add_rmsnorm.restype = i
    lib.ap_add_rmsnorm.argtypes = [vp, vp, vp, vp, i, i, f, vp]
    lib.ap_rope_cache.restype = i
    lib.ap_rope_cache.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, i, i, vp]
    lib.ap_decode_attention.restype = i
    lib.ap_decode_attention.argtypes = [vp, i, vp, vp, vp, vp, i, i, i, i, i, f, i, vp, vp]
    lib.ap_decode_attention_rope.restype = i
    lib.ap_decode_attention_rope.argtypes = [vp, i, vp, vp, vp, vp, vp, i, i, i, i, i, f, i, vp, vp]
    lib.ap_decode_attention_scratch_bytes.restype = ctypes.c_size_t
    lib.ap_decode_attention_scratch_bytes.argtypes = [i, i, i, i]
    lib._decoder_ready = True
    return lib


def _check(lib, rc, what):
    if rc != 0:
        raise RuntimeError(f"{what}: {lib.ap_strerror(rc).decode()}")


def _shard_module(m: AnyPrecisionLinear, style: str, rank: int, world: int) -> AnyPrecisionLinear:
    """This rank's shard of a layer as a module of its own: rows ``[n0, n1)`` for a column-parallel layer,
    input columns ``[k0, k1)`` (re-packed when the shard's last group is partial) with the full tables for
    a row-parallel one (``tensor_parallel.shard_linear``)."""
    from .tensor_parallel import shard_linear
    luts = {b: getattr(m, f"lut{b}") for b in m.supported_bits if hasattr(m, f"lut{b}")}
    sh = shard_linear(m.qweight, luts, style, rank, world)
    out = AnyPrecisionLinear(sh.in_features, sh.out_features, list(m.supported_bits), bias=False,
                             precisions=list(m.precisions), device="meta")
    out.qweight = sh.qweight.contiguous()
    for b in m.supported_bits:
        if b in sh.luts:
            setattr(out, f"lut{b}", sh.luts[b].contiguous())
        elif hasattr(out, f"lut{b}"):
            delattr(out, f"lut{b}")
    if m.bias is not None:
        raise ValueError("sharding layers with a bias is not supported")
    out.precision = m.precision
    return out


class _Layer:
    __slots__ = ("qkv", "o", "gate_up", "down", "in_norm", "post_norm", "k_cache", "v_cache")


class AnyPrecisionLlama:
    """``spec``: model dimensions.  ``layers``: an iterable giving, per decoder layer, a dict with the seven
    ``AnyPrecisionLinear`` modules (keys ``q_proj, k_proj, v_proj, o_proj, gate_proj, up_proj, down_proj``;
    ``qkv_proj`` / ``gate_up_proj`` may stand for the already stacked ones) and the two norm weights
    (``input_layernorm``, ``post_attention_layernorm``).

    Tensor parallelism (``tp_world`` > 1, one process per GPU, no counterpart in the reference): the layers
    handed in are this rank's shards: q/k/v/gate/up hold ``heads / tp_world`` (``kv_heads / tp_world``)
    heads and ``ffn / tp_world`` rows, o/down the matching input columns, tables of o/down and everything
    unquantised replicated.  The outputs of o and down are summed over the ranks: by ``allreduce`` (a
    ``comm.OneShotAllReduce``) in decode steps, by the process group for the prompt."""

    def __init__(self, spec: LlamaSpec, layers, embed: torch.Tensor, final_norm: torch.Tensor, lm_head: torch.Tensor,
                 device, batch: int = 1, max_seq: int = 1024, tp_world: int = 1, allreduce=None, group=None):
        self.spec, self.batch, self.max_seq = spec, batch, max_seq
        self.device = torch.device(device)
        self.lib = _ops()
        dev, s = self.device, spec
        if tp_world < 1 or s.heads % tp_world or s.kv_heads % tp_world or s.ffn % tp_world:
            raise ValueError("tp_world must divide heads, kv_heads and ffn")
        self.tp_world, self.allreduce, self.group = tp_world, allreduce, group
        self.heads, self.kv_heads = s.heads // tp_world, s.kv_heads // tp_world        # this rank's
        self.ffn = s.ffn // tp_world
        self.embed = embed.to(dev, torch.float16).contiguous()
        self.final_norm = final_norm.to(dev, torch.float16).contiguous()
        self.lm_head = lm_head.to(dev, torch.float16).contiguous()
        self.layers = []
        for src in layers:
            L = _Layer()
            L.qkv = src["qkv_proj"].to(dev) if "qkv_proj" in src else \
                AnyPrecisionLinear.fuse([src["q_proj"].to(dev), src["k_proj"].to(dev), src["v_proj"].to(dev)])
            L.o = src["o_proj"].to(dev)
            L.gate_up = src["gate_up_proj"].to(dev) if "gate_up_proj" in src else \
                AnyPrecisionLinear.fuse_gated(src["gate_proj"].to(dev), src["up_proj"].to(dev))
            if not getattr(L.gate_up, "gated", False):
                raise ValueError("gate_up_proj must come from AnyPrecisionLinear.fuse_gated (rows stacked tile by tile)")
            L.down = src["down_proj"].to(dev)
            if L.qkv.out_features != (self.heads + 2 * self.kv_heads) * s.head_dim or L.down.in_features != self.ffn:
                raise ValueError("layer shapes do not match the model dimensions (and tp_world)")
            L.in_norm = src["input_layernorm"].to(dev, torch.float16).contiguous()
            L.post_norm = src["post_attention_layernorm"].to(dev, torch.float16).contiguous()
            self.layers.append(L)
            src.clear()                                      # the separate q/k/v, gate/up operands are not kept
        self.precisions = list(self.layers[0].o.precisions)
        self.precision = max(self.precisions)
        # rotary tables: [max_seq][cos(head_dim / 2) | sin(head_dim / 2)] in fp32
        inv = 1.0 / (s.rope_theta ** (torch.arange(0, s.head_dim, 2, dtype=torch.float64) / s.head_dim))
        ang = torch.arange(max_seq, dtype=torch.float64)[:, None] * inv[None, :]
        self.cos_sin = torch.cat([ang.cos(), ang.sin()], dim=1).to(torch.float32).to(dev).contiguous()
        self._allocate_state()

    def _allocate_state(self):
        """KV caches and the decode step's buffers, all on the device so that a captured step can be replayed."""
        dev, s, batch, max_seq = self.device, self.spec, self.batch, self.max_seq
        for L in self.layers:
            L.k_cache = torch.zeros((batch, self.kv_heads, max_seq, s.head_dim), dtype=torch.float16, device=dev)
            L.v_cache = torch.zeros_like(L.k_cache)
        self.pos = torch.zeros(batch, dtype=torch.int32, device=dev)          # position of the token being processed
        self.tok = torch.zeros(batch, dtype=torch.int64, device=dev)
        self.h = torch.empty((batch, s.hidden), dtype=torch.float16, device=dev)
        self.y = torch.empty_like(self.h)
        self.act = torch.empty((batch, self.ffn), dtype=torch.float16, device=dev)
        self.ssq = torch.zeros((batch, s.hidden // 16), dtype=torch.float32, device=dev)     # per-tile sums of squares of h
        self.attn = torch.empty((batch, self.heads * s.head_dim), dtype=torch.float16, device=dev)
        # a decode step has few heads: cut each head's cached positions over enough blocks for about two per SM
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        self.attn_splits = max(1, min(16, (2 * sms) // (batch * self.heads), max_seq // 64))
        self.attn_scratch = None
        if self.attn_splits > 1:
            nbytes = self.lib.ap_decode_attention_scratch_bytes(batch, self.heads, s.head_dim, self.attn_splits)
            self.attn_scratch = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
        self._graphs = {}
        self.fold_norms = True                              # False: every norm a launch of its own (the prompt's path)
        self._side = None                                   # the stream decode graphs are captured and replayed on

    # ------------------------------------------------------------------------------------ construction
    @classmethod
    def random_init(cls, spec: LlamaSpec, device, supported_bits=(3, 4, 5, 6, 7, 8), seed: int = 0, batch: int = 1,
                    max_seq: int = 1024, tp_rank: int = 0, tp_world: int = 1, allreduce=None, group=None):
        """Random weights of the right architecture: uniform parent codes (drawn directly as random
        bitplanes; q+k+v and gate+up as the stacked operands they end up as), per-row sorted N(0, 0.02)
        tables, N(0, 0.02) fp16 embeddings and ``lm_head``, unit norms.  With ``tp_world`` > 1 every rank
        draws its own shard; what is replicated (tables of o/down, embeddings, ``lm_head``) comes from a
        generator seeded alike on all ranks."""
        from . import packing
        dev = torch.device(device)
        gen = torch.Generator(device=dev).manual_seed(seed * 1000 + 17 * tp_rank + 1)      # this rank's shards
        common = torch.Generator(device=dev).manual_seed(seed * 1000)                      # replicated tensors
        bits = list(supported_bits)
        heads, kv, ffn, D = spec.heads // tp_world, spec.kv_heads // tp_world, spec.ffn // tp_world, spec.head_dim
        shapes = {"qkv_proj": ((heads + 2 * kv) * D, spec.hidden, gen), "o_proj": (spec.hidden, heads * D, common),
                  "gate_up_proj": (2 * ffn, spec.hidden, gen), "down_proj": (spec.hidden, ffn, common)}

        def layer_dicts():
            for _ in range(spec.layers):
                d = {}
                for name, (N, K, lut_gen) in shapes.items():
                    m = AnyPrecisionLinear(K, N, bits, bias=False, device="meta")
                    m.qweight = packing.random_qweight(max(bits), N, K, device=dev, generator=gen)
                    for b in bits:
                        setattr(m, f"lut{b}", packing.random_lut(N, b, device=dev, generator=lut_gen))
                    d[name] = m
                d["qkv_proj"].split_sizes = [heads * D, kv * D, kv * D]
                d["gate_up_proj"].gated = True              # random rows: any stacking order is as good as another
                d["input_layernorm"] = torch.ones(spec.hidden, dtype=torch.float16, device=dev)
                d["post_attention_layernorm"] = torch.ones(spec.hidden, dtype=torch.float16, device=dev)
                yield d

        embed = (torch.randn((spec.vocab, spec.hidden), device=dev, generator=common) * 0.02).half()
        head = (torch.randn((spec.vocab, spec.hidden), device=dev, generator=common) * 0.02).half()
        return cls(spec, layer_dicts(), embed, torch.ones(spec.hidden, dtype=torch.float16, device=dev), head, dev, batch,
                   max_seq, tp_world=tp_world, allreduce=allreduce, group=group)

    @classmethod
    def from_packed(cls, path: str, device, precisions=None, batch: int = 1, max_seq: int = 1024, tp_rank: int = 0,
                    tp_world: int = 1, allreduce=None, group=None):
        """Build the model from a packed checkpoint directory written by the reference's packer (Llama
        architecture: ``arch_config`` must name the seven Llama projections).  With ``tp_world`` > 1 every
        rank reads the whole checkpoint and keeps its shard of every layer."""
        from . import checkpoint
        config, linears, rest = checkpoint.load_linears(path, precisions=precisions, device=None)
        arch = config["anyprec"]["arch_config"]
        spec = LlamaSpec.from_hf_config(config)
        prefix = f"{arch['model_name']}.{arch['layers_name']}"
        styles = {"q_proj": "col", "k_proj": "col", "v_proj": "col", "gate_proj": "col", "up_proj": "col",
                  "o_proj": "row", "down_proj": "row"}

        def layer_dicts():
            for L in range(spec.layers):
                d = {}
                for full in arch["module_names"]:
                    d[full.split(".")[-1]] = linears.pop(f"{prefix}.{L}.{full}")
                missing = set(styles) - set(d)
                if missing:
                    raise ValueError(f"layer {L}: the checkpoint does not hold {sorted(missing)} (not a Llama-style model?)")
                if tp_world > 1:
                    d = {name: _shard_module(m.to(device), styles[name], tp_rank, tp_world) for name, m in d.items()}
                d["input_layernorm"] = rest[f"{prefix}.{L}.input_layernorm.weight"]
                d["post_attention_layernorm"] = rest[f"{prefix}.{L}.post_attention_layernorm.weight"]
                yield d

        embed = rest[f"{arch['model_name']}.embed_tokens.weight"]
        head = rest.get("lm_head.weight", embed)
        return cls(spec, layer_dicts(), embed, rest[f"{arch['model_name']}.norm.weight"], head, device, batch, max_seq,
                   tp_world=tp_world, allreduce=allreduce, group=group)

    def with_batch(self, batch: int, max_seq: int | None = None):
        """A second model over the SAME weights (modules and tables are shared, nothing is copied) with KV
        caches, buffers and decode graphs of its own for another batch size."""
        other = object.__new__(type(self))
        other.__dict__.update(self.__dict__)
        other.batch, other.max_seq = batch, max_seq or self.max_seq
        other.layers = []
        for L in self.layers:
            M = _Layer()
            for name in ("qkv", "o", "gate_up", "down", "in_norm", "post_norm"):
                setattr(M, name, getattr(L, name))
            other.layers.append(M)
        if other.max_seq != self.max_seq:
            s = self.spec
            inv = 1.0 / (s.rope_theta ** (torch.arange(0, s.head_dim, 2, dtype=torch.float64) / s.head_dim))
            ang = torch.arange(other.max_seq, dtype=torch.float64)[:, None] * inv[None, :]
            other.cos_sin = torch.cat([ang.cos(), ang.sin()], dim=1).to(torch.float32).to(self.device).contiguous()
        other._allocate_state()
        return other

    # ------------------------------------------------------------------------------------ precision
    def set_precision(self, precision: int):
        if precision not in self.precisions:
            raise RuntimeError(f"{self.precisions}-bit precisions are supported but {precision}-bit was specified.")
        for L in self.layers:
            for m in (L.qkv, L.o, L.gate_up, L.down):
                m.set_precision(precision)
        self.precision = precision

    # ------------------------------------------------------------------------------------ building blocks
    def _stream(self):
        return torch.cuda.current_stream(self.device).cuda_stream

    def _add_rmsnorm(self, h, delta, weight, y):
        rows = h.shape[0]
        _check(self.lib, self.lib.ap_add_rmsnorm(h.data_ptr(), delta.data_ptr() if delta is not None else None,
                                                 weight.data_ptr(), y.data_ptr(), rows, self.spec.hidden,
                                                 self.spec.rms_eps, self._stream()), "ap_add_rmsnorm")

    def _reduce(self, t, decode: bool):
        """Sum a row-parallel output over the ranks, in place."""
        if self.tp_world > 1:
            if decode and self.allreduce is not None:
                self.allreduce(t)
            else:
                import torch.distributed as dist
                dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
        return t

    def _layer_tail(self, L, h, y, attn, decode: bool):
        """o_proj, residual + norm, gate/up, SiLU * up, down; returns the MLP output (the caller adds it)."""
        o = self._reduce(L.o(attn), decode)
        self._add_rmsnorm(h, o, L.post_norm, y)
        rows = y.shape[0]
        act = self.act[:rows] if rows <= self.batch else torch.empty((rows, self.ffn), dtype=torch.float16, device=self.device)
        L.gate_up.forward_gated(y, out=act)
        return self._reduce(L.down(act), decode)

    # ------------------------------------------------------------------------------------ prefill
    @torch.inference_mode()
    def prefill(self, input_ids: torch.Tensor) -> torch.Tensor:
        """Run the prompt ``[batch, T]`` through the model, fill the KV caches for positions 0..T-1 and
        return the logits of the last position ``[batch, vocab]``.  The linears see ``batch * T`` rows,
        i.e. their prefill path."""
        s, B = self.spec, self.batch
        if input_ids.shape[0] != B:
            raise ValueError(f"the model was built for batch {B}")
        T = input_ids.shape[1]
        if T > self.max_seq:
            raise ValueError("prompt longer than the KV cache")
        with torch.cuda.device(self.device):
            ids = input_ids.to(self.device)
            h = self.embed[ids].reshape(B * T, s.hidden).contiguous()
            y = torch.empty_like(h)
            pos = torch.arange(T, device=self.device, dtype=torch.int32).repeat(B)
            mlp = None
            for L in self.layers:
                self._add_rmsnorm(h, mlp, L.in_norm, y)
                qkv = L.qkv(y)                                             # [B*T, (H + 2 KV) * D]
                _check(self.lib, self.lib.ap_rope_cache(qkv.data_ptr(), self.cos_sin.data_ptr(), pos.data_ptr(),
                                                        L.k_cache.data_ptr(), L.v_cache.data_ptr(), B * T, T, self.heads,
                                                        self.kv_heads, s.head_dim, self.max_seq, self._stream()), "ap_rope_cache")
                q = qkv[:, :self.heads * s.head_dim].reshape(B, T, self.heads, s.head_dim).transpose(1, 2)   # [B, H, T, D]
                k, v = L.k_cache[:, :, :T], L.v_cache[:, :, :T]
                attn = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.kv_heads != self.heads)
                attn = attn.transpose(1, 2).reshape(B * T, self.heads * s.head_dim)
                mlp = self._layer_tail(L, h, y, attn, decode=False)
            self._add_rmsnorm(h, mlp, self.final_norm, y)
            last = y.view(B, T, s.hidden)[:, -1]
            self.pos.fill_(T)
            return last @ self.lm_head.T

    # ------------------------------------------------------------------------------------ decode
    def _attention(self, L, qkv):
        """Rotary embedding of q and k, the cache write and the attention itself: one launch."""
        s = self.spec
        _check(self.lib, self.lib.ap_decode_attention_rope(
            qkv.data_ptr(), qkv.shape[1], self.cos_sin.data_ptr(), L.k_cache.data_ptr(), L.v_cache.data_ptr(),
            self.pos.data_ptr(), self.attn.data_ptr(), self.batch, self.heads, self.kv_heads, s.head_dim, self.max_seq,
            1.0 / math.sqrt(s.head_dim), self.attn_splits,
            self.attn_scratch.data_ptr() if self.attn_scratch is not None else None, self._stream()),
            "ap_decode_attention_rope")

    def _folded_norms(self):
        """Whether a decode step can fold every residual add + RMSNorm into the launches around it (on one GPU
        into the products' epilogues; across tensor-parallel ranks the add goes into the one-shot all-reduce
        that sums a row-parallel output): at most eight sequences, shapes the decode kernel takes."""
        if self.batch > 8:
            return False
        if self.tp_world > 1 and (self.allreduce is None or not hasattr(self.allreduce, "collect") or
                                  self.allreduce.residual_blocks(self.batch, self.spec.hidden) == 0):
            return False                                   # the process group's all-reduce has no folded form
        return all(m.bias is None and m.in_features % 128 == 0 and m.out_features % 16 == 0
                   for L in self.layers for m in (L.qkv, L.o, L.gate_up, L.down))

    def _decode_step_folded(self):
        """The decode step with five launches per layer: q+k+v (scaled by the norm's rsqrt in its epilogue),
        attention (rotation and cache write inside), o (residual add, norm weights and sums of squares in its
        epilogue), gate+up (scaled, SiLU * up in its epilogue), down (as o, with the next layer's norm).  The
        first norm is the stand-alone kernel; the last one's scale is positive and the same for all logits of a
        sequence, so the arg-max needs none."""
        s = self.spec
        h, y, ssq = self.h, self.y, self.ssq
        tp = self.tp_world > 1
        blocks = self.allreduce.residual_blocks(self.batch, s.hidden) if tp else None   # partial sums per row in ssq

        def add_and_scale(layer, x, norm_weight):
            if tp:                                           # this rank's partial product goes from the kernel's epilogue into
                layer.forward_push(x, self.allreduce)       # every rank's inbox; the collect sums and adds
                self.allreduce.collect(y, h, norm_weight, ssq)
            else:
                layer.forward_residual(x, h, norm_weight, ssq, out=y)

        h.copy_(self.embed[self.tok])
        self._add_rmsnorm(h, None, self.layers[0].in_norm, y)
        for li, L in enumerate(self.layers):
            qkv = L.qkv(y) if li == 0 else L.qkv.forward_prenorm(y, ssq, s.hidden, s.rms_eps, blocks=blocks)
            self._attention(L, qkv)
            add_and_scale(L.o, self.attn, L.post_norm)
            L.gate_up.forward_prenorm(y, ssq, s.hidden, s.rms_eps, out=self.act, blocks=blocks)
            nxt = self.layers[li + 1].in_norm if li + 1 < len(self.layers) else self.final_norm
            add_and_scale(L.down, self.act, nxt)
        logits = y @ self.lm_head.T
        self.tok.copy_(logits.argmax(dim=-1))
        self.pos.add_(1)

    @torch.inference_mode()
    def last_logits(self) -> torch.Tensor:
        """fp32 logits ``[batch, vocab]`` of the decode step that ran last (the step itself keeps only their
        arg-max).  After a step with folded norms ``self.y`` is the residual stream times the last norm's
        weights without the division by its root mean square, which is applied here."""
        y = self.y.float()
        if self.fold_norms and self._folded_norms():
            y = y * torch.rsqrt(self.h.float().pow(2).mean(-1, keepdim=True) + self.spec.rms_eps)
        return y @ self.lm_head.float().T

    def _decode_step(self):
        """One token per sequence: reads ``self.tok`` and ``self.pos``, writes the next token to ``self.tok``
        and advances ``self.pos``.  Everything it touches lives on the device (graph-replayable)."""
        if self.fold_norms and self._folded_norms():
            return self._decode_step_folded()
        s, B = self.spec, self.batch
        self.h.copy_(self.embed[self.tok])
        mlp = None
        for L in self.layers:
            self._add_rmsnorm(self.h, mlp, L.in_norm, self.y)
            qkv = L.qkv(self.y)                                              # decode kernel: B <= 8 rows
            self._attention(L, qkv)
            mlp = self._layer_tail(L, self.h, self.y, self.attn, decode=True)
        self._add_rmsnorm(self.h, mlp, self.final_norm, self.y)
        logits = self.y @ self.lm_head.T
        self.tok.copy_(logits.argmax(dim=-1))
        self.pos.add_(1)

    def _graph(self, precision):
        """The captured decode step of ``precision``.  Must be called on the side stream the graphs live on
        (``generate`` does): the split-K scratch of the linears belongs to the stream that captures."""
        g = self._graphs.get(precision)
        if g is None:
            stream = torch.cuda.current_stream(self.device)
            _ext.reserve_workspace(self.device)
            pos0, tok0 = self.pos.clone(), self.tok.clone()
            self._decode_step()                                  # warm-up outside the capture (allocations, tensor maps)
            torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                self._decode_step()
            self.pos.copy_(pos0)
            self.tok.copy_(tok0)
            self._graphs[precision] = g
        return g

    @torch.inference_mode()
    def generate(self, input_ids: torch.Tensor, max_new_tokens: int, precision: int | None = None,
                 use_graph: bool = True) -> torch.Tensor:
        """Greedy generation: ``[batch, T]`` prompt -> ``[batch, T + max_new_tokens]``.  ``precision``
        applies to this call only, as in the reference's ``generate`` (AnyPrecisionForCausalLM.py:99-111)."""
        prev = self.precision
        if precision is not None:
            self.set_precision(precision)
        try:
            with torch.cuda.device(self.device):
                T = input_ids.shape[1]
                if T + max_new_tokens > self.max_seq:
                    raise ValueError("prompt + new tokens exceed the KV cache")
                logits = self.prefill(input_ids)
                out = [logits.argmax(dim=-1)]
                self.tok.copy_(out[0])
                if use_graph and max_new_tokens > 1:
                    if self._side is None:
                        self._side = torch.cuda.Stream(self.device)
                    stream = self._side
                    stream.wait_stream(torch.cuda.current_stream(self.device))
                    with torch.cuda.stream(stream):
                        g = self._graph(self.precision)
                        for _ in range(max_new_tokens - 1):
                            g.replay()
                            out.append(self.tok.clone())
                    torch.cuda.current_stream(self.device).wait_stream(stream)
                else:
                    for _ in range(max_new_tokens - 1):
                        self._decode_step()
                        out.append(self.tok.clone())
                return torch.cat([input_ids.to(self.device), torch.stack(out, dim=1)], dim=1)
        finally:
            self.set_precision(prev)
