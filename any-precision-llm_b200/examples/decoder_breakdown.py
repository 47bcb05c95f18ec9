"""Where a decode step of the random-init Llama-2-7B decoder spends its time: the captured step is timed whole
and again with groups of its kernels replaced by no-ops (results are then meaningless; only the time counts).

    python any-precision-llm_b200/examples/decoder_breakdown.py [w_bits]
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

import torch

from anyprec_b200.decoder import AnyPrecisionLlama, LlamaSpec
from anyprec_b200.modules.AnyPrecisionLinear import AnyPrecisionLinear


def main():
    w = int(sys.argv[1]) if len(sys.argv) > 1 else 4
    spec = LlamaSpec.llama2_7b()
    model = AnyPrecisionLlama.random_init(spec, "cuda", seed=1, batch=1, max_seq=640)
    ids = torch.randint(0, spec.vocab, (1, 512), generator=torch.Generator().manual_seed(1))
    model.set_precision(w)

    def timed(label):
        model._graphs.clear()
        logits = model.prefill(ids)
        model.tok.copy_(logits.argmax(-1))
        torch.cuda.synchronize()
        if model._side is None:
            model._side = torch.cuda.Stream()
        with torch.cuda.stream(model._side):
            g = model._graph(w)
            for _ in range(5):
                g.replay()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(100):
                g.replay()
            b.record()
        torch.cuda.synchronize()
        print(f"{label}: {a.elapsed_time(b) / 100:.3f} ms per token", flush=True)

    class Without:
        """The library with some entry points answering 0 without launching anything."""

        def __init__(self, lib, skip):
            self._lib, self._skip = lib, skip

        def __getattr__(self, name):
            if name in self._skip:
                return lambda *args: 0
            return getattr(self._lib, name)

    real = model.lib
    timed(f"w_bits {w}: whole step")
    model.lib = Without(real, {"ap_decode_attention_rope"})
    timed("without attention (with rotary embedding and cache write inside)")
    model.lib = real
    forward = AnyPrecisionLinear.forward
    outs = {}

    def no_linear(self, x, **kwargs):
        key = (x.shape[0], self.out_features)
        if key not in outs:
            outs[key] = torch.zeros(key, dtype=torch.float16, device=x.device)
        return outs[key]

    def no_fused(self, x, *args, out=None, **kwargs):
        if out is not None:
            return out
        full = no_linear(self, x)
        return full[:, :self.out_features // 2] if getattr(self, "gated", False) else full

    saved = {name: getattr(AnyPrecisionLinear, name) for name in ("forward_gated", "forward_prenorm", "forward_residual")}
    AnyPrecisionLinear.forward = no_linear
    for name in saved:
        setattr(AnyPrecisionLinear, name, no_fused)
    timed("without the linears (attention, first norm, lm_head and embedding left)")
    AnyPrecisionLinear.forward = forward
    for name, fn in saved.items():
        setattr(AnyPrecisionLinear, name, fn)
    model.fold_norms = False
    timed("whole step with every norm a launch of its own (fold_norms = False)")


if __name__ == "__main__":
    main()
