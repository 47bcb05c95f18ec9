"""Benchmark of the bitplane GEMV hot path (matmul_kbit) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line is printed by rank 0.

Workload at N = 1: the Llama-2-7B linear-layer set (q/k/v/o 4096x4096, gate/up 11008x4096,
down 4096x11008), every layer an 8-bit-parent any-precision layer, swept over w_bits 3..8 at
batch 1.  A *step* is one pass of matmul_kbit over the whole weight set for every w_bits:
`--layers` decoder layers' worth of distinct weights (default 4: 28 linears, 0.8 GB of planes,
so consecutive launches never find their operands in the 126 MB L2).  Operands are seeded
synthetic data with the reference's layout and value distributions (uniform parent codes drawn
directly as random bitplanes, per-row sorted N(0, 0.02) fp16 tables, N(0, 1) fp16 activations).

`value` is the algorithmic bytes of all launches in the timed region divided by its duration,
operands resident in HBM, launches replayed from one CUDA graph per step.  `e2e` is the same
quantity through the public operator API (any_precision_ext.matmul_kbit) with activations
coming from pinned host memory and results copied back, copies inside the timed region.

At N > 1 the workload is the Llama-2-70B linear-layer set, tensor-parallel over the ranks
(q/k/v/gate/up split on N, o/down split on K with an all-reduce of the row-parallel outputs);
value is again total algorithmic bytes over the max-over-ranks time.  The same workload on one
GPU (`tp1_llama2_70b` in the N = 1 line) anchors the 1/2/4/8 curve, and `curve` holds w_bits
3, 4, 8 at batch 1 and 8 with the decode rate the linear stack alone would allow.

`--impl reference` times the reference semantics on the host cores instead: the reference's own
dequantisation kernel source compiled for the CPU (oracle/_ref; else the oracle port) followed by
an fp32 torch.matmul, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "any-precision-llm_b200")
for _p in (ROOT, PKG):
    if _p not in sys.path:
        sys.path.insert(0, _p)

METRIC = "bitplane_gemv_hbm_gbs"
UNIT = "GB/s"
W_BITS = (3, 4, 5, 6, 7, 8)
# DRAM bytes moved per algorithmic byte by the decode kernel, from hardware counters of single launches
# (see profiles/): the kernel reads every operand once and writes the output once.
DRAM_TRAFFIC_RATIO = 1.002
LLAMA2_7B_SET = [("q_proj", 4096, 4096), ("k_proj", 4096, 4096), ("v_proj", 4096, 4096), ("o_proj", 4096, 4096),
                 ("gate_proj", 11008, 4096), ("up_proj", 11008, 4096), ("down_proj", 4096, 11008)]
# name, N, K, parallel style
LLAMA2_70B_SET = [("q_proj", 8192, 8192, "col"), ("k_proj", 1024, 8192, "col"), ("v_proj", 1024, 8192, "col"),
                  ("o_proj", 8192, 8192, "row"), ("gate_proj", 28672, 8192, "col"), ("up_proj", 28672, 8192, "col"),
                  ("down_proj", 8192, 28672, "row")]


def gemv_bytes(M: int, N: int, K: int, w: int) -> int:
    """Algorithmic bytes of one matmul_kbit: planes + that precision's table + activations in + out."""
    return N * K * w // 8 + N * (1 << w) * 2 + M * K * 2 + M * N * 2


def measured_peak_tflops():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"]), "measured"
    except (OSError, KeyError, ValueError):
        return 1590.0, "fallback"


def prefill_figures(torch, ext, packing, device):
    """Secondary figures for the prefill side of the path (tensor roofline): the fused dequantise + tcgen05
    kernel and the two-step dequant_kbit + library GEMM on Llama-3-8B layer shapes (64, 256 and 2048 tokens), w_bits 4, three distinct
    layers per CUDA graph, CUDA events.  Reported beside the headline, not part of it."""
    peak, kind = measured_peak_tflops()
    gen = torch.Generator(device=device).manual_seed(77)
    out = []
    for N, K, M in ((14336, 4096, 64), (14336, 4096, 256), (4096, 4096, 2048)):
        qs = [packing.random_qweight(8, N, K, device=device, generator=gen) for _ in range(3)]
        luts = [packing.random_lut(N, 4, device=device, generator=gen) for _ in range(3)]
        x = torch.randn((M, K), device=device, generator=gen).to(torch.float16)
        y = torch.empty((M, N), device=device, dtype=torch.float16)
        W = torch.empty((N, K), device=device, dtype=torch.float16)

        def fused():
            for i in range(3):
                ext.gemm_kbit(x, qs[i], luts[i], 4, out=y)

        def two_step():
            for i in range(3):
                ext.dequant_kbit(qs[i], luts[i], 4, out=W)
                torch.matmul(x, W.T, out=y)

        row = {"layer": f"{N}x{K}", "tokens": M, "w_bits": 4}
        for name, fn in (("fused_tcgen05", fused), ("dequant_plus_library_gemm", two_step)):
            fn()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            st = torch.cuda.Stream(device)
            with torch.cuda.stream(st):
                fn()
                torch.cuda.synchronize()
                with torch.cuda.graph(g, stream=st):
                    fn()
            torch.cuda.synchronize()
            for _ in range(3):
                g.replay()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(10):
                g.replay()
            b.record()
            torch.cuda.synchronize()
            us = a.elapsed_time(b) * 1e3 / 30
            tf = 2.0 * M * N * K / us / 1e6
            row[name] = {"us": round(us, 1), "tflops": round(tf, 1), "frac_of_tensor_peak": round(tf / peak, 3)}
            del g
        out.append(row)
        del qs, luts, W
    return {"peak_tflops": peak, "peak_kind": kind, "cases": out}


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20", "-i",
                 str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                smax = float(parts[1])
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm)}


# --------------------------------------------------------------------------------------------- ours
def build_weight_set(torch, packing, shapes, layers, device, seed):
    gen = torch.Generator(device=device).manual_seed(seed)
    weights = []
    for layer in range(layers):
        for name, N, K in shapes:
            q = packing.random_qweight(8, N, K, device=device, generator=gen)
            luts = {w: packing.random_lut(N, w, device=device, generator=gen) for w in W_BITS}
            weights.append((name, N, K, q, luts))
    return weights


def run_ours(args):
    import torch
    import torch.distributed as dist

    import any_precision_ext as ext
    from anyprec_b200 import packing

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    ext.load_library()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            raise SystemExit("for --gpus N > 1 launch with: python -m torch.distributed.run --nproc-per-node N bench.py ...")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    if world > 1:
        line = tensor_parallel_figures(args, rank, world, device, args.layers, full=True)
        torch.cuda.empty_cache()
        decoder70 = decoder_70b_figures(args, rank, world, device)
        if rank == 0:
            line["decoder_llama2_70b"] = decoder70
            print(json.dumps(line))
        # A captured graph holds collective work; leave without the process-group destructor (it can block
        # on a communicator that graphs still use).  Only the benchmark process ends this way.
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)

    M = args.batch
    weights = build_weight_set(torch, packing, LLAMA2_7B_SET, args.layers, device, seed=1000)
    gen = torch.Generator(device=device).manual_seed(7)
    xs = {K: torch.randn((M, K), device=device, generator=gen).to(torch.float16) for K in (4096, 11008)}
    outs = {N: torch.empty((M, N), device=device, dtype=torch.float16) for N in (4096, 11008)}

    def one_pass(w):
        for _, N, K, q, luts in weights:
            ext.matmul_kbit(xs[K], q, luts[w], w, out=outs[N])

    def one_step():
        for w in W_BITS:
            one_pass(w)

    launches_per_step = len(weights) * len(W_BITS)
    bytes_per_w = {w: sum(gemv_bytes(M, N, K, w) for _, N, K, _, _ in weights) for w in W_BITS}
    bytes_per_step = sum(bytes_per_w.values())

    # Capture one step into a CUDA graph (kernels are launched on the capturing stream).
    stream = torch.cuda.Stream(device)
    with torch.cuda.stream(stream):
        one_step()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            one_step()
        per_w_graphs = {}
        for w in W_BITS:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                one_pass(w)
            per_w_graphs[w] = g
    torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)      # started before warm-up: nvidia-smi needs ~0.1 s to deliver samples
    sampler.start()
    for _ in range(args.warmup):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ms_total = e0.elapsed_time(e1)

    # Per-w_bits breakdown (same weights, same launches, timed per precision).
    per_w = {}
    for w in W_BITS:
        for _ in range(2):
            per_w_graphs[w].replay()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        reps = max(3, args.steps)
        for _ in range(reps):
            per_w_graphs[w].replay()
        b.record()
        torch.cuda.synchronize()
        gbs = bytes_per_w[w] * reps / (a.elapsed_time(b) * 1e-3) / 1e9
        per_w[str(w)] = round(gbs, 1)
    clocks = sampler.stop()

    ms_per_step = ms_total / args.steps
    value = bytes_per_step / (ms_per_step * 1e-3) / 1e9
    peak, peak_kind = measured_peak_gbs()

    # Secondary figure: the same weights with q/k/v and gate/up stacked by rows (one launch each, as a
    # decoder that fuses those layers would call the operator).  Same planes and tables, fewer launches.
    fused_sets = []
    per_layer = len(LLAMA2_7B_SET)
    for l0 in range(0, len(weights), per_layer):
        group = {name: (N, K, q, luts) for name, N, K, q, luts in weights[l0:l0 + per_layer]}
        for names in (("q_proj", "k_proj", "v_proj"), ("o_proj",), ("gate_proj", "up_proj"), ("down_proj",)):
            q, luts = packing.concat_rows([group[n][2] for n in names], [group[n][3] for n in names])
            fused_sets.append((q.shape[1], group[names[0]][1], q, luts))
    fouts = {N: torch.empty((M, N), device=device, dtype=torch.float16) for N in {f[0] for f in fused_sets}}

    def fused_step():
        for w in W_BITS:
            for N, K, q, luts in fused_sets:
                ext.matmul_kbit(xs[K], q, luts[w], w, out=fouts[N])

    with torch.cuda.stream(stream):
        fused_step()
        torch.cuda.synchronize()
        fgraph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(fgraph, stream=stream):
            fused_step()
    torch.cuda.synchronize()
    for _ in range(args.warmup):
        fgraph.replay()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(args.steps):
        fgraph.replay()
    b.record()
    torch.cuda.synchronize()
    fused_bytes = sum(gemv_bytes(M, N, K, w) for w in W_BITS for N, K, _, _ in fused_sets)
    fused_value = fused_bytes * args.steps / (a.elapsed_time(b) * 1e-3) / 1e9
    del fgraph, fused_sets

    # End to end through the operator API: activations from pinned host memory, result back to host.
    x_host = {K: torch.randn((M, K), generator=torch.Generator().manual_seed(K)).to(torch.float16).pin_memory()
              for K in (4096, 11008)}
    y_host = {N: torch.empty((M, N), dtype=torch.float16).pin_memory() for N in (4096, 11008)}
    x_dev = {K: torch.empty((M, K), device=device, dtype=torch.float16) for K in (4096, 11008)}

    def e2e_step():
        # one step end to end: this step's activations come from pinned host memory, every layer is
        # one call of the public operator, the step's results go back to pinned host memory
        h2d = d2h = 0
        for K in x_dev:
            x_dev[K].copy_(x_host[K], non_blocking=True)
            h2d += M * K * 2
        for w in W_BITS:
            for _, N, K, q, luts in weights:
                ext.matmul_kbit(x_dev[K], q, luts[w], w, out=outs[N])
        for N in y_host:
            y_host[N].copy_(outs[N], non_blocking=True)
            d2h += M * N * 2
        torch.cuda.current_stream().synchronize()           # the host has the step's result
        return h2d, d2h

    e2e_steps = max(1, min(args.steps, 5))
    e2e_step()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(e2e_steps):
        h2d, d2h = e2e_step()
    b.record()
    torch.cuda.synchronize()
    e2e_gbs = bytes_per_step * e2e_steps / (a.elapsed_time(b) * 1e-3) / 1e9

    # The same step as a serving loop runs it: the copies and the operator calls captured once into a CUDA
    # graph (the operator allocates nothing when `out` is given), one replay plus a stream synchronise per
    # step.  Reported beside `e2e`, which stays the eager figure.
    gstream = torch.cuda.Stream()
    egraph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(gstream):
        with torch.cuda.graph(egraph, stream=gstream):
            for K in x_dev:
                x_dev[K].copy_(x_host[K], non_blocking=True)
            for w in W_BITS:
                for _, N, K, q, luts in weights:
                    ext.matmul_kbit(x_dev[K], q, luts[w], w, out=outs[N])
            for N in y_host:
                y_host[N].copy_(outs[N], non_blocking=True)
        egraph.replay()
        gstream.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(gstream)
        for _ in range(e2e_steps):
            egraph.replay()
            gstream.synchronize()                            # the host has the step's result
        b.record(gstream)
        gstream.synchronize()
    e2e_graph_gbs = bytes_per_step * e2e_steps / (a.elapsed_time(b) * 1e-3) / 1e9
    del egraph

    prefill = prefill_figures(torch, ext, packing, device)
    # The tensor-parallel workload (Llama-2-70B layer set) on this one GPU: the anchor of the 1/2/4/8 curve.
    tp1 = tensor_parallel_figures(args, 0, 1, device, args.layers, full=False)
    decoder = decoder_figures(args, device)
    decoder70 = decoder_70b_figures(args, 0, 1, device)
    quantizer = quantizer_figures(device)
    cpu = cpu_baseline_sample(kind_pref="port", seconds_hint=15)

    line = {
        "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"llama2-7b linear-layer set x{args.layers} layers, matmul_kbit M={M}, w_bits 3..8 sweep",
                   "batch": M, "launches_per_step": launches_per_step,
                   "bytes_per_step": bytes_per_step, "l2": "inputs larger than L2 (0.8 GB of planes per pass)"},
        "fused_qkv_gateup": {"value": round(fused_value, 1), "unit": UNIT, "launches_per_step": 4 * args.layers * len(W_BITS),
                             "note": "same weights, q+k+v and gate+up stacked by rows (packing.concat_rows)"},
        "prefill": prefill,
        "tp1_llama2_70b": tp1,
        "decoder_llama2_7b": decoder,
        "decoder_llama2_70b": decoder70,
        "quantizer": quantizer,
        "per_w_bits_gbs": per_w,
        "per_w_bits_frac_of_measured_peak": {k: round(v / peak, 3) for k, v in per_w.items()},
        "roofline": {"bound": "hbm", "achieved": round(value, 1), "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                     "frac": round(value / peak, 4), "frac_of_nominal_8tbs": round(value / 8000.0, 4),
                     "traffic": round(bytes_per_step / launches_per_step * DRAM_TRAFFIC_RATIO),
                     "traffic_unit": "bytes per launch (mean over the step's launches)",
                     "algorithmic_bytes_per_launch": round(bytes_per_step / launches_per_step),
                     "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of single M=1 launches: 4096x4096 at "
                                       "w_bits 3, 4, 8 (1.003, 1.003, 1.001 x the algorithmic bytes), 11008x4096 at 3, 4 (1.0013, "
                                       "1.0008), 4096x11008 at 4, 8 (1.0015, 1.0014); scaled by bytes"},
        "cpu_baseline": cpu,
        "e2e": {"value": round(e2e_gbs, 1), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "e2e_cuda_graph": {"value": round(e2e_graph_gbs, 1), "unit": UNIT,
                           "note": "the e2e step (pinned-host copies in and out, every layer one operator call) captured "
                                   "once and replayed per step with a stream synchronise; `e2e` is the eager figure"},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks,
    }
    print(json.dumps(line))
    return line




# ------------------------------------------------------------------------------------- quantiser
def quantizer_figures(device):
    """Seed (3-bit) + upscale (to 8-bit) quantisation of the three Llama-2-7B layer shapes on the GPU
    (`ap_seed_upscale`, one thread block per row), in rows and weights per second, with the CPU checker's
    row routine timed on a few rows of the same data beside it (one core, plain Python + numpy)."""
    import numpy as np
    import torch

    from anyprec_b200 import quantize
    from oracle import seed_upscale as su

    out = {}
    gen = torch.Generator(device=device).manual_seed(4000)
    for N, K in ((4096, 4096), (11008, 4096), (4096, 11008)):
        w = (torch.randn((N, K), device=device, generator=gen) * 0.02).half().float()
        s = torch.randn((N, K), device=device, generator=gen) ** 2
        quantize.seed_and_upscale_layer(w, s)                                  # warm-up (module load, allocations)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        luts, codes = quantize.seed_and_upscale_layer(w, s)
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b)
        rows = 4
        wn, sn = w[:rows].cpu().numpy(), s[:rows].cpu().numpy()
        t0 = time.perf_counter()
        ref_luts, ref_codes = su.seed_and_upscale_layer(wn, sn, 3, 8, blocked=True)
        cpu_s = (time.perf_counter() - t0) / rows
        same = bool(np.array_equal(codes[:rows].cpu().numpy(), ref_codes)) and all(
            np.array_equal(luts[bit][:rows].cpu().numpy().view(np.uint16), ref_luts[bit].view(np.uint16)) for bit in ref_luts)
        out[f"{N}x{K}"] = {"gpu_ms": round(ms, 2), "rows_per_s": round(N / ms * 1e3), "weights_per_s": round(N * K / ms * 1e3),
                           "cpu_checker_rows_per_s_one_core": round(1.0 / cpu_s, 1), "first_rows_equal_checker": same}
    return {"what": "seed 3-bit + upscale to 8-bit per-row tables and codes (quantize.py:85-187 of the reference), fp32 in, "
                    "fp16-valued N(0, 0.02) weights, squared-normal sensitivities", "layers": out}


# ------------------------------------------------------------------------------------- whole-model decode
def decoder_figures(args, device):
    """Decode rate of a whole random-init Llama-2-7B decoder whose linears are any-precision layers: a
    512-token prompt of uniform random token ids, then 128 greedy steps at batch 1, for every w_bits.
    `generate_tok_s` is the wall-clock method of the reference's demo (new tokens over the whole generate call,
    prompt included, synchronised at both ends); `decode_tok_s` times the 127 replayed decode steps alone
    with CUDA events.  `bound_tok_s` is what the measured HBM peak allows for the bytes a step must read
    (planes, that precision's tables, fp16 lm_head; KV cache and activations not counted)."""
    import torch

    from anyprec_b200.decoder import AnyPrecisionLlama, LlamaSpec

    spec = LlamaSpec.llama2_7b()
    prompt, new = 512, 128
    model = AnyPrecisionLlama.random_init(spec, device, seed=2000, batch=1, max_seq=prompt + new)
    ids = torch.randint(0, spec.vocab, (1, prompt), generator=torch.Generator().manual_seed(2))
    peak, _ = measured_peak_gbs()
    per_layer = [(spec.heads * spec.head_dim + 2 * spec.kv_heads * spec.head_dim, spec.hidden), (spec.hidden, spec.hidden),
                 (2 * spec.ffn, spec.hidden), (spec.hidden, spec.ffn)]
    out = {}
    for w in W_BITS:
        model.generate(ids, 4, precision=w)                                   # captures this precision's decode graph
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        toks = model.generate(ids, new, precision=w)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        assert toks.shape == (1, prompt + new)
        # the decode steps alone
        model.set_precision(w)
        logits = model.prefill(ids)
        model.tok.copy_(logits.argmax(-1))
        torch.cuda.synchronize()
        with torch.cuda.stream(model._side):
            g = model._graph(w)                                               # cached by the generate calls above
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(new - 1):
                g.replay()
            b.record()
        torch.cuda.synchronize()
        step_ms = a.elapsed_time(b) / (new - 1)
        step_bytes = spec.layers * sum(N * K * w // 8 + N * (1 << w) * 2 for N, K in per_layer) + spec.vocab * spec.hidden * 2
        out[str(w)] = {"generate_tok_s": round(new / wall, 1), "decode_tok_s": round(1e3 / step_ms, 1),
                       "decode_ms_per_token": round(step_ms, 4), "bound_tok_s": round(peak * 1e9 / step_bytes, 1),
                       "frac_of_bound": round(1e3 / step_ms / (peak * 1e9 / step_bytes), 3)}
    del model
    torch.cuda.empty_cache()
    return {"model": "random-init Llama-2-7B decoder (32 layers, hidden 4096, 32 heads, FFN 11008, vocab 32000), every "
                     "linear an 8-bit-parent any-precision layer; five launches per layer (q+k+v, attention with rotation and cache write, "
                     "o, gate+up with SiLU * up, down; residual adds and norms in their epilogues); one CUDA graph per precision",
            "prompt_tokens": prompt, "new_tokens": new, "batch": 1, "per_w_bits": out}


def decoder_70b_figures(args, rank, world, device):
    """Decode rate of a whole random-init Llama-2-70B decoder (80 layers, hidden 8192, 64 heads / 8 KV heads,
    FFN 28672) tensor-parallel over `world` ranks: a 1024-token prompt of uniform random token ids, then greedy
    decode steps at batch 1 and batch 8, w_bits 3, 4 and 8.  q/k/v/gate/up are split on their rows (heads, FFN
    rows), o/down on their input columns with the one-shot all-reduce in the captured decode step and the process
    group's all-reduce for the prompt.  Times are the max over ranks; `bound_tok_s` is what the measured HBM peak
    allows for the bytes ONE rank must read per step (its planes and tables, the replicated fp16 lm_head)."""
    import torch
    import torch.distributed as dist

    from anyprec_b200.decoder import AnyPrecisionLlama, LlamaSpec

    spec = LlamaSpec.llama2_70b()
    prompt, new = 1024, 33
    allreduce = None
    if world > 1:
        from anyprec_b200.comm import OneShotAllReduce
        allreduce = OneShotAllReduce(8 * spec.hidden * 2, device)
    big = AnyPrecisionLlama.random_init(spec, device, supported_bits=(3, 4, 8), seed=4100, batch=8, max_seq=prompt + new,
                                        tp_rank=rank, tp_world=world, allreduce=allreduce)
    peak, _ = measured_peak_gbs()
    local = [(m.out_features, m.in_features) for L in big.layers[:1] for m in (L.qkv, L.o, L.gate_up, L.down)]
    out = {}
    for batch in (1, 8):
        model = big if batch == 8 else big.with_batch(1)
        ids = torch.randint(0, spec.vocab, (batch, prompt), generator=torch.Generator().manual_seed(3))
        for w in (3, 4, 8):
            model.generate(ids, 3, precision=w)                               # captures this precision's decode graph
            model.set_precision(w)
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            t0 = time.perf_counter()
            logits = model.prefill(ids)
            torch.cuda.synchronize()
            prefill_ms = (time.perf_counter() - t0) * 1e3
            model.tok.copy_(logits.argmax(-1))
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            with torch.cuda.stream(model._side):
                g = model._graph(w)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(new - 1):
                    g.replay()
                b.record()
            torch.cuda.synchronize()
            t = torch.tensor([a.elapsed_time(b) / (new - 1), prefill_ms], device=device, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            step_ms = float(t[0])
            step_bytes = spec.layers * sum(N * K * w // 8 + N * (1 << w) * 2 for N, K in local) + spec.vocab * spec.hidden * 2
            bound = batch * peak * 1e9 / step_bytes
            out[f"batch{batch}_w{w}"] = {"decode_tok_s": round(batch * 1e3 / step_ms, 1), "decode_ms_per_step": round(step_ms, 3),
                                         "prefill_ms": round(float(t[1]), 1), "bound_tok_s": round(bound, 1),
                                         "frac_of_bound": round(batch * 1e3 / step_ms / bound, 3)}
    if allreduce is not None:
        wait_expired = allreduce.wait_expired()
        allreduce.close()
    else:
        wait_expired = False
    del big, model
    torch.cuda.empty_cache()
    return {"model": "random-init Llama-2-70B decoder (80 layers, hidden 8192, 64 heads, 8 KV heads, FFN 28672, vocab 32000), "
                     "every linear an 8-bit-parent any-precision layer",
            "parallelism": f"tp{world}", "prompt_tokens": prompt, "decode_steps_timed": new - 1,
            "allreduce_wait_expired": bool(wait_expired), "cases": out}

# ----------------------------------------------------------------------------- tensor-parallel workload
def tensor_parallel_figures(args, rank, world, device, layers, full):
    """Decode-step linear stack of Llama-2-70B over `world` ranks (world = 1: the whole layers on one GPU).

    Per decoder layer: q+k+v (column-parallel, stacked by rows into one launch) -> o (row-parallel,
    all-reduce) -> gate+up (column, stacked) -> down (row, all-reduce).  The full-size operands are never
    materialised: each rank draws its own shard directly (uniform codes are i.i.d. bits, so a shard of
    random planes is a random shard).  Before anything is timed one row-parallel layer's all-reduced output
    is checked against a rank-order fp32 sum of the gathered partial results (`tp_check`).

    Returns the JSON line (world > 1, rank 0; None on other ranks) or, for world = 1, the secondary object
    that the one-GPU line carries."""
    import torch
    import torch.distributed as dist

    import any_precision_ext as ext
    from anyprec_b200 import packing
    from anyprec_b200.tensor_parallel import LinearShard, shard_bounds, shard_forward, stack_column_shards

    M = args.batch
    gen = torch.Generator(device=device).manual_seed(4000 + rank)
    shards = []
    for _ in range(layers):
        for name, N, K, style in LLAMA2_70B_SET:
            if style == "col":
                n0, n1 = shard_bounds(N, world, rank, 16)
                q = packing.random_qweight(8, n1 - n0, K, device=device, generator=gen)
                luts = {w: packing.random_lut(n1 - n0, w, device=device, generator=gen) for w in W_BITS}
                shards.append((name, LinearShard("col", q, luts, (n0, n1), (0, K))))
            else:
                k0, k1 = shard_bounds(K, world, rank, 128)
                q = packing.random_qweight(8, N, k1 - k0, device=device, generator=gen)
                lgen = torch.Generator(device=device).manual_seed(5000 + len(shards))   # replicated tables
                luts = {w: packing.random_lut(N, w, device=device, generator=lgen) for w in W_BITS}
                shards.append((name, LinearShard("row", q, luts, (0, N), (k0, k1))))
    fuse = os.environ.get("AP_TP_FUSE", "1") != "0"
    if fuse:
        shards = stack_column_shards(shards)

    hidden = LLAMA2_70B_SET[0][2]
    max_m = 8
    x_full = torch.randn((max_m, hidden), device=device, generator=torch.Generator(device=device).manual_seed(9)).half()
    bufs = {}
    for name, sh in shards:
        bufs.setdefault((sh.style, sh.out_features), torch.empty((max_m, sh.out_features), device=device, dtype=torch.float16))
        bufs.setdefault(("in", sh.in_features), torch.randn((max_m, sh.in_features), device=device).half())

    # Row-parallel outputs are summed by the one-shot peer-memory kernel unless asked otherwise
    # (AP_TP_ALLREDUCE=nccl) or its set-up fails on this machine, which the JSON line then says.
    allreduce, allreduce_kind = None, "none (one rank)"
    if world > 1:
        allreduce_kind = "nccl"
        if os.environ.get("AP_TP_ALLREDUCE", "oneshot") == "oneshot":
            try:
                from anyprec_b200.comm import OneShotAllReduce
                allreduce = OneShotAllReduce(max_m * max(sh.out_features for _, sh in shards if sh.style == "row") * 2, device)
                allreduce_kind = "one-shot over peer memory (ap_allreduce_oneshot)"
            except Exception as exc:                                   # noqa: BLE001 - reported, not hidden
                allreduce_kind = f"nccl (one-shot set-up failed: {type(exc).__name__}: {exc})"[:200]
        kinds = [None] * world
        dist.all_gather_object(kinds, allreduce is not None)
        if not all(kinds):                                             # all ranks or none
            allreduce = None
            if allreduce_kind.startswith("one-shot"):
                allreduce_kind = "nccl (one-shot set-up failed on another rank)"

    # tp_check: one row-parallel layer, every precision of the curve, batch 1 and 8
    tp_check = "not applicable (one rank)"
    if world > 1:
        name, sh = next((n, s) for n, s in shards if s.style == "row")
        good = True
        for m in (1, 8):
            for w in (3, 4, 8):
                xin = bufs[("in", sh.in_features)][:m]
                part = ext.matmul_kbit(xin, sh.qweight, sh.luts[w], w)
                gathered = [torch.empty_like(part) for _ in range(world)]
                dist.all_gather(gathered, part)
                want = torch.zeros_like(part, dtype=torch.float32)
                for r in range(world):
                    want += gathered[r].float()                       # rank order, fp32: what the kernel does
                got = shard_forward(xin, sh, w, ext.matmul_kbit, allreduce=allreduce)
                if allreduce is not None:
                    good = good and torch.equal(got, want.to(torch.float16))
                else:
                    good = good and torch.allclose(got.float(), want, rtol=2e-2, atol=2e-2 * float(want.abs().max()))
        flag = torch.tensor([1.0 if good else 0.0], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        tp_check = "ok" if float(flag[0]) == 1.0 else "FAILED"
        if tp_check != "ok":
            raise SystemExit(f"tp_check failed on {name}: the all-reduced row-parallel output differs from the sum of the partials")

    push_ok = allreduce is not None and hasattr(allreduce, "push_target") and os.environ.get("AP_TP_PUSH", "1") != "0"

    def one_pass(w, m, do_gemv=True, do_reduce=True):
        for name, sh in shards:
            xin = (x_full if sh.style == "col" else bufs[("in", sh.in_features)])[:m]
            out = bufs[(sh.style, sh.out_features)][:m]
            if do_gemv and do_reduce and sh.style == "row" and world > 1 and push_ok and m <= 8:
                # the product stores its tiles straight into every rank's inbox; the collecting half sums
                ext.matmul_kbit(xin, sh.qweight, sh.luts[w], w, push=allreduce.push_target)
                allreduce.collect(out)
                continue
            if do_gemv:
                ext.matmul_kbit(xin, sh.qweight, sh.luts[w], w, out=out)
            if do_reduce and sh.style == "row" and world > 1:
                if allreduce is not None:
                    allreduce(out)
                else:
                    dist.all_reduce(out, op=dist.ReduceOp.SUM)

    def local_bytes(w, m):
        return sum(gemv_bytes(m, sh.out_features, sh.in_features, w) for _, sh in shards)

    def total_bytes(w, m):
        # whole-job algorithmic bytes: what all ranks together stream (tables of row-parallel layers are
        # replicated and counted once per rank, because every rank reads them)
        t = torch.tensor([float(local_bytes(w, m))], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t)
        return float(t[0])

    stream = torch.cuda.Stream(device)
    ext.reserve_workspace(device)

    def timed(fn, steps, warmup):
        """Capture fn into a graph on `stream`, replay it warmup + steps times; ms per replay, max over ranks."""
        with torch.cuda.stream(stream):
            ext.reserve_workspace(device)
            fn()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                fn()
        torch.cuda.synchronize()
        for _ in range(warmup):
            g.replay()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        ms = torch.tensor([e0.elapsed_time(e1) / steps], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        del g
        return float(ms[0])

    peak, peak_kind = measured_peak_gbs()
    sampler = ClockSampler(device.index if device.index is not None else 0)
    sampler.start()
    time.sleep(0.3)                                                    # nvidia-smi needs a moment to deliver samples
    ms_per_step = timed(lambda: [one_pass(w, M) for w in W_BITS], args.steps, args.warmup)
    clocks = sampler.stop()
    bytes_per_step = sum(total_bytes(w, M) for w in W_BITS)
    value = bytes_per_step / (ms_per_step * 1e-3) / 1e9

    # The curve BASELINE.json asks for: w_bits 3, 4, 8 at batch 1 and 8; per-GPU roofline fraction and the
    # decode rate the linear stack alone would allow for the 80-layer model (attention, norms and sampling
    # not included).
    curve = {}
    short = max(3, args.steps // 2)
    for m in (1, 8):
        for w in (3, 4, 8):
            ms = timed(lambda: one_pass(w, m), short, 3)
            gbs = total_bytes(w, m) / (ms * 1e-3) / 1e9
            curve[f"batch{m}_w{w}"] = {
                "ms_per_pass": round(ms, 4), "gbs": round(gbs, 1), "per_gpu_frac_of_peak": round(gbs / world / peak, 4),
                "us_per_decoder_layer": round(ms * 1e3 / layers, 2),
                "tok_s_linear_stack_80_layers": round(m / (ms * 1e-3 / layers * 80), 1)}
    breakdown = None
    if world > 1:
        gemv_ms = timed(lambda: [one_pass(w, M, do_reduce=False) for w in W_BITS], short, 3)
        red_ms = timed(lambda: [one_pass(w, M, do_gemv=False) for w in W_BITS], short, 3)
        breakdown = {"gemv_only_ms_per_step": round(gemv_ms, 4), "allreduce_only_ms_per_step": round(red_ms, 4),
                     "both_ms_per_step": round(ms_per_step, 4),
                     "note": "the same step captured without the all-reduces and without the GEMVs (there every "
                             "all-reduce is the one-kernel form; in the timed step the row-parallel products store "
                             "their tiles into the ranks' inboxes themselves and the all-reduce only collects)"}

    launches = len(shards) * len(W_BITS)
    config = {"workload": f"llama2-70b linear-layer set x{layers} layers, tensor-parallel tp{world} "
                          f"(q/k/v/gate/up on N, o/down on K + all-reduce), matmul_kbit M={M}, w_bits 3..8 sweep",
              "allreduce": allreduce_kind + (" fed by the products' epilogues (ap_matmul_kbit_push + ap_allreduce_oneshot_collect)"
                                             if push_ok else ""), "tp_check": tp_check,
              "fused_layers": "q+k+v and gate+up stacked by rows (one launch each)" if fuse else "none",
              "batch": M, "parallelism": f"tp{world}", "launches_per_step_per_rank": launches,
              "allreduces_per_step": (2 * layers * len(W_BITS)) if world > 1 else 0, "bytes_per_step": bytes_per_step,
              "l2": "inputs larger than L2"}
    if not full:
        return {"value": round(value, 1), "unit": UNIT, "ms_per_step": round(ms_per_step, 4),
                "frac_of_peak": round(value / peak, 4), "config": config, "curve": curve,
                "note": "the N > 1 workload on one GPU (no all-reduce): the TP = 1 point of the scaling curve"}

    # end to end through the operator API with host activations (copies inside the timed region)
    x_host = torch.randn((M, hidden)).half().pin_memory()
    y_host = torch.empty((M, hidden), dtype=torch.float16).pin_memory()
    x_dev = torch.empty((M, hidden), device=device, dtype=torch.float16)

    def e2e_step():
        h2d = d2h = 0
        for w in W_BITS:
            for name, sh in shards:
                if sh.style == "col":
                    x_dev.copy_(x_host, non_blocking=True)
                    h2d += x_host.numel() * 2
                    shard_forward(x_dev, sh, w, ext.matmul_kbit)
                else:
                    y = shard_forward(bufs[("in", sh.in_features)][:M], sh, w, ext.matmul_kbit, allreduce=allreduce)
                    y_host.copy_(y, non_blocking=True)
                    d2h += y.numel() * 2
        torch.cuda.current_stream().synchronize()
        return h2d, d2h

    e2e_step()
    torch.cuda.synchronize()
    dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_steps = max(1, min(args.steps, 3))
    a.record()
    for _ in range(e2e_steps):
        h2d, d2h = e2e_step()
    b.record()
    torch.cuda.synchronize()
    ems = torch.tensor([a.elapsed_time(b)], device=device, dtype=torch.float64)
    dist.all_reduce(ems, op=dist.ReduceOp.MAX)
    e2e_gbs = bytes_per_step * e2e_steps / (float(ems[0]) * 1e-3) / 1e9
    if rank != 0:
        return None
    return {
        "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic", "config": config,
        "roofline": {"bound": "hbm", "achieved": round(value / world, 1), "peak": peak, "peak_kind": peak_kind,
                     "unit": "GB/s per GPU", "frac": round(value / world / peak, 4), "traffic": None},
        "curve": curve, "breakdown": breakdown,
        "e2e": {"value": round(e2e_gbs, 1), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": (launches + (2 * layers * len(W_BITS))) * args.steps,
        "clocks": clocks,
    }


# --------------------------------------------------------------------------------------------- CPU arms
def cpu_baseline_sample(kind_pref: str, seconds_hint: float):
    """Time the reference semantics on the host cores on a bounded sample: the 4096 x 4096
    layer at every w_bits, batch 1 (bitplane unpack + table gather + fp32 product)."""
    import numpy as np

    from oracle import oracle

    N = K = 4096
    rng = np.random.default_rng(0)
    q = rng.integers(-2 ** 31, 2 ** 31, size=(8, N, K // 32), dtype=np.int64).astype(np.int32)
    x = rng.normal(size=(1, K)).astype(np.float16)
    cores = oracle.usable_cpus()
    oracle.c_set_threads(cores)
    total_bytes, total_s = 0, 0.0
    t_start = time.perf_counter()
    for w in W_BITS:
        lut = np.sort(rng.normal(0, 0.02, size=(N, 1 << w)).astype(np.float32), axis=1).astype(np.float16)
        oracle.c_matmul(x, q, lut, w)                       # warm
        reps = 0
        t0 = time.perf_counter()
        while True:
            oracle.c_matmul(x, q, lut, w)
            reps += 1
            dt = time.perf_counter() - t0
            if dt > seconds_hint / len(W_BITS) / 2 or reps >= 20:
                break
        total_bytes += gemv_bytes(1, N, K, w) * reps
        total_s += dt
        if time.perf_counter() - t_start > 2 * seconds_hint:
            break
    oracle.c_set_threads(min(8, cores))
    return {"value": round(total_bytes / total_s / 1e9, 3), "unit": UNIT, "cores": cores, "kind": "port",
            "sample": "one 4096x4096 layer, batch 1, w_bits 3..8, oracle C port (unpack + table gather + dot), OpenMP"}


def run_reference(args):
    """The reference arm: the reference's own CPU code path for this computation."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    import numpy as np
    import torch

    from oracle import oracle

    cores = oracle.usable_cpus()
    torch.set_num_threads(cores)
    oracle.c_set_threads(cores)
    use_ref = oracle.reflib() is not None
    N = K = 4096
    rng = np.random.default_rng(0)
    q = rng.integers(-2 ** 31, 2 ** 31, size=(8, N, K // 32), dtype=np.int64).astype(np.int32)
    x = torch.from_numpy(rng.normal(size=(1, K)).astype(np.float16)).float()
    luts = {w: np.sort(rng.normal(0, 0.02, size=(N, 1 << w)).astype(np.float32), axis=1).astype(np.float16)
            for w in W_BITS}
    bytes_per_step = sum(gemv_bytes(1, N, K, w) for w in W_BITS)

    def step():
        for w in W_BITS:
            Wd = oracle.ref_dequant(q, luts[w], w) if use_ref else oracle.c_dequant(q, luts[w], w)
            torch.matmul(x, torch.from_numpy(Wd).float().T)

    for _ in range(args.warmup):
        step()
    steps = args.steps
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = time.perf_counter() - t0
    value = bytes_per_step * steps / dt / 1e9
    kind = "reference" if use_ref else "port"
    sample = ("one 4096x4096 layer per step, batch 1, w_bits 3..8: " +
              ("reference dequant_kbit_store source compiled for the host (oracle/_ref)" if use_ref else "oracle C port") +
              " + fp32 torch.matmul")
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": round(dt / steps * 1e3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "llama2-7b linear-layer set, matmul_kbit M=1, w_bits 3..8 sweep (bounded sample: the "
                               "4096x4096 layer)", "batch": 1},
        "cpu_baseline": {"value": round(value, 3), "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": round(value, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--layers", type=int, default=4, help="decoder layers' worth of distinct weights per pass")
    ap.add_argument("--batch", type=int, default=1, help="activation rows M (1..8)")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
