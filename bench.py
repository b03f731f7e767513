#!/usr/bin/env python
"""Benchmark of the Metis NVFP4 linear-layer hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one forward + backward of ONE Metis linear layer (rank-r bf16 low-rank product + NVFP4
residual, mean-centred activations and gradients, stochastic-rounding backward: the GRPO default
configuration) on a fixed batch of synthetic tokens, through the public `BitLinear` module.
Workload: M = 16384 tokens, K = N = 4096, r = 128, bf16 -- the largest square shape of the GEMM
shape sweep with a low-rank term.  value = algorithmic TFLOP/s, (6 M N K + 6 M r (K+N)) / step time,
summed over all GPUs (token batch sharded, weights replicated; for N > 1 the weight gradients are
all-reduced with NCCL inside the step, as a data-parallel trainer would).

The JSON line also carries
  e2e          the same step through the same API with HOST inputs: pinned host -> device copies of
               x and grad_out (double-buffered, the next step's copy overlapping the current step)
               and a device -> host read of a checksum, every step, inside the timed region
  roofline     the tcgen05 GEMM kernel alone (CUDA events around back-to-back launches of the
               forward residual GEMM with its fused rank-r product) against 4 x the measured dense bf16
               rate, the dense NVFP4 : bf16 ratio of the part
  quant        the HBM-bound kernels alone: fused RMSNorm->NVFP4 and the plain quantizer at hidden
               4096 x 65536 tokens, algorithmic GB/s against the measured copy bandwidth
  cpu_baseline the same layer on this host's cores on a slice of the same workload: the reference's own
               BitLinear where oracle/build_ref.py has placed its modules in oracle/_ref ("reference"), else
               the restated oracle oracle/metis_layer.py ("port"); `config1` adds the baseline's first
               configuration (2048^3, rank 64, fp32), forward and backward, all threads and one thread
  value_cached_weights  the step with the opt-in packed-weight cache (the headline re-quantizes the weights
               every step, the reference's default)

`--impl reference` times that CPU implementation as the whole job (rank 0 only).
`--only gemm_yardstick` times the vendor library's block-scaled NVFP4 GEMM (torch._scaled_mm) at the
benchmark's shapes: what a library kernel reaches on the same box and clocks (never on the product path).
`--only gemm_sustained` runs both for seconds with clocks and power sampled; `--only gemm_accounting` (needs
the timing-knobs build) says where a GEMM tile's cycles go; `--only step_timeline` lists the kernels of one
graph replay of the step in start order.
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
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

M_TOKENS, HIDDEN_K, HIDDEN_N, RANK = 16384, 4096, 4096, 128
OVERLAP_SMS = 16                      # SMs (and NCCL CTAs) the GEMMs of the backward leave to the gradient all-reduce (N > 1)
QUANT_ROWS, QUANT_COLS = 65536, 4096
METRIC = "metis_nvfp4_linear_fwd_bwd_tflops"
BYTES_PER_ELEM_BF16 = 2.5625          # 2 (bf16 in) + 0.5 (codes) + 1/16 (E4M3 scale)
BYTES_PER_ELEM_DUAL_BF16 = 3.125      # one read, two packed outputs (row-major and transposed)
# DRAM bytes (read + write) of one forward GEMM launch, from an ncu capture of the same kernel on
# M = 8192 (31.6 MB read + 21.4 MB written) scaled by the rows processed; the profile summary
# profiles/nvfp4_gemm_pair_8192x4096x4096_r128.md holds the capture and its command.
GEMM_DRAM_BYTES_PER_LAUNCH = int(52.9e6 * M_TOKENS / 8192)      # 31.57 MB read + 21.36 MB written at M = 8192
GEMM_DRAM_SOURCE = ("ncu dram__bytes_read.sum + dram__bytes_write.sum at M = 8192, scaled by M; below the algorithmic bytes "
                    "because the part of the output still in L2 when the kernel ends is not counted")


def layer_flops(M, N, K, r):
    return 6 * M * N * K + 6 * M * r * (K + N)


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], bf16_sustained=d.get("bf16_tflops_sustained"),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_sustained=1400.0, source="fallback")


# ---- clocks during the timed region -----------------------------------------------------------------

class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                self.rows.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()          # the exact process started above
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        busy = [c for c in sm if c > 0.5 * max(mx, default=1)] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---- CPU arm ------------------------------------------------------------------------------------------------

def _cpu_factors(N, K, r, g):
    """A rank-r split without the (slow, one-time) exact SVD: random factors of the right scale."""
    import torch
    W = torch.randn(N, K, generator=g) / K ** 0.5
    U = torch.randn(N, r, generator=g) / N ** 0.5
    V = torch.randn(r, K, generator=g) / K ** 0.5
    s = torch.rand(r, generator=g) + 0.5
    return U, s, V, W - U @ torch.diag(s) @ V


def cpu_kind():
    """"reference": the reference's own BitLinear (oracle/_ref, placed there by oracle/build_ref.py where a
    checkout exists); "port": the restated oracle (oracle/metis_layer.py)."""
    from oracle import build_ref
    return "reference" if build_ref.available() else "port"


def cpu_layer_times(tokens, K, N, r, steps, warmup, threads, kind, outliers=True):
    """fwd and bwd of one Metis layer on the host for `tokens` tokens, fp32, mean mode, RTN forward and
    stochastic-rounding backward (the port rounds to nearest in the backward too); median seconds of
    the forward and of the backward."""
    import torch
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(1, tokens, K, generator=g)
    if outliers:
        x[..., torch.randperm(K, generator=g)[: max(1, K // 100)]] *= 20
    grad = torch.randn(1, tokens, N, generator=g)
    U, s, V, R = _cpu_factors(N, K, r, g)
    fwd, bwd = [], []
    if kind == "reference":
        from oracle import ref_layer
        layer = ref_layer.assemble(U, s, V, R)
        xin = x.requires_grad_(True)
        for i in range(warmup + steps):
            for p in layer.parameters():
                p.grad = None
            xin.grad = None
            t0 = time.perf_counter()
            y = layer(xin)
            t1 = time.perf_counter()
            y.backward(grad)
            t2 = time.perf_counter()
            if i >= warmup:
                fwd.append(t1 - t0); bwd.append(t2 - t1)
    else:
        from oracle import metis_layer as ML
        for i in range(warmup + steps):
            t0 = time.perf_counter()
            y, saved = ML.forward(x, U, s, V, R, None, threads=threads)
            t1 = time.perf_counter()
            ML.backward(grad, saved, U, s, has_bias=False, threads=threads)
            t2 = time.perf_counter()
            if i >= warmup:
                fwd.append(t1 - t0); bwd.append(t2 - t1)
    return statistics.median(fwd), statistics.median(bwd)


def cpu_c1_lines(kind, threads):
    """Configuration 1 of the baseline (x [2048 x 2048] fp32 with 1 % outlier channels, rank 64) on the
    host: forward and backward separately, all threads and one thread."""
    M = K = N = 2048
    r = 64
    f_fwd = 2 * M * N * K + 2 * M * r * (K + N)
    out = {"shape": "M=K=N=2048, rank 64, fp32", "kind": kind}
    for label, thr, steps, warm in (("all_threads", threads, 5, 2), ("one_thread", 1, 2, 1)):
        fwd, bwd = cpu_layer_times(M, K, N, r, steps, warm, thr, kind)
        out[label] = {"threads": thr, "fwd_ms": round(fwd * 1e3, 1), "bwd_ms": round(bwd * 1e3, 1),
                      "fwd_tflops": round(f_fwd / fwd / 1e12, 4), "bwd_tflops": round(2 * f_fwd / bwd / 1e12, 4),
                      "timed_steps": steps}
    return out


def run_reference_arm(args):
    """The CPU implementation of the path as the whole job: every step is forward + backward of the same
    layer on a sample of the token batch, sized from one probe step so that the run ends within about
    two minutes; ms_per_step is the time of what ran."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = len(os.sched_getaffinity(0))
    kind = cpu_kind()
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    probe_tokens = 1024
    f, b = cpu_layer_times(probe_tokens, HIDDEN_K, HIDDEN_N, RANK, 1, 1, threads, kind)
    per_token = (f + b) / probe_tokens
    tokens = M_TOKENS
    while tokens > probe_tokens and per_token * tokens * (steps + warmup) > 120.0:
        tokens //= 2
    fwd, bwd = cpu_layer_times(tokens, HIDDEN_K, HIDDEN_N, RANK, steps, warmup, threads, kind)
    sec = fwd + bwd
    tf = layer_flops(tokens, HIDDEN_N, HIDDEN_K, RANK) / sec / 1e12
    sample = (f"{tokens} of {M_TOKENS} tokens per step, same N, K, r, fp32 on {threads} host threads; "
              f"ms_per_step is the time of that sample")
    config = workload_config(1)
    config["sample_tokens_per_step"] = tokens
    config["parallelism"] = "one host process (the CPU arm does not shard)"
    line = {
        "impl": "reference", "metric": METRIC, "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4 (simulated in fp32)",
        "data": "synthetic", "config": config,
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": kind, "sample": sample,
                         "fwd_ms": fwd * 1e3, "bwd_ms": bwd * 1e3},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus, n_layers=1):
    what = "one Metis NVFP4 linear layer" if n_layers == 1 else f"{n_layers} stacked Metis NVFP4 linear layers"
    return {"workload": f"{what} fwd+bwd, M={M_TOKENS} tokens per GPU, K={HIDDEN_K}, N={HIDDEN_N}, "
                        f"rank {RANK}, bf16, mean mode, RTN forward / stochastic-rounding backward",
            "tokens_per_gpu": M_TOKENS, "in_features": HIDDEN_K, "out_features": HIDDEN_N, "rank": RANK,
            "parallelism": f"dp{n_gpus} (tokens sharded, weights replicated" + (", NCCL all-reduce of weight grads)" if n_gpus > 1 else ")"),
            "l2": "inputs larger than L2 (x and grad_out are 128 MiB each)"}


# ---- one kernel alone -----------------------------------------------------------------------------------------

GEMM_SWEEP = [(M, N, K) for (N, K) in ((4096, 4096), (14336, 4096), (4096, 14336)) for M in (16, 128, 4096, 16384)]


def run_gemm_sweep(args):
    """`--only gemm_sweep`: the GEMM shape grid (decode to training token counts, square and MLP shapes),
    each with and without the fused rank-128 product; one JSON line per shape."""
    import torch
    from fp4_post_b200 import ops
    from fp4_post_b200.graphs import GraphedStep
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    for M, N, K in GEMM_SWEEP:
        qa = ops.nvfp4_quantize(torch.randn(M, K, device=dev, dtype=torch.bfloat16))
        qb = ops.nvfp4_quantize(torch.randn(N, K, device=dev, dtype=torch.bfloat16) / K ** 0.5)
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        line = {"only": "gemm_sweep", "M": M, "N": N, "K": K}
        for rank in (0, args.rank):
            lr = None
            if rank:
                lr = (torch.randn(M, rank, device=dev, dtype=torch.bfloat16), torch.randn(N, rank, device=dev, dtype=torch.bfloat16))
            fn = lambda: ops.nvfp4_gemm(qa, qb, lowrank=lr, out=out)
            # `steps` launches replayed as one CUDA graph: the small shapes take less GPU time than
            # Python needs to issue them, so eager back-to-back calls would time the host
            def burst():
                for _ in range(args.steps):
                    fn()
            graphed = GraphedStep(burst, warmup=1)
            graphed()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graphed()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / args.steps
            del graphed
            key = f"r{rank}"
            line[key + "_us"] = round(ms * 1e3, 2)
            line[key + "_tflops"] = round(2 * M * N * (K + rank) / ms / 1e9, 1)
            # operand + output bytes: what a decode-sized product is bound by
            line[key + "_gbs"] = round((M * K * 0.5625 + N * K * 0.5625 + M * N * 2 + rank * (M + N) * 2) / ms / 1e6, 1)
        print(json.dumps(line), flush=True)


RMSNORM_SWEEP = [(tokens, hidden) for hidden in (1536, 3584, 4096) for tokens in (1024, 8192, 65536)]
# rollout-sized inputs: up to 32 rows take the one-launch cluster kernels, 33 and more the streaming ones
DECODE_QUANT_SWEEP = [(tokens, hidden) for hidden in (1536, 3584, 4096) for tokens in (1, 16, 32, 33, 128)]


def run_rmsnorm_sweep(args, shapes=None, tag="rmsnorm_sweep"):
    """`--only rmsnorm_sweep` (training token counts) and `--only decode_quant_sweep` (rollout sizes): the fused RMSNorm -> NVFP4 quantizer (and the plain row quantizer on the
    same input) over hidden x tokens; bf16 activations Student-t (nu = 3) plus a per-channel mean
    ~N(0, 2), gamma ~N(1, 0.1), eps 1e-6.  Algorithmic GB/s: 2.5625 bytes per element."""
    import torch
    from fp4_post_b200 import ops
    from fp4_post_b200.graphs import GraphedStep
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0)
    for tokens, hidden in (shapes or RMSNORM_SWEEP):
        z = torch.randn(tokens, hidden, device=dev, generator=g)
        chi = torch.randn(3, tokens, hidden, device=dev, generator=g).pow(2).sum(0)
        x = (z / (chi / 3).sqrt() + 2.0 * torch.randn(1, hidden, device=dev, generator=g)).to(torch.bfloat16)
        del z, chi
        gamma = (1.0 + 0.1 * torch.randn(hidden, device=dev, generator=g)).to(torch.bfloat16)
        line = {"only": tag, "tokens": tokens, "hidden": hidden}
        for name, fn in (("rmsnorm_quant", lambda: ops.rmsnorm_nvfp4_quantize(x, gamma, 1e-6)),
                         ("quant_rows", lambda: ops.nvfp4_quantize(x))):
            def burst():
                for _ in range(args.steps):
                    fn()
            graphed = GraphedStep(burst, warmup=1)
            graphed()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graphed()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / args.steps
            graphed.release()
            line[name + "_us"] = round(ms * 1e3, 2)
            line[name + "_gbs"] = round(tokens * hidden * BYTES_PER_ELEM_BF16 / ms / 1e6, 1)
        print(json.dumps(line), flush=True)


DECODE_LAYER_SWEEP = [(4096, 4096), (4096, 14336), (14336, 4096)]     # (K, N): attention and MLP projections


def run_decode_layer(args):
    """`--only decode_layer`: the rollout forward of one Metis layer (no_grad: shared activation
    quantizer, FP4 product with V, rank-r scale, FP4 residual product with the fused bf16 side
    product; weights from the packed cache) at 1-128 tokens, `steps` forwards replayed as one CUDA
    graph.  `weights_gbs`: packed weight bytes (R and V: 0.5625 B per element) over the time."""
    import torch
    import fp4_post_b200
    from fp4_post_b200.graphs import GraphedStep
    fp4_post_b200.install_reference_aliases()
    from Metis.Metis.bitlinear import BitLinear
    from grpo.grpo import MetisArgs
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    for K, N in DECODE_LAYER_SWEEP:
        margs = MetisArgs(forward_svd_rank=RANK, activation_lowrank_svd=RANK, backward_lowrank_svd=RANK, cache_quantized_weight=True)
        margs.device = dev
        layer = BitLinear(K, N, args=margs, bias=False, dtype=torch.bfloat16, compute_dtype=torch.bfloat16)
        with torch.no_grad():
            layer.warmup_linear.weight.copy_(torch.randn(N, K, device=dev) / K ** 0.5)
        layer.layer_name = f"decode.{K}x{N}"
        layer.split()
        for tokens in (1, 16, 32, 128):
            x = torch.randn(1, tokens, K, device=dev, dtype=torch.bfloat16)

            def burst():
                with torch.no_grad():
                    for _ in range(args.steps):
                        y = layer(x)
                return y
            graphed = GraphedStep(burst, warmup=2)
            graphed()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graphed()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / args.steps
            graphed.release()
            print(json.dumps({"only": "decode_layer", "tokens": tokens, "K": K, "N": N, "rank": RANK,
                              "forward_us": round(ms * 1e3, 2),
                              "weights_gbs": round((N * K + RANK * K) * 0.5625 / ms / 1e6, 1)}), flush=True)
        del layer


def run_decode_block(args):
    """`--only decode_block`: the rollout forward (no_grad, packed-weight cache) of ONE decoder block of the 7B
    configuration at 1-128 tokens, `steps` forwards replayed as one CUDA graph: the seven Metis projections with
    their fused norms, attention over the tokens of the call.  `grouped`: q/k/v and gate/up issued as parallel
    branches behind their shared quantization (forward_group) against one projection after the other."""
    import torch
    import fp4_post_b200
    from fp4_post_b200.graphs import GraphedStep
    fp4_post_b200.install_reference_aliases()
    from fp4_post_b200.decoder import Block, QWEN2_7B
    from Metis.Metis import bitlinear
    from grpo.grpo import MetisArgs, replace_linear_with_metis
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    cfg = QWEN2_7B
    blk = Block(cfg, fuse_norms=True).to(dev).to(torch.bfloat16)
    margs = MetisArgs(forward_svd_rank=RANK, activation_lowrank_svd=RANK, backward_lowrank_svd=RANK, cache_quantized_weight=True)
    margs.device = dev
    replace_linear_with_metis(blk, dtype=torch.bfloat16, metis_args=margs, compute_dtype=torch.bfloat16)
    for tokens in (1, 16, 32, 128):
        x = torch.randn(1, tokens, cfg.hidden, device=dev, dtype=torch.bfloat16)
        ang = torch.zeros(1, 1, tokens, cfg.head_dim, device=dev, dtype=torch.bfloat16)
        cos, sin = ang.cos(), ang.sin()
        out = {"only": "decode_block", "tokens": tokens, "hidden": cfg.hidden, "ffn": cfg.ffn, "rank": RANK}
        for grouped in (False, True):
            bitlinear.GROUP_BRANCHES = grouped

            def burst():
                with torch.no_grad():
                    for _ in range(args.steps):
                        y = blk(x, cos, sin)
                return y
            graphed = GraphedStep(burst, warmup=2)
            graphed()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graphed()
            e1.record()
            torch.cuda.synchronize()
            out["grouped_us" if grouped else "sequential_us"] = round(e0.elapsed_time(e1) / args.steps * 1e3, 2)
            graphed.release()
        bitlinear.GROUP_BRANCHES = True
        print(json.dumps(out), flush=True)


def run_gemm_yardstick(args):
    """`--only gemm_yardstick`: cuBLASLt's NVFP4 GEMM (e2m1 codes, E4M3 scales per 16 elements, through
    torch._scaled_mm) on random codes and unit scales; one JSON line per shape.  A yardstick for the
    tensor-core roofline on this box, not part of the library."""
    import torch
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    fp4, e4m3 = getattr(torch, "float4_e2m1fn_x2", None), torch.float8_e4m3fn
    for M, N, K in ((16384, 4096, 4096), (16384, 14336, 4096), (16384, 4096, 14336), (4096, 4096, 4096)):
        line = {"only": "gemm_yardstick", "M": M, "N": N, "K": K}
        try:
            if fp4 is None:
                raise RuntimeError("this torch has no float4_e2m1fn_x2")
            a = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, device=dev).view(fp4)
            b = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=dev).view(fp4)
            pad = lambda rows: (rows + 127) // 128 * 128
            sa = torch.ones(pad(M) * ((K // 16 + 3) // 4 * 4), device=dev).to(e4m3)
            sb = torch.ones(pad(N) * ((K // 16 + 3) // 4 * 4), device=dev).to(e4m3)
            fn = lambda: torch._scaled_mm(a, b.t(), sa, sb, out_dtype=torch.bfloat16)
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.steps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / args.steps
            line.update(ms_per_call=round(ms, 4), tflops=round(2 * M * N * K / ms / 1e9, 1))
        except Exception as exc:                      # the yardstick is optional: say why it is missing
            line["unavailable"] = f"{type(exc).__name__}: {str(exc)[:200]}"
        print(json.dumps(line), flush=True)


def _sustained(fn, name, index, seconds=2.5, burst=50):
    """Runs `fn` back to back for `seconds` (bursts captured in a CUDA graph) with the GPU's clocks and power
    sampled beside it; one dict with the time per call of a short burst and of the long run."""
    import torch
    from fp4_post_b200.graphs import GraphedStep

    def many():
        for _ in range(burst):
            fn()
    g = GraphedStep(many, warmup=1)
    g()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(); g(); e1.record()
    torch.cuda.synchronize()
    burst_ms = e0.elapsed_time(e1) / burst
    reps = max(3, int(seconds * 1e3 / (burst_ms * burst)))
    with ClockSampler(index) as clocks:
        time.sleep(0.3)
        clocks.rows.clear()                          # samples of the loaded GPU only
        e0.record()
        for _ in range(reps):
            g()
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / (reps * burst)
    rows = clocks.rows[2:] if len(clocks.rows) > 6 else clocks.rows
    power = [float(r[2]) for r in rows if r[2].replace(".", "", 1).isdigit()]
    g.release()
    time.sleep(1.0)
    return {"variant": name, "burst_us": round(burst_ms * 1e3, 2), "sustained_us": round(ms * 1e3, 2),
            "power_w_median": statistics.median(power) if power else None, "clocks": clocks.summary()}


def run_gemm_sustained(args):
    """`--only gemm_sustained`: the forward GEMM shape in a seconds-long loop, this library's kernel and the vendor
    library's block-scaled NVFP4 GEMM (torch._scaled_mm) on the SAME codes and scales, with SM clock and board
    power sampled during each loop.  Both run into the board's power limit; what differs is the clock they are
    left with and the cycles they need."""
    import torch
    from fp4_post_b200 import ops
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    M, N, K = args.rows, args.n, args.cols
    a = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=dev, dtype=torch.bfloat16) / K ** 0.5
    qa, qb = ops.nvfp4_quantize(a), ops.nvfp4_quantize(b)
    out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    lr = (torch.randn(M, args.rank, device=dev, dtype=torch.bfloat16), torch.randn(N, args.rank, device=dev, dtype=torch.bfloat16))
    lines = [_sustained(lambda: ops.nvfp4_gemm(qa, qb, out=out), "this library, no side product", 0),
             _sustained(lambda: ops.nvfp4_gemm(qa, qb, lowrank=lr, out=out), f"this library, rank-{args.rank} side product", 0)]
    fp4 = getattr(torch, "float4_e2m1fn_x2", None)
    if fp4 is not None:
        try:
            A, B = qa.codes.view(fp4), qb.codes.view(fp4)
            sa, sb = qa.scales.view(torch.float8_e4m3fn), qb.scales.view(torch.float8_e4m3fn)
            lines.append(_sustained(lambda: torch._scaled_mm(A, B.t(), sa, sb, out_dtype=torch.bfloat16),
                                    "vendor library (torch._scaled_mm), same codes and scales, no side product", 0))
        except Exception as exc:
            lines.append({"variant": "vendor library", "unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"})
    lines.append(_sustained(lambda: torch.matmul(a, b.t(), out=out), "torch.matmul bf16 (cuBLAS)", 0))
    for line in lines:
        line.update(only="gemm_sustained", M=M, N=N, K=K)
        if "sustained_us" in line:
            flops = 2 * M * N * (K + (args.rank if "rank-" in line["variant"] else 0))
            line["tflops_burst"] = round(flops / line["burst_us"] / 1e6, 1)
            line["tflops_sustained"] = round(flops / line["sustained_us"] / 1e6, 1)
        print(json.dumps(line), flush=True)


def run_gemm_accounting(args):
    """`--only gemm_accounting`: where the cycles of a 256 x 256 tile of the CTA-pair GEMM go.  Needs the build
    with the timing knobs (python -m fp4_post_b200.build --timing-knobs): parts of the kernel are switched off
    one at a time and the issuing warp of CTA 0 counts its own cycles (clock64) and nanoseconds (globaltimer).
    Two K per variant separate the cost per 256-element stage from the fixed cost per tile."""
    import torch
    from fp4_post_b200 import build as build_mod, cabi
    if not build_mod.KNOBS_LIB.exists():
        print(json.dumps({"only": "gemm_accounting", "unavailable": "build it first: python -m fp4_post_b200.build --timing-knobs"}))
        return
    cabi.LIB_PATH = build_mod.KNOBS_LIB
    from fp4_post_b200 import ops
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    M, N, rank = args.rows, args.n, 0
    NO_MMA, NO_LOAD, NO_EPILOGUE, NO_STORE, PROFILE, NO_SCALE_COPY = 2, 4, 16, 32, 128, 0x10000
    variants = (("everything", 0), ("no scale copies", NO_SCALE_COPY), ("no stores of D", NO_STORE), ("no epilogue arithmetic or stores", NO_EPILOGUE),
                ("no loads", NO_LOAD), ("no loads, no scale copies", NO_LOAD | NO_SCALE_COPY),
                ("MMAs only (no loads, scale copies, epilogue)", NO_LOAD | NO_SCALE_COPY | NO_EPILOGUE), ("loads only (no MMAs)", NO_MMA))
    results = {}
    for K in (4096, 8192):
        qa = ops.nvfp4_quantize(torch.randn(M, K, device=dev, dtype=torch.bfloat16))
        qb = ops.nvfp4_quantize(torch.randn(N, K, device=dev, dtype=torch.bfloat16) / K ** 0.5)
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        st = torch.zeros(8, dtype=torch.int32, device=dev)
        for name, bits in variants:
            for _ in range(3):
                ops.nvfp4_gemm(qa, qb, out=out, _debug=bits, status=st)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.steps):
                ops.nvfp4_gemm(qa, qb, out=out, _debug=bits | PROFILE, status=st)
            e1.record()
            torch.cuda.synchronize()
            w = st.tolist()
            cyc, ns, tiles = w[2], w[3], max(w[6], 1)
            results[(name, K)] = {"us_per_launch": round(e0.elapsed_time(e1) / args.steps * 1e3, 1), "sm_mhz_in_kernel": round(cyc / max(ns, 1) * 1e3),
                                  "kcycles_per_tile": round(cyc / tiles / 1e3, 2), "tiles_of_cta0": tiles}
    for name, _ in variants:
        lo, hi = results[(name, 4096)], results[(name, 8192)]
        per_stage = (hi["kcycles_per_tile"] - lo["kcycles_per_tile"]) * 1e3 / 16
        print(json.dumps({"only": "gemm_accounting", "M": M, "N": N, "variant": name, "K4096": lo, "K8192": hi,
                          "cycles_per_stage": round(per_stage), "fixed_kcycles_per_tile": round(lo["kcycles_per_tile"] - 16 * per_stage / 1e3, 2),
                          "note": "a stage is 4 MMAs of 256x256x64 per CTA pair: 512 tensor-pipe cycles"}), flush=True)


def run_step_timeline(args):
    """`--only step_timeline`: start, duration and name of every kernel of ONE graph replay of the default training
    step (torch profiler), in start order, and the time between the first start and the last end."""
    import torch
    from torch.profiler import profile, ProfilerActivity
    from fp4_post_b200.graphs import GraphedStep
    from fp4_post_b200.Metis.Metis.bitlinear import BitLinear
    from fp4_post_b200.grpo.grpo import MetisArgs
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    M, K, N, R = args.rows, args.cols, args.n, args.rank
    margs = MetisArgs(forward_svd_rank=R, activation_lowrank_svd=R, backward_lowrank_svd=R, cache_quantized_weight=False)
    margs.device = dev
    layer = BitLinear(K, N, args=margs, bias=False, dtype=torch.bfloat16, compute_dtype=torch.bfloat16)
    with torch.no_grad():
        layer.warmup_linear.weight.copy_(torch.randn(N, K, device=dev) / K ** 0.5)
    layer.layer_name = "p"
    layer.split()
    x = torch.randn(1, M, K, device=dev, dtype=torch.bfloat16).requires_grad_(True)
    g = torch.randn(1, M, N, device=dev, dtype=torch.bfloat16)
    params = list(layer.parameters())

    def step():
        for p in params:
            p.grad = None
        x.grad = None
        y = layer(x)
        y.backward(g)
        return y
    gs = GraphedStep(step, warmup=3)
    for _ in range(5):
        gs()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        gs()
    e1.record()
    torch.cuda.synchronize()
    print(json.dumps({"only": "step_timeline", "ms_per_step": e0.elapsed_time(e1) / args.steps}), flush=True)
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        gs(); gs()
        torch.cuda.synchronize()
    ev = sorted((e for e in prof.events() if e.device_type.name == "CUDA" and e.device_time > 0), key=lambda e: e.time_range.start)
    ev = ev[len(ev) // 2:]                            # the second replay
    t0 = ev[0].time_range.start
    print(f"{'start us':>9} {'dur us':>8}  kernel")
    for e in ev:
        print(f"{e.time_range.start - t0:9.1f} {e.device_time:8.1f}  {e.name[:100]}")
    print(f"span {max(e.time_range.end for e in ev) - t0:.1f} us, {len(ev)} kernels and memsets")
    gs.release()


def run_decoder_step(args):
    """`--only c4` / `--only c5_update`: one training step (forward, next-token loss, backward) of a Qwen2-style
    decoder with random weights whose seven projections per block are Metis rank-r NVFP4 layers, on synthetic
    token ids; data-parallel over the ranks of the job (tokens sharded, NCCL all-reduce of every gradient).
    c4: 1.5B shape, rank 64, batch 8 x 1024 per job.  c5_update: 7B shape, rank 128, 2 x 768 per GPU (a slice of
    the policy update of the rollout configuration).  One JSON line: tokens/s, the Metis layers' algorithmic
    TFLOP/s over the whole step time, and the share of device time spent in this library's kernels.
    The rank-r factors come from a randomized SVD instead of the exact one (196 exact SVDs take minutes):
    same shapes, same work per step."""
    import torch
    import torch.distributed as dist
    import fp4_post_b200
    from fp4_post_b200 import cabi, ops
    from fp4_post_b200.decoder import QWEN2_1P5B, QWEN2_7B, Decoder
    from fp4_post_b200.dp import GradientReducer, allreduce_gradients
    from fp4_post_b200.graphs import GraphedStep
    from fp4_post_b200.grpo.grpo import MetisArgs, replace_linear_with_metis
    from fp4_post_b200.Metis.Metis.bitlinear import BitLinear

    cabi.lib()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("NCCL_MAX_CTAS", str(OVERLAP_SMS))
        os.environ.setdefault("METIS_LAUNCH_OVERLAP", "0")
        dist.init_process_group("nccl", device_id=dev)
    if args.only == "c4":
        cfg, r, batch, seq = QWEN2_1P5B, 64, max(1, 8 // world), 1024
    else:
        cfg, r, batch, seq = QWEN2_7B, 128, 2, 768
    if args.layers > 1 or args.layers_set:
        cfg = type(cfg)(**{**cfg.__dict__, "layers": args.layers})          # a shallower stack for quick runs
    torch.manual_seed(0)
    with torch.device(dev):
        model = Decoder(cfg, fuse_norms=not args.no_fused_norm).to(torch.bfloat16)
    margs = MetisArgs(forward_svd_rank=r, activation_lowrank_svd=r, backward_lowrank_svd=r)
    margs.device = dev
    exact_svd = torch.linalg.svd

    def quick_svd(w, full_matrices=False):
        # randomized range finder, then the exact SVD of the small projected matrix
        omega = torch.randn(w.shape[1], r + 8, device=w.device, dtype=w.dtype)
        q, _ = torch.linalg.qr(w @ omega)
        ub, sv, vh = exact_svd(q.T @ w, full_matrices=False)
        return q @ ub, sv, vh
    torch.linalg.svd = quick_svd
    try:
        replace_linear_with_metis(model, dtype=torch.bfloat16, metis_args=margs, compute_dtype=torch.bfloat16)
    finally:
        torch.linalg.svd = exact_svd
    params = list(model.parameters())
    metis_params = {id(p) for m in model.modules() if isinstance(m, BitLinear) for p in m.parameters()}
    other = [p for p in params if id(p) not in metis_params]
    g = torch.Generator(device=dev).manual_seed(1 + rank)
    ids = torch.randint(0, cfg.vocab, (batch, seq), device=dev, generator=g)
    if world > 1:
        GradientReducer(overlap_sms=OVERLAP_SMS, across_layers=True).attach()

    def step():
        for p in params:
            p.grad = None
        loss = model.loss(ids)
        loss.backward()
        if world > 1:
            allreduce_gradients(other)              # norms, embedding, lm_head: what the fused backward does not see
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(2):
        step()
    barrier()
    mode = "eager"
    runner = step
    if not args.no_graph:
        try:
            runner = GraphedStep(step, warmup=1)
            runner()
            mode = "one CUDA graph per step"
        except Exception as exc:                    # capture is an optimisation: say why it was not taken
            mode = f"eager (capture failed: {type(exc).__name__}: {str(exc)[:120]})"
            runner = step
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        runner()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    # share of device time in this library's kernels: one profiled eager step
    share = None
    if rank == 0:
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            step()
            torch.cuda.synchronize()
        ours = sum(e.device_time_total for e in prof.key_averages() if e.key.startswith(("void metis::", "metis::")))
        total = sum(e.device_time_total for e in prof.key_averages())
        share = ours / max(total, 1e-9)
        top = sorted(prof.key_averages(), key=lambda e: -e.device_time_total)[:14]
        top_kernels = [{"kernel": e.key[:70], "launches": e.count, "ms": round(e.device_time_total / 1e3, 2)} for e in top]
    if rank == 0:
        tokens = world * batch * seq
        lin = 3 * cfg.linear_flops_per_token(r) * tokens
        print(json.dumps({"only": args.only, "n_gpus": world, "tokens_per_step": tokens, "batch_per_gpu": batch, "seq_len": seq,
                          "layers": cfg.layers, "hidden": cfg.hidden, "rank": r, "ms_per_step": ms,
                          "tokens_per_s": tokens / ms * 1e3, "metis_linear_tflops": lin / ms / 1e9,
                          "share_of_device_time_in_library_kernels": share, "device_ms_of_one_eager_step": round(total / 1e3, 1),
                          "top_kernels_of_one_eager_step": top_kernels, "launch_mode": mode,
                          "fused_norms": not args.no_fused_norm, "data": "synthetic token ids, random weights"}), flush=True)
    if world > 1:
        if isinstance(runner, GraphedStep):
            runner.release()
        torch.cuda.synchronize()
        dist.destroy_process_group()


def run_single_kernel(args):
    """`--only K`: a few launches of one kernel on [rows, cols] bf16 (GEMM: M = rows, K = cols, N = n),
    timed with CUDA events.  Small enough to sit under an ncu capture."""
    import torch
    from fp4_post_b200 import ops
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    rows, cols = args.rows, args.cols
    x = torch.randn(rows, cols, device=dev, dtype=torch.bfloat16)
    if args.only == "gemm":
        w = torch.randn(args.n, cols, device=dev, dtype=torch.bfloat16) / cols ** 0.5
        qa, qb = ops.nvfp4_quantize(x), ops.nvfp4_quantize(w)
        lr = None
        if args.rank:
            lr = (torch.randn(rows, args.rank, device=dev, dtype=torch.bfloat16),
                  torch.randn(args.n, args.rank, device=dev, dtype=torch.bfloat16))
        out = torch.empty(rows, args.n, device=dev, dtype=torch.bfloat16)
        fn = lambda: ops.nvfp4_gemm(qa, qb, lowrank=lr, out=out)
        work, unit = 2 * rows * args.n * (cols + args.rank) / 1e12, "TFLOP/s"
    else:
        gamma = torch.ones(cols, device=dev, dtype=torch.bfloat16)
        x_mean = ops.col_mean(x)
        fn = {"quant_rows": lambda: ops.nvfp4_quantize(x),
              "quant_transposed": lambda: ops.nvfp4_quantize(x, transpose=True),
              "quant_dual": lambda: ops.nvfp4_quantize_dual(x),
              "quant_dual_sr": lambda: ops.nvfp4_quantize_dual(x, stochastic=True, seed=1, offset=1, mean=x_mean),
              # the form the output gradient takes in the training step: the token sums of the transposed output too
              "quant_dual_sr_sums": lambda: ops.nvfp4_quantize_dual(x, stochastic=True, seed=1, offset=1, mean=x_mean, token_sums=True),
              "rmsnorm_quant": lambda: ops.rmsnorm_nvfp4_quantize(x, gamma, 1e-6)}[args.only]
        work, unit = rows * cols * (BYTES_PER_ELEM_DUAL_BF16 if args.only.startswith("quant_dual") else BYTES_PER_ELEM_BF16) / 1e9, "GB/s"
    for _ in range(max(1, args.warmup)):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    print(json.dumps({"only": args.only, "rows": rows, "cols": cols, "n": args.n, "rank": args.rank,
                      "ms_per_call": ms, "value": work / (ms / 1e3), "unit": unit}), flush=True)


# ---- GPU arm ------------------------------------------------------------------------------------------------

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--only", default=None, choices=["quant_rows", "quant_transposed", "quant_dual", "quant_dual_sr", "quant_dual_sr_sums", "rmsnorm_quant", "gemm", "gemm_sweep", "gemm_yardstick", "gemm_sustained", "gemm_accounting", "step_timeline", "rmsnorm_sweep", "decode_quant_sweep", "decode_layer", "decode_block", "c4", "c5_update"],
                    help="time one kernel alone on a small case (the command used for ncu captures)")
    ap.add_argument("--layers", type=int, default=1,
                    help="stack this many Metis layers (the headline is 1): with several GPUs the gradient all-reduce "
                         "of layer k then runs beside the backward of layer k-1")
    ap.add_argument("--no-graph", action="store_true", help="decoder steps: issue from Python instead of one CUDA graph")
    ap.add_argument("--no-fused-norm", action="store_true", help="decoder steps: plain RMSNorm modules instead of the fused norm -> quantizer entry")
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--cols", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--rank", type=int, default=128)
    args = ap.parse_args()
    args.layers_set = "--layers" in sys.argv
    if args.only in ("c4", "c5_update"):
        return run_decoder_step(args)
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.only == "gemm_sweep":
        return run_gemm_sweep(args)
    if args.only == "gemm_yardstick":
        return run_gemm_yardstick(args)
    if args.only == "gemm_sustained":
        return run_gemm_sustained(args)
    if args.only == "gemm_accounting":
        return run_gemm_accounting(args)
    if args.only == "step_timeline":
        return run_step_timeline(args)
    if args.only == "rmsnorm_sweep":
        return run_rmsnorm_sweep(args)
    if args.only == "decode_block":
        return run_decode_block(args)
    if args.only == "decode_layer":
        return run_decode_layer(args)
    if args.only == "decode_quant_sweep":
        return run_rmsnorm_sweep(args, DECODE_QUANT_SWEEP, "decode_quant_sweep")
    if args.only:
        return run_single_kernel(args)

    import torch
    import torch.distributed as dist
    import fp4_post_b200
    from fp4_post_b200 import cabi, ops
    from fp4_post_b200.dp import GradientReducer
    from fp4_post_b200.graphs import GraphedStep
    from fp4_post_b200.Metis.Metis.bitlinear import BitLinear
    from fp4_post_b200.grpo.grpo import MetisArgs

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the NVFP4 path has no CPU fallback "
                         "(use --impl reference for the CPU arm)")
    cabi.lib()                                     # fail loudly if the library is not built
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("NCCL_MAX_CTAS", str(OVERLAP_SMS))       # the collective fits beside the capped GEMM
        # plain launches beside captured collectives: the configuration the multi-GPU numbers were taken in
        # (programmatic serialization changes nothing for the training step on one GPU)
        os.environ.setdefault("METIS_LAUNCH_OVERLAP", "0")
        dist.init_process_group("nccl", device_id=dev)
    warmup = max(3, args.warmup)
    peaks = measured_peaks()

    # ---- the layer ----------------------------------------------------------------------------------------------
    torch.manual_seed(0)
    # The reference's default flags (src/grpo/grpo.py:62-103): the packed-weight cache is OFF, so every step
    # quantizes R and V again (row-major for the forward, transposed for the input gradient), as a training
    # loop whose optimizer changes the weights every step has to.
    margs = MetisArgs(forward_svd_rank=RANK, activation_lowrank_svd=RANK, backward_lowrank_svd=RANK,
                      cache_quantized_weight=False)
    margs.device = dev
    n_layers = max(1, args.layers)
    layers = []
    for i in range(n_layers):
        lyr = BitLinear(HIDDEN_K, HIDDEN_N, args=margs, bias=False, dtype=torch.bfloat16, compute_dtype=torch.bfloat16)
        with torch.no_grad():
            lyr.warmup_linear.weight.copy_(torch.randn(HIDDEN_N, HIDDEN_K, device=dev) / HIDDEN_K ** 0.5)
        lyr.layer_name = f"bench.layer{i}"
        lyr.split()                                # exact SVD once, outside the timed region
        layers.append(lyr)
    layer = layers[0]
    params = [p for lyr in layers for p in lyr.parameters()]

    g = torch.Generator(device="cpu").manual_seed(1 + rank)
    x_host = torch.randn(1, M_TOKENS, HIDDEN_K, generator=g).to(torch.bfloat16)
    x_host[..., torch.randperm(HIDDEN_K, generator=g)[: HIDDEN_K // 100]] *= 20      # 1 % outlier channels
    g_host = torch.randn(1, M_TOKENS, HIDDEN_N, generator=g).to(torch.bfloat16)
    x_host, g_host = x_host.pin_memory(), g_host.pin_memory()
    x_dev = x_host.to(dev).requires_grad_(True)
    g_dev = g_host.to(dev)
    flops = n_layers * layer_flops(M_TOKENS, HIDDEN_N, HIDDEN_K, RANK)

    def step(x, grad):
        for p in params:
            p.grad = None
        x.grad = None
        y = x
        for lyr in layers:
            y = lyr(y)
        y.backward(grad)
        return y

    if world > 1:
        # What DDP does for this layer, started inside the backward pass: the all-reduce of the residual
        # weight's gradient begins when that gradient exists and runs beside the input-gradient GEMM
        # (and, with several layers, beside the backward of the layers below), which leave it OVERLAP_SMS
        # SMs; the wait is at the end of the backward pass; the collectives are captured with the step.
        GradientReducer(overlap_sms=OVERLAP_SMS, across_layers=True).attach()
    graphs = []                                    # released before the process group is destroyed

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        """n calls between events on the current stream; ms per call, max over ranks."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1) / n
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    with ClockSampler(local) as clocks:
        time.sleep(0.3)                            # let the sampler start before the GPU gets busy
        for _ in range(warmup):
            step(x_dev, g_dev)
        # The timed step is one CUDA-graph launch: the ~35 kernels and the torch ops between them are
        # captured once (fp4_post_b200/graphs.py) instead of being issued from Python every step.
        def eager_step():
            step(x_dev, g_dev)
        ms_eager = timed(eager_step, max(3, args.steps // 5))                        # the same step issued from Python
        launches0 = ops.launch_count()
        graphed = GraphedStep(lambda: step(x_dev, g_dev), warmup=1)
        launches_per_step = (ops.launch_count() - launches0) // 2          # one warm-up run + the capture
        graphs.append(graphed)
        for _ in range(3):
            graphed()
        ms_step = timed(graphed, args.steps)
        launches = launches_per_step * args.steps

        # the same step with the opt-in packed-weight cache (weights that do not change between steps:
        # evaluation, rollout, frozen layers): their four quantizations leave the step
        def set_weight_cache(on):
            for lyr in layers:
                for m in (lyr.warmup_linear, lyr.vlinear):
                    m.cache_quantized_weight = on
                    m._quantized_weight_cache = None
        set_weight_cache(True)
        for _ in range(2):
            step(x_dev, g_dev)
        cached = GraphedStep(lambda: step(x_dev, g_dev), warmup=1, pool=graphed.pool())
        graphs.append(cached)
        cached()
        ms_cached = timed(cached, max(3, args.steps // 2))
        set_weight_cache(False)
        # N > 1: the same step without the gradient all-reduce; the difference is what the collective costs the step
        ms_local = None
        if world > 1:
            GradientReducer.detach()
            for _ in range(2):
                step(x_dev, g_dev)
            local_graph = GraphedStep(lambda: step(x_dev, g_dev), warmup=1, pool=graphed.pool())
            graphs.append(local_graph)
            local_graph()
            ms_local = timed(local_graph, max(3, args.steps // 2))
            GradientReducer(overlap_sms=OVERLAP_SMS, across_layers=True).attach()
        # and in the mode whose gradients meet the 1e-3 bar against the reference's own (the reference's
        # wiring: native quantizers, dequantized operands, torch.matmul), issued from Python
        ms_dense = None
        if world == 1:
            from fp4_post_b200.Metis.Metis.bitlinear import LinearLowbitFunction
            LinearLowbitFunction.gemm_mode = "dense"
            try:
                for _ in range(2):
                    step(x_dev, g_dev)
                ms_dense = timed(eager_step, 3)
            finally:
                LinearLowbitFunction.gemm_mode = "packed"

        # ---- end to end: host inputs, checksum back -------------------------------------------------------------
        # Inputs arrive the way a training input pipeline delivers them: two device buffers, the copy
        # of step k+1 on a side stream while step k computes.  The timed region starts with nothing in
        # flight and contains exactly one host -> device copy of x and grad_out per step (the first
        # one exposed, the others overlapped) and one device -> host checksum read per step.
        copy_stream = torch.cuda.Stream(device=dev)
        bufs = [(torch.empty_like(x_dev).requires_grad_(True), torch.empty_like(g_dev)) for _ in range(2)]
        ready = [torch.cuda.Event() for _ in range(2)]
        consumed = [torch.cuda.Event() for _ in range(2)]

        def issue_copy(i):
            with torch.cuda.stream(copy_stream), torch.no_grad():
                copy_stream.wait_event(consumed[i])          # the step that last read this buffer is done
                bufs[i][0].copy_(x_host, non_blocking=True)
                bufs[i][1].copy_(g_host, non_blocking=True)
                ready[i].record(copy_stream)

        def checked_step(i):
            y = step(*bufs[i])
            return y.float().abs().mean() + bufs[i][0].grad.float().abs().mean()

        e2e_graphs = [GraphedStep(lambda i=i: checked_step(i), warmup=1, pool=graphed.pool()) for i in range(2)]
        graphs.extend(e2e_graphs)

        def e2e_run(n):
            main = torch.cuda.current_stream()
            total = 0.0
            issue_copy(0)
            for k in range(n):
                i = k & 1
                if k + 1 < n:
                    issue_copy(1 - i)
                main.wait_event(ready[i])
                check = e2e_graphs[i]()
                consumed[i].record(main)
                total += float(check.item())
            return total

        for i in range(2):
            consumed[i].record(torch.cuda.current_stream())
        e2e_run(2)
        n_e2e = max(3, args.steps // 2)
        ms_e2e = timed(lambda: e2e_run(n_e2e), 1) / n_e2e

        # ---- kernel-level lines (rank 0's GPU; every rank runs them so that nobody idles) ----------------------
        shared = layer._get_shared_quantized_input(x_dev.detach())
        rq = layer.warmup_linear._get_quantized_weight(layer.warmup_linear.weight)
        t_acc = torch.randn(M_TOKENS, RANK, device=dev, dtype=torch.bfloat16)
        u16 = layer.ulinear.weight.detach().to(torch.bfloat16)
        out = torch.empty(M_TOKENS, HIDDEN_N, device=dev, dtype=torch.bfloat16)
        gemm = lambda: ops.nvfp4_gemm(shared.q, rq.q, lowrank=(t_acc, u16), out=out)
        def burst_ms(fn, n):
            """average device time of one call: n calls captured into one CUDA graph (a kernel that runs
            for 0.1 ms would otherwise be timed together with the gap Python leaves between launches)"""
            def burst():
                for _ in range(n):
                    fn()
            g = GraphedStep(burst, warmup=1, pool=graphed.pool())
            g()
            ms = timed(g, 3) / n
            g.release()
            return ms

        ms_gemm = burst_ms(gemm, 20)
        gemm_flops = 2 * M_TOKENS * HIDDEN_N * HIDDEN_K + 2 * M_TOKENS * HIDDEN_N * RANK

        xq = torch.randn(QUANT_ROWS, QUANT_COLS, device=dev, dtype=torch.bfloat16)
        gamma = torch.ones(QUANT_COLS, device=dev, dtype=torch.bfloat16)
        quant_lines = {}
        for name, fn in (("rmsnorm_quant", lambda: ops.rmsnorm_nvfp4_quantize(xq, gamma, 1e-6)),
                         ("quant_rows", lambda: ops.nvfp4_quantize(xq)),
                         ("quant_transposed", lambda: ops.nvfp4_quantize(xq, transpose=True)),
                         ("quant_dual", lambda: ops.nvfp4_quantize_dual(xq))):
            ms = burst_ms(fn, 10)
            gbs = QUANT_ROWS * QUANT_COLS * (BYTES_PER_ELEM_DUAL_BF16 if name == "quant_dual" else BYTES_PER_ELEM_BF16) / ms / 1e6
            quant_lines[name] = {"gbs": round(gbs, 1), "ms": round(ms, 4), "frac_of_hbm_copy": round(gbs / peaks["hbm_gbs"], 4)}
        del xq
    clock_summary = clocks.summary()

    # ---- CPU baseline on this host's cores (rank 0, N = 1 only) ----------------------------------------------
    cpu = None
    if rank == 0 and world == 1:
        threads = len(os.sched_getaffinity(0))
        tokens, kind = 2048, cpu_kind()
        fwd, bwd = cpu_layer_times(tokens, HIDDEN_K, HIDDEN_N, RANK, steps=2, warmup=1, threads=threads, kind=kind)
        cpu = {"value": layer_flops(tokens, HIDDEN_N, HIDDEN_K, RANK) / (fwd + bwd) / 1e12, "unit": "TFLOP/s", "cores": threads,
               "kind": kind, "sample": f"{tokens} of {M_TOKENS} tokens, same N, K, r, fp32, 2 timed steps after 1 warm-up",
               "config1": cpu_c1_lines(kind, threads)}

    grad_bytes = sum(p.numel() * p.element_size() for p in params)
    if rank == 0:
        fp4_peak = 4.0 * peaks["bf16_tflops"]
        achieved = gemm_flops / ms_gemm / 1e9
        line = {
            "metric": METRIC, "value": world * flops / ms_step / 1e9, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3, fp32 accumulate) + bf16 rank-r",
            "data": "synthetic", "config": workload_config(world, n_layers),
            "e2e": {"value": world * flops / ms_e2e / 1e9, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": x_host.numel() * 2 + g_host.numel() * 2, "d2h_bytes_per_step": 8,
                    "ms_per_step": ms_e2e},
            "value_cached_weights": world * flops / ms_cached / 1e9, "ms_per_step_cached_weights": ms_cached,
            "gemm_mode": {"timed": "packed: FP4 operands on the tensor-core GEMM; dX and dW contract over operands re-quantized along "
                                   "N and along tokens (same expectation as the reference's gradients, rel-L2 up to 0.25 from them; "
                                   "tests/test_layer_gpu.py)",
                          "dense_ms_per_step": ms_dense,
                          "dense": "reference wiring (fake-quantized operands, torch.matmul): gradients within 1e-3 of the reference's"},
            "allreduce": None if ms_local is None else {
                "ms_per_step_without": ms_local, "exposed_ms": ms_step - ms_local, "bytes_per_step": grad_bytes,
                "bus_gbs_if_fully_exposed": 2 * (world - 1) / world * grad_bytes / max(ms_step - ms_local, 1e-6) / 1e6,
                "dtype": "gradients travel in the parameters' dtype (bf16)"},
            "gpu_launches": launches, "launch_mode": "one CUDA graph per step" + (" (NCCL all-reduce of the weight gradients captured inside)" if world > 1 else ""), "ms_per_step_eager": ms_eager,
            "clocks": clock_summary,
            "roofline": {"bound": "tensor", "kernel": "nvfp4_gemm_pair_kernel (CTA pairs, 256x256 tiles) forward residual GEMM + fused rank-128 product",
                         "achieved": achieved, "peak": fp4_peak, "unit": "TFLOP/s", "frac": achieved / fp4_peak,
                         "traffic": GEMM_DRAM_BYTES_PER_LAUNCH, "traffic_source": GEMM_DRAM_SOURCE, "peak_source": f"4 x {peaks['source']} dense bf16 burst ({peaks['bf16_tflops']} TFLOP/s)",
                         "frac_of_nominal_9000": achieved / 9000.0, "ms_per_launch": ms_gemm,
                         "step_frac": flops / ms_step / 1e9 / fp4_peak, "step_frac_of_nominal_9000": flops / ms_step / 1e9 / 9000.0,
                         "hbm_kernels": quant_lines, "hbm_peak_gbs": peaks["hbm_gbs"]},
            "quant": quant_lines,
            "hbm_peak_gbs": peaks["hbm_gbs"],
            "cpu_baseline": cpu,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        for g in graphs:                           # graphs that hold captured NCCL kernels go first
            g.release()
        torch.cuda.synchronize()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
