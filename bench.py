#!/usr/bin/env python
"""Benchmark of the NVFP4 linear path on B200.

A step is one pass over the four linears of a Wan2.2-TI2V-5B-shaped DiT block
at M = 27280 tokens (QKV 3072->9216, attention-out 3072->3072, FFN-up
3072->14336 with fused GELU-tanh, FFN-down 14336->3072): for every linear the
bf16 activation is quantized to NVFP4 (tensor amax + pack) and multiplied with
the pre-quantized weight on the tcgen05 tensor cores.  Inputs are seeded
synthetic tensors of the named shapes (Student-t(4)*0.5 activations, N(0,0.02^2)
weights with 0.1% x20 outliers).

    python bench.py --gpus N --steps K --warmup W          # this library
    python bench.py --impl reference ...                   # CPU restatement of the reference path

Prints one JSON line (rank 0).  With N > 1 (under torchrun) every rank runs the
block linears on its own token shard -- they need no collective -- and the value
is the whole-job aggregate over the slowest rank's device time.  The same line
carries ``dit_step``: one denoising step of the Wan2.2-A14B-shaped DiT (40 blocks,
32760 tokens) on the N GPUs, token-sharded with the head/sequence exchange around
self-attention -- the one part of the workload that communicates.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CONFIG_NAME = "wan2.2-ti2v-5b block linears, M=27280 (qkv, attn_out, ffn_up+gelu, ffn_down)"
FP4_TO_BF16_PEAK_RATIO = 4.0  # nominal dense peaks 9 PFLOP/s (FP4) : 2.25 PFLOP/s (bf16)
SUSTAINED_SECONDS = 2.0


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"],
                    bf16_tflops_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0,
                source="fallback")


def profiled_gemm_traffic():
    """DRAM bytes per launch and the algorithmic bytes of the same launch, from the committed
    ncu summary of the GEMM kernel (a line `traffic_bytes_per_launch: X algorithmic_bytes: Y`)."""
    path = os.path.join(ROOT, "profiles", "nvfp4_gemm_kernel_8192x9216x3072.md")
    try:
        m = re.search(r"traffic_bytes_per_launch:\s*([0-9.eE+]+)\s+algorithmic_bytes:\s*([0-9.eE+]+)",
                      open(path).read())
        return (float(m.group(1)), float(m.group(2)), os.path.relpath(path, ROOT)) if m else None
    except OSError:
        return None


class ClockSampler:
    """Samples SM clock, power and throttle reasons through NVML (read-only) while running."""

    def __init__(self, index: int, period_s: float = 0.005):
        self.index, self.period = index, period_s
        self.samples, self.power, self.reasons = [], [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nvml = None

    def _run(self):
        n = self.nvml
        names = {
            getattr(n, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(n, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(n, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(n, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                try:
                    self.power.append(n.nvmlDeviceGetPowerUsage(self.handle) / 1000.0)
                except Exception:
                    pass
                try:
                    mask = n.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                except Exception:
                    mask = n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self.nvml is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable"]}
        out = {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
               "reasons": sorted(self.reasons), "samples": len(self.samples),
               "sm_mhz_min": min(self.samples)}
        if self.power:
            out["power_w_median"] = round(statistics.median(self.power), 1)
        return out


def bind_to_gpu_numa_node(index: int):
    """Run this process on the CPUs NVML names as closest to GPU `index`, so that the pinned
    staging buffers allocated afterwards sit on that GPU's NUMA node.  Changes only this
    process's own CPU affinity; returns a short description for the report."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        cpus = {64 * i + b for i, w in enumerate(mask) for b in range(64) if (w >> b) & 1}
        cpus &= set(os.sched_getaffinity(0))
        if cpus and len(cpus) < len(os.sched_getaffinity(0)):
            os.sched_setaffinity(0, cpus)
            return f"{len(cpus)} CPUs nearest GPU {index}"
        return "all CPUs are equally near (one NUMA node)"
    except Exception as e:  # NVML or affinity calls unavailable: report, do not fail
        return f"not bound ({type(e).__name__})"


# ------------------------------------------------------------ CPU reference --

def cpu_baseline_report(full: bool):
    """The CPU baseline legs (oracle/cpu_baseline.py): the block linears at M = 4096 tokens with
    the weights quantized once and with the weights re-quantized every forward as the reference
    does, and -- when `full` -- the single-linear configuration in full and the reference's
    literal per-element loop on a 256 x 3072 slice.  Returns (object for the JSON line, runner)."""
    from oracle import cpu_baseline as B
    threads = B.use_all_cores()
    bl = B.BlockLinearsM4096(4096)
    prep = bl.prepare_weights()
    bl.run(False)                                   # warm-up
    t_once = min(bl.run(False) for _ in range(2))
    t_requant = bl.run(True)
    sample = ("M = 4096 of 27280 tokens through all four linears (quantize + dequantize the "
              "activation, fp32 matmul on all cores, bias/GELU, bf16), weights quantized once "
              "outside the timed call; TFLOP/s is a rate, so it stands for the full M unscaled")
    obj = {"value": bl.flops / t_once / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
           "sample": sample, "threads_used": threads, "ms_per_pass_m4096": t_once * 1e3,
           "extrapolated_ms_m27280": t_once * 1e3 * 27280 / 4096,
           "weights_requantized_every_forward": {
               "value": bl.flops / t_requant / 1e12, "unit": "TFLOP/s",
               "ms_per_pass_m4096": t_requant * 1e3,
               "note": "as the reference does on every forward (nvfp4_linear.cpp:123-152)"},
           "weight_quantization_once_ms": prep * 1e3}
    if full:
        obj["config1_single_linear_full"] = B.config1_full()
        obj["reference_literal_path"] = B.literal_slice(256, 3072)
    return obj, bl


def run_reference(args, rank: int):
    if rank != 0:
        return
    # the launcher may have exported OMP_NUM_THREADS=1: the thread counts are set explicitly
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    obj, bl = cpu_baseline_report(full=False)
    for _ in range(max(1, min(args.warmup, 2))):
        bl.run(False)
    times = [bl.run(False) for _ in range(args.steps)]
    t = sum(times) / len(times)
    value = bl.flops / t / 1e12
    obj["value"] = value
    line = {
        "impl": "reference", "metric": "NVFP4 GEMM TFLOPS", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp4_e2m1", "data": "synthetic",
        "config": {"workload": CONFIG_NAME, "sample": obj["sample"]},
        "threads_used": obj["threads_used"],
        "cpu_baseline": obj,
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "native_library_loaded": "blackwell_diffusion_rtx6000_5090_i2v_b200._native" in sys.modules,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------- DiT step leg --

def dit_step_report(world: int, rank: int, local_rank: int, steps: int = 3):
    """One denoising step of the Wan2.2-A14B-shaped DiT (40 blocks, 32760 tokens, text 512 x 4096)
    on the `world` GPUs: unsharded on one GPU, token-sharded with the peer-store head/sequence
    exchange on several.  CUDA-event latency (max over ranks), rank 0's per-component device time,
    bytes each rank sends per step and, on several GPUs, the same box's single-GPU step for the
    strong-scaling ratio."""
    import torch
    import torch.distributed as dist
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import dit, nvfp4, ulysses

    cfg = dit.WAN22_A14B
    C, Fr, H, W = 16, 21, 60, 104
    tokens = Fr * (H // 2) * (W // 2)
    group = dist.group.WORLD if world > 1 else None
    model = dit.WanDiT(cfg, device=f"cuda:{local_rank}", seed=1238)
    g = torch.Generator(device="cuda").manual_seed(4321)
    latent = torch.randn(C, Fr, H, W, generator=g, device="cuda").to(torch.bfloat16)
    text = torch.randn(512, cfg.text_dim, generator=g, device="cuda").to(torch.bfloat16)

    def fence():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        out = []
        for _ in range(n):
            fence()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            fence()
            t = torch.tensor([e0.elapsed_time(e1)], device="cuda")
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            out.append(float(t))
        return out

    def step():
        return model.forward(latent, 500.0, text, group=group, exchange="peer")

    with torch.no_grad():
        step()                                            # warm-up: tables, exchange buffers
        nvfp4.check_status()                              # a rank that never showed up ends the leg here
        times = timed(step, steps)
        nvfp4.check_status()
        dit.TIMELINE = dit.Timeline()
        dit.TIMELINE.mark("start")
        step()
        dit.TIMELINE.mark("other")
        parts = dit.TIMELINE.totals_ms()
        dit.TIMELINE = None
        n1_ms = None
        if world > 1:
            fence()
            if rank == 0:                                 # the same box's single-GPU step
                single = lambda: model.forward(latent, 500.0, text)   # noqa: E731
                single()
                ts = []
                for _ in range(2):
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    single()
                    e1.record()
                    torch.cuda.synchronize()
                    ts.append(e0.elapsed_time(e1))
                n1_ms = min(ts)
            fence()
    ms = statistics.median(times)
    gemm_ms = sum(v for k, v in parts.items() if k.startswith("gemm")) + parts.get("text_kv", 0.0)
    sent = ulysses.exchange_bytes_per_rank(tokens, cfg.heads, cfg.head_dim, world) * len(model.blocks) \
        if world > 1 else 0
    report = {
        "workload": f"wan2.2 a14b shape, {len(model.blocks)} blocks, {tokens} tokens, text 512x{cfg.text_dim}, "
                    "all linears NVFP4, bf16 attention (torch SDPA), random init, seeded inputs",
        "n_gpus": world, "tokens_per_rank": tokens // world,
        "parallelism": f"ulysses x{world} (tokens sharded, weights replicated)" if world > 1 else "single GPU",
        "exchange": "peer stores + flag waits (no collective in the block)" if world > 1 else None,
        "ms_per_step": round(ms, 3), "all_ms": [round(t, 3) for t in times], "steps": steps, "warmup": 1,
        "components_ms_rank0": {k: round(v, 3) for k, v in sorted(parts.items())},
        "gemm_tflops_per_gpu": round(model.linear_flops(tokens) / world / (gemm_ms * 1e-3) / 1e12, 1),
        "linear_tflop": round(model.linear_flops(tokens) / 1e12, 1),
        "attention_tflop": round(model.attention_flops(tokens) / 1e12, 1),
    }
    if world > 1:
        x_ms = parts.get("exchange", 0.0)
        carry_ms = x_ms + parts.get("qk_norm_rope", 0.0)
        report.update({
            "exchange_ms": round(x_ms, 3),
            "exchange_note": "return kernel + both flag waits (includes waiting for the slowest "
                             "rank); the q|k|v stores ride in the q/k norm + RoPE kernel",
            "bytes_sent_per_rank_per_step": sent,
            "nvlink_gbs_over_exchange_and_rope_time": round(sent / (carry_ms * 1e-3) / 1e9, 1) if carry_ms else None,
            "n1_ms_same_box": round(n1_ms, 3) if n1_ms else None,
            "strong_scaling_vs_n1": round(n1_ms / (world * ms), 3) if n1_ms else None,
        })
    del model
    torch.cuda.empty_cache()
    return report


# ------------------------------------------------------------------ GPU arm --

def attention_report():
    """The package's tcgen05 attention kernel beside the library kernel on the Wan 2.2 5B
    self-attention shape (27280 tokens, 24 heads of 128): four alternating rounds of three launches."""
    import torch
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import dit
    from blackwell_diffusion_rtx6000_5090_i2v_b200.synthetic import student_t_bf16
    L, H = 27280, 24
    qkv = student_t_bf16((L, 3 * H * 128), 13, device="cuda")
    q, k, v = (t.view(L, H, 128) for t in qkv.split(H * 128, dim=-1))
    out = torch.empty(L, H, 128, dtype=torch.bfloat16, device="cuda")
    amax = torch.zeros(1, device="cuda")
    old = dit.ATTENTION_BACKEND
    dit.ATTENTION_BACKEND = "library"

    def timed(fn, n=3):
        r = fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            r = fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n, r

    # the two kernels take turns, so that neither is always the one measured on the warmer GPU;
    # the best round of each is reported, all rounds are listed
    own_ms, lib_ms = [], []
    try:
        for _ in range(4):
            ms, o_own = timed(lambda: dit.attention_native(q, k, v, amax=amax.zero_(), out=out))
            own_ms.append(ms)
            ms, o_lib = timed(lambda: dit.attention(q, k, v))
            lib_ms.append(ms)
    finally:
        dit.ATTENTION_BACKEND = old
    ms_own, ms_lib = min(own_ms), min(lib_ms)
    flops = 4.0 * L * L * H * 128
    peaks = measured_peaks()
    own, lib = flops / ms_own / 1e9, flops / ms_lib / 1e9
    return {"kernel": "attention_kernel (tcgen05, bf16, max|o| folded in)", "bound": "tensor",
            "workload": f"[{L}, {H}, 128] self-attention, non-causal, q/k/v as column blocks of one "
                        "[L, 3*H*128] tensor",
            "achieved": own, "unit": "TFLOP/s", "ms": ms_own, "peak": peaks["bf16_tflops"],
            "frac": own / peaks["bf16_tflops"], "peak_source": f"{peaks['source']} cuBLAS bf16 burst",
            "library": {"kernel": "F.scaled_dot_product_attention", "achieved": lib, "ms": ms_lib},
            "frac_of_library": own / lib,
            "rounds_ms": {"own": [round(t, 3) for t in own_ms], "library": [round(t, 3) for t in lib_ms]},
            "max_abs_diff_vs_library": float((o_own.float() - o_lib.float()).abs().max()),
            "amax_matches_output": float(amax) == float(o_own.float().abs().max())}


def run_ours(args, rank: int, local_rank: int, world: int):
    import torch
    import torch.distributed as dist
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import _native as N
    from blackwell_diffusion_rtx6000_5090_i2v_b200.synthetic import outlier_weight_bf16, student_t_bf16
    from blackwell_diffusion_rtx6000_5090_i2v_b200.block_linears import (
        WAN22_TI2V_5B, HostStagedLinears, WanBlockLinears, wan_block_specs)

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    numa = bind_to_gpu_numa_node(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = WAN22_TI2V_5B
    M = cfg["tokens"]
    specs = wan_block_specs(cfg["dim"], cfg["ffn"])
    seed = 1234 + 2 + 1000 * rank
    weights = {s.name: outlier_weight_bf16((s.n, s.k), seed + 10 + i) for i, s in enumerate(specs)}
    biases = {s.name: (torch.randn(s.n, generator=torch.Generator().manual_seed(seed + 20 + i))
                       * 0.01).to(torch.bfloat16) for i, s in enumerate(specs)}
    runner = WanBlockLinears(specs, M, weights, biases, device=dev)
    # activations resident in HBM before the timed region; ffn_down consumes ffn_up's output
    inputs = {s.name: student_t_bf16((M, s.k), seed + 30 + i, device=dev)
              for i, s in enumerate(specs) if s.name != "ffn_down"}

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        runner.step(inputs)
    barrier()
    N.check_status(dev)

    # ---- exactly K steps: the headline value (a burst figure: tens of milliseconds) ----
    gemm_events = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        barrier()
        e0.record()
        for _ in range(args.steps):
            runner.step(inputs, gemm_events)
        e1.record()
        barrier()
    N.check_status(dev)
    ms_total = e0.elapsed_time(e1)
    gemm_ms = sum(a.elapsed_time(b) for a, b in gemm_events)

    if world > 1:
        t = torch.tensor([ms_total, gemm_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total, gemm_ms = float(t[0]), float(t[1])
    ms_step = ms_total / args.steps
    value = world * runner.flops_per_step / (ms_step * 1e-3) / 1e12

    # ---- quantizer alone (HBM roofline), activations larger than L2 ----
    st = torch.cuda.current_stream().cuda_stream
    q0, q1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    big = runner.out["ffn_up"]  # [M, 14336] bf16 = 782 MB, left by the last step
    qa = runner.act["ffn_down"]
    reps = 10
    for _ in range(3):
        N.lib.nvfp4_quantize_bf16(big.data_ptr(), qa.m, qa.k, qa.amax.data_ptr(),
                                  qa.data.data_ptr(), None, qa.sf.data_ptr(),
                                  qa.gscale.data_ptr(), st)
    q0.record()
    for _ in range(reps):
        N.lib.nvfp4_quantize_bf16(big.data_ptr(), qa.m, qa.k, qa.amax.data_ptr(),
                                  qa.data.data_ptr(), None, qa.sf.data_ptr(),
                                  qa.gscale.data_ptr(), st)
    q1.record()
    torch.cuda.synchronize()
    quant_gbs = 2.5625 * qa.m * qa.k / (q0.elapsed_time(q1) / reps * 1e-3) / 1e9

    # ---- fused LayerNorm + adaLN modulation + quantize (both sweeps), the block's norm1 shape ----
    xin = runner.out["attn_out"]                      # [M, dim] bf16
    rows_n, dim = xin.shape
    gsc = torch.Generator(device="cuda").manual_seed(77)
    ada_scale = torch.randn(dim, generator=gsc, device="cuda") * 0.1
    ada_shift = torch.randn(dim, generator=gsc, device="cuda") * 0.1
    qn = runner.act["qkv"]                            # packed buffers of a [M, dim] activation
    stats = torch.empty(2 * rows_n, dtype=torch.float32, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def fused_norm_quantize():
        N.check(N.lib.nvfp4_norm_mod_amax_bf16(xin.data_ptr(), rows_n, dim, None, None,
                                               ada_scale.data_ptr(), ada_shift.data_ptr(), 0, 1e-6,
                                               stats.data_ptr(), qn.amax.data_ptr(), None,
                                               runner.status.data_ptr(), st), "norm amax")
        N.check(N.lib.nvfp4_norm_mod_quantize_bf16(xin.data_ptr(), rows_n, dim, None, None,
                                                   ada_scale.data_ptr(), ada_shift.data_ptr(),
                                                   stats.data_ptr(), qn.amax.data_ptr(),
                                                   qn.data.data_ptr(), None, qn.sf.data_ptr(),
                                                   qn.gscale.data_ptr(), runner.status.data_ptr(), st),
                "norm quantize")

    fused_ms = []
    for i in range(3 + reps):
        flush.zero_()                                 # L2 flush; also keeps the GPU ahead of the host
        q0.record()
        fused_norm_quantize()
        q1.record()
        torch.cuda.synchronize()
        if i >= 3:
            fused_ms.append(q0.elapsed_time(q1))
    fused_ms = sorted(fused_ms)[len(fused_ms) // 2]
    fused_alg_gbs = 2.5625 * xin.numel() / (fused_ms * 1e-3) / 1e9
    fused_moved_gbs = 4.5625 * xin.numel() / (fused_ms * 1e-3) / 1e9
    del flush

    # ---- the same steps repeated for at least two seconds: the sustained figure, with the SM
    # clock sampled every 5 ms (a 1 kW part settles well below its idle-boost clock) ----
    sus_events = []
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sus_steps = 0
    with ClockSampler(local_rank) as sus_clocks:
        barrier()
        t_start = time.perf_counter()
        s0.record()
        while True:
            for _ in range(args.steps):
                runner.step(inputs, sus_events)
            sus_steps += args.steps
            torch.cuda.current_stream().synchronize()
            if time.perf_counter() - t_start >= (0.0 if args.skip_e2e else SUSTAINED_SECONDS):
                break
        s1.record()
        barrier()
    sus_ms_total = s0.elapsed_time(s1)
    # the clock is still settling in the first half of the window: GEMM events from the second
    late = sus_events[len(sus_events) // 2 // len(specs) * len(specs):]
    late_steps = len(late) / len(specs)
    sus_gemm_ms = sum(a.elapsed_time(b) for a, b in late)
    sus_gemm_flops = runner.flops_per_step * late_steps
    if world > 1:
        t = torch.tensor([sus_ms_total / sus_steps], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sus_ms_step = float(t[0])
    else:
        sus_ms_step = sus_ms_total / sus_steps
    # let the power controller release the clocks again before the library is timed
    if not args.skip_e2e:
        time.sleep(1.0)

    if args.skip_e2e:
        if rank == 0:
            print(json.dumps({"metric": "NVFP4 GEMM TFLOPS", "value": value, "unit": "TFLOP/s",
                              "ms_per_step": ms_step, "quantizer_gbs": quant_gbs,
                              "gemm_tflops": runner.flops_per_step * args.steps / (gemm_ms * 1e-3) / 1e12,
                              "note": "--skip-e2e: partial line, not a bench result"}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- library reference: cuBLASLt block-scaled FP4 through torch._scaled_mm, same packed
    # operands, same stream, back to back (not on the product path; reported beside the number),
    # and the same library on one large square problem as a MEASURED FP4 throughput of this box
    lib_ref, fp4_measured = None, None
    if rank == 0:
        def time_lib(f, n=10):
            for _ in range(3):
                f()
            l0, l1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            l0.record()
            for _ in range(n):
                f()
            l1.record()
            torch.cuda.synchronize()
            return l0.elapsed_time(l1) / n
        try:
            ms_lib, per_lib = 0.0, {}
            for s_ in specs:
                q, w = runner.act[s_.name], runner.w[s_.name]
                A = q.data.view(q.m, s_.k // 2).view(torch.float4_e2m1fn_x2)
                B = w._data.view(s_.n, s_.k // 2).view(torch.float4_e2m1fn_x2)
                sa = q.sf.view(torch.float8_e4m3fn)
                sb = w._scales_swz.view(torch.float8_e4m3fn)
                t_ = time_lib(lambda: torch._scaled_mm(A, B.t(), sa, sb, out_dtype=torch.bfloat16))
                ms_lib += t_
                per_lib[s_.name] = round(2.0 * M * s_.n * s_.k / t_ / 1e9, 1)
            lib_ref = {"what": "torch._scaled_mm (cuBLASLt NVFP4) on the same four packed GEMMs, "
                               "each timed alone over 10 back-to-back launches",
                       "tflops": runner.flops_per_step / (ms_lib * 1e-3) / 1e12,
                       "per_linear_tflops": per_lib}
        except Exception as e:  # library path unavailable for these shapes: report, do not fail
            lib_ref = {"unavailable": repr(e)[:160]}
        try:
            S = 16384
            A = torch.randint(0, 256, (S, S // 2), dtype=torch.uint8, device=dev).view(torch.float4_e2m1fn_x2)
            B = torch.randint(0, 256, (S, S // 2), dtype=torch.uint8, device=dev).view(torch.float4_e2m1fn_x2)
            nsf = N.lib.nvfp4_swizzled_scale_bytes(S, S)
            sa = torch.full((nsf,), 0x38, dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
            sb = torch.full((nsf,), 0x38, dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
            t_ = time_lib(lambda: torch._scaled_mm(A, B.t(), sa, sb, out_dtype=torch.bfloat16), 5)
            fp4_measured = 2.0 * S ** 3 / t_ / 1e9
            del A, B, sa, sb
        except Exception:
            fp4_measured = None

    # ---- end to end through the public API with host buffers ----
    e2e_steps = max(3, args.steps // 4)
    host_in = {s.name: torch.empty(M, s.k, dtype=torch.bfloat16).pin_memory() for s in specs}
    host_out = {s.name: torch.empty(M, s.n, dtype=torch.bfloat16).pin_memory() for s in specs}
    for s in specs:
        src = inputs.get(s.name, runner.out["ffn_up"])
        host_in[s.name].copy_(src)
    h2d = sum(t.numel() * 2 for t in host_in.values())
    d2h = sum(t.numel() * 2 for t in host_out.values())
    staged = HostStagedLinears(runner)

    def e2e_step():
        staged.step(host_in, host_out)

    e2e_step()
    staged.wait()
    barrier()
    x0, x1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    x0.record()
    for _ in range(e2e_steps):
        e2e_step()
    staged.wait()
    x1.record()
    barrier()
    e2e_ms = x0.elapsed_time(x1) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t[0])
    e2e_value = world * runner.flops_per_step / (e2e_ms * 1e-3) / 1e12

    # ---- one DiT step of the A14B shape on these GPUs (frees the block-linears buffers first) ----
    n_gemm = len(gemm_events)
    gemm_tflops = runner.flops_per_step * args.steps / (gemm_ms * 1e-3) / 1e12
    per_linear = {}
    for i, s_ in enumerate(specs):
        ms_i = sum(a.elapsed_time(b) for a, b in gemm_events[i::len(specs)]) / args.steps
        per_linear[s_.name] = round(2.0 * M * s_.n * s_.k / ms_i / 1e9, 1)
    flops_per_step, kernels_per_step = runner.flops_per_step, runner.kernels_per_step
    qa_shape = (qa.m, qa.k)
    del staged, host_in, host_out, runner, inputs, gemm_events, sus_events, late, big, xin, qa, qn
    torch.cuda.empty_cache()
    attention = None
    if rank == 0 and not args.skip_dit:
        try:
            attention = attention_report()
        except Exception as e:
            attention = {"failed": f"{type(e).__name__}: {str(e)[:300]}"}
        torch.cuda.empty_cache()
    dit_step = None
    if not args.skip_dit:
        try:
            dit_step = dit_step_report(world, rank, local_rank)
        except Exception as e:   # report the failure in the line instead of losing the line
            dit_step = {"failed": f"{type(e).__name__}: {str(e)[:300]}"}

    if rank == 0:
        peaks = measured_peaks()
        fp4_peak = FP4_TO_BF16_PEAK_RATIO * peaks["bf16_tflops"]
        sus_gemm_tflops = sus_gemm_flops / (sus_gemm_ms * 1e-3) / 1e12 if sus_gemm_ms else None
        sus_clk = sus_clocks.summary()
        traffic = profiled_gemm_traffic()
        alg_bytes_avg = sum(M * s.k / 2 * 1.125 + s.n * s.k / 2 * 1.125 + 2.0 * M * s.n
                            for s in specs) / len(specs)
        line = {
            "metric": "NVFP4 GEMM TFLOPS", "value": value, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp4_e2m1", "data": "synthetic",
            "config": {"workload": CONFIG_NAME, "tokens_per_gpu": M,
                       "step": "per linear: amax + NVFP4 quantize of the bf16 activation, then "
                               "tcgen05 block-scaled GEMM with fused bias (+GELU); weights "
                               "pre-quantized",
                       "l2": "inputs_exceed_l2 (each step streams >3 GB of activations and outputs)",
                       "parallelism": f"token-sharded x{world}, weights replicated, no collective "
                                      "(the communicating workload is dit_step)"},
            "gpu_launches": kernels_per_step * args.steps,
            "roofline": {
                "kernel": "nvfp4_gemm_kernel", "bound": "tensor", "achieved": gemm_tflops,
                "peak": fp4_peak, "unit": "TFLOP/s", "frac": gemm_tflops / fp4_peak,
                "peak_source": f"4 x {peaks['source']} cuBLAS bf16 burst "
                               f"({peaks['bf16_tflops']} TF/s); nominal dense FP4:bf16 = 9:2.25; "
                               "MEASURED_PEAKS.json holds no FP4 figure",
                "peak_measured_fp4": fp4_measured,
                "peak_measured_fp4_source": "cuBLASLt NVFP4 (torch._scaled_mm) on 16384^3, this run, "
                                            "5 back-to-back launches",
                "frac_of_measured_fp4": gemm_tflops / fp4_measured if fp4_measured else None,
                "frac_of_nominal_9pf": gemm_tflops / 9000.0,
                "launches": n_gemm, "avg_launch_ms": gemm_ms / n_gemm,
                "flops_per_launch_avg": flops_per_step / len(specs),
                "per_linear_tflops": per_linear,
                "library_reference": lib_ref,
                "traffic": (traffic[0] * alg_bytes_avg / traffic[1]) if traffic else None,
                "traffic_source": (f"{traffic[2]}: ncu dram read+write {traffic[0]:.3g} B for "
                                   f"{traffic[1]:.3g} algorithmic bytes, scaled by algorithmic bytes "
                                   f"to this workload's average launch ({alg_bytes_avg:.3g} B)")
                if traffic else "no profile summary found",
            },
            "sustained": {
                "what": f"the same step repeated for {sus_ms_total / 1e3:.2f} s ({sus_steps} steps), "
                        "SM clock sampled every 5 ms",
                "value": world * flops_per_step / (sus_ms_step * 1e-3) / 1e12, "unit": "TFLOP/s",
                "ms_per_step": sus_ms_step, "gemm_tflops": sus_gemm_tflops,
                "gemm_frac_of_4x_bf16_sustained":
                    sus_gemm_tflops / (FP4_TO_BF16_PEAK_RATIO * peaks["bf16_tflops_sustained"])
                    if sus_gemm_tflops else None,
                "clocks": sus_clk,
                "gemm_ms_per_step_x_sm_mhz":
                    (sus_gemm_ms / late_steps) * sus_clk["sm_mhz"]
                    if sus_gemm_ms and sus_clk.get("sm_mhz") else None,
            },
            "quantizer": {"kernel": "quantize_bf16_kernel", "bound": "hbm", "achieved": quant_gbs,
                          "peak": peaks["hbm_gbs"], "unit": "GB/s",
                          "frac": quant_gbs / peaks["hbm_gbs"], "peak_source": peaks["source"],
                          "workload": f"[{qa_shape[0]}, {qa_shape[1]}] bf16 -> nibbles + swizzled E4M3 "
                                      "scales, 2.5625 B/element"},
            "fused_norm_quantizer": {
                "kernel": "norm_mod_kernel (two sweeps)", "bound": "hbm", "achieved": fused_alg_gbs,
                "moved": fused_moved_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": fused_alg_gbs / peaks["hbm_gbs"], "frac_moved": fused_moved_gbs / peaks["hbm_gbs"],
                "us": fused_ms * 1e3,
                "workload": f"[{rows_n}, {dim}] bf16 LayerNorm + (1+scale)x+shift -> nibbles + "
                            "swizzled scales; 2.5625 B/element algorithmic, 4.5625 moved (x read "
                            "twice, recompute variant); L2 flushed before each timing"},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "steps": e2e_steps, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "api": "HostStagedLinears.step on pinned host buffers (copy-in, compute and "
                           "copy-out streams overlapped)",
                    "limit": "host link: every rank moves 2.9 GB per step over PCIe "
                             "(copy-out alone needs ~29 ms at 55 GB/s); on several GPUs the ranks "
                             "share the host's memory and PCIe roots, so the aggregate does not "
                             "scale with N",
                    "cpu_binding": numa},
            "clocks": clocks.summary(),
            "attention": attention,
            "dit_step": dit_step,
        }
        if world == 1 and not args.skip_cpu:
            line["cpu_baseline"] = cpu_baseline_report(full=True)[0]
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--skip-e2e", action="store_true",
                    help="leave out the host-buffer leg, the DiT step and the CPU baseline (profiler runs)")
    ap.add_argument("--skip-dit", action="store_true", help="leave out the DiT-step leg")
    ap.add_argument("--skip-cpu", action="store_true", help="leave out the CPU baseline leg")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if world != args.gpus and world == 1 and args.gpus > 1:
        # launched without torchrun: re-exec under it, one rank per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
               f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1", "--master-port",
               os.environ.get("MASTER_PORT", "29517"), os.path.abspath(__file__), "--gpus",
               str(args.gpus), "--steps", str(args.steps), "--warmup", str(args.warmup)]
        for flag in ("skip_e2e", "skip_dit", "skip_cpu"):
            if getattr(args, flag):
                cmd.append("--" + flag.replace("_", "-"))
        sys.exit(subprocess.call(cmd))
    run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
