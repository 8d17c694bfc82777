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
same workload on its own token shard -- the path needs no collective -- and the
value is the whole-job aggregate over the slowest rank's device time.
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
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CONFIG_NAME = "wan2.2-ti2v-5b block linears, M=27280 (qkv, attn_out, ffn_up+gelu, ffn_down)"
FP4_TO_BF16_PEAK_RATIO = 4.0  # nominal dense peaks 9 PFLOP/s (FP4) : 2.25 PFLOP/s (bf16)


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


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while running."""

    def __init__(self, index: int):
        self.index = index
        self.samples, self.reasons = [], set()
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
                    mask = n.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                except Exception:
                    mask = n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.02)

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
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons)}


# ------------------------------------------------------------ CPU reference --

def cpu_reference_sample(rows: int = 96):
    """The reference's CPU arithmetic for the path (host fake-quantizer + matmul,
    fx/src/s4/nvfp4/linear/nvfp4_linear.cpp:61-152) restated in oracle/nvfp4_oracle.c,
    timed with all host threads on a bounded sample: `rows` tokens of each of the four
    block linears (weights quantized inside the timed call, as the reference does every
    forward).  Returns (run, flops, cores, description); run() executes the sample once and
    returns its wall time in seconds."""
    import numpy as np
    import torch
    from oracle import nvfp4_oracle as O
    from blackwell_diffusion_rtx6000_5090_i2v_b200.block_linears import WAN22_TI2V_5B, wan_block_specs
    from blackwell_diffusion_rtx6000_5090_i2v_b200.synthetic import outlier_weight_bf16, student_t_bf16

    def bits_of(t):
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)

    O.lib()
    specs = wan_block_specs(WAN22_TI2V_5B["dim"], WAN22_TI2V_5B["ffn"])
    data = []
    for i, s in enumerate(specs):
        x = bits_of(student_t_bf16((rows, s.k), 1300 + i))
        w = bits_of(outlier_weight_bf16((s.n, s.k), 1400 + i))
        b = bits_of((torch.randn(s.n) * 0.01).to(torch.bfloat16))
        data.append((s, x, w, b))
    flops = sum(2 * rows * s.n * s.k for s in specs)

    def run():
        t0 = time.perf_counter()
        for s, x, w, b in data:
            O.linear(x, w, b, act=1 if s.gelu else 0)
        return time.perf_counter() - t0

    return run, flops, os.cpu_count(), (f"{rows} of 27280 tokens through all four linears, "
                                         "operand quantization included, OpenMP over all host threads")


def run_reference(args, rank: int):
    if rank != 0:
        return
    run, flops, cores, sample = cpu_reference_sample()
    for _ in range(max(1, min(args.warmup, 2))):
        run()
    times = [run() for _ in range(args.steps)]
    t = sum(times) / len(times)
    value = flops / t / 1e12
    line = {
        "impl": "reference", "metric": "NVFP4 GEMM TFLOPS", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp4_e2m1", "data": "synthetic",
        "config": {"workload": CONFIG_NAME, "sample": sample},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ GPU arm --

def run_ours(args, rank: int, local_rank: int, world: int):
    import torch
    import torch.distributed as dist
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import _native as N
    from blackwell_diffusion_rtx6000_5090_i2v_b200.synthetic import outlier_weight_bf16, student_t_bf16
    from blackwell_diffusion_rtx6000_5090_i2v_b200.block_linears import (
        WAN22_TI2V_5B, WanBlockLinears, wan_block_specs)

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
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
    # operands, same stream, back to back (not on the product path; reported beside the number)
    lib_ref = None
    if rank == 0:
        try:
            ms_lib = 0.0
            for s_ in specs:
                q, w = runner.act[s_.name], runner.w[s_.name]
                Mp = q.m
                A = q.data.view(Mp, s_.k // 2).view(torch.float4_e2m1fn_x2)
                B = w._data.view(s_.n, s_.k // 2).view(torch.float4_e2m1fn_x2)
                sa = q.sf.view(torch.float8_e4m3fn)
                sb = w._scales_swz.view(torch.float8_e4m3fn)
                f = lambda: torch._scaled_mm(A, B.t(), sa, sb, out_dtype=torch.bfloat16)  # noqa: E731
                for _ in range(3):
                    f()
                l0, l1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                l0.record()
                for _ in range(10):
                    f()
                l1.record()
                torch.cuda.synchronize()
                ms_lib += l0.elapsed_time(l1) / 10
            lib_ref = {"what": "torch._scaled_mm (cuBLASLt NVFP4) on the same four packed GEMMs, "
                               "each timed alone over 10 back-to-back launches",
                       "tflops": runner.flops_per_step / (ms_lib * 1e-3) / 1e12}
        except Exception as e:  # library path unavailable for these shapes: report, do not fail
            lib_ref = {"unavailable": repr(e)[:160]}

    # ---- end to end through the public API with host buffers ----
    e2e_steps = max(3, args.steps // 4)
    host_in = {s.name: torch.empty(M, s.k, dtype=torch.bfloat16).pin_memory() for s in specs}
    host_out = {s.name: torch.empty(M, s.n, dtype=torch.bfloat16).pin_memory() for s in specs}
    for s in specs:
        src = inputs.get(s.name, runner.out["ffn_up"])
        host_in[s.name].copy_(src)
    h2d = sum(t.numel() * 2 for t in host_in.values())
    d2h = sum(t.numel() * 2 for t in host_out.values())

    from blackwell_diffusion_rtx6000_5090_i2v_b200.block_linears import HostStagedLinears
    staged = HostStagedLinears(runner)

    def e2e_step():
        staged.step(host_in, host_out)

    e2e_step()
    staged.wait()
    barrier()
    t0 = time.perf_counter()
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

    if rank == 0:
        peaks = measured_peaks()
        n_gemm = len(gemm_events)
        gemm_tflops = runner.flops_per_step * args.steps / (gemm_ms * 1e-3) / 1e12
        fp4_peak = FP4_TO_BF16_PEAK_RATIO * peaks["bf16_tflops"]
        per_linear = {}
        for i, s_ in enumerate(specs):
            ms_i = sum(a.elapsed_time(b) for a, b in gemm_events[i::len(specs)]) / args.steps
            per_linear[s_.name] = round(2.0 * M * s_.n * s_.k / ms_i / 1e9, 1)
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
                       "parallelism": f"token-sharded x{world}, weights replicated, no collective"},
            "gpu_launches": runner.kernels_per_step * args.steps,
            "roofline": {
                "kernel": "nvfp4_gemm_kernel", "bound": "tensor", "achieved": gemm_tflops,
                "peak": fp4_peak, "unit": "TFLOP/s", "frac": gemm_tflops / fp4_peak,
                "peak_source": f"4 x {peaks['source']} cuBLAS bf16 burst "
                               f"({peaks['bf16_tflops']} TF/s); nominal dense FP4:bf16 = 9:2.25",
                "frac_of_nominal_9pf": gemm_tflops / 9000.0,
                "launches": n_gemm, "avg_launch_ms": gemm_ms / n_gemm,
                "flops_per_launch_avg": runner.flops_per_step / len(specs),
                "per_linear_tflops": per_linear,
                "library_reference": lib_ref,
                "traffic": 3.46e8,
                "traffic_source": "ncu dram read+write of the M=8192,N=9216,K=3072 capture "
                                  "(122 MB for 181 MB algorithmic) scaled by algorithmic bytes to "
                                  "the average launch of this workload (513 MB); bytes per launch",
            },
            "quantizer": {"kernel": "quantize_bf16_kernel", "bound": "hbm", "achieved": quant_gbs,
                          "peak": peaks["hbm_gbs"], "unit": "GB/s",
                          "frac": quant_gbs / peaks["hbm_gbs"], "peak_source": peaks["source"],
                          "workload": f"[{qa.m}, {qa.k}] bf16 -> nibbles + swizzled E4M3 scales, "
                                      "2.5625 B/element"},
            "fused_norm_quantizer": {
                "kernel": "norm_mod_kernel (two sweeps)", "bound": "hbm", "achieved": fused_alg_gbs,
                "moved": fused_moved_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": fused_alg_gbs / peaks["hbm_gbs"], "frac_moved": fused_moved_gbs / peaks["hbm_gbs"],
                "workload": f"[{xin.shape[0]}, {dim}] bf16 LayerNorm + (1+scale)x+shift -> nibbles + "
                            "swizzled scales; 2.5625 B/element algorithmic, 4.5625 moved (x read "
                            "twice, recompute variant); L2 flushed before each timing"},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "steps": e2e_steps, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "api": "HostStagedLinears.step on pinned host buffers (copy-in, compute and "
                           "copy-out streams overlapped)"},
            "clocks": clocks.summary(),
        }
        if world == 1:
            run, flops, cores, sample = cpu_reference_sample()
            run()
            t = min(run() for _ in range(2))
            line["cpu_baseline"] = {"value": flops / t / 1e12, "unit": "TFLOP/s", "cores": cores,
                                    "kind": "port", "sample": sample}
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
                    help="leave out the host-buffer leg and the CPU baseline (profiler runs)")
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
        sys.exit(subprocess.call(cmd))
    run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
