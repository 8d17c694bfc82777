"""GEMM and quantizer sweep over the Wan 2.2 linear shapes:
``python -m blackwell_diffusion_rtx6000_5090_i2v_b200.sweep [--out table.md]``.

M in {256, 1024, 4096, 16384, 32760, 65536} x (N, K) in the eight linear shapes of the 5B and
14B models; operands bf16 N(0, 1) before quantization (seeded).  Per cell: NVFP4 GEMM TFLOP/s
(2 M N K / CUDA-event time, operands pre-quantized) and its fraction of the FP4 peak; per (M, K):
quantizer GB/s (amax pass + pack pass, 2.5625 B/element algorithmic) and its fraction of the HBM
peak.  L2 is flushed before every timed launch.  Peaks come from ``MEASURED_PEAKS.json`` beside
the package when present (FP4 peak = 4 x the measured bf16 burst figure), else nominal.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch

from . import _native as N
from .nvfp4 import FP4Tensor, fp4_gemm
from .synthetic import randn_bf16

MS = (256, 1024, 4096, 16384, 32760, 65536)
NKS = ((3072, 3072), (9216, 3072), (14336, 3072), (3072, 14336),
       (5120, 5120), (15360, 5120), (13824, 5120), (5120, 13824))


def _peaks():
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return 4.0 * float(p["bf16_tflops"]), float(p["hbm_gbs"]), "measured (FP4 = 4 x bf16 burst)"
    except (OSError, KeyError, ValueError):
        return 9000.0, 8000.0, "nominal"


def _median_ms(fn, flush, iters):
    fn()
    ts = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return statistics.median(ts)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--iters", type=int, default=7)
    ap.add_argument("--out", default=None, help="also write the tables to this file")
    a = ap.parse_args(argv)
    torch.cuda.set_device(0)
    fp4_peak, hbm_peak, src = _peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    lines = [f"peaks: FP4 {fp4_peak:.0f} TFLOP/s, HBM {hbm_peak:.0f} GB/s ({src}); "
             f"median of {a.iters} launches, L2 flushed before each", "",
             "GEMM TFLOP/s (fraction of FP4 peak)", "",
             "| M \\ (N, K) | " + " | ".join(f"{n}x{k}" for n, k in NKS) + " |",
             "|---|" + "---|" * len(NKS)]
    weights = {nk: FP4Tensor.from_bfloat16(randn_bf16(nk, 100 + i, device="cuda"), linear_scales=False)
               for i, nk in enumerate(NKS)}
    acts = {}
    quant = {}
    for m in MS:
        row = [f"| {m} |"]
        for (n, k) in NKS:
            if (m, k) not in acts:
                x = randn_bf16((m, k), 7 + k, device="cuda")
                qa = FP4Tensor.from_bfloat16(x, linear_scales=False)
                acts[(m, k)] = qa
                st = N.stream_ptr()

                def q(x=x, qa=qa, m=m, k=k, st=st):
                    N.lib.nvfp4_amax_bf16(x.data_ptr(), m * k, qa._amax.data_ptr(), st)
                    N.lib.nvfp4_quantize_bf16(x.data_ptr(), m, k, qa._amax.data_ptr(),
                                              qa._data.data_ptr(), None, qa._scales_swz.data_ptr(),
                                              qa._gscale.data_ptr(), st)
                quant[(m, k)] = _median_ms(q, flush, a.iters)
                del x
            out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
            qa, qb = acts[(m, k)], weights[(n, k)]
            ms = _median_ms(lambda: fp4_gemm(qa, qb, out=out), flush, a.iters)
            tf = 2.0 * m * n * k / ms / 1e9
            row.append(f" {tf:.0f} ({tf / fp4_peak:.2f}) |")
            del out
        lines.append("".join(row))
        for key in [key for key in acts if key[0] == m]:
            del acts[key]
    N.check_status()
    ks = sorted({k for _, k in NKS})
    lines += ["", "Quantizer (amax + pack) GB/s algorithmic, 2.5625 B/element; one pass each over the "
              "input (fraction of HBM peak; the two passes move 4.5625 B/element)", "",
              "| M \\ K | " + " | ".join(str(k) for k in ks) + " |", "|---|" + "---|" * len(ks)]
    for m in MS:
        row = [f"| {m} |"]
        for k in ks:
            gbs = 2.5625 * m * k / quant[(m, k)] / 1e6
            moved = 4.5625 * m * k / quant[(m, k)] / 1e6
            row.append(f" {gbs:.0f} alg / {moved:.0f} moved ({moved / hbm_peak:.2f}) |")
        lines.append("".join(row))
    text = "\n".join(lines)
    print(text, flush=True)
    if a.out:
        with open(a.out, "w") as f:
            f.write(text + "\n")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
