"""The timed CPU baseline of the NVFP4 linear path -- TEST / BENCHMARK INFRASTRUCTURE ONLY.

What the reference computes on the CPU for this path is its host fake-quantizer followed by a
matmul (fx/src/s4/nvfp4/linear/nvfp4_linear.cpp:61-152).  Three timed forms:

* :func:`config1_full` -- the single NVFP4 linear (X [4096, 3072], W [3072, 3072], bias) in full:
  quantize both operands (``nvfp4_oracle.c``, OpenMP), dequantize to fp32, ``torch.matmul`` on
  all cores, bias, round to bf16;
* :func:`block_linears_m4096` -- the four block linears of the Wan2.2-TI2V-5B shape at
  M = 4096 tokens, weights quantized once outside the timed call, and again with the weights
  re-quantized inside every call as the reference does on every forward (:123-152);
* :func:`literal_slice` -- a transliteration of the reference's own loop structure
  (:61-119: one host read per element to find each block's maximum, another per element to
  scale and round it, rounding by a scan of the eight E2M1 magnitudes) on a 256 x 3072 slice.
  It is timed once and extrapolated; as in the reference, its rounding breaks ties towards the
  smaller magnitude and its scale is an unrounded fp32 number, so its values are NOT the
  parity oracle's.

Only ``bench.py`` (the ``cpu_baseline`` leg and ``--impl reference``) and tests import this.
"""
from __future__ import annotations

import os
import time

import numpy as np
import torch

from blackwell_diffusion_rtx6000_5090_i2v_b200.shapes import WAN22_TI2V_5B, wan_block_specs
from blackwell_diffusion_rtx6000_5090_i2v_b200.synthetic import (outlier_weight_bf16, randn_bf16,
                                                                 student_t_bf16)
from oracle import nvfp4_oracle as O


def use_all_cores() -> int:
    """Pin the thread counts explicitly (launchers export OMP_NUM_THREADS=1); returns the count."""
    n = os.cpu_count() or 1
    torch.set_num_threads(n)
    return min(O.set_threads(n), torch.get_num_threads())


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def _quant_dequant(bits: np.ndarray) -> torch.Tensor:
    packed, scales, amax = O.quantize(bits)
    return torch.from_numpy(O.dequantize_f32(packed, scales, amax))


def _finish(acc: torch.Tensor, bias: torch.Tensor, gelu: bool) -> torch.Tensor:
    y = acc + bias.float()
    if gelu:
        y = torch.nn.functional.gelu(y, approximate="tanh")
    return y.to(torch.bfloat16)


def config1_full() -> dict:
    """One NVFP4 linear, X [4096, 3072] N(0,1), W [3072, 3072] N(0, 0.02^2), b N(0, 0.01^2)."""
    M, N, K = 4096, 3072, 3072
    x, w, b = randn_bf16((M, K), 1235), randn_bf16((N, K), 1236, 0.02), randn_bf16((N,), 1237, 0.01)
    xb, wb = _bits(x), _bits(w)
    t0 = time.perf_counter()
    px, sx, ax = O.quantize(xb)
    pw, sw, aw = O.quantize(wb)
    t1 = time.perf_counter()
    xq = torch.from_numpy(O.dequantize_f32(px, sx, ax))
    wq = torch.from_numpy(O.dequantize_f32(pw, sw, aw))
    t2 = time.perf_counter()
    _finish(xq @ wq.t(), b, False)
    t3 = time.perf_counter()
    total = t3 - t0
    return {"shape": [M, N, K], "quantize_ms": (t1 - t0) * 1e3, "dequantize_ms": (t2 - t1) * 1e3,
            "matmul_ms": (t3 - t2) * 1e3, "total_ms": total * 1e3,
            "tflops": 2.0 * M * N * K / total / 1e12}


class BlockLinearsM4096:
    """The four block linears at M = 4096 (of 27280) tokens on the CPU."""

    def __init__(self, rows: int = 4096):
        self.rows = rows
        self.specs = wan_block_specs(WAN22_TI2V_5B["dim"], WAN22_TI2V_5B["ffn"])
        self.x, self.w, self.b, self.wq = {}, {}, {}, {}
        for i, s in enumerate(self.specs):
            self.x[s.name] = _bits(student_t_bf16((rows, s.k), 1300 + i))
            self.w[s.name] = _bits(outlier_weight_bf16((s.n, s.k), 1400 + i))
            self.b[s.name] = (torch.randn(s.n, generator=torch.Generator().manual_seed(1500 + i))
                              * 0.01).to(torch.bfloat16)
        self.flops = sum(2.0 * rows * s.n * s.k for s in self.specs)

    def prepare_weights(self) -> float:
        t0 = time.perf_counter()
        for s in self.specs:
            self.wq[s.name] = _quant_dequant(self.w[s.name])
        return time.perf_counter() - t0

    def run(self, requantize_weights: bool) -> float:
        """One pass over the four linears; returns seconds."""
        t0 = time.perf_counter()
        for s in self.specs:
            xq = _quant_dequant(self.x[s.name])
            wq = _quant_dequant(self.w[s.name]) if requantize_weights else self.wq[s.name]
            _finish(xq @ wq.t(), self.b[s.name], s.gelu)
        return time.perf_counter() - t0


_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def _round_like_the_reference(v: float) -> float:
    """nvfp4_linear.cpp:40-58: clamp to +-6, then the first of the eight magnitudes at minimal
    distance (a tie keeps the smaller one)."""
    v = max(-6.0, min(6.0, v))
    a = abs(v)
    best, best_d = 0.0, float("inf")
    for m in _E2M1:
        d = abs(a - m)
        if d < best_d:
            best, best_d = m, d
    return -best if v < 0 else best


def literal_slice(rows: int = 256, cols: int = 3072) -> dict:
    """The reference's loop structure on a [rows, cols] slice: per-element host reads
    (``tensor[row][col].item()``) for the block maximum and again for the scaled, rounded value
    (nvfp4_linear.cpp:87-116).  Returns the time and an extrapolation to a [27280, 3072]
    activation."""
    x = student_t_bf16((rows, cols), 1300)
    t0 = time.perf_counter()
    amax = float(x.abs().max().item())
    enc_g = 1.0 if amax == 0.0 or amax == float("inf") else min(448.0 * 6.0 / amax, 3.4028234663852886e38)
    dec_g = 1.0 / enc_g
    blocks = (cols + 15) // 16
    scales = torch.empty(rows, blocks, dtype=torch.float32)
    out = torch.empty_like(x)
    for r in range(rows):
        for blk in range(blocks):
            c0, c1 = blk * 16, min(blk * 16 + 16, cols)
            bmax = 0.0
            for c in range(c0, c1):
                bmax = max(bmax, abs(x[r][c].item()))
            sf = max(-448.0, min(448.0, bmax / 6.0 * enc_g))
            scales[r][blk] = sf
            enc = 1.0 / (sf * dec_g) if sf != 0.0 else float("inf")
            for c in range(c0, c1):
                out[r][c] = _round_like_the_reference(x[r][c].item() * enc) if sf != 0.0 else 0.0
    dt = time.perf_counter() - t0
    per_elem = dt / (rows * cols)
    return {"slice": [rows, cols], "seconds": dt, "ns_per_element": per_elem * 1e9,
            "extrapolated_seconds_27280x3072": per_elem * 27280 * 3072,
            "note": "reference literal path (one host read per element), extrapolated"}
