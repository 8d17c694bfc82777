"""Regenerates tests/golden/nvfp4_cases.npz from the CPU oracle.

    python tests/golden/make_golden.py

Inputs are seeded; the file stores bf16 inputs as uint16 bit patterns together
with the oracle's packed nibbles, E4M3 scales, tensor amax, FP32 tensor scale,
the dequantized values and one small linear output, so that both the oracle
(CPU test) and the CUDA path (GPU test) are checked against fixed bytes.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from helpers import bits_of, outlier_weight_bf16, randn_bf16, student_t_bf16  # noqa: E402
from oracle import nvfp4_oracle as O  # noqa: E402


def main():
    out = {}
    cases = {
        "normal": randn_bf16((48, 256), 1234),
        "student_t": student_t_bf16((40, 512), 1235),
        "weights": outlier_weight_bf16((64, 256), 1236),
        "tiny_blocks": randn_bf16((16, 128), 1237) * torch.logspace(-12, 2, 128).to(torch.bfloat16),
    }
    edge = torch.zeros(8, 64, dtype=torch.bfloat16)
    edge[1, :] = 1.0
    edge[2, ::2] = -3.0
    edge[3, 5] = 3.3895313892515355e38  # bf16 max
    edge[4, :16] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0,
                                 -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0])
    edge[5, 16:32] = 1e-30
    cases["edge"] = edge
    for name, x in cases.items():
        xb = bits_of(x)
        packed, scales, amax = O.quantize(xb)
        out[f"{name}.x"] = xb
        out[f"{name}.packed"] = packed
        out[f"{name}.scales"] = scales
        out[f"{name}.amax"] = np.float32(amax)
        out[f"{name}.gscale"] = np.float32(O.global_decode_scale(amax))
        out[f"{name}.dequant_bf16"] = O.dequantize_bf16(packed, scales, amax)
    # one small linear: Y = X W^T + b through dequantize-then-matmul
    x = randn_bf16((24, 256), 2001)
    w = randn_bf16((32, 256), 2002, 0.02)
    b = randn_bf16((32,), 2003, 0.01)
    out["linear.x"], out["linear.w"], out["linear.b"] = bits_of(x), bits_of(w), bits_of(b)
    out["linear.y"] = O.linear(bits_of(x), bits_of(w), bits_of(b))
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)),
                                     "nvfp4_cases.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
