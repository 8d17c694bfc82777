"""Writes the reference kernel's E4M3 block scales for the golden cases.

    python tests/golden/make_ref_scales.py [--out tests/golden/ref_te_scales.npz]

Needs a B200 and ``oracle/_ref/libref_quant_te.so`` (the reference's own
``block_1d_quantization_kernel_te``, fx/src/s4/nvfp4/quantization_te.cu:92-135, compiled from the
reference tree by ``oracle/Makefile``).  For every input of ``nvfp4_cases.npz`` it runs that
kernel with the case's tensor amax and stores the scale bytes it produced, plus the kernel's own
element bytes for the record (the reference's live kernels emit a linear 4-bit code, not E2M1, so
those are not a parity target).  The committed output pins the scale recipe for a checkout that
has neither a GPU nor the reference tree.
"""
import argparse
import ctypes as C
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import nvfp4_oracle as O  # noqa: E402

CASES = ("normal", "student_t", "weights", "tiny_blocks", "edge")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(HERE, "ref_te_scales.npz"))
    args = ap.parse_args()
    ref = O.reference_te()
    if ref is None:
        raise SystemExit("oracle/_ref/libref_quant_te.so is missing: run `make -C oracle REF=...`")
    g = np.load(os.path.join(HERE, "nvfp4_cases.npz"))
    out = {}
    for name in CASES:
        xb = g[f"{name}.x"]
        amax = float(g[f"{name}.amax"])
        x = torch.from_numpy(xb.view(np.int16).copy()).view(torch.bfloat16).cuda()
        n = x.numel()
        packed = torch.zeros(n // 2, dtype=torch.uint8, device="cuda")
        scales = torch.zeros(n // 16, dtype=torch.uint8, device="cuda")
        rc = ref.ref_te_quantize(x.data_ptr(), packed.data_ptr(), scales.data_ptr(), n, C.c_float(amax), None)
        torch.cuda.synchronize()
        if rc != 0:
            raise SystemExit(f"{name}: reference kernel launch failed with CUDA error {rc}")
        out[f"{name}.scales"] = scales.cpu().numpy().reshape(xb.shape[0], -1)
        out[f"{name}.ref_linear_codes"] = packed.cpu().numpy().reshape(xb.shape[0], -1)
        out[f"{name}.amax"] = np.float32(amax)
    np.savez_compressed(args.out, **out)
    print("wrote", len(out), "arrays to", args.out)


if __name__ == "__main__":
    main()
