"""Shared input generators and comparisons for the parity tests."""
import numpy as np
import torch


def bits_of(t: torch.Tensor) -> np.ndarray:
    """bf16 tensor -> uint16 bit patterns (numpy), any device."""
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def from_bits(b: np.ndarray, device="cpu") -> torch.Tensor:
    return torch.from_numpy(b.view(np.int16).copy()).view(torch.bfloat16).to(device)


from blackwell_diffusion_rtx6000_5090_i2v_b200.synthetic import (  # noqa: E402,F401
    outlier_weight_bf16, randn_bf16, student_t_bf16)


def rel_fro(a: torch.Tensor, b: torch.Tensor) -> float:
    a = a.double()
    b = b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))
