"""Shared input generators and comparisons for the parity tests."""
import numpy as np
import torch


def bits_of(t: torch.Tensor) -> np.ndarray:
    """bf16 tensor -> uint16 bit patterns (numpy), any device."""
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def from_bits(b: np.ndarray, device="cpu") -> torch.Tensor:
    return torch.from_numpy(b.view(np.int16).copy()).view(torch.bfloat16).to(device)


def randn_bf16(shape, seed, scale=1.0, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16).to(device)


def student_t_bf16(shape, seed, df=4.0, scale=0.5, device="cpu"):
    """Heavy-tailed activations: Student-t(df) * scale."""
    g = torch.Generator().manual_seed(seed)
    z = torch.randn(shape, generator=g)
    chi = torch.zeros(shape)
    for _ in range(int(df)):
        chi += torch.randn(shape, generator=g) ** 2
    return (z / torch.sqrt(chi / df) * scale).to(torch.bfloat16).to(device)


def outlier_weight_bf16(shape, seed, std=0.02, frac=1e-3, mult=20.0, device="cpu"):
    """N(0, std^2) weights with a Bernoulli(frac) mask of entries multiplied by mult."""
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(shape, generator=g) * std
    mask = torch.rand(shape, generator=g) < frac
    return torch.where(mask, w * mult, w).to(torch.bfloat16).to(device)


def rel_fro(a: torch.Tensor, b: torch.Tensor) -> float:
    a = a.double()
    b = b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))
