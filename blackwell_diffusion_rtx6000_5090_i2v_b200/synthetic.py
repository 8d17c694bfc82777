"""Seeded synthetic tensors with the shapes and value distributions of the
benchmark configurations (no Wan 2.2 weights, prompts or videos are used)."""
from __future__ import annotations

import torch


def randn_bf16(shape, seed, scale=1.0, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16).to(device)


def student_t_bf16(shape, seed, df=4.0, scale=0.5, device="cpu"):
    """Heavy-tailed activations: Student-t(df) * scale (stresses the block scales)."""
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
