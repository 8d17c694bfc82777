"""Drop-in for the reference's ``nvfp4_linear_cpp`` extension module.

Mirrors the functions bound at ``fx/src/s4/nvfp4/linear/nvfp4_gemm_kernel.cu:
223-268``: ``gemm``, ``gemv``, ``batched_gemm``, ``forward``, ``backward``,
``are_dimensions_aligned``, ``get_padded_dimensions`` and
``estimate_padding_overhead``.  Differences that matter on B200:

* no pad-to-128 copy (nvfp4_gemm_kernel.cu:51-64): ragged M is handled inside
  the GEMM by TMA zero fill and clipped stores;
* the bias add is fused into the GEMM epilogue (reference: a separate op,
  nvfp4_gemm_kernel.cu:140-142);
* weights are quantized once per version of the weight tensor and cached
  (the reference re-quantizes every forward).
"""
from __future__ import annotations

import weakref
from typing import List, Optional, Tuple

import torch

from .nvfp4 import FP4Tensor, fp4_gemm

_PFX = "[fxy] [ops] [nvfp4]"

# id(weight) -> (weakref, version, data_ptr, FP4Tensor)
_weight_cache: dict = {}


def quantized_weight(weight: torch.Tensor) -> FP4Tensor:
    """NVFP4 copy of a ``[N, K]`` bf16 weight, reused until the tensor is
    modified in place, reallocated or freed."""
    try:
        version = weight._version
    except RuntimeError:
        # tensors created under torch.inference_mode() track no version: an in-place change
        # could not be noticed, so they are quantized on every call
        return FP4Tensor.from_bfloat16(weight.detach(), linear_scales=False)
    key = id(weight)
    hit = _weight_cache.get(key)
    if hit is not None:
        ref, cached_version, ptr, q = hit
        if ref() is weight and cached_version == version and ptr == weight.data_ptr():
            return q
    q = FP4Tensor.from_bfloat16(weight.detach(), linear_scales=False)
    _weight_cache[key] = (weakref.ref(weight, lambda _r, k=key: _weight_cache.pop(k, None)),
                          version, weight.data_ptr(), q)
    return q


def _check_pair(input_matrix: torch.Tensor, weight_matrix: torch.Tensor) -> None:
    # nvfp4_gemm_kernel.cu:25-39
    if not (input_matrix.is_cuda and weight_matrix.is_cuda):
        raise RuntimeError(f"{_PFX} Tensors must be on CUDA device")
    if input_matrix.dtype != torch.bfloat16 or weight_matrix.dtype != torch.bfloat16:
        raise RuntimeError(f"{_PFX} Tensors must be BFloat16")
    if input_matrix.dim() != 2 or weight_matrix.dim() != 2:
        raise RuntimeError(f"{_PFX} Tensors must be 2D matrices")
    if weight_matrix.size(1) != input_matrix.size(1):
        raise RuntimeError(f"{_PFX} Inner dimensions must match: {input_matrix.size(1)} vs "
                           f"{weight_matrix.size(1)}")


def _pad_k(t: torch.Tensor, mult: int = 32) -> torch.Tensor:
    k = t.size(1)
    if k % mult == 0:
        return t.contiguous()
    return torch.nn.functional.pad(t, (0, mult - k % mult))


def gemm(input_matrix: torch.Tensor, weight_matrix: torch.Tensor, alpha: float = 1.0,
         beta: float = 0.0, *, cache_weight: bool = False, **epilogue) -> torch.Tensor:
    """``alpha * input @ weight.T`` with both operands quantized to NVFP4
    (``nvfp4_gemm``, nvfp4_gemm_kernel.cu:21-65).  ``beta`` multiplies an
    all-zero C in the reference and is accepted for signature parity."""
    _check_pair(input_matrix, weight_matrix)
    n = weight_matrix.size(0)
    x, w = input_matrix, weight_matrix
    if x.size(1) % 32 != 0:           # K tail: zero columns add nothing to the sum
        x, w, cache_weight = _pad_k(x), _pad_k(w), False
    n_pad = (n + 7) // 8 * 8
    if n_pad != n:                    # N tail: extra zero weight rows, sliced off below
        w, cache_weight = torch.nn.functional.pad(w, (0, 0, 0, n_pad - n)), False
        if epilogue:
            raise RuntimeError(f"{_PFX} fused epilogue needs N to be a multiple of 8")
    a = FP4Tensor.from_bfloat16(x, linear_scales=False)
    b = quantized_weight(w) if cache_weight else FP4Tensor.from_bfloat16(w, linear_scales=False)
    out = fp4_gemm(a, b, alpha, 0.0, **epilogue)
    return out if n_pad == n else out[:, :n]


def gemv(input_vector: torch.Tensor, weight_matrix: torch.Tensor,
         alpha: float = 1.0) -> torch.Tensor:
    """nvfp4_gemm_kernel.cu:67-87: a one-row GEMM."""
    x = input_vector.unsqueeze(0) if input_vector.dim() == 1 else input_vector
    if x.size(0) != 1:
        x = x.t()
    return gemm(x.contiguous(), weight_matrix, alpha, 0.0).squeeze(0)


def batched_gemm(input_batch: torch.Tensor, weight_matrix: torch.Tensor,
                 alpha: float = 1.0) -> torch.Tensor:
    """nvfp4_gemm_kernel.cu:89-107."""
    if input_batch.dim() != 3:
        raise RuntimeError(f"{_PFX} Input must be 3D for batched GEMM")
    b, m, k = input_batch.shape
    out = gemm(input_batch.reshape(b * m, k), weight_matrix, alpha, 0.0)
    return out.reshape(b, m, weight_matrix.size(0))


def linear(input: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, *,
           gelu: bool = False, gate: Optional[torch.Tensor] = None,
           residual: Optional[torch.Tensor] = None,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``residual + gate * act(input @ weight.T + bias)`` over flattened batch
    dims: quantize the activation, one tcgen05 GEMM with everything else fused
    into its epilogue."""
    if input.dim() < 2:
        raise RuntimeError(f"{_PFX} Input must be at least 2D, got {input.dim()}D")
    if weight.dim() != 2:
        raise RuntimeError(f"{_PFX} Weight must be 2D, got {weight.dim()}D")
    in_features = input.size(-1)
    if weight.size(1) != in_features:
        raise RuntimeError(f"{_PFX} Weight shape mismatch")
    batch_dims = list(input.shape[:-1])
    x2 = input.reshape(-1, in_features)
    n = weight.size(0)
    if bias is not None and bias.numel() == 0:
        bias = None
    ep = {}
    if bias is not None:
        ep["bias"] = bias.contiguous()
    if gelu:
        ep["gelu"] = True
    if gate is not None:
        ep["gate"] = gate
    if residual is not None:
        ep["C"] = residual.reshape(-1, n)
    if out is not None:
        ep["out"] = out.reshape(-1, n)
    if n % 8 != 0 and ep:
        # ragged N: run the plain GEMM and finish the few extra ops in torch
        y = gemm(x2, weight, 1.0, 0.0, cache_weight=False)
        if bias is not None:
            y = y + bias.unsqueeze(0)
        if gelu:
            y = torch.nn.functional.gelu(y, approximate="tanh")
        if gate is not None:
            y = y * gate.to(y.dtype)
        if residual is not None:
            y = y + residual.reshape(-1, n)
        return y.reshape(batch_dims + [n])
    beta = 1.0 if residual is not None else 0.0
    _check_pair(x2, weight)
    y = _gemm_beta(x2, weight, beta, ep)
    return y.reshape(batch_dims + [n])


def _gemm_beta(x2, weight, beta, ep):
    if x2.size(1) % 32 != 0:
        x2, weight, cached = _pad_k(x2), _pad_k(weight), False
    else:
        cached = True
    a = FP4Tensor.from_bfloat16(x2, linear_scales=False)
    b = quantized_weight(weight) if cached else FP4Tensor.from_bfloat16(weight, linear_scales=False)
    return fp4_gemm(a, b, 1.0, beta, **ep)


def forward(input: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor,
            scale_input: torch.Tensor, scale_weight: torch.Tensor) -> torch.Tensor:
    """``nvfp4_linear_forward`` (nvfp4_gemm_kernel.cu:109-149).  The two scale
    arguments are reserved and ignored, as in the reference (:111-112)."""
    return linear(input, weight, bias)


def backward(grad_output: torch.Tensor, input: torch.Tensor, weight: torch.Tensor,
             scale_input: torch.Tensor, scale_weight: torch.Tensor,
             scale_grad_output: torch.Tensor, needs_input_grad: bool, needs_weight_grad: bool,
             needs_bias_grad: bool) -> List[Optional[torch.Tensor]]:
    """``nvfp4_linear_backward`` (nvfp4_gemm_kernel.cu:151-196): both gradient
    GEMMs run through the same FP4 path.  The reference's weight-gradient call
    passes operands whose inner dimensions disagree (:187); the product meant
    there, ``grad_output.T @ input``, is what is computed here."""
    in_features = input.size(-1)
    out_features = weight.size(0)
    x2 = input.reshape(-1, in_features)
    go = grad_output.reshape(-1, out_features).to(torch.bfloat16)
    grad_input = grad_weight = grad_bias = None
    if needs_input_grad:
        grad_input = gemm(go.contiguous(), weight.t().contiguous(), 1.0, 0.0).reshape(input.shape)
    if needs_weight_grad:
        grad_weight = gemm(go.t().contiguous(), x2.t().contiguous(), 1.0, 0.0)
    if needs_bias_grad:
        grad_bias = go.sum(0)
    return [grad_input, grad_weight, grad_bias]


def are_dimensions_aligned(M: int, N: int, K: int) -> bool:  # nvfp4_gemm_kernel.cu:201-203
    return M % 128 == 0 and N % 128 == 0 and K % 128 == 0


def get_padded_dimensions(M: int, N: int, K: int) -> Tuple[int, int, int]:  # :206-209
    return ((M + 127) // 128 * 128, (N + 127) // 128 * 128, (K + 127) // 128 * 128)


def estimate_padding_overhead(M: int, N: int, K: int) -> float:  # :212-218
    mp, np_, kp = get_padded_dimensions(M, N, K)
    original = M * K + N * K + M * N
    return float(mp * kp + np_ * kp + mp * np_ - original) / original
