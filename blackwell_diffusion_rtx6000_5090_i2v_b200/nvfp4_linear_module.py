"""Drop-in for ``fx/src/s4/nvfp4/linear/nvfp4_linear_module.py``:
``NVFP4LinearFunction`` and ``NVFP4Linear`` with the same constructor
arguments, parameters and buffers, running on the B200 kernels."""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
from torch import Tensor

from . import nvfp4_linear_cpp


class NVFP4LinearFunction(torch.autograd.Function):
    """nvfp4_linear_module.py:9-46."""

    @staticmethod
    def forward(ctx, input: Tensor, weight: Tensor, bias: Optional[Tensor], scale_input: Tensor,
                scale_weight: Tensor) -> Tensor:
        ctx.save_for_backward(input, weight, scale_input, scale_weight)
        ctx.needs_bias_grad = bias is not None
        if bias is None:
            bias = torch.empty(0, device=input.device, dtype=input.dtype)
        return nvfp4_linear_cpp.forward(input, weight, bias, scale_input, scale_weight)

    @staticmethod
    def backward(ctx, grad_output: Tensor):
        input, weight, scale_input, scale_weight = ctx.saved_tensors
        scale_grad_output = torch.ones_like(scale_input)
        grad_input, grad_weight, grad_bias = nvfp4_linear_cpp.backward(
            grad_output, input, weight, scale_input, scale_weight, scale_grad_output,
            ctx.needs_input_grad[0], ctx.needs_input_grad[1], ctx.needs_bias_grad)
        return grad_input, grad_weight, grad_bias, None, None


class NVFP4Linear(nn.Module):
    """NVFP4 linear layer (nvfp4_linear_module.py:49-106): bf16 ``weight``
    ``[out, in]``, optional bf16 ``bias``, and the reserved ``scale_weight``
    buffer.  In inference (no grad) the forward skips autograd bookkeeping and
    the dummy ``scale_input`` allocation the reference makes every call."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True,
                 block_size: int = 32):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.block_size = block_size
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=torch.bfloat16))
        if bias:
            self.bias = nn.Parameter(torch.empty(out_features, dtype=torch.bfloat16))
        else:
            self.register_parameter("bias", None)
        self.register_buffer(
            "scale_weight",
            torch.ones((out_features * in_features + block_size - 1) // block_size,
                       dtype=torch.float32))
        self.reset_parameters()

    def reset_parameters(self):
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))
        if self.bias is not None:
            fan_in, _ = nn.init._calculate_fan_in_and_fan_out(self.weight)
            bound = 1 / math.sqrt(fan_in) if fan_in > 0 else 0
            nn.init.uniform_(self.bias, -bound, bound)

    def forward(self, input: Tensor) -> Tensor:
        if input.dtype != torch.bfloat16:
            input = input.to(torch.bfloat16)
        if not torch.is_grad_enabled() or not (input.requires_grad or self.weight.requires_grad):
            return nvfp4_linear_cpp.linear(input, self.weight, self.bias)
        input_numel = input.numel() // input.size(-1) * self.in_features
        scale_input = torch.ones((input_numel + self.block_size - 1) // self.block_size,
                                 device=input.device, dtype=torch.float32)
        return NVFP4LinearFunction.apply(input, self.weight, self.bias, scale_input,
                                         self.scale_weight)

    @classmethod
    def from_linear(cls, linear: nn.Linear, block_size: int = 32) -> "NVFP4Linear":
        """An NVFP4Linear holding ``linear``'s weight and bias (cast to bf16), on its device."""
        out = cls(linear.in_features, linear.out_features, linear.bias is not None, block_size)
        out = out.to(linear.weight.device)
        with torch.no_grad():
            out.weight.copy_(linear.weight.to(torch.bfloat16))
            if linear.bias is not None:
                out.bias.copy_(linear.bias.to(torch.bfloat16))
        out.weight.requires_grad_(linear.weight.requires_grad)
        out.train(linear.training)
        return out

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, "
                f"bias={self.bias is not None}, format=nvfp4")


class NVFP4InferenceConfig:
    """Stands where the reference passes torchao's config of the same name to ``quantize_``
    (fx/src/s4/models/wan22/wan_loader.py:613-616): which linears to convert."""

    def __init__(self, min_features: int = 32, skip: tuple = ()):
        self.min_features = min_features
        self.skip = tuple(skip)          # substrings of module paths to leave alone

    def wants(self, name: str, module: nn.Module) -> bool:
        return (type(module) is nn.Linear and module.in_features % 32 == 0
                and module.out_features % 8 == 0
                and min(module.in_features, module.out_features) >= self.min_features
                and not any(s in name for s in self.skip))


def quantize_(model: nn.Module, config: Optional[NVFP4InferenceConfig] = None, filter_fn=None) -> nn.Module:
    """In place, replace every ``nn.Linear`` the config wants (and ``filter_fn(module, name)``
    accepts, when given) by an :class:`NVFP4Linear` with the same weights -- the call shape of
    ``torchao.quantization.quantize_`` as the reference uses it on the DiT
    (wan_loader.py:613-616).  Linears whose sizes the GEMM cannot take stay as they are.
    Returns the model."""
    config = config or NVFP4InferenceConfig()

    def walk(parent: nn.Module, prefix: str) -> None:
        for child_name, child in list(parent.named_children()):
            path = f"{prefix}.{child_name}" if prefix else child_name
            if config.wants(path, child) and (filter_fn is None or filter_fn(child, path)):
                setattr(parent, child_name, NVFP4Linear.from_linear(child))
            else:
                walk(child, path)

    if config.wants("", model) and (filter_fn is None or filter_fn(model, "")):
        return NVFP4Linear.from_linear(model)
    walk(model, "")
    return model
