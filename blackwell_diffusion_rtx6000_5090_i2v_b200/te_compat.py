"""``te.Linear``-shaped front end of the NVFP4 linear.

The reference's production model builds every DiT linear as
``transformer_engine.pytorch.Linear`` and switches it to NVFP4 from outside with
``te.fp8_autocast(enabled=True, fp8_recipe=NVFP4BlockScaling(fp4_format=Format.E2M1))``
(fx/src/s4/models/wan22/wan_transformer_megaupload.py:46,162-165,210-212,260-262,379,403;
fx/src/s4/models/wan22/bench_te_nvfp4.py:96-105,120-122,142;
fx/src/s4/benchmarks/transformer_engine_fp4_linear.py:14-43).  TransformerEngine itself is not
part of that repository.  This module offers the few names those call sites use, with the same
constructor and context-manager arguments, on top of :class:`NVFP4Linear`:

    import blackwell_diffusion_rtx6000_5090_i2v_b200.te_compat as te
    from blackwell_diffusion_rtx6000_5090_i2v_b200.te_compat import Format, NVFP4BlockScaling

    lin = te.Linear(3072, 9216, bias=True, params_dtype=torch.bfloat16).cuda()
    y_bf16 = lin(x)                                        # outside the context: plain bf16
    with te.fp8_autocast(enabled=True, fp8_recipe=NVFP4BlockScaling(fp4_format=Format.E2M1)):
        y_fp4 = lin(x)                                     # NVFP4 quantize + tcgen05 GEMM

Only the NVFP4 recipe is served; any other recipe raises, as nothing else is built here.
"""
from __future__ import annotations

import contextlib
import enum
import threading
from typing import Optional

import torch
import torch.nn.functional as F

from .nvfp4_linear_module import NVFP4Linear


class Format(enum.Enum):
    """The recipe formats the reference names (bench_te_nvfp4.py:96; megaupload.py:600)."""
    E2M1 = "e2m1"
    E4M3 = "e4m3"
    HYBRID = "hybrid"


class NVFP4BlockScaling:
    """Recipe object: E2M1 elements, one E4M3 scale per 16 elements, FP32 tensor scale."""

    def __init__(self, fp4_format: Format = Format.E2M1):
        if fp4_format is not Format.E2M1:
            raise ValueError("NVFP4BlockScaling: only Format.E2M1 exists for 4-bit elements")
        self.fp4_format = fp4_format

    def __repr__(self) -> str:
        return "NVFP4BlockScaling(fp4_format=Format.E2M1)"


_state = threading.local()


def _active_recipe():
    return getattr(_state, "recipe", None)


@contextlib.contextmanager
def fp8_autocast(enabled: bool = True, fp8_recipe=None, **_ignored):
    """Inside the context, :class:`Linear` modules run on the NVFP4 path.  ``fp8_recipe`` must be
    an :class:`NVFP4BlockScaling` (the default when ``enabled`` and none is given)."""
    if enabled and fp8_recipe is None:
        fp8_recipe = NVFP4BlockScaling()
    if enabled and not isinstance(fp8_recipe, NVFP4BlockScaling):
        raise NotImplementedError(f"fp8_autocast: recipe {fp8_recipe!r} is not served; only "
                                  "NVFP4BlockScaling is")
    previous = _active_recipe()
    _state.recipe = fp8_recipe if enabled else None
    try:
        yield
    finally:
        _state.recipe = previous


class Linear(NVFP4Linear):
    """``te.Linear(in_features, out_features, bias=True, params_dtype=...)``: bf16 parameters;
    ``forward(inp)`` is a plain bf16 linear outside :func:`fp8_autocast` and the NVFP4 linear
    inside it.  Further TransformerEngine keyword arguments (sequence-parallel and
    tensor-parallel options, fused weight-gradient accumulation ...) have no meaning for a
    single-GPU inference linear and are refused rather than silently dropped."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True,
                 params_dtype: Optional[torch.dtype] = None, device=None, **unsupported):
        if unsupported:
            raise TypeError(f"te_compat.Linear: unsupported arguments {sorted(unsupported)}")
        if params_dtype not in (None, torch.bfloat16):
            raise TypeError("te_compat.Linear: parameters are bf16 (params_dtype=torch.bfloat16)")
        super().__init__(in_features, out_features, bias=bias)
        if device is not None:
            self.to(device)

    def forward(self, inp: torch.Tensor, is_first_microbatch: Optional[bool] = None) -> torch.Tensor:
        if _active_recipe() is None:
            return F.linear(inp.to(torch.bfloat16), self.weight, self.bias)
        return super().forward(inp)
