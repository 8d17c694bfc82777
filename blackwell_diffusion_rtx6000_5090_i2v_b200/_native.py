"""ctypes binding of libnvfp4_b200.so -- the only route to the CUDA kernels.

There is no CPU or PyTorch fallback: if the library is missing the import of
this module raises, and every failed call raises ``RuntimeError``.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libnvfp4_b200.so")

if not os.path.exists(_LIB_PATH):
    raise ImportError(
        f"{_LIB_PATH} is missing: build it with "
        "`python -m blackwell_diffusion_rtx6000_5090_i2v_b200.build` "
        "(there is no fallback path)")

lib = C.CDLL(_LIB_PATH)

_p, _i64, _f, _i = C.c_void_p, C.c_int64, C.c_float, C.c_int

# name -> (restype, argtypes); must list every symbol include/nvfp4_b200.h declares
SIGNATURES = {
    "nvfp4_status_string": (C.c_char_p, [_i]),
    "nvfp4_version": (_i, []),
    "nvfp4_init": (_i, [_i, C.POINTER(_i), C.POINTER(_i)]),
    "nvfp4_amax_bf16": (_i, [_p, _i64, _p, _p]),
    "nvfp4_swizzled_scale_bytes": (_i64, [_i64, _i64]),
    "nvfp4_quantize_bf16": (_i, [_p, _i64, _i64, _p, _p, _p, _p, _p, _p]),
    "nvfp4_quantize_bf16_amax": (_i, [_p, _p, _p, _i64, _f, _p]),
    "nvfp4_dequantize_bf16": (_i, [_p, _p, _i64, _i64, _p, _p, _p]),
    "nvfp4_dequantize_bf16_amax": (_i, [_p, _p, _p, _i64, _f, _p]),
    "nvfp4_swizzle_scales": (_i, [_p, _i64, _i64, _p, _p]),
    "nvfp4_gemm": (_i, [_p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _f, _f, _p, _p, _p, _i, _p,
                        _p, _p, _p]),
    "nvfp4_gemm_set_tiling": (_i, [_i]),
    "nvfp4_gemm_stacked": (_i, [_p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _p, _p, _p, _p]),
    "nvfp4_norm_mod_amax_bf16": (_i, [_p, _i64, _i64, _p, _p, _p, _p, _i, _f, _p, _p, _p, _p, _p]),
    "nvfp4_norm_mod_quantize_bf16": (_i, [_p, _i64, _i64, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p,
                                          _p, _p]),
    "nvfp4_qk_norm_rope_bf16": (_i, [_p, _p, _p, _i64, _i64, _i, _i, _p, _p, _f, _p, _p, _p, _p,
                                     _i64, _i64, _p, _p]),
    "nvfp4_qk_norm_rope_exchange_bf16": (_i, [_p, _p, _p, _i64, _i64, _i, _i, _p, _p, _f, _p, _p, _i,
                                              _i64, _p, _i, _p, _p]),
    "nvfp4_exchange_sync_bytes": (_i64, []),
    "nvfp4_exchange_wait": (_i, [_p, _i, _i, _i64, _p, _p, _p]),
    "nvfp4_attn_return_exchange_bf16": (_i, [_p, _i64, _i64, _i64, _i, _i, _p, _p, _i, _i, _p]),
    "nvfp4_attention_bf16": (_i, [_p, _i64, _i64, _p, _i64, _i64, _p, _i64, _i64, _i64, _i64, _i, _i, _f,
                                  _p, _i64, _i64, _p, _p, _p]),
    "nvfp4_linear_bf16_static": (_i, [_p, _i64, _i64, _p, _p, _p, _i64, _p, _i, _p, _p, _p]),
    "nvfp4_linear_bf16_static_max_elements": (_i64, []),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args

OK = 0
ACT_NONE, ACT_GELU_TANH = 0, 1


def status_string(rc: int) -> str:
    return lib.nvfp4_status_string(int(rc)).decode()


def check(rc: int, what: str, prefix: str = "[s4] [nvfp4]") -> None:
    if rc != OK:
        raise RuntimeError(f"{prefix} {what}: {status_string(rc)} (status {rc})")


def stream_ptr() -> int:
    """The current torch CUDA stream as a cudaStream_t value."""
    return torch.cuda.current_stream().cuda_stream


def ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


_status_words: dict[int, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 the GEMM kernel sets when a bounded wait expires."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    w = _status_words.get(idx)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status_words[idx] = w
    return w


def check_status(device: torch.device | None = None) -> None:
    """Synchronise and raise if any GEMM on ``device`` reported a timeout."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    w = status_word(device)
    v = int(w.item())
    if v != 0:
        w.zero_()
        raise RuntimeError(f"[s4] [nvfp4] [gemm] device-side wait timed out at 0x{v:x}")
