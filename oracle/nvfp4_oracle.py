"""ctypes front-end of the plain-C NVFP4 oracle -- TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the benchmark's CPU-baseline leg import this
module; the shipped CUDA path never does.  Arrays are numpy: bf16 travels as
its uint16 bit pattern.  Each wrapper names the oracle function it calls; the
reference citations live beside those functions in ``nvfp4_oracle.c``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_TK = None
_REF = None


def build(quiet: bool = True) -> None:
    """Compile the checkers with ``make`` (oracle/Makefile)."""
    subprocess.run(["make", "-C", _HERE], check=True,
                   stdout=subprocess.DEVNULL if quiet else None)


def _load(name: str):
    path = os.path.join(_HERE, name)
    if not os.path.exists(path):
        build()
    return C.CDLL(path)


def lib():
    global _LIB
    if _LIB is None:
        L = _load("libnvfp4_oracle.so")
        p = C.c_void_p
        i64 = C.c_int64
        L.nvfp4_oracle_f32_to_e4m3.restype = C.c_uint8
        L.nvfp4_oracle_f32_to_e4m3.argtypes = [C.c_float]
        L.nvfp4_oracle_e4m3_to_f32.restype = C.c_float
        L.nvfp4_oracle_e4m3_to_f32.argtypes = [C.c_uint8]
        L.nvfp4_oracle_f32_to_e2m1.restype = C.c_uint8
        L.nvfp4_oracle_f32_to_e2m1.argtypes = [C.c_float]
        L.nvfp4_oracle_e2m1_to_f32.restype = C.c_float
        L.nvfp4_oracle_e2m1_to_f32.argtypes = [C.c_uint8]
        L.nvfp4_oracle_div6_mismatches.restype = C.c_int64
        L.nvfp4_oracle_div6_mismatches.argtypes = [p, i64]
        L.nvfp4_oracle_amax_bf16.restype = C.c_float
        L.nvfp4_oracle_amax_bf16.argtypes = [p, i64]
        L.nvfp4_oracle_global_encode_scale.restype = C.c_float
        L.nvfp4_oracle_global_encode_scale.argtypes = [C.c_float]
        L.nvfp4_oracle_global_decode_scale.restype = C.c_float
        L.nvfp4_oracle_global_decode_scale.argtypes = [C.c_float]
        L.nvfp4_oracle_quantize.restype = None
        L.nvfp4_oracle_quantize.argtypes = [p, i64, i64, C.c_float, p, p]
        L.nvfp4_oracle_dequantize_f32.restype = None
        L.nvfp4_oracle_dequantize_f32.argtypes = [p, p, i64, i64, C.c_float, p]
        L.nvfp4_oracle_dequantize_bf16.restype = None
        L.nvfp4_oracle_dequantize_bf16.argtypes = [p, p, i64, i64, C.c_float, p]
        L.nvfp4_oracle_swizzled_scale_bytes.restype = i64
        L.nvfp4_oracle_swizzled_scale_bytes.argtypes = [i64, i64]
        L.nvfp4_oracle_swizzle_scales.restype = None
        L.nvfp4_oracle_swizzle_scales.argtypes = [p, i64, i64, p]
        L.nvfp4_oracle_matmul_nt.restype = None
        L.nvfp4_oracle_matmul_nt.argtypes = [p, p, p, i64, i64, i64, C.c_int, p, p, p, p]
        L.nvfp4_oracle_set_threads.restype = C.c_int
        L.nvfp4_oracle_set_threads.argtypes = [C.c_int]
        L.nvfp4_oracle_linear.restype = C.c_int
        L.nvfp4_oracle_linear.argtypes = [p, p, p, i64, i64, i64, C.c_int, p]
        _LIB = L
    return _LIB


def set_threads(n: int) -> int:
    """OpenMP threads of the oracle's loops; returns the number in effect."""
    return int(lib().nvfp4_oracle_set_threads(int(n)))


def toolkit():
    """The CUDA toolkit's host converters (oracle/toolkit_cvt.cpp)."""
    global _TK
    if _TK is None:
        T = _load("libtoolkit_cvt.so")
        T.tk_f32_to_e4m3.restype = C.c_uint8
        T.tk_f32_to_e4m3.argtypes = [C.c_float]
        T.tk_e4m3_to_f32.restype = C.c_float
        T.tk_e4m3_to_f32.argtypes = [C.c_uint8]
        T.tk_f32_to_e2m1.restype = C.c_uint8
        T.tk_f32_to_e2m1.argtypes = [C.c_float]
        T.tk_f32x2_to_e2m1x2.restype = C.c_uint8
        T.tk_f32x2_to_e2m1x2.argtypes = [C.c_float, C.c_float]
        T.tk_f32_to_e4m3_many.restype = None
        T.tk_f32_to_e4m3_many.argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
        T.tk_f32_to_e2m1_many.restype = None
        T.tk_f32_to_e2m1_many.argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
        _TK = T
    return _TK


def reference_te():
    """The reference's own quantization_te.cu built into oracle/_ref (needs a
    GPU to call).  Returns None when the prebuilt library is absent."""
    global _REF
    if _REF is None:
        path = os.path.join(_HERE, "_ref", "libref_quant_te.so")
        if not os.path.exists(path):
            return None
        R = C.CDLL(path)
        p = C.c_void_p
        R.ref_te_quantize.restype = C.c_int
        R.ref_te_quantize.argtypes = [p, p, p, C.c_int64, C.c_float, p]
        R.ref_te_dequantize.restype = C.c_int
        R.ref_te_dequantize.argtypes = [p, p, p, C.c_int64, C.c_float, p]
        _REF = R
    return _REF


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _u16(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a)
    assert a.dtype == np.uint16, "bf16 travels as uint16 bit patterns"
    return a


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return r


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def amax(x_bits: np.ndarray) -> float:
    x_bits = _u16(x_bits)
    return float(lib().nvfp4_oracle_amax_bf16(_ptr(x_bits), x_bits.size))


def global_encode_scale(a: float) -> float:
    return float(lib().nvfp4_oracle_global_encode_scale(a))


def global_decode_scale(a: float) -> float:
    return float(lib().nvfp4_oracle_global_decode_scale(a))


def quantize(x_bits: np.ndarray, global_amax: float | None = None):
    """-> (packed uint8 [rows, cols/2], scales uint8 [rows, cols/16], amax)."""
    x_bits = _u16(x_bits)
    rows, cols = x_bits.shape
    assert cols % 16 == 0
    if global_amax is None:
        global_amax = amax(x_bits)
    packed = np.empty((rows, cols // 2), np.uint8)
    scales = np.empty((rows, cols // 16), np.uint8)
    lib().nvfp4_oracle_quantize(_ptr(x_bits), rows, cols, global_amax, _ptr(packed), _ptr(scales))
    return packed, scales, global_amax


def dequantize_f32(packed, scales, global_amax: float) -> np.ndarray:
    rows, half = packed.shape
    out = np.empty((rows, half * 2), np.float32)
    lib().nvfp4_oracle_dequantize_f32(_ptr(np.ascontiguousarray(packed)),
                                      _ptr(np.ascontiguousarray(scales)), rows, half * 2,
                                      global_amax, _ptr(out))
    return out


def dequantize_bf16(packed, scales, global_amax: float) -> np.ndarray:
    rows, half = packed.shape
    out = np.empty((rows, half * 2), np.uint16)
    lib().nvfp4_oracle_dequantize_bf16(_ptr(np.ascontiguousarray(packed)),
                                       _ptr(np.ascontiguousarray(scales)), rows, half * 2,
                                       global_amax, _ptr(out))
    return out


def swizzle_scales(scales: np.ndarray, cols: int) -> np.ndarray:
    rows = scales.shape[0]
    n = lib().nvfp4_oracle_swizzled_scale_bytes(rows, cols)
    out = np.empty(n, np.uint8)
    lib().nvfp4_oracle_swizzle_scales(_ptr(np.ascontiguousarray(scales)), rows, cols, _ptr(out))
    return out


def matmul_nt(xq: np.ndarray, wq: np.ndarray, bias_bits=None, act: int = 0, gate=None,
              residual_bits=None, want_f32: bool = False):
    """Y[M,N] = epilogue(xq[M,K] @ wq[N,K]^T); returns bf16 bits (and fp32)."""
    xq = np.ascontiguousarray(xq, np.float32)
    wq = np.ascontiguousarray(wq, np.float32)
    M, K = xq.shape
    N = wq.shape[0]
    y = np.empty((M, N), np.uint16)
    yf = np.empty((M, N), np.float32) if want_f32 else None
    b = _u16(bias_bits) if bias_bits is not None else None
    g = np.ascontiguousarray(gate, np.float32) if gate is not None else None
    r = _u16(residual_bits) if residual_bits is not None else None
    lib().nvfp4_oracle_matmul_nt(_ptr(xq), _ptr(wq), _ptr(b) if b is not None else None, M, N, K,
                                 act, _ptr(g) if g is not None else None,
                                 _ptr(r) if r is not None else None, _ptr(y),
                                 _ptr(yf) if yf is not None else None)
    return (y, yf) if want_f32 else y


def linear(x_bits, w_bits, bias_bits=None, act: int = 0) -> np.ndarray:
    """Whole CPU linear (quantize both operands, dequantize, matmul, bias)."""
    x_bits = _u16(x_bits)
    w_bits = _u16(w_bits)
    M, K = x_bits.shape
    N = w_bits.shape[0]
    y = np.empty((M, N), np.uint16)
    b = _u16(bias_bits) if bias_bits is not None else None
    rc = lib().nvfp4_oracle_linear(_ptr(x_bits), _ptr(w_bits), _ptr(b) if b is not None else None,
                                   M, N, K, act, _ptr(y))
    if rc != 0:
        raise MemoryError("oracle scratch allocation failed")
    return y
