"""Drop-in for the reference's ``nvfp4`` extension module on B200.

Same names, argument order, defaults and error behaviour as the pybind11
module of ``fx/src/s4/nvfp4/bindings.cpp:12-135`` (``init``,
``QuantizationMode``, ``FP4Tensor``, ``blackwell_fp4_gemm``, ``fp4_gemm``,
``gemm_fp4_quantized``, ``is_aligned``, ``get_aligned_dims``, ``benchmark``),
backed by the hand-written sm_100a kernels behind the C ABI of
``include/nvfp4_b200.h``.  Additive extras: ``FP4Tensor.global_scale()``, the
swizzled scale accessor, ``out=`` and the fused-epilogue keywords of the GEMM
entry points, and ``torch.library`` ops under the ``nvfp4_b200`` namespace.

Nothing here computes on the CPU and nothing synchronises with the host.
"""
from __future__ import annotations

import enum
from typing import Optional, Sequence

import torch

from . import _native as N

__version__ = "1.0.0"
__cuda_arch__ = "sm_100a"  # the reference reports "sm_120" (bindings.cpp:134)

FP4_E2M1_MAX = 6.0     # fx/src/s4/nvfp4/tensor.h:11
FP8_E4M3_MAX = 448.0   # fx/src/s4/nvfp4/tensor.h:12
FP4_BLOCK_SIZE = 16    # fx/src/s4/nvfp4/tensor.h:13


def init() -> None:
    """Check the current device.  The reference's ``init`` throws below compute
    capability 12 (bindings.cpp:23-27); this build requires exactly 10.x."""
    import ctypes as C
    if not torch.cuda.is_available():
        raise RuntimeError("[s4] [nvfp4] NVFP4 requires a CUDA device (SM_100)")
    dev = torch.cuda.current_device()
    major, minor = C.c_int(0), C.c_int(0)
    rc = N.lib.nvfp4_init(dev, C.byref(major), C.byref(minor))
    if rc != N.OK:
        raise RuntimeError("[s4] [nvfp4] NVFP4 requires SM_100. Current device: SM_"
                           f"{major.value}{minor.value}")
    print("[s4] [nvfp4] Initialized on", torch.cuda.get_device_name(dev),
          "with compute capability", major.value, ".", minor.value)


class QuantizationMode(enum.Enum):
    """fx/src/s4/nvfp4/tensor.h:15-20.  Only ``block_1d`` is NVFP4."""
    block_1d = 0
    block_2d = 1
    per_tensor = 2
    per_channel = 3


def _require_block_1d(mode: QuantizationMode, what: str) -> None:
    if mode is not QuantizationMode.block_1d:
        # same outcome as the reference's own NVFP4 build, whose other modes
        # throw (fx/src/s4/nvfp4/quantization_te_clean.cu:285-344)
        pretty = {QuantizationMode.block_2d: "Block 2D", QuantizationMode.per_tensor: "Per-tensor",
                  QuantizationMode.per_channel: "Per-channel"}[mode]
        raise RuntimeError(f"{pretty} {what} not yet implemented in clean version")


class PackedBuffers:
    """Preallocated device buffers for the packed form of a bf16 ``[rows, cols]`` activation
    (additive: the ``out=`` form of the quantizers; the reference allocates on every call,
    fx/src/s4/nvfp4/tensor.cpp:7-16, kernel.cu:109-110,140-142).  A quantizer given one writes
    into it and returns an :class:`FP4Tensor` that aliases it; the caller keeps that tensor only
    until the next quantizer call with the same buffers."""

    def __init__(self, rows: int, cols: int, device, linear_scales: bool = False):
        if cols % FP4_BLOCK_SIZE != 0:
            raise RuntimeError("[s4] [nvfp4] [tensor] cols must be a multiple of 16")
        self.rows, self.cols, self.device = rows, cols, torch.device(device)
        with torch.cuda.device(self.device):
            self.data = torch.empty(rows * cols // 2, dtype=torch.uint8, device=self.device)
            self.scales_swz = torch.empty(N.lib.nvfp4_swizzled_scale_bytes(rows, cols), dtype=torch.uint8,
                                          device=self.device)
            self.scales = (torch.empty(rows * cols // FP4_BLOCK_SIZE, dtype=torch.uint8, device=self.device)
                           if linear_scales else None)
            self.amax = torch.empty(1, dtype=torch.float32, device=self.device)
            self.gscale = torch.empty(1, dtype=torch.float32, device=self.device)
            self.stats = torch.empty(rows, 2, dtype=torch.float32, device=self.device)   # fused norm
        self.device = self.data.device       # with its index, as tensors report it

    def matches(self, rows: int, cols: int, device) -> bool:
        return (rows, cols) == (self.rows, self.cols) and torch.device(device) == self.device


class FP4Tensor:
    """Owning packed NVFP4 tensor (fx/src/s4/nvfp4/tensor.h:22-115).

    ``quantized_data()`` is uint8 ``[ceil(n/2)]`` (two E2M1 codes per byte, even
    element in the low nibble) and ``scale_factors()`` uint8 ``[ceil(n/16)]``
    (E4M3 bits, linear row-major), exactly the reference's buffers
    (tensor.cpp:7-16).  The FP32 per-tensor scale, which the reference computes
    but never stores, is kept in a one-element device tensor.
    """

    __slots__ = ("_data", "_scales", "_scales_swz", "_amax", "_gscale", "_shape", "_mode",
                 "_device", "_rows", "_cols", "_numel")

    def __init__(self):
        raise TypeError("use FP4Tensor.from_bfloat16")

    # ------------------------------------------------------------ create --
    @staticmethod
    def from_bfloat16(input: torch.Tensor,
                      mode: QuantizationMode = QuantizationMode.block_1d,
                      *, linear_scales: bool = True, swizzled_scales: bool = True,
                      amax: Optional[torch.Tensor] = None, amax_hook=None,
                      out: Optional[PackedBuffers] = None) -> "FP4Tensor":
        """``amax`` (additive): a one-element fp32 device tensor already holding max|input|,
        e.g. from the GEMM that produced ``input``; the amax pass is then skipped.
        ``amax_hook`` (additive): called with the amax tensor between the amax pass and the
        packing pass, e.g. to all-reduce the maximum over the shards of a sharded tensor.
        ``out`` (additive): preallocated buffers of the input's ``[rows, cols]``; nothing is
        allocated and the result aliases them."""
        if input.dtype != torch.bfloat16:
            raise RuntimeError("[s4] [nvfp4] [tensor] Input must be BFloat16")
        if not input.is_cuda:
            raise RuntimeError("[s4] [nvfp4] [tensor] Input must be on CUDA device")
        _require_block_1d(mode, "quantization")
        self = object.__new__(FP4Tensor)
        self._shape = list(input.shape)
        self._mode = mode
        self._device = input.device
        n = input.numel()
        self._numel = n
        with torch.cuda.device(input.device):
            x = input.contiguous()
            last = x.shape[-1] if x.dim() >= 1 and n > 0 else 0
            if n > 0 and last % FP4_BLOCK_SIZE == 0:
                rows, cols = n // last, last
            else:
                # blocks run over the flattened tensor (tensor.cpp:8-10); a ragged
                # tail block is completed with zeros, which leave its amax unchanged
                n_pad = (n + FP4_BLOCK_SIZE - 1) // FP4_BLOCK_SIZE * FP4_BLOCK_SIZE
                if n_pad != n:
                    x = torch.nn.functional.pad(x.reshape(-1), (0, n_pad - n))
                rows, cols = (1, n_pad) if n_pad else (0, 0)
            self._rows, self._cols = rows, cols
            dev = input.device
            if amax is not None and (amax.dtype != torch.float32 or amax.numel() != 1
                                     or amax.device != dev):
                raise RuntimeError("[s4] [nvfp4] [tensor] amax must be a one-element float32 "
                                   "tensor on the input's device")
            if out is not None:
                if not out.matches(rows, cols, dev) or (linear_scales and out.scales is None):
                    raise RuntimeError("[s4] [nvfp4] [tensor] out buffers do not match the input")
                self._amax = amax if amax is not None else out.amax
                self._gscale, self._data = out.gscale, out.data
                self._scales = out.scales if linear_scales else None
                self._scales_swz = out.scales_swz
            else:
                self._amax = amax if amax is not None else torch.empty(1, dtype=torch.float32,
                                                                       device=dev)
                self._gscale = torch.empty(1, dtype=torch.float32, device=dev)
                self._data = torch.empty(rows * cols // 2, dtype=torch.uint8, device=dev)
                self._scales = (torch.empty(rows * cols // FP4_BLOCK_SIZE, dtype=torch.uint8, device=dev)
                                if linear_scales else None)
                self._scales_swz = (torch.empty(N.lib.nvfp4_swizzled_scale_bytes(rows, cols),
                                                dtype=torch.uint8, device=dev)
                                    if swizzled_scales and rows * cols > 0 else None)
            st = N.stream_ptr()
            if amax is None:
                N.check(N.lib.nvfp4_amax_bf16(N.ptr(x), rows * cols, N.ptr(self._amax), st),
                        "[tensor] amax")
                if amax_hook is not None:
                    amax_hook(self._amax)
            N.check(N.lib.nvfp4_quantize_bf16(N.ptr(x), rows, cols, N.ptr(self._amax),
                                              N.ptr(self._data), N.ptr(self._scales),
                                              N.ptr(self._scales_swz), N.ptr(self._gscale), st),
                    "[tensor] quantize")
        return self

    @staticmethod
    def from_norm_mod(x: torch.Tensor, *, weight: Optional[torch.Tensor] = None,
                      bias: Optional[torch.Tensor] = None, scale: Optional[torch.Tensor] = None,
                      shift: Optional[torch.Tensor] = None, rms: bool = False, eps: float = 1e-6,
                      linear_scales: bool = False, return_normed: bool = False, amax_hook=None,
                      out: Optional[PackedBuffers] = None):
        """Quantize ``bf16(norm(x) * weight + bias) * (1 + scale) + shift`` without ever
        writing that tensor: the fused producer in front of the DiT block's linears
        (fx/src/s4/models/wan22/wan_transformer.py:204-206,210,218-220).  ``x`` is bf16
        ``[..., cols]``; the per-column vectors are fp32 ``[cols]``.  With ``return_normed`` the
        bf16 tensor is also produced and returned beside the packed one."""
        if x.dtype != torch.bfloat16:
            raise RuntimeError("[s4] [nvfp4] [tensor] Input must be BFloat16")
        if not x.is_cuda:
            raise RuntimeError("[s4] [nvfp4] [tensor] Input must be on CUDA device")
        cols = x.shape[-1]
        if cols % FP4_BLOCK_SIZE != 0 or cols > 16384:
            raise RuntimeError("[s4] [nvfp4] [tensor] fused norm needs cols % 16 == 0, cols <= 16384")
        dev = x.device
        vecs = []
        for name, v in (("weight", weight), ("bias", bias), ("scale", scale), ("shift", shift)):
            if v is not None:
                v = v.reshape(-1)
                if v.numel() != cols or v.dtype != torch.float32 or v.device != dev:
                    raise RuntimeError(f"[s4] [nvfp4] [tensor] {name} must be float32 [{cols}] on {dev}")
                v = v.contiguous()
            vecs.append(v)
        self = object.__new__(FP4Tensor)
        self._shape = list(x.shape)
        self._mode = QuantizationMode.block_1d
        self._device = dev
        self._numel = x.numel()
        rows = self._numel // cols
        self._rows, self._cols = rows, cols
        with torch.cuda.device(dev):
            xc = x.contiguous()
            if out is not None:
                if not out.matches(rows, cols, dev) or (linear_scales and out.scales is None):
                    raise RuntimeError("[s4] [nvfp4] [tensor] out buffers do not match the input")
                self._amax, self._gscale, self._data = out.amax, out.gscale, out.data
                self._scales = out.scales if linear_scales else None
                self._scales_swz, stats = out.scales_swz, out.stats
            else:
                self._amax = torch.empty(1, dtype=torch.float32, device=dev)
                self._gscale = torch.empty(1, dtype=torch.float32, device=dev)
                self._data = torch.empty(rows * cols // 2, dtype=torch.uint8, device=dev)
                self._scales = (torch.empty(rows * cols // FP4_BLOCK_SIZE, dtype=torch.uint8, device=dev)
                                if linear_scales else None)
                self._scales_swz = torch.empty(N.lib.nvfp4_swizzled_scale_bytes(rows, cols),
                                               dtype=torch.uint8, device=dev)
                stats = torch.empty(rows, 2, dtype=torch.float32, device=dev)
            normed = torch.empty_like(xc) if return_normed else None
            st = N.stream_ptr()
            status = N.ptr(N.status_word(dev))
            w_, b_, sc_, sh_ = (N.ptr(v) for v in vecs)
            N.check(N.lib.nvfp4_norm_mod_amax_bf16(N.ptr(xc), rows, cols, w_, b_, sc_, sh_,
                                                   1 if rms else 0, float(eps), N.ptr(stats),
                                                   N.ptr(self._amax), N.ptr(normed), status, st),
                    "[tensor] norm+amax")
            if amax_hook is not None:
                amax_hook(self._amax)
            N.check(N.lib.nvfp4_norm_mod_quantize_bf16(N.ptr(xc), rows, cols, w_, b_, sc_, sh_,
                                                       N.ptr(stats), N.ptr(self._amax),
                                                       N.ptr(self._data), N.ptr(self._scales),
                                                       N.ptr(self._scales_swz),
                                                       N.ptr(self._gscale), status, st),
                    "[tensor] norm+quantize")
        return (self, normed) if return_normed else self

    @staticmethod
    def from_packed(data: torch.Tensor, scales: torch.Tensor, amax: torch.Tensor,
                    global_scale: torch.Tensor, shape: Sequence[int]) -> "FP4Tensor":
        """Re-create a packed tensor from stored parts (additive: the reference never stores
        one): ``data`` uint8 ``[numel/2]``, ``scales`` uint8 linear ``[numel/16]``, ``amax`` and
        ``global_scale`` one-element fp32, all on one CUDA device; ``shape`` with a last
        dimension that is a multiple of 16.  The tensor-core scale layout is rebuilt on first use."""
        shape = [int(v) for v in shape]
        if len(shape) < 1 or shape[-1] % FP4_BLOCK_SIZE != 0:
            raise RuntimeError("[s4] [nvfp4] [tensor] stored shape needs a last dimension % 16 == 0")
        numel = 1
        for v in shape:
            numel *= v
        dev = data.device
        if not data.is_cuda or data.dtype != torch.uint8 or scales.dtype != torch.uint8 or \
                data.numel() != numel // 2 or scales.numel() != numel // FP4_BLOCK_SIZE:
            raise RuntimeError("[s4] [nvfp4] [tensor] stored buffers do not match the shape")
        for t in (scales, amax, global_scale):
            if t.device != dev:
                raise RuntimeError("[s4] [nvfp4] [tensor] stored buffers must share one device")
        if amax.dtype != torch.float32 or global_scale.dtype != torch.float32 or \
                amax.numel() != 1 or global_scale.numel() != 1:
            raise RuntimeError("[s4] [nvfp4] [tensor] amax / global_scale must be one-element float32")
        self = object.__new__(FP4Tensor)
        self._shape, self._mode, self._device, self._numel = shape, QuantizationMode.block_1d, dev, numel
        self._cols = shape[-1]
        self._rows = numel // self._cols
        self._data = data.contiguous().reshape(-1)
        self._scales = scales.contiguous().reshape(-1)
        self._scales_swz = None
        self._amax = amax.contiguous().reshape(1)
        self._gscale = global_scale.contiguous().reshape(1)
        return self

    def snapshot(self) -> "FP4Tensor":
        """A second handle on the same packed buffers with its own copy of the amax / tensor-scale
        slots (additive; callers that keep a packed tensor while its producer reuses those
        one-element slots for the next tensor)."""
        other = object.__new__(FP4Tensor)
        for name in self.__slots__:
            setattr(other, name, getattr(self, name))
        other._amax, other._gscale = self._amax.clone(), self._gscale.clone()
        return other

    # ------------------------------------------------------------ access --
    def to_bfloat16(self) -> torch.Tensor:
        """Dequantize (fx/src/s4/nvfp4/tensor.h:53-72)."""
        with torch.cuda.device(self._device):
            flat = torch.empty(self._rows * self._cols, dtype=torch.bfloat16, device=self._device)
            scales = self.scale_factors_full()
            N.check(N.lib.nvfp4_dequantize_bf16(N.ptr(self._data), N.ptr(scales), self._rows,
                                                self._cols, N.ptr(self._amax), N.ptr(flat),
                                                N.stream_ptr()), "[tensor] dequantize")
        return flat[: self._numel].reshape(self._shape)

    def quantized_data(self) -> torch.Tensor:
        """Packed FP4 bytes, ``[(numel+1)//2]`` (alias, tensor.h:74-76)."""
        return self._data[: (self._numel + 1) // 2]

    def scale_factors_full(self) -> torch.Tensor:
        if self._scales is None:
            raise RuntimeError("[s4] [nvfp4] [tensor] linear scale factors were not requested")
        return self._scales

    def scale_factors(self) -> torch.Tensor:
        """E4M3 block scales as uint8, ``[ceil(numel/16)]`` (alias, tensor.h:78-80)."""
        return self.scale_factors_full()

    def scale_factors_swizzled(self) -> torch.Tensor:
        """Scales in the tensor-core layout the GEMM consumes (built on demand)."""
        if self._scales_swz is None:
            with torch.cuda.device(self._device):
                self._scales_swz = torch.empty(
                    N.lib.nvfp4_swizzled_scale_bytes(self._rows, self._cols), dtype=torch.uint8,
                    device=self._device)
                N.check(N.lib.nvfp4_swizzle_scales(N.ptr(self.scale_factors_full()), self._rows,
                                                   self._cols, N.ptr(self._scales_swz),
                                                   N.stream_ptr()), "[tensor] swizzle")
        return self._scales_swz

    def global_scale(self) -> torch.Tensor:
        """FP32 per-tensor scale amax/(6*448) as a one-element device tensor."""
        return self._gscale

    def global_amax(self) -> torch.Tensor:
        return self._amax

    def shape(self) -> Sequence[int]:
        return list(self._shape)

    def numel(self) -> int:
        return self._numel

    def memory_usage(self) -> int:
        """tensor.h:93-97: packed bytes plus scale bytes."""
        return (self._numel + 1) // 2 + (self._numel + FP4_BLOCK_SIZE - 1) // FP4_BLOCK_SIZE

    def __repr__(self) -> str:  # bindings.cpp:55-67
        dims = ", ".join(str(d) for d in self._shape)
        return f"FP4Tensor(shape=[{dims}], memory={self.memory_usage()} bytes)"


# ------------------------------------------------------------------ GEMM --

def _gemm_packed(a: FP4Tensor, b: FP4Tensor, alpha: float, beta: float,
                 c: Optional[torch.Tensor], bias: Optional[torch.Tensor],
                 gate: Optional[torch.Tensor], gelu: bool,
                 out: Optional[torch.Tensor],
                 out_amax: Optional[torch.Tensor] = None) -> torch.Tensor:
    a_shape, b_shape = a.shape(), b.shape()
    if len(a_shape) != 2 or len(b_shape) != 2:
        raise RuntimeError("[s4] [nvfp4] [gemm] Inputs must be 2D matrices")
    if a_shape[1] != b_shape[1]:
        raise RuntimeError("[s4] [nvfp4] [gemm] Inner dimensions must match")
    M, K = a_shape
    Nn = b_shape[0]
    dev = a._device
    if b._device != dev:
        raise RuntimeError("[s4] [nvfp4] [gemm] Operands must be on the same device")
    if K % 32 != 0 or Nn % 8 != 0:
        raise RuntimeError("[s4] [nvfp4] [gemm] K must be a multiple of 32 and N of 8")
    if out is None:
        out = torch.empty((M, Nn), dtype=torch.bfloat16, device=dev)
    elif out.shape != (M, Nn) or out.dtype != torch.bfloat16 or not out.is_contiguous():
        raise RuntimeError("[s4] [nvfp4] [gemm] out must be a contiguous BFloat16 [M, N] tensor")
    for name, t, shape, dt in (("C", c, (M, Nn), torch.bfloat16), ("bias", bias, (Nn,), torch.bfloat16),
                               ("gate", gate, (Nn,), torch.float32)):
        if t is not None and (tuple(t.shape) != shape or t.dtype != dt or not t.is_contiguous()
                              or t.device != dev):
            raise RuntimeError(f"[s4] [nvfp4] [gemm] {name} must be contiguous {dt} {list(shape)}")
    with torch.cuda.device(dev):
        rc = N.lib.nvfp4_gemm(N.ptr(a._data), N.ptr(b._data), N.ptr(a.scale_factors_swizzled()),
                              N.ptr(b.scale_factors_swizzled()), N.ptr(a._gscale),
                              N.ptr(b._gscale), M, Nn, K, float(alpha), float(beta), N.ptr(c),
                              N.ptr(bias), N.ptr(gate),
                              N.ACT_GELU_TANH if gelu else N.ACT_NONE, N.ptr(out),
                              N.ptr(out_amax), N.ptr(N.status_word(dev)), N.stream_ptr())
    N.check(rc, "[gemm] launch")
    return out


def fp4_gemm(A: FP4Tensor, B: FP4Tensor, alpha: float = 1.0, beta: float = 0.0, *,
             C: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
             gate: Optional[torch.Tensor] = None, gelu: bool = False,
             out: Optional[torch.Tensor] = None,
             out_amax: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``alpha * A @ B.T + beta * C`` on pre-quantized operands
    (fx/src/s4/nvfp4/tensor.h:126-143).  The reference always passes a zero C
    (kernel.cu:109), which is what ``C=None`` means here.  ``out_amax`` (a one-element
    fp32 device tensor) receives max|output|, sparing the next quantizer its amax pass."""
    if out_amax is not None and (out_amax.dtype != torch.float32 or out_amax.numel() != 1):
        raise RuntimeError("[s4] [nvfp4] [gemm] out_amax must be a one-element float32 tensor")
    if C is not None and beta == 0.0:
        # beta keeps the reference's default of 0, under which a C would be silently ignored
        raise RuntimeError("[s4] [nvfp4] [gemm] C given with beta == 0: pass the beta to apply")
    return _gemm_packed(A, B, alpha, beta, C, bias, gate, gelu, out, out_amax)


class StackedWeights:
    """Several packed ``[rows, K]`` weights stacked along N so that one GEMM launch serves them
    all, each keeping its own FP32 tensor scale (additive; ``nvfp4_gemm_stacked``).  Used for
    the text K/V projections of all DiT blocks, computed once per step before the block loop
    as the reference's TE model does (fx/src/s4/models/wan22/wan_transformer_megaupload.py:
    379-382,411-426).  ``rows`` must be a multiple of 256.  The given tensors are re-pointed
    at their slices of the stacked buffers, so the weights are not held twice."""

    def __init__(self, weights: Sequence[FP4Tensor], biases: Optional[Sequence[torch.Tensor]] = None):
        first = weights[0]
        rows, k = first.shape()
        if rows % 256 != 0:
            raise RuntimeError("[s4] [nvfp4] [gemm] stacked weights need rows % 256 == 0")
        for w in weights:
            if w.shape() != [rows, k] or w._device != first._device:
                raise RuntimeError("[s4] [nvfp4] [gemm] stacked weights must share shape and device")
        self.rows, self.k, self.count, self.device = rows, k, len(weights), first._device
        self.data = torch.cat([w._data for w in weights])
        self.scales_swz = torch.cat([w.scale_factors_swizzled() for w in weights])
        self.gscales = torch.cat([w._gscale for w in weights])
        self.bias = torch.cat([b.reshape(-1) for b in biases]).contiguous() if biases is not None else None
        nd, ns = first._data.numel(), first._scales_swz.numel()
        for i, w in enumerate(weights):
            w._data = self.data[i * nd:(i + 1) * nd]
            w._scales_swz = self.scales_swz[i * ns:(i + 1) * ns]
            w._gscale = self.gscales[i:i + 1]

    def gemm(self, a: FP4Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``[M, K]`` packed activation -> bf16 ``[M, rows * count]``; columns
        ``[i*rows, (i+1)*rows)`` are ``a @ weight_i.T + bias_i``."""
        m, k = a.shape()
        if k != self.k or a._device != self.device:
            raise RuntimeError("[s4] [nvfp4] [gemm] Inner dimensions must match")
        n = self.rows * self.count
        if out is None:
            out = torch.empty((m, n), dtype=torch.bfloat16, device=self.device)
        with torch.cuda.device(self.device):
            rc = N.lib.nvfp4_gemm_stacked(N.ptr(a._data), N.ptr(self.data),
                                          N.ptr(a.scale_factors_swizzled()), N.ptr(self.scales_swz),
                                          N.ptr(a._gscale), N.ptr(self.gscales), self.rows, m, n, k,
                                          N.ptr(self.bias), N.ptr(out),
                                          N.ptr(N.status_word(self.device)), N.stream_ptr())
        N.check(rc, "[gemm] stacked launch")
        return out


def gemm_fp4_quantized(A: torch.Tensor, B: torch.Tensor, alpha: float = 1.0, beta: float = 0.0,
                       mode: QuantizationMode = QuantizationMode.block_1d, **kw) -> torch.Tensor:
    """Quantize both bf16 operands, then ``fp4_gemm`` (tensor.h:145-154)."""
    a = FP4Tensor.from_bfloat16(A, mode, linear_scales=False)
    b = FP4Tensor.from_bfloat16(B, mode, linear_scales=False)
    return fp4_gemm(a, b, alpha, beta, **kw)


def blackwell_fp4_gemm(A: torch.Tensor, B: torch.Tensor, alpha: float = 1.0,
                       beta: float = 0.0, **kw) -> torch.Tensor:
    """bf16 ``[M,K] x [N,K] -> [M,N]`` with automatic quantization
    (declared at fx/src/s4/nvfp4/kernel.cuh:8-10, bound at bindings.cpp:70-73).
    Unlike the reference, dimensions need not be multiples of 128."""
    for t in (A, B):
        if not t.is_cuda:
            raise RuntimeError("[fxy] [ops] [nvfp4] Tensors must be on CUDA device")
        if t.dtype != torch.bfloat16:
            raise RuntimeError("[fxy] [ops] [nvfp4] Tensors must be BFloat16")
        if t.dim() != 2:
            raise RuntimeError("[fxy] [ops] [nvfp4] Tensors must be 2D matrices")
    return gemm_fp4_quantized(A, B, alpha, beta, **kw)


def is_aligned(M: int, N: int, K: int) -> bool:  # bindings.cpp:86-91
    return M % 128 == 0 and N % 128 == 0 and K % 128 == 0


def get_aligned_dims(M: int, N: int, K: int):  # bindings.cpp:93-99
    return ((M + 127) // 128 * 128, (N + 127) // 128 * 128, (K + 127) // 128 * 128)


def benchmark(A: torch.Tensor, B: torch.Tensor, iterations: int = 100):
    """``(avg_ms, TFLOPS)`` of ``blackwell_fp4_gemm`` (bindings.cpp:101-130):
    10 warm-up runs, then ``iterations`` timed runs, 2*M*N*K flops each.  Timed
    with CUDA events on the current stream instead of the host clock."""
    for _ in range(10):
        blackwell_fp4_gemm(A, B, 1.0, 0.0)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iterations):
        blackwell_fp4_gemm(A, B, 1.0, 0.0)
    end.record()
    torch.cuda.synchronize()
    avg_ms = start.elapsed_time(end) / iterations
    M, K = A.shape
    tflops = 2.0 * M * B.shape[0] * K / avg_ms / 1e9
    return avg_ms, tflops


_TILINGS = {"auto": 0, "uniform": 1, "alternating": 2}


def set_gemm_tiling(mode: str = "auto") -> None:
    """How the GEMM cuts N (additive; a tuning and test knob): ``"uniform"`` 256-wide tiles,
    ``"alternating"`` 256/192-wide tiles on two disjoint accumulators, ``"auto"`` (default) by
    shape.  The results are bit-identical either way."""
    if mode not in _TILINGS:
        raise RuntimeError(f"[s4] [nvfp4] [gemm] unknown tiling {mode!r}")
    N.check(N.lib.nvfp4_gemm_set_tiling(_TILINGS[mode]), "[gemm] tiling")


def check_status() -> None:
    """Synchronise and raise if a GEMM kernel reported an expired wait."""
    N.check_status()


# ------------------------------------------------- torch.library registration --
# The reference binds plain pybind11 functions; registering the same entry
# points as torch custom ops lets graph capture and export see them as opaque
# nodes with known output shapes.

@torch.library.custom_op("nvfp4_b200::quantize", mutates_args=())
def _quantize_op(x: torch.Tensor) -> list[torch.Tensor]:
    t = FP4Tensor.from_bfloat16(x)
    return [t._data, t._scales, t._scales_swz, t._amax, t._gscale]


@_quantize_op.register_fake
def _(x):
    n = x.numel()
    rows, cols = (n // x.shape[-1], x.shape[-1]) if n and x.shape[-1] % 16 == 0 else (1, (n + 15) // 16 * 16)
    swz = ((rows + 255) // 256 * 2) * (((cols // 16) + 15) // 16 * 4) * 512
    u8 = dict(dtype=torch.uint8, device=x.device)
    f32 = dict(dtype=torch.float32, device=x.device)
    return [torch.empty(rows * cols // 2, **u8), torch.empty(rows * cols // 16, **u8),
            torch.empty(swz, **u8), torch.empty(1, **f32), torch.empty(1, **f32)]


@torch.library.custom_op("nvfp4_b200::linear", mutates_args=())
def _linear_op(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
               gelu: bool) -> torch.Tensor:
    from . import nvfp4_linear_cpp
    return nvfp4_linear_cpp.linear(x, weight, bias, gelu=gelu)


@_linear_op.register_fake
def _(x, weight, bias, gelu):
    return x.new_empty((*x.shape[:-1], weight.shape[0]))
