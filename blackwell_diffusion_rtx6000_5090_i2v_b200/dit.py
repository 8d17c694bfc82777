"""Shape-faithful Wan 2.2 DiT step whose linears all run on the NVFP4 path.

Random-initialised (no checkpoint is used) model with the block structure of
the reference transformer (fx/src/s4/models/wan22/wan_transformer.py:189-225
for the block, :389-441 for the step): adaLN-modulated self-attention with q/k
RMSNorm across heads and 3-D RoPE, cross-attention over the text context, and a
GELU-tanh feed-forward.  It exists to measure the step latency of the
benchmark configurations and to check the NVFP4 path end to end, not as a
model implementation: attention is torch's scaled-dot-product attention in
bf16 and the small embedders are torch ops.

Two ways of evaluating a linear share the same packed weights:
  * ``nvfp4``   -- fused norm+modulation+quantize, tcgen05 FP4 GEMM with bias /
                   GELU / gate / residual in its epilogue, fused q/k RMSNorm +
                   RoPE between the QKV linear and attention (the product path);
  * ``dequant`` -- quantize, dequantize both operands to fp32, fp32 matmul (no
                   TF32), then the same elementwise ops in torch: the
                   dequantize-then-matmul formulation, used as the comparison
                   for the cosine check.  Operands stay fp32 on purpose: FP4
                   re-quantization of the next linear's input turns a
                   perturbation of relative size e into an error of about
                   sqrt(e * step), so a comparison path that rounds its operands
                   to bf16 (2^-9 per value) drifts by percents within a few
                   linears and would measure its own rounding, not the kernel.

With a process group the token sequence is sharded over the ranks (weights
replicated) and only self-attention communicates (``ulysses.py``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import _native as N
from . import ulysses
from .nvfp4 import FP4Tensor, PackedBuffers, StackedWeights, fp4_gemm


@dataclass(frozen=True)
class WanDiTConfig:
    dim: int
    heads: int
    ffn: int
    layers: int
    in_channels: int
    out_channels: int
    text_dim: int = 4096
    freq_dim: int = 256
    head_dim: int = 128
    patch: Tuple[int, int, int] = (1, 2, 2)
    eps: float = 1e-6
    rope_theta: float = 10000.0


# Wan2.2-TI2V-5B shape: latent [48, 31, 44, 80] -> 27280 tokens
WAN22_TI2V_5B = WanDiTConfig(dim=3072, heads=24, ffn=14336, layers=30, in_channels=48,
                             out_channels=48)
# Wan2.2-A14B shape (one expert): latent [16, 21, 60, 104] -> 32760 tokens
WAN22_A14B = WanDiTConfig(dim=5120, heads=40, ffn=13824, layers=40, in_channels=16,
                          out_channels=16)


def _cosine(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double().flatten(), b.double().flatten()
    return float(torch.dot(a, b) / (a.norm() * b.norm()))


class Timeline:
    """Per-component device time of a step: ``mark(label)`` charges the time since the previous
    mark to ``label``.  Events only; nothing synchronizes until :meth:`totals_ms`."""

    def __init__(self):
        self.events: List[Tuple[str, torch.cuda.Event]] = []

    def mark(self, label: str) -> None:
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self.events.append((label, e))

    def totals_ms(self) -> Dict[str, float]:
        torch.cuda.synchronize()
        out: Dict[str, float] = {}
        for (_, e0), (label, e1) in zip(self.events, self.events[1:]):
            out[label] = out.get(label, 0.0) + e0.elapsed_time(e1)
        return out


TIMELINE: Optional[Timeline] = None     # set by the step benchmark; None costs nothing


def _mark(label: str) -> None:
    if TIMELINE is not None:
        TIMELINE.mark(label)


# Tensor amax of every activation the NVFP4 path quantizes, by linear name: filled while
# AMAX_RECORD is a dict, and forced onto the comparison model's quantizers while AMAX_PIN is one
# (the comparison then shares only the per-tensor FP32 scale with the NVFP4 path; block scales
# and elements are still derived from its own activations).
AMAX_RECORD: Optional[Dict[str, torch.Tensor]] = None
AMAX_PIN: Optional[Dict[str, torch.Tensor]] = None
# The packed activation itself (nibbles, linear scales, amax) of every linear, by name: filled
# by either evaluation mode while QUANT_RECORD is a dict; while QUANT_PIN is one, the comparison
# model feeds each linear the recorded packed activation instead of quantizing its own input
# (everything else -- matmul, epilogue, norms, attention, residual stream -- stays its own).
QUANT_RECORD: Optional[Dict[str, FP4Tensor]] = None
QUANT_PIN: Optional[Dict[str, FP4Tensor]] = None


def _want_linear_scales() -> bool:
    return QUANT_RECORD is not None


def _record_amax(lin: "PackedLinear", t: FP4Tensor) -> FP4Tensor:
    if AMAX_RECORD is not None:
        AMAX_RECORD[lin.name] = t.global_amax().clone()
    if QUANT_RECORD is not None:
        QUANT_RECORD[lin.name] = t.snapshot()
    return t


def flip_stats(a: Dict[str, FP4Tensor], b: Dict[str, FP4Tensor]) -> Dict[str, Dict[str, float]]:
    """Per linear name present in both records: the fraction of element codes and of block
    scale bytes that differ between the two packed activations, and whether the tensor amax
    does -- where two trajectories of the step part ways, and through which of the three."""
    out = {}
    for name, ta in a.items():
        tb = b.get(name)
        if tb is None or ta.shape() != tb.shape():
            continue
        da, db = ta.quantized_data(), tb.quantized_data()
        nib = ((da ^ db) & 0x0F).ne(0).float().mean() + ((da ^ db) & 0xF0).ne(0).float().mean()
        out[name] = {"nibbles_differ": float(nib) / 2,
                     "block_scales_differ": float(ta.scale_factors().ne(tb.scale_factors()).float().mean()),
                     "amax_differs": bool(ta.global_amax().item() != tb.global_amax().item())}
    return out


_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def dequant_f32(t: FP4Tensor) -> torch.Tensor:
    """fp32 ``e2m1 * (float(sf) / S_enc)`` of a packed tensor that carries linear scales, in
    torch ops (comparison path only; formula of fx/src/s4/nvfp4/quantization_te.cu:149-160)."""
    rows, cols = t._rows, t._cols
    b = t.quantized_data().view(rows, cols // 2)
    tbl = torch.tensor(_E2M1 + tuple(-v for v in _E2M1), dtype=torch.float32, device=b.device)
    vals = torch.stack([tbl[(b & 0xF).long()], tbl[(b >> 4).long()]], dim=-1).view(rows, cols)
    amax = t.global_amax().float()
    fmax = torch.finfo(torch.float32).max
    s_enc = torch.clamp(torch.tensor(448.0 * 6.0, device=b.device) / amax, max=fmax)
    s_enc = torch.where((amax == 0) | (s_enc == 0), torch.ones_like(s_enc), s_enc)
    sf = t.scale_factors().view(torch.float8_e4m3fn).float().view(rows, cols // 16) / s_enc
    return (vals.view(rows, cols // 16, 16) * sf.unsqueeze(-1)).view(rows, cols)


class PackedLinear:
    """A linear whose weight lives only in packed NVFP4 form (bias in bf16)."""

    def __init__(self, n: int, k: int, gen: torch.Generator, device, std: float = 0.02,
                 bias: bool = True, name: str = ""):
        w = (torch.randn(n, k, generator=gen, device=device) * std).to(torch.bfloat16)
        self.n, self.k, self.name = n, k, name
        self.w = FP4Tensor.from_bfloat16(w, linear_scales=True)
        self.bias = ((torch.randn(n, generator=gen, device=device) * 0.01).to(torch.bfloat16)
                     if bias else None)

    def nvfp4(self, a: FP4Tensor, **epilogue) -> torch.Tensor:
        return fp4_gemm(a, self.w, bias=self.bias, **epilogue)

    def dequant(self, x: torch.Tensor, *, gelu: bool = False, gate: Optional[torch.Tensor] = None,
                residual: Optional[torch.Tensor] = None, reorder: bool = False) -> torch.Tensor:
        """Quantize x, dequantize both operands, matmul: the comparison path.  ``reorder``
        reverses the K axis of both operands -- the same sum in another order, which serves as
        the control for how much a last-bit change in a GEMM moves the step output."""
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        if QUANT_PIN is not None and self.name in QUANT_PIN:
            xt = QUANT_PIN[self.name]
        else:
            pinned = AMAX_PIN.get(self.name) if AMAX_PIN is not None else None
            xt = FP4Tensor.from_bfloat16(x2, linear_scales=True, amax=pinned)
        if QUANT_RECORD is not None:
            QUANT_RECORD[self.name] = xt.snapshot()
        xq = dequant_f32(xt)
        wq = dequant_f32(self.w)
        if reorder:
            xq, wq = xq.flip(-1).contiguous(), wq.flip(-1).contiguous()
        tf32 = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False
        try:
            y = torch.matmul(xq, wq.t())
        finally:
            torch.backends.cuda.matmul.allow_tf32 = tf32
        if self.bias is not None:
            y = y + self.bias.float()
        if gelu:
            y = F.gelu(y, approximate="tanh")
        if gate is not None:
            y = y * gate
        if residual is not None:
            y = y + residual.float()
        return y.to(torch.bfloat16)


def rope_tables(cfg: WanDiTConfig, grid: Tuple[int, int, int], device) -> Tuple[torch.Tensor, torch.Tensor]:
    """3-D rotary tables ``[L, head_dim]`` (cos, sin): per axis the 1-D table of
    fx/src/s4/models/wan_22/wan_attention_static.py:49-58 (inverse frequencies
    theta^(-2i/d), each frequency repeated for its pair), axes t/h/w taking 44/42/42 of the
    128 head dims (fx/src/s4/models/wan22/wan_transformer.py:274-275,309-335)."""
    f, h, w = grid
    hd = cfg.head_dim
    h_dim = w_dim = 2 * (hd // 6)
    t_dim = hd - h_dim - w_dim

    def axis(dim, n):
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, dim, 2, dtype=torch.float64) / dim))
        ang = torch.arange(n, dtype=torch.float64).unsqueeze(1) * inv.unsqueeze(0)
        ang = ang.repeat_interleave(2, dim=1)            # [n, dim]: (a0, a0, a1, a1, ...)
        return ang.cos().float(), ang.sin().float()

    ct, st = axis(t_dim, f)
    ch, sh = axis(h_dim, h)
    cw, sw = axis(w_dim, w)
    cos = torch.cat([ct.view(f, 1, 1, -1).expand(f, h, w, -1), ch.view(1, h, 1, -1).expand(f, h, w, -1),
                     cw.view(1, 1, w, -1).expand(f, h, w, -1)], dim=-1).reshape(f * h * w, hd)
    sin = torch.cat([st.view(f, 1, 1, -1).expand(f, h, w, -1), sh.view(1, h, 1, -1).expand(f, h, w, -1),
                     sw.view(1, 1, w, -1).expand(f, h, w, -1)], dim=-1).reshape(f * h * w, hd)
    return cos.to(device), sin.to(device)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x ``[L, H, D]``; pairs (even, odd) rotate by the pair's angle
    (fx/src/s4/models/wan22/wan_transformer.py:61-75)."""
    xf = x.float()
    x1, x2 = xf[..., 0::2], xf[..., 1::2]
    c, s = cos[:, None, 0::2], sin[:, None, 1::2]
    out = torch.empty_like(xf)
    out[..., 0::2] = x1 * c - x2 * s
    out[..., 1::2] = x1 * s + x2 * c
    return out.to(x.dtype)


def pack_rope_table(cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``[L, D]`` cos / sin tables -> fp32 ``[L, D/2, 2]`` holding, for each rotated pair, the
    two entries :func:`apply_rope` uses (``cos[:, 0::2]`` and ``sin[:, 1::2]``)."""
    return torch.stack([cos[:, 0::2], sin[:, 1::2]], dim=-1).contiguous()


def qk_norm_rope(qkv: torch.Tensor, heads: int, head_dim: int, gain_q: Optional[torch.Tensor],
                 gain_k: Optional[torch.Tensor], eps: float, cos_sin: torch.Tensor,
                 packed: bool = False):
    """RMSNorm across heads of q and k, then the rotary embedding, in one kernel over the
    ``[L, 3*dim]`` output of the QKV linear (the fused form of ``rms_norm`` + ``apply_rope``
    below).  Returns ``(q, k, v)`` as ``[L, heads, head_dim]`` tensors -- v is a view of
    ``qkv`` -- or, with ``packed``, one ``[L, heads, 3*head_dim]`` tensor holding q | k | v per
    head, the layout the head/sequence exchange sends."""
    L, three_dim = qkv.shape
    dim = heads * head_dim
    if three_dim != 3 * dim or qkv.dtype != torch.bfloat16 or not qkv.is_contiguous():
        raise RuntimeError("qk_norm_rope: qkv must be a contiguous bf16 [L, 3*heads*head_dim] tensor")
    if cos_sin.shape != (L, head_dim // 2, 2) or cos_sin.dtype != torch.float32 or \
            not cos_sin.is_contiguous():
        raise RuntimeError("qk_norm_rope: cos_sin must be a contiguous fp32 [L, head_dim/2, 2] tensor")
    base = qkv.data_ptr()
    st = N.stream_ptr()
    status = N.ptr(N.status_word(qkv.device))
    if packed:
        out = torch.empty(L, heads, 3 * head_dim, dtype=torch.bfloat16, device=qkv.device)
        o = out.data_ptr()
        N.check(N.lib.nvfp4_qk_norm_rope_bf16(base, base + 2 * dim, base + 4 * dim, 3 * dim, L, heads,
                                              head_dim, N.ptr(gain_q), N.ptr(gain_k), float(eps),
                                              N.ptr(cos_sin), o, o + 2 * head_dim, o + 4 * head_dim,
                                              3 * dim, 3 * head_dim, status, st), "qk_norm_rope")
        return out
    q = torch.empty(L, heads, head_dim, dtype=torch.bfloat16, device=qkv.device)
    k = torch.empty_like(q)
    N.check(N.lib.nvfp4_qk_norm_rope_bf16(base, base + 2 * dim, None, 3 * dim, L, heads, head_dim,
                                          N.ptr(gain_q), N.ptr(gain_k), float(eps), N.ptr(cos_sin),
                                          q.data_ptr(), k.data_ptr(), None, dim, head_dim, status, st),
            "qk_norm_rope")
    return q, k, qkv[:, 2 * dim:].view(L, heads, head_dim)


def rms_norm_fused(x: torch.Tensor, heads: int, head_dim: int, gain: Optional[torch.Tensor],
                   eps: float) -> torch.Tensor:
    """RMSNorm over the last axis of a bf16 ``[L, heads*head_dim]`` tensor (rows may be a strided
    view, e.g. a column block of a wider matrix) with the same kernel (no rotation); returns a
    contiguous ``[L, heads, head_dim]``."""
    L, dim = x.shape
    if dim != heads * head_dim or x.dtype != torch.bfloat16 or x.stride(1) != 1 or \
            x.stride(0) % 8 != 0 or x.data_ptr() % 16 != 0:
        raise RuntimeError("rms_norm_fused: x must be a bf16 [L, heads*head_dim] tensor with unit "
                           "inner stride and 16-byte aligned rows")
    out = torch.empty(L, heads, head_dim, dtype=torch.bfloat16, device=x.device)
    N.check(N.lib.nvfp4_qk_norm_rope_bf16(x.data_ptr(), None, None, x.stride(0), L, heads, head_dim,
                                          N.ptr(gain), None, float(eps), None, out.data_ptr(), None,
                                          None, dim, head_dim, N.ptr(N.status_word(x.device)),
                                          N.stream_ptr()), "rms_norm")
    return out


def rms_norm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * gain).to(x.dtype)


def layer_norm(x: torch.Tensor, eps: float, weight=None, bias=None) -> torch.Tensor:
    return F.layer_norm(x.float(), (x.shape[-1],), weight, bias, eps)


# "library": torch's scaled_dot_product_attention; "native": this package's tcgen05 kernel
ATTENTION_BACKEND = "library"


def attention_native(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                     amax: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The package's own attention kernel (head dimension 128): ``[Lq, H, D]`` x ``[Lk, H, D]`` ->
    ``[Lq, H, D]`` bf16, non-causal, scale 1/sqrt(D); q, k, v may be strided views (last
    dimension contiguous).  ``amax``: a zeroed one-element fp32 tensor that receives max|o|."""
    Lq, H, D = q.shape
    Lk = k.shape[0]
    for t in (q, k, v):
        if t.dtype != torch.bfloat16 or t.stride(2) != 1 or t.shape[1:] != (H, D):
            raise ValueError("attention_native wants bf16 [L, H, D] tensors with a contiguous last dimension")
    if out is None:
        out = torch.empty(Lq, H, D, dtype=torch.bfloat16, device=q.device)
    N.check(N.lib.nvfp4_attention_bf16(
        q.data_ptr(), q.stride(0), q.stride(1), k.data_ptr(), k.stride(0), k.stride(1),
        v.data_ptr(), v.stride(0), v.stride(1), Lq, Lk, H, D, 1.0 / D ** 0.5, out.data_ptr(),
        out.stride(0), out.stride(1), None if amax is None else amax.data_ptr(),
        N.ptr(N.status_word(q.device)), N.stream_ptr()), "attention")
    return out


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """``[Lq, H, D]`` x ``[Lk, H, D]`` -> ``[Lq, H, D]``, bf16, non-causal, scale 1/sqrt(D)."""
    if ATTENTION_BACKEND == "native":
        return attention_native(q, k, v)
    o = F.scaled_dot_product_attention(q.transpose(0, 1).unsqueeze(0), k.transpose(0, 1).unsqueeze(0),
                                       v.transpose(0, 1).unsqueeze(0))
    return o.squeeze(0).transpose(0, 1)


class ActivationScratch:
    """Packed-activation buffers of a step, one set per activation shape: every quantizer of the
    block loop writes into them instead of allocating (the ``out=`` form; the block-linears
    runner preallocates the same way)."""

    def __init__(self, device):
        self.device = device
        self._bufs: Dict[Tuple[int, int], PackedBuffers] = {}

    def get(self, rows: int, cols: int) -> PackedBuffers:
        key = (rows, cols)
        if key not in self._bufs:
            self._bufs[key] = PackedBuffers(rows, cols, self.device)
        return self._bufs[key]


class WanBlock:
    def __init__(self, cfg: WanDiTConfig, gen: torch.Generator, device, name: str = "block"):
        d = cfg.dim
        self.cfg = cfg
        self.qkv = PackedLinear(3 * d, d, gen, device, name=f"{name}.qkv")
        self.attn_out = PackedLinear(d, d, gen, device, name=f"{name}.attn_out")
        self.cross_q = PackedLinear(d, d, gen, device, name=f"{name}.cross_q")
        self.cross_kv = PackedLinear(2 * d, d, gen, device, name=f"{name}.cross_kv")
        self.cross_out = PackedLinear(d, d, gen, device, name=f"{name}.cross_out")
        self.ffn_up = PackedLinear(cfg.ffn, d, gen, device, name=f"{name}.ffn_up")
        self.ffn_down = PackedLinear(d, cfg.ffn, gen, device, name=f"{name}.ffn_down")
        ones = lambda: torch.ones(d, device=device)  # noqa: E731
        self.g_q, self.g_k, self.g_cq, self.g_ck = ones(), ones(), ones(), ones()  # unit RMSNorm gains
        self.norm2_w, self.norm2_b = ones(), torch.zeros(d, device=device)
        self.scale_shift_table = torch.randn(6, d, generator=gen, device=device) / d ** 0.5
        self._amax = torch.empty(1, dtype=torch.float32, device=device)

    # ---------------------------------------------------------------- parts --
    def _self_attention_fused(self, qkv, cos_sin, group, px=None):
        """nvfp4 path: one kernel between the QKV linear and attention (or the exchange).
        Returns ``(o [L, dim], amax of o or None)``."""
        cfg = self.cfg
        L = qkv.shape[0]
        dim = cfg.dim
        base = qkv.data_ptr()
        if px is not None:
            # exchange by stores into peer memory, fused into the norm + RoPE kernel; its last
            # CTA raises the flags the wait below polls
            N.check(N.lib.nvfp4_qk_norm_rope_exchange_bf16(
                base, base + 2 * dim, base + 4 * dim, 3 * dim, L, cfg.heads, cfg.head_dim,
                N.ptr(self.g_q), N.ptr(self.g_k), float(cfg.eps), N.ptr(cos_sin),
                px.qkv_ptrs[px.turn], px.P, px.rank * px.Lp, px.sync_ptrs, px.rank,
                N.ptr(N.status_word(qkv.device)), N.stream_ptr()), "qk_norm_rope_exchange")
            _mark("qk_norm_rope")
            px.wait(0)
            q, k, v = px.qkv[px.turn].split(cfg.head_dim, dim=-1)
            _mark("exchange")
            o = attention(q, k, v)
            _mark("self_attention")
            o, amax = px.return_attention_output(o)
            _mark("exchange")
            return o.reshape(L, cfg.dim), amax
        if group is None:
            q, k, v = qk_norm_rope(qkv, cfg.heads, cfg.head_dim, self.g_q, self.g_k, cfg.eps, cos_sin)
            _mark("qk_norm_rope")
        else:
            # the kernel writes its pieces grouped by destination rank, [P, L/P, H/P, 3D]: the
            # all-to-all's send buffer, with no packing copy in between
            import ctypes
            P = dist.get_world_size(group)
            Hp = cfg.heads // P
            send = torch.empty(P, L, Hp, 3 * cfg.head_dim, dtype=torch.bfloat16, device=qkv.device)
            ptrs = (ctypes.c_void_p * P)(*[send[r].data_ptr() for r in range(P)])
            N.check(N.lib.nvfp4_qk_norm_rope_exchange_bf16(
                base, base + 2 * dim, base + 4 * dim, 3 * dim, L, cfg.heads, cfg.head_dim,
                N.ptr(self.g_q), N.ptr(self.g_k), float(cfg.eps), N.ptr(cos_sin), ptrs, P, 0, None, 0,
                N.ptr(N.status_word(qkv.device)), N.stream_ptr()), "qk_norm_rope (send layout)")
            _mark("qk_norm_rope")
            q, k, v = ulysses.all_to_all_packed(send, group).split(cfg.head_dim, dim=-1)
            _mark("exchange")
        amax = None
        if ATTENTION_BACKEND == "native" and group is None:
            # the kernel folds max|o| into its epilogue: the quantizer in front of the
            # attention-out linear gets its amax from here
            amax = self._amax.zero_()
            o = attention_native(q, k, v, amax=amax)
        else:
            o = attention(q, k, v)
        _mark("self_attention")
        if group is not None:
            o = ulysses.heads_to_seq(o.contiguous(), group)
            _mark("exchange")
        return o.reshape(L, cfg.dim), amax

    def _self_attention(self, q, k, v, cos, sin, group):
        cfg = self.cfg
        L = q.shape[0]
        q = apply_rope(rms_norm(q, self.g_q, cfg.eps).view(L, cfg.heads, cfg.head_dim), cos, sin)
        k = apply_rope(rms_norm(k, self.g_k, cfg.eps).view(L, cfg.heads, cfg.head_dim), cos, sin)
        v = v.reshape(L, cfg.heads, cfg.head_dim)
        _mark("qk_norm_rope")
        if group is not None:
            # token shards -> head shards: one packed exchange for q, k, v
            qkv = ulysses.seq_to_heads(torch.cat([q, k, v], dim=-1), group)
            q, k, v = qkv.split(cfg.head_dim, dim=-1)
            _mark("exchange")
        o = attention(q, k, v)
        _mark("self_attention")
        if group is not None:
            o = ulysses.heads_to_seq(o.contiguous(), group)
            _mark("exchange")
        return o.reshape(L, cfg.dim)

    def _cross_kv(self, ctx: torch.Tensor, mode: str):
        cfg = self.cfg
        kv = (self.cross_kv.nvfp4(_record_amax(self.cross_kv, FP4Tensor.from_bfloat16(
            ctx, linear_scales=_want_linear_scales())))
              if mode == "nvfp4" else self.cross_kv.dequant(ctx, reorder=mode == "dequant_reordered"))
        return self._split_text_kv(kv)

    def _split_text_kv(self, kv: torch.Tensor, fused: bool = False):
        """``[C, 2*dim]`` projection of the text context -> normalised k and v, ``[C, heads, D]``.
        ``fused``: the RMSNorm of k by the library's kernel (one launch, straight off the column
        block of the stacked projection) instead of the separate torch ops."""
        cfg = self.cfg
        k, v = kv.chunk(2, dim=-1)
        C = kv.shape[0]
        kn = (rms_norm_fused(k, cfg.heads, cfg.head_dim, self.g_ck, cfg.eps) if fused
              else rms_norm(k, self.g_ck, cfg.eps).view(C, cfg.heads, cfg.head_dim))
        return kn, v.reshape(C, cfg.heads, cfg.head_dim)

    # -------------------------------------------------------------- forward --
    def forward(self, x: torch.Tensor, ctx: torch.Tensor, temb6: torch.Tensor, cos, sin,
                mode: str = "nvfp4", group=None, cos_sin: Optional[torch.Tensor] = None,
                px: Optional[ulysses.PeerExchange] = None, text_kv=None,
                amax_hook=None, scratch: Optional["ActivationScratch"] = None) -> torch.Tensor:
        """``text_kv``: this block's cross-attention ``(k, v)`` when the step computed them
        for all blocks ahead of the loop.  ``amax_hook(t)``: called on every activation's
        one-element amax tensor between the amax pass and the packing pass (sharded runs use it
        to all-reduce the maximum, which makes every shard quantize with the full tensor's
        scale).  ``scratch``: preallocated buffers for the packed activations (shared by all
        blocks of a step: each packed activation is consumed by the GEMM that follows it)."""
        cfg = self.cfg
        mod = self.scale_shift_table + temb6.float()
        shift_msa, scale_msa, gate_msa, c_shift, c_scale, c_gate = (m.contiguous() for m in mod)
        L = x.shape[0]
        if mode == "nvfp4":
            if cos_sin is None:
                cos_sin = pack_rope_table(cos, sin)
            _mark("other")
            ls = _want_linear_scales()
            # a recording keeps the packed tensors, so it gets fresh ones
            buf = (lambda t, cols: scratch.get(t.shape[0], cols)) if scratch is not None and not ls \
                else (lambda t, cols: None)
            a = _record_amax(self.qkv, FP4Tensor.from_norm_mod(x, scale=scale_msa, shift=shift_msa,
                                                               eps=cfg.eps, amax_hook=amax_hook,
                                                               linear_scales=ls, out=buf(x, cfg.dim)))
            _mark("norm_quantize")
            qkv = self.qkv.nvfp4(a)
            _mark("gemm_qkv")
            o, o_amax = self._self_attention_fused(qkv, cos_sin, group, px)
            if o_amax is not None and amax_hook is not None:
                amax_hook(o_amax)
            # with the peer exchange the return kernel has already taken max|o|
            oq = _record_amax(self.attn_out, FP4Tensor.from_bfloat16(
                o.contiguous(), linear_scales=ls, amax=o_amax,
                amax_hook=None if o_amax is not None else amax_hook, out=buf(o, cfg.dim)))
            _mark("quantize")
            x = self.attn_out.nvfp4(oq, gate=gate_msa, C=x, beta=1.0)
            _mark("gemm_attn_out")
            a = _record_amax(self.cross_q, FP4Tensor.from_norm_mod(
                x, weight=self.norm2_w, bias=self.norm2_b, eps=cfg.eps, amax_hook=amax_hook,
                linear_scales=ls, out=buf(x, cfg.dim)))
            _mark("norm_quantize")
            q = self.cross_q.nvfp4(a)
            _mark("gemm_cross_q")
            q = rms_norm_fused(q, cfg.heads, cfg.head_dim, self.g_cq, cfg.eps)
            _mark("qk_norm_rope")
            if text_kv is None:
                text_kv = self._cross_kv(ctx, mode)
                _mark("text_kv")
            ck, cv = text_kv
            o = attention(q, ck, cv).reshape(L, cfg.dim)
            _mark("cross_attention")
            oq = _record_amax(self.cross_out, FP4Tensor.from_bfloat16(o.contiguous(), linear_scales=ls,
                                                                      amax_hook=amax_hook,
                                                                      out=buf(o, cfg.dim)))
            _mark("quantize")
            x = self.cross_out.nvfp4(oq, C=x, beta=1.0)
            _mark("gemm_cross_out")
            a = _record_amax(self.ffn_up, FP4Tensor.from_norm_mod(x, scale=c_scale, shift=c_shift,
                                                                  eps=cfg.eps, amax_hook=amax_hook,
                                                                  linear_scales=ls, out=buf(x, cfg.dim)))
            _mark("norm_quantize")
            hid = self.ffn_up.nvfp4(a, gelu=True, out_amax=self._amax)
            _mark("gemm_ffn_up")
            if amax_hook is not None:
                amax_hook(self._amax)
            hq = _record_amax(self.ffn_down, FP4Tensor.from_bfloat16(hid, linear_scales=ls,
                                                                     amax=self._amax,
                                                                     out=buf(hid, cfg.ffn)))
            _mark("quantize")
            x = self.ffn_down.nvfp4(hq, gate=c_gate, C=x, beta=1.0)
            _mark("gemm_ffn_down")
            return x
        # comparison path: same ops, linears by dequantize-then-matmul
        ro = mode == "dequant_reordered"
        h = (layer_norm(x, cfg.eps) * (1 + scale_msa) + shift_msa).to(x.dtype)
        q, k, v = self.qkv.dequant(h, reorder=ro).chunk(3, dim=-1)
        o = self._self_attention(q, k, v, cos, sin, group)
        x = self.attn_out.dequant(o, gate=gate_msa, residual=x, reorder=ro)
        h = layer_norm(x, cfg.eps, self.norm2_w, self.norm2_b).to(x.dtype)
        q = rms_norm(self.cross_q.dequant(h, reorder=ro), self.g_cq, cfg.eps).view(L, cfg.heads, cfg.head_dim)
        ck, cv = self._cross_kv(ctx, mode)
        o = attention(q, ck, cv).reshape(L, cfg.dim)
        x = self.cross_out.dequant(o, residual=x, reorder=ro)
        h = (layer_norm(x, cfg.eps) * (1 + c_scale) + c_shift).to(x.dtype)
        hid = self.ffn_up.dequant(h, gelu=True, reorder=ro)
        return self.ffn_down.dequant(hid, gate=c_gate, residual=x, reorder=ro)


class WanDiT:
    """One denoising step of the DiT (timestep + text conditioning -> blocks -> output head)."""

    def __init__(self, cfg: WanDiTConfig, device="cuda", seed: int = 1234, layers: Optional[int] = None):
        self.cfg = cfg
        self.device = torch.device(device)
        gen = torch.Generator(device=self.device).manual_seed(seed)
        d = cfg.dim
        pt, ph, pw = cfg.patch
        self.patch_w = (torch.randn(d, cfg.in_channels, pt, ph, pw, generator=gen, device=self.device)
                        * 0.02).to(torch.bfloat16)
        self.patch_b = torch.zeros(d, dtype=torch.bfloat16, device=self.device)
        self.time_in = PackedLinear(d, cfg.freq_dim, gen, self.device, name="time_in")
        self.time_hidden = PackedLinear(d, d, gen, self.device, name="time_hidden")
        self.time_proj = PackedLinear(6 * d, d, gen, self.device, name="time_proj")
        self.text_in = PackedLinear(d, cfg.text_dim, gen, self.device, name="text_in")
        self.text_hidden = PackedLinear(d, d, gen, self.device, name="text_hidden")
        self.blocks: List[WanBlock] = [WanBlock(cfg, gen, self.device, name=f"blocks.{i}")
                                       for i in range(layers if layers is not None else cfg.layers)]
        # The text context is the same for every block, so the cross-attention K/V projections
        # of ALL blocks (each with its own weight) run as one stacked GEMM ahead of the block
        # loop, as the reference's TE model hoists them
        # (fx/src/s4/models/wan22/wan_transformer_megaupload.py:379-382,411-426), instead of
        # one launch-bound 512-row GEMM inside every block.
        self.text_kv = (StackedWeights([b.cross_kv.w for b in self.blocks],
                                       [b.cross_kv.bias for b in self.blocks])
                        if (2 * d) % 256 == 0 and self.blocks else None)
        self._rope: Dict[Tuple[int, int, int], Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = {}
        self._px: Dict[Tuple[int, int], ulysses.PeerExchange] = {}
        self._scratch = ActivationScratch(self.device)
        self.out_table = torch.randn(2, d, generator=gen, device=self.device) / d ** 0.5
        self.proj_out = PackedLinear(cfg.out_channels * pt * ph * pw, d, gen, self.device, name="proj_out")

    def _lin(self, lin: PackedLinear, x: torch.Tensor, mode: str, **kw) -> torch.Tensor:
        if mode == "nvfp4":
            return lin.nvfp4(_record_amax(lin, FP4Tensor.from_bfloat16(x.contiguous(),
                                                                       linear_scales=_want_linear_scales())),
                             gelu=kw.get("gelu", False))
        return lin.dequant(x, gelu=kw.get("gelu", False), reorder=mode == "dequant_reordered")

    def _conditions(self, t: float, text: torch.Tensor, mode: str):
        cfg = self.cfg
        half = cfg.freq_dim // 2
        freqs = torch.exp(-math.log(10000.0) * torch.arange(half, device=self.device) / half)
        ang = t * freqs
        t_freq = torch.cat([ang.cos(), ang.sin()]).to(torch.bfloat16).unsqueeze(0)   # [1, 256]
        temb = self._lin(self.time_hidden, F.silu(self._lin(self.time_in, t_freq, mode)), mode)
        temb6 = self._lin(self.time_proj, F.silu(temb), mode).view(6, cfg.dim)
        ctx = self._lin(self.text_hidden, self._lin(self.text_in, text, mode, gelu=True), mode)
        return temb.view(cfg.dim), temb6, ctx

    def _embed(self, latent: torch.Tensor, t: float, text: torch.Tensor, mode: str):
        cfg = self.cfg
        pt, ph, pw = cfg.patch
        C, Fr, H, W = latent.shape
        grid = (Fr // pt, H // ph, W // pw)
        x = F.conv3d(latent.unsqueeze(0), self.patch_w, self.patch_b, stride=cfg.patch)
        x = x.flatten(2).squeeze(0).t().contiguous()                  # [L, dim]
        if grid not in self._rope:          # tables depend on the grid only: built once
            cos, sin = rope_tables(cfg, grid, self.device)
            self._rope[grid] = (cos, sin, pack_rope_table(cos, sin))
        cos, sin, cos_sin = self._rope[grid]
        temb, temb6, ctx = self._conditions(t, text, mode)
        return x, cos, sin, cos_sin, temb, temb6, ctx, grid

    def _head(self, x: torch.Tensor, temb: torch.Tensor, mode: str, amax_hook=None) -> torch.Tensor:
        cfg = self.cfg
        shift, scale = (m.contiguous() for m in (self.out_table + temb.float()))
        if mode == "nvfp4":
            return self.proj_out.nvfp4(_record_amax(self.proj_out, FP4Tensor.from_norm_mod(
                x, scale=scale, shift=shift, eps=cfg.eps, amax_hook=amax_hook,
                linear_scales=_want_linear_scales())))
        return self.proj_out.dequant((layer_norm(x, cfg.eps) * (1 + scale) + shift).to(x.dtype),
                                     reorder=mode == "dequant_reordered")

    def _unpatchify(self, y: torch.Tensor, grid) -> torch.Tensor:
        cfg = self.cfg
        pt, ph, pw = cfg.patch
        f, h, w = grid
        y = y.reshape(f, h, w, pt, ph, pw, cfg.out_channels).permute(6, 0, 3, 1, 4, 2, 5)
        return y.reshape(cfg.out_channels, f * pt, h * ph, w * pw)

    def _text_kv_all(self, ctx: torch.Tensor):
        """Cross-attention ``(k, v)`` of every block from one stacked GEMM over the text context."""
        two_d = 2 * self.cfg.dim
        ctx_q = FP4Tensor.from_bfloat16(ctx.contiguous(), linear_scales=_want_linear_scales())
        for blk in self.blocks:
            _record_amax(blk.cross_kv, ctx_q)
        kv = self.text_kv.gemm(ctx_q)
        return [blk._split_text_kv(kv[:, i * two_d:(i + 1) * two_d], fused=True)
                for i, blk in enumerate(self.blocks)]

    def forward(self, latent: torch.Tensor, t: float, text: torch.Tensor, mode: str = "nvfp4",
                group: Optional[dist.ProcessGroup] = None, exchange: str = "nccl",
                amax_sync: bool = False) -> torch.Tensor:
        y, grid = self.forward_tokens(latent, t, text, mode, group, exchange, amax_sync)
        return self.gather_tokens(y, grid, group)

    def gather_tokens(self, y: torch.Tensor, grid, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
        """The ranks' token shards of the head's output -> the full ``[C_out, F, H, W]`` on every
        rank (one all-gather; nothing to do on a single GPU)."""
        if group is not None and dist.get_world_size(group) > 1:
            parts = [torch.empty_like(y) for _ in range(dist.get_world_size(group))]
            dist.all_gather(parts, y.contiguous(), group=group)
            y = torch.cat(parts, dim=0)
        return self._unpatchify(y, grid)

    def forward_tokens(self, latent: torch.Tensor, t: float, text: torch.Tensor, mode: str = "nvfp4",
                       group: Optional[dist.ProcessGroup] = None, exchange: str = "nccl",
                       amax_sync: bool = False):
        """The step up to and including the output head: ``(this rank's rows of the head's output,
        token grid)``; ``gather_tokens`` finishes it.
        latent ``[C, F, H, W]`` bf16, text ``[512, 4096]`` bf16 -> ``[C_out, F, H, W]``.
        With ``group`` each rank processes its contiguous shard of the token sequence and
        returns the full output (gathered) on every rank.  ``exchange``: ``"nccl"`` (two
        all-to-alls per block) or ``"peer"`` (stores into peer memory fused into the q/k norm +
        RoPE kernel and a return kernel after attention, ordered by flags; NVFP4 mode, ranks of
        one node).  ``amax_sync``: every sharded activation is quantized with the maximum of
        the shards' amax (a 4-byte all-reduce per quantizer) instead of its own shard's, i.e.
        with the FP32 tensor scale the unsharded model uses."""
        x, cos, sin, cos_sin, temb, temb6, ctx, grid = self._embed(latent, t, text, mode)
        L = x.shape[0]
        P = dist.get_world_size(group) if group is not None else 1
        if P > 1:
            if L % P != 0:
                raise ValueError(f"tokens ({L}) must divide by the world size ({P})")
            r = dist.get_rank(group)
            sl = slice(r * (L // P), (r + 1) * (L // P))
            x, cos, sin, cos_sin = x[sl].contiguous(), cos[sl], sin[sl], cos_sin[sl].contiguous()
        px = None
        if P > 1 and exchange == "peer" and mode == "nvfp4":
            key = (L, id(group))
            if key not in self._px:
                self._px[key] = ulysses.PeerExchange(L, self.cfg.heads, self.cfg.head_dim, group, self.device)
            px = self._px[key]
        hook = None
        if P > 1 and amax_sync and mode == "nvfp4":
            def hook(amax_t: torch.Tensor) -> None:
                dist.all_reduce(amax_t, op=dist.ReduceOp.MAX, group=group)
        kvs = None
        if mode == "nvfp4" and self.text_kv is not None:
            _mark("other")
            kvs = self._text_kv_all(ctx)
            _mark("text_kv")
        for i, blk in enumerate(self.blocks):
            x = blk.forward(x, ctx, temb6, cos, sin, mode, group if P > 1 else None, cos_sin, px,
                            kvs[i] if kvs is not None else None, hook, self._scratch)
        return self._head(x, temb, mode, hook), grid

    def capture(self, latent: torch.Tensor, t: float, text: torch.Tensor,
                group: Optional[dist.ProcessGroup] = None):
        """Record one NVFP4 step into a CUDA graph (the static-shape capture of
        fx/src/s4/models/wan_22/wan_attention_static.py:566-630).  Returns ``(graph, out)``:
        ``graph.replay()`` re-runs the step on whatever ``latent`` and ``text`` then contain
        (same tensors, same timestep) and leaves the result in ``out``.  Everything the step
        launches is capturable: the library's kernels run on the current stream, never
        synchronise with the host, and take their temporaries from the torch allocator.

        With ``group`` the sharded step with the peer-store exchange is recorded: its flag waits
        keep their epochs in device memory, so every replay waits for the peers' matching replay
        (all ranks must replay the same number of times).  ``out`` is then this rank's rows of the
        head's output and ``(graph, out, grid)`` is returned; ``gather_tokens(out, grid, group)``
        (an all-gather, outside the graph) completes the step."""
        sharded = group is not None and dist.get_world_size(group) > 1
        kw = dict(group=group, exchange="peer") if sharded else {}
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            self.forward_tokens(latent, t, text, **kw)   # warm-up: tables, status word, lazy buffers
        torch.cuda.current_stream(self.device).wait_stream(side)
        if sharded:
            torch.cuda.synchronize(self.device)
            dist.barrier(group)                          # every rank's warm-up step has finished
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out, grid = self.forward_tokens(latent, t, text, **kw)
            if not sharded:
                out = self._unpatchify(out, grid)
        if sharded:
            return graph, out, grid
        return graph, out

    def compare_blocks(self, latent: torch.Tensor, t: float, text: torch.Tensor
                       ) -> List[Tuple[float, float]]:
        """Every block evaluated both ways FROM THE SAME INPUT (the NVFP4 trajectory's): per
        block ``(cosine of the outputs, cosine of the block's own contribution out - in)``.
        This is the per-block statement of parity; the free-running step comparison on top of
        it also measures how fast FP4 re-quantization amplifies last-bit differences."""
        x, cos, sin, cos_sin, temb, temb6, ctx, grid = self._embed(latent, t, text, "nvfp4")
        out = []
        kvs = self._text_kv_all(ctx) if self.text_kv is not None else None
        for i, blk in enumerate(self.blocks):
            y = blk.forward(x, ctx, temb6, cos, sin, "nvfp4", None, cos_sin,
                            text_kv=kvs[i] if kvs is not None else None)
            ref = blk.forward(x, ctx, temb6, cos, sin, "dequant")
            out.append((_cosine(y, ref), _cosine(y.float() - x.float(), ref.float() - x.float())))
            x = y
        return out

    def linear_flops(self, tokens: int, text_tokens: int = 512) -> float:
        cfg = self.cfg
        d = cfg.dim
        per_block = 2 * tokens * (3 * d * d + d * d + d * d + d * d + 2 * cfg.ffn * d) \
            + 2 * text_tokens * 2 * d * d
        return per_block * len(self.blocks)

    def attention_flops(self, tokens: int, text_tokens: int = 512) -> float:
        cfg = self.cfg
        return len(self.blocks) * 4 * cfg.dim * tokens * (tokens + text_tokens)
