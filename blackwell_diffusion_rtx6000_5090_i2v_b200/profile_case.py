"""Small fixed cases of the hot kernels, for timing or for a profiler capture.

    python -m blackwell_diffusion_rtx6000_5090_i2v_b200.profile_case gemm --m 8192 --n 9216 --k 3072
    python -m blackwell_diffusion_rtx6000_5090_i2v_b200.profile_case quantize --m 27280 --k 3072
    python -m blackwell_diffusion_rtx6000_5090_i2v_b200.profile_case norm --m 27280 --k 3072
    python -m blackwell_diffusion_rtx6000_5090_i2v_b200.profile_case rope --m 27280 --k 3072
    python -m blackwell_diffusion_rtx6000_5090_i2v_b200.profile_case return --m 32760 --k 5120
    python -m blackwell_diffusion_rtx6000_5090_i2v_b200.profile_case attention --m 27280 --k 3072

Each case holds well under a few GB on the device, launches the kernel
``--iters`` times after ``--warmup`` launches, and prints the CUDA-event time.
"""
from __future__ import annotations

import argparse

import torch

from . import _native as N
from .nvfp4 import FP4Tensor, fp4_gemm
from .synthetic import outlier_weight_bf16, student_t_bf16


def _time(fn, warmup, iters):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "quantize", "amax", "norm", "rope", "return", "attention"])
    ap.add_argument("--tiling", choices=["auto", "uniform", "alternating"], default="auto")
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=9216)
    ap.add_argument("--k", type=int, default=3072)
    ap.add_argument("--gelu", action="store_true")
    ap.add_argument("--bias", action="store_true")
    ap.add_argument("--gate", action="store_true", help="per-column fp32 gate in the epilogue")
    ap.add_argument("--residual", action="store_true", help="+ C (bf16 [m, n]) in the epilogue")
    ap.add_argument("--library", action="store_true", help="attention: time the library kernel instead")
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args()
    torch.cuda.set_device(0)
    x = student_t_bf16((a.m, a.k), 7, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    if a.kernel == "gemm":
        from .nvfp4 import set_gemm_tiling
        set_gemm_tiling(a.tiling)
        w = outlier_weight_bf16((a.n, a.k), 8, device="cuda")
        qa = FP4Tensor.from_bfloat16(x, linear_scales=False)
        qb = FP4Tensor.from_bfloat16(w, linear_scales=False)
        out = torch.empty(a.m, a.n, dtype=torch.bfloat16, device="cuda")
        bias = torch.zeros(a.n, dtype=torch.bfloat16, device="cuda") if a.bias else None
        gate = torch.ones(a.n, dtype=torch.float32, device="cuda") if a.gate else None
        res = student_t_bf16((a.m, a.n), 9, device="cuda") if a.residual else None
        ms = _time(lambda: fp4_gemm(qa, qb, 1.0, 1.0 if a.residual else 0.0, out=out, gelu=a.gelu,
                                    bias=bias, gate=gate, C=res), a.warmup, a.iters)
        N.check_status()
        print(f"gemm M={a.m} N={a.n} K={a.k}: {ms:.4f} ms, "
              f"{2.0 * a.m * a.n * a.k / ms / 1e9:.1f} TFLOP/s")
    elif a.kernel == "rope":
        # q/k RMSNorm + rotary embedding over a [m, 3k] QKV tensor (k = heads * 128)
        from . import dit
        heads = a.k // 128
        cfg = dit.WanDiTConfig(dim=a.k, heads=heads, ffn=a.k, layers=1, in_channels=16, out_channels=16)
        qkv = student_t_bf16((a.m, 3 * a.k), 11, device="cuda")
        cos, sin = dit.rope_tables(cfg, (1, 1, a.m), "cuda")
        cs = dit.pack_rope_table(cos, sin)
        gq = torch.ones(a.k, device="cuda")
        ms = _time(lambda: dit.qk_norm_rope(qkv, heads, 128, gq, gq, 1e-6, cs), a.warmup, a.iters)
        N.check_status()
        nbytes = 2 * (2.0 + 2.0) * a.m * a.k          # q and k, read + written
        print(f"qk_norm_rope [{a.m}, 3x{a.k}]: {ms:.4f} ms, {nbytes / ms / 1e6:.1f} GB/s")
    elif a.kernel == "attention":
        # self-attention over m tokens, k/128 heads of 128, q/k/v as the column blocks of one
        # [m, 3k] projection output
        from . import dit
        heads = a.k // 128
        qkv = student_t_bf16((a.m, 3 * a.k), 13, device="cuda")
        q, k, v = (t.view(a.m, heads, 128) for t in qkv.split(a.k, dim=-1))
        out = torch.empty(a.m, heads, 128, dtype=torch.bfloat16, device="cuda")
        amax = torch.zeros(1, device="cuda")
        dit.ATTENTION_BACKEND = "library"
        fn = (lambda: dit.attention(q, k, v)) if a.library else \
            (lambda: dit.attention_native(q, k, v, amax=amax, out=out))
        ms = _time(fn, a.warmup, a.iters)
        N.check_status()
        print(f"attention [{a.m}, {heads}, 128] ({'library' if a.library else 'native'}): {ms:.4f} ms, "
              f"{4.0 * a.m * a.m * a.k / ms / 1e9:.1f} TFLOP/s")
    elif a.kernel == "return":
        # the attention-output return exchange on one GPU (one rank: every store is local), then
        # the flag wait that also reduces the amax: [m, k/128 heads, 128] -> the same buffer layout
        import ctypes
        heads = a.k // 128
        o = x.view(a.m, heads, 128)
        out = torch.empty_like(o)
        sync = torch.zeros(N.lib.nvfp4_exchange_sync_bytes() // 4, dtype=torch.int32, device="cuda")
        amax = torch.zeros(1, device="cuda")
        outs = (ctypes.c_void_p * 1)(out.data_ptr())
        syncs = (ctypes.c_void_p * 1)(sync.data_ptr())

        def run():
            N.check(N.lib.nvfp4_attn_return_exchange_bf16(o.data_ptr(), o.stride(0), o.stride(1), a.m,
                                                          heads, 128, outs, syncs, 1, 0, st), "return")
            N.check(N.lib.nvfp4_exchange_wait(sync.data_ptr(), 1, 1, 1_000_000_000, amax.data_ptr(),
                                              N.ptr(N.status_word(x.device)), st), "wait")
        ms = _time(run, a.warmup, a.iters)
        N.check_status()
        assert torch.equal(out, o) and float(amax) == float(o.abs().max())
        print(f"attention return [{a.m}, {heads}, 128]: {ms:.4f} ms, {4.0 * a.m * a.k / ms / 1e6:.1f} GB/s "
              "(read + write)")
    elif a.kernel == "norm":
        # LayerNorm + adaLN modulation + quantize: both sweeps per iteration
        g = torch.Generator(device="cuda").manual_seed(9)
        scale = torch.randn(a.k, generator=g, device="cuda") * 0.1
        shift = torch.randn(a.k, generator=g, device="cuda") * 0.1
        ms = _time(lambda: FP4Tensor.from_norm_mod(x, scale=scale, shift=shift), a.warmup, a.iters)
        N.check_status()
        n = a.m * a.k
        print(f"norm+mod+quantize [{a.m}, {a.k}]: {ms:.4f} ms, algorithmic {2.5625 * n / ms / 1e6:.1f} "
              f"GB/s, moved {4.5625 * n / ms / 1e6:.1f} GB/s")
    else:
        q = FP4Tensor.from_bfloat16(x, linear_scales=False)
        if a.kernel == "quantize":
            fn = lambda: N.lib.nvfp4_quantize_bf16(  # noqa: E731
                x.data_ptr(), a.m, a.k, q._amax.data_ptr(), q._data.data_ptr(), None,
                q._scales_swz.data_ptr(), q._gscale.data_ptr(), st)
            nbytes = 2.5625 * a.m * a.k
        else:
            fn = lambda: N.lib.nvfp4_amax_bf16(x.data_ptr(), a.m * a.k, q._amax.data_ptr(), st)  # noqa: E731
            nbytes = 2.0 * a.m * a.k
        ms = _time(fn, a.warmup, a.iters)
        print(f"{a.kernel} [{a.m}, {a.k}]: {ms:.4f} ms, {nbytes / ms / 1e6:.1f} GB/s")


if __name__ == "__main__":
    main()
