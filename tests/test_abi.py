"""The C-ABI library loads on a machine without a GPU, exports every symbol the
public header declares, and rejects bad arguments before touching a device."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "nvfp4_b200.h")


def _declared():
    text = open(HEADER).read()
    return sorted(set(re.findall(r"NVFP4_API[^;]*?\b(nvfp4_\w+)\s*\(", text)))


def test_header_symbols_exported():
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import _native
    names = _declared()
    assert len(names) >= 11
    for n in names:
        assert hasattr(_native.lib, n), n
    assert set(names) == set(_native.SIGNATURES), "ctypes table and header disagree"


def test_status_strings_and_version():
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import _native
    assert _native.status_string(0) == "ok"
    assert "aligned" in _native.status_string(2)
    assert "10.x" in _native.status_string(3)
    assert _native.lib.nvfp4_version() >= 100


def test_swizzled_bytes_formula():
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import _native
    f = _native.lib.nvfp4_swizzled_scale_bytes
    assert f(128, 64) == 2 * 4 * 512       # rows pad to 256, K-blocks pad to 16
    assert f(27280, 3072) == 214 * 48 * 512
    assert f(300, 320) == 4 * 8 * 512


def test_argument_validation_without_device():
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import _native
    L = _native.lib
    # cols not a multiple of 16, null pointers, negative sizes: rejected on the host
    assert L.nvfp4_quantize_bf16(None, 4, 24, None, None, None, None, None, None) == 1
    assert L.nvfp4_quantize_bf16_amax(None, None, None, 17, 1.0, None) == 1
    assert L.nvfp4_gemm(None, None, None, None, None, None, 8, 12, 64, 1.0, 0.0, None, None,
                        None, 0, None, None, None, None) == 1  # N % 8
    assert L.nvfp4_gemm(None, None, None, None, None, None, 8, 16, 48, 1.0, 0.0, None, None,
                        None, 0, None, None, None, None) == 1  # K % 32
    assert L.nvfp4_gemm(None, None, None, None, None, None, 8, 16, 64, 1.0, 0.0, None, None,
                        None, 7, None, None, None, None) == 1  # unknown activation
    assert L.nvfp4_gemm(None, None, None, None, None, None, 8, 16, 64, 1.0, 0.0, None, None,
                        None, 0, None, None, None, None) == 1  # null operands
    assert L.nvfp4_gemm(None, None, None, None, None, None, 0, 16, 64, 1.0, 0.0, None, None,
                        None, 0, None, None, None, None) == 0  # empty problem is a no-op
    assert L.nvfp4_amax_bf16(None, 16, None, None) == 1
    # extents whose product would wrap a 64-bit integer are refused before anything is multiplied
    assert L.nvfp4_quantize_bf16(None, 1 << 40, 1 << 40, None, None, None, None, None, None) == 1
    assert L.nvfp4_dequantize_bf16(None, None, 1 << 40, 1 << 40, None, None, None) == 1
    assert L.nvfp4_swizzle_scales(None, 1 << 40, 1 << 40, None, None) == 1
    # the fused norm quantizer stores 8-byte words of nibbles: a packed pointer that is only
    # 4-byte aligned is refused on the host (status 2), nothing is launched
    fake = 0x10000
    assert L.nvfp4_norm_mod_quantize_bf16(fake, 4, 64, None, None, None, None, fake, fake, fake + 4,
                                          None, None, None, None, None) == 2
    assert L.nvfp4_norm_mod_quantize_bf16(fake + 8, 4, 64, None, None, None, None, fake, fake, fake,
                                          None, None, None, None, None) == 2   # x itself
    # attention: head dimension, key count, scale, pointers, strides and alignment are all
    # checked before the device is looked at

    def attn(q=fake, hd=128, lq=256, lk=256, scale=0.1, qs=384, o=fake, heads=1):
        return L.nvfp4_attention_bf16(q, qs, 128, fake, 384, 128, fake, 384, 128, lq, lk, heads, hd, scale,
                                      o, 128, 128, None, None, None)
    assert attn(hd=64) == 1
    assert attn(lk=0) == 1
    assert attn(lq=-1) == 1
    assert attn(scale=0.0) == 1
    assert attn(heads=0) == 1
    assert attn(q=None) == 1
    assert attn(o=None) == 1
    assert attn(qs=64) == 1              # token stride shorter than a head
    assert attn(qs=132) == 2             # token stride not a multiple of 16 bytes
    assert attn(q=fake + 8) == 2
    assert attn(lq=0) == 0               # no queries: a no-op


def test_host_api_mirrors_reference_names():
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import nvfp4, nvfp4_linear_cpp, nvfp4_linear_module
    for name in ("init", "QuantizationMode", "FP4Tensor", "blackwell_fp4_gemm", "fp4_gemm",
                 "gemm_fp4_quantized", "is_aligned", "get_aligned_dims", "benchmark",
                 "__version__", "__cuda_arch__"):
        assert hasattr(nvfp4, name), name
    assert [m.name for m in nvfp4.QuantizationMode] == ["block_1d", "block_2d", "per_tensor",
                                                        "per_channel"]
    for name in ("gemm", "gemv", "batched_gemm", "forward", "backward", "are_dimensions_aligned",
                 "get_padded_dimensions", "estimate_padding_overhead"):
        assert hasattr(nvfp4_linear_cpp, name), name
    assert nvfp4.is_aligned(128, 256, 384) and not nvfp4.is_aligned(100, 256, 384)
    assert nvfp4.get_aligned_dims(100, 129, 1) == (128, 256, 128)
    assert nvfp4_linear_cpp.get_padded_dimensions(100, 129, 1) == (128, 256, 128)
    assert nvfp4.FP4_E2M1_MAX == 6.0 and nvfp4.FP8_E4M3_MAX == 448.0 and nvfp4.FP4_BLOCK_SIZE == 16
    lin = nvfp4_linear_module.NVFP4Linear(64, 48, bias=True)
    assert lin.weight.shape == (48, 64) and lin.weight.dtype.__str__() == "torch.bfloat16"
    assert lin.scale_weight.numel() == (48 * 64 + 31) // 32


def test_input_checks_raise_like_the_reference():
    import torch
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import nvfp4
    with pytest.raises(RuntimeError, match="Input must be BFloat16"):
        nvfp4.FP4Tensor.from_bfloat16(torch.zeros(4, 16))
    with pytest.raises(RuntimeError, match="Input must be on CUDA device"):
        nvfp4.FP4Tensor.from_bfloat16(torch.zeros(4, 16, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError, match="Tensors must be on CUDA device"):
        nvfp4.blackwell_fp4_gemm(torch.zeros(4, 16, dtype=torch.bfloat16),
                                 torch.zeros(4, 16, dtype=torch.bfloat16))
