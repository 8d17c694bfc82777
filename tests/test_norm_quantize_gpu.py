"""GPU tests of the fused norm + adaLN + NVFP4 quantizer: its bytes equal the plain quantizer
applied to the bf16 tensor the same arithmetic produces, and that tensor matches a torch fp32
reference of the reference model's norm -> modulation -> cast chain."""
import numpy as np
import pytest
import torch

from helpers import bits_of, randn_bf16, student_t_bf16

pytestmark = pytest.mark.gpu


def _torch_chain(x, weight, bias, scale, shift, rms, eps):
    xf = x.float()
    if rms:
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    else:
        y = torch.nn.functional.layer_norm(xf, (x.shape[-1],), None, None, eps)
    if weight is not None:
        y = y * weight
    if bias is not None:
        y = y + bias
    if scale is not None:
        y = y * (1 + scale)
    if shift is not None:
        y = y + shift
    return y.to(torch.bfloat16)


@pytest.mark.parametrize("rows,cols,rms,affine,mod", [
    (300, 3072, False, False, True),     # norm1 / norm3 of the 5B-shaped block
    (129, 5120, False, True, False),     # norm2 (affine, no modulation), 14B width
    (64, 14336, True, True, True),       # widest row held in registers
    (33, 48, True, False, False),        # a row shorter than one warp pass
    (17, 3088, False, False, True),      # odd number of scale blocks per row: one block per thread
    (5, 16384, False, True, True),       # the widest supported row, all four vectors
    (2049, 1024, True, False, True),     # many short rows, ragged last group
])
def test_fused_norm_quantize(oracle, rows, cols, rms, affine, mod):
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import nvfp4 as nv
    g = torch.Generator().manual_seed(rows + cols)
    x = student_t_bf16((rows, cols), rows, scale=1.5, device="cuda")
    vec = lambda s: (torch.randn(cols, generator=g) * s).cuda()  # noqa: E731
    weight = 1 + vec(0.1) if affine else None
    bias = vec(0.1) if affine else None
    scale = vec(0.2) if mod else None
    shift = vec(0.2) if mod else None
    t, h = nv.FP4Tensor.from_norm_mod(x, weight=weight, bias=bias, scale=scale, shift=shift,
                                      rms=rms, linear_scales=True, return_normed=True)
    # (1) the packed result is exactly the quantizer's view of h
    q = nv.FP4Tensor.from_bfloat16(h)
    assert float(t.global_amax().item()) == float(q.global_amax().item())
    assert torch.equal(t.quantized_data(), q.quantized_data())
    assert torch.equal(t.scale_factors(), q.scale_factors())
    assert torch.equal(t.scale_factors_swizzled(), q.scale_factors_swizzled())
    assert float(t.global_scale().item()) == float(q.global_scale().item())
    # and the CPU oracle's, from the same h
    packed, scales, amax = oracle.quantize(bits_of(h))
    assert np.array_equal(t.quantized_data().cpu().numpy(), packed.reshape(-1))
    assert np.array_equal(t.scale_factors().cpu().numpy(), scales.reshape(-1))
    # (2) h matches the fp32 torch chain to bf16 rounding (different summation order)
    ref = _torch_chain(x, weight, bias, scale, shift, rms, 1e-6)
    diff = (h.float() - ref.float()).abs()
    tol = 2.0 ** -7 * ref.float().abs() + 1e-3
    assert bool((diff <= tol).all())
    assert float((h != ref).float().mean()) < 0.02


def test_fused_norm_feeds_the_gemm(oracle):
    """norm -> modulation -> QKV linear, fused against unfused, through the GEMM."""
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import nvfp4 as nv
    x = randn_bf16((500, 3072), 5, device="cuda")
    w = nv.FP4Tensor.from_bfloat16(randn_bf16((1024, 3072), 6, 0.02, device="cuda"))
    scale = (torch.randn(3072, generator=torch.Generator().manual_seed(7)) * 0.1).cuda()
    shift = (torch.randn(3072, generator=torch.Generator().manual_seed(8)) * 0.1).cuda()
    a, h = nv.FP4Tensor.from_norm_mod(x, scale=scale, shift=shift, return_normed=True)
    y_fused = nv.fp4_gemm(a, w)
    y_plain = nv.fp4_gemm(nv.FP4Tensor.from_bfloat16(h), w)
    nv.check_status()
    assert torch.equal(y_fused, y_plain)


def test_fused_norm_rejects_bad_shapes():
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import nvfp4 as nv
    with pytest.raises(RuntimeError, match="cols"):
        nv.FP4Tensor.from_norm_mod(torch.zeros(4, 24, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(RuntimeError, match="float32"):
        nv.FP4Tensor.from_norm_mod(torch.zeros(4, 32, dtype=torch.bfloat16, device="cuda"),
                                   scale=torch.zeros(32, dtype=torch.bfloat16, device="cuda"))
