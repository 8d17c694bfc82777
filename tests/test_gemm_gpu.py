"""GPU parity of the tcgen05 block-scaled FP4 GEMM and the linear built on it,
through the C ABI, against the dequantize-then-matmul oracle.  Tolerance:
relative Frobenius error <= 1e-2 against that path on the same inputs."""
import os

import numpy as np
import pytest
import torch

from helpers import bits_of, from_bits, outlier_weight_bf16, randn_bf16, rel_fro, student_t_bf16

pytestmark = pytest.mark.gpu
TOL = 1e-2
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "nvfp4_cases.npz")


@pytest.fixture(scope="module", params=["uniform", "alternating"])
def nv(request):
    """Every test of this file runs under both N tilings of the GEMM."""
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import nvfp4
    nvfp4.set_gemm_tiling(request.param)
    yield nvfp4
    nvfp4.set_gemm_tiling("auto")


def _oracle_gemm(oracle, x, w, bias=None, act=0, gate=None, residual=None):
    px, sx, ax = oracle.quantize(bits_of(x))
    pw, sw, aw = oracle.quantize(bits_of(w))
    xq = oracle.dequantize_f32(px, sx, ax)
    wq = oracle.dequantize_f32(pw, sw, aw)
    _, y = oracle.matmul_nt(xq, wq, bits_of(bias) if bias is not None else None, act,
                            gate.numpy() if gate is not None else None,
                            bits_of(residual) if residual is not None else None, want_f32=True)
    return torch.from_numpy(y)


def _gpu_dequant_matmul(nv, a, b):
    """fp32 matmul of the dequantized operands on the GPU (for sizes the CPU oracle
    cannot finish in seconds); dequantized values are exact in bf16 x bf16 -> fp32 only up
    to the bf16 rounding of the operands, hence used with its own looser bound."""
    return a.to_bfloat16().float() @ b.to_bfloat16().float().t()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 256), (128, 256, 1024),
                                   (256, 512, 512), (1, 8, 32), (15, 16, 96), (17, 264, 160),
                                   (127, 128, 128), (129, 384, 288), (300, 1032, 544),
                                   (512, 3072, 3072)])
def test_gemm_matches_oracle(nv, oracle, M, N, K):
    x = randn_bf16((M, K), 100 + M)
    w = randn_bf16((N, K), 200 + N, 0.02)
    y = nv.gemm_fp4_quantized(x.cuda(), w.cuda())
    nv.check_status()
    ref = _oracle_gemm(oracle, x, w)
    assert y.shape == (M, N) and y.dtype == torch.bfloat16
    assert rel_fro(y.float().cpu(), ref) <= TOL


def test_gemm_many_tiles_per_cta(nv, oracle):
    # more tiles than SMs: every CTA walks several tiles and both accumulators
    M, N, K = 1100, 9216, 256
    x = randn_bf16((M, K), 1)
    w = randn_bf16((N, K), 2, 0.02)
    a = nv.FP4Tensor.from_bfloat16(x.cuda())
    b = nv.FP4Tensor.from_bfloat16(w.cuda())
    y = nv.fp4_gemm(a, b)
    nv.check_status()
    ref = _oracle_gemm(oracle, x, w)
    assert rel_fro(y.float().cpu(), ref) <= TOL
    # per 128x256 tile as well: a misplaced tile would hide in the global norm
    yc = y.float().cpu()
    for m0 in range(0, M, 128):
        for n0 in range(0, N, 1024):
            assert rel_fro(yc[m0:m0 + 128, n0:n0 + 1024], ref[m0:m0 + 128, n0:n0 + 1024]) <= 2 * TOL


def test_fused_epilogue(nv, oracle):
    M, N, K = 200, 512, 512
    x = student_t_bf16((M, K), 3)
    w = outlier_weight_bf16((N, K), 4)
    bias = randn_bf16((N,), 5, 0.01)
    gate = torch.randn(N, generator=torch.Generator().manual_seed(6))
    res = randn_bf16((M, N), 7)
    a = nv.FP4Tensor.from_bfloat16(x.cuda())
    b = nv.FP4Tensor.from_bfloat16(w.cuda())
    for kw, okw in (
        (dict(bias=bias.cuda()), dict(bias=bias)),
        (dict(bias=bias.cuda(), gelu=True), dict(bias=bias, act=1)),
        (dict(bias=bias.cuda(), gate=gate.cuda(), C=res.cuda(), beta=1.0),
         dict(bias=bias, gate=gate, residual=res)),
        (dict(bias=bias.cuda(), gelu=True, gate=gate.cuda(), C=res.cuda(), beta=1.0),
         dict(bias=bias, act=1, gate=gate, residual=res)),
    ):
        beta = kw.pop("beta", 0.0)
        y = nv.fp4_gemm(a, b, 1.0, beta, **kw)
        nv.check_status()
        ref = _oracle_gemm(oracle, x, w, **okw)
        assert rel_fro(y.float().cpu(), ref) <= TOL, kw.keys()


def test_alpha_and_out_argument(nv, oracle):
    M, N, K = 64, 256, 128
    x = randn_bf16((M, K), 8)
    w = randn_bf16((N, K), 9)
    a = nv.FP4Tensor.from_bfloat16(x.cuda())
    b = nv.FP4Tensor.from_bfloat16(w.cuda())
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    y = nv.fp4_gemm(a, b, 0.5, 0.0, out=out)
    assert y.data_ptr() == out.data_ptr()
    ref = 0.5 * _oracle_gemm(oracle, x, w)
    assert rel_fro(y.float().cpu(), ref) <= TOL


def test_config1_linear(nv, oracle):
    """Single NVFP4 linear, X [4096,3072] N(0,1), W [3072,3072] N(0,0.02^2), b N(0,0.01^2):
    packed bytes and scales bit-exact on a row slice, Y against the fp32 dequant matmul
    (CPU oracle on 256 rows, GPU dequant-matmul on all rows)."""
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import nvfp4_linear_cpp
    x = randn_bf16((4096, 3072), 1235)
    w = randn_bf16((3072, 3072), 1236, 0.02)
    bias = randn_bf16((3072,), 1237, 0.01)
    xd, wd, bd = x.cuda(), w.cuda(), bias.cuda()
    y = nvfp4_linear_cpp.forward(xd, wd, bd, torch.ones(1, device="cuda"), torch.ones(1, device="cuda"))
    nv.check_status()
    assert y.shape == (4096, 3072)
    a = nv.FP4Tensor.from_bfloat16(xd)
    b = nv.FP4Tensor.from_bfloat16(wd)
    px, sx, ax = oracle.quantize(bits_of(x))
    pw, sw, aw = oracle.quantize(bits_of(w))
    assert np.array_equal(a.quantized_data().cpu().numpy(), px.reshape(-1))
    assert np.array_equal(a.scale_factors().cpu().numpy(), sx.reshape(-1))
    assert np.array_equal(b.quantized_data().cpu().numpy(), pw.reshape(-1))
    assert np.array_equal(b.scale_factors().cpu().numpy(), sw.reshape(-1))
    rows = slice(1000, 1256)
    xq = oracle.dequantize_f32(px[rows], sx[rows], ax)
    wq = oracle.dequantize_f32(pw, sw, aw)
    _, ref = oracle.matmul_nt(xq, wq, bits_of(bias), want_f32=True)
    assert rel_fro(y[rows].float().cpu(), torch.from_numpy(ref)) <= TOL
    full = _gpu_dequant_matmul(nv, a, b) + bd.float()
    assert rel_fro(y.float(), full) <= TOL


def test_golden_linear(nv):
    g = np.load(GOLDEN)
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import nvfp4_linear_cpp
    x, w, b = (from_bits(g[f"linear.{k}"]).cuda() for k in ("x", "w", "b"))
    y = nvfp4_linear_cpp.linear(x, w, b)
    ref = from_bits(g["linear.y"]).float()
    assert rel_fro(y.float().cpu(), ref) <= TOL


@pytest.mark.parametrize("N,K,gelu", [(9216, 3072, False), (3072, 3072, False),
                                      (14336, 3072, True), (3072, 14336, False)])
def test_config2_block_linears_full_size(nv, N, K, gelu):
    """Wan2.2-TI2V-5B block linears at M = 27280 (Student-t activations, outlier weights):
    against the GPU fp32 dequant-matmul on row bands, plus linearity in alpha."""
    M = 27280
    x = student_t_bf16((M, K), 60, device="cuda")
    w = outlier_weight_bf16((N, K), 61, device="cuda")
    a = nv.FP4Tensor.from_bfloat16(x, linear_scales=True)
    b = nv.FP4Tensor.from_bfloat16(w, linear_scales=True)
    y = nv.fp4_gemm(a, b, gelu=gelu)
    nv.check_status()
    ad, bd = a.to_bfloat16().float(), b.to_bfloat16().float()
    for r0 in (0, 13568, M - 400):
        ref = ad[r0:r0 + 400] @ bd.t()
        if gelu:
            ref = torch.nn.functional.gelu(ref, approximate="tanh")
        assert rel_fro(y[r0:r0 + 400].float(), ref) <= TOL
    if not gelu:
        y2 = nv.fp4_gemm(a, b, 2.0)
        assert rel_fro(y2.float(), 2.0 * y.float()) <= 4e-3  # two bf16 roundings


def test_reference_statistical_bounds(nv):
    # fx/src/s4/nvfp4/test_gemm.cpp:81-82: mean relative error vs bf16 matmul below 0.3
    A = randn_bf16((512, 1024), 70, device="cuda")
    B = randn_bf16((768, 1024), 71, device="cuda")
    y = nv.blackwell_fp4_gemm(A, B)
    ref = (A.float() @ B.float().t())
    rel = float((y.float() - ref).abs().mean() / ref.abs().mean())
    assert rel < 0.3
    assert torch.isfinite(y.float()).all()


def test_error_cases(nv):
    # fx/src/s4/nvfp4/test_gemm.cpp:232-263
    A = nv.FP4Tensor.from_bfloat16(randn_bf16((64, 128), 72, device="cuda"))
    B = nv.FP4Tensor.from_bfloat16(randn_bf16((64, 256), 73, device="cuda"))
    with pytest.raises(RuntimeError, match="Inner dimensions must match"):
        nv.fp4_gemm(A, B)
    one_d = nv.FP4Tensor.from_bfloat16(randn_bf16((128,), 74, device="cuda"))
    with pytest.raises(RuntimeError, match="2D matrices"):
        nv.fp4_gemm(one_d, B)


def test_linear_module_and_ops(nv, oracle):
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import nvfp4_linear_cpp
    from blackwell_diffusion_rtx6000_5090_i2v_b200.nvfp4_linear_module import NVFP4Linear
    torch.manual_seed(0)
    lin = NVFP4Linear(256, 136, bias=True).cuda()
    x = randn_bf16((3, 50, 256), 80, device="cuda")
    with torch.no_grad():
        y = lin(x)
        y_again = lin(x)  # cached weight
    assert y.shape == (3, 50, 136)
    assert torch.equal(y, y_again)
    ref = _oracle_gemm(oracle, x.reshape(-1, 256).cpu(), lin.weight.detach().cpu(),
                       bias=lin.bias.detach().cpu())
    assert rel_fro(y.reshape(-1, 136).float().cpu(), ref) <= TOL
    # in-place weight update invalidates the cached quantized copy
    with torch.no_grad():
        lin.weight.mul_(2.0)
        y2 = lin(x)
    assert not torch.equal(y, y2)
    # autograd path: forward equals the no-grad path; backward returns finite grads
    xg = x.clone().requires_grad_(True)
    yg = lin(xg)
    yg.float().sum().backward()
    assert torch.equal(yg.detach(), y2)
    assert xg.grad.shape == x.shape and torch.isfinite(xg.grad.float()).all()
    assert lin.weight.grad.shape == lin.weight.shape and lin.bias.grad.shape == lin.bias.shape
    gi_ref = torch.ones(150, 136, device="cuda") @ lin.weight.detach().float()
    assert rel_fro(xg.grad.reshape(150, 256).float(), gi_ref) < 0.3
    # gemv / batched_gemm and the registered torch ops
    v = randn_bf16((256,), 81, device="cuda")
    assert nvfp4_linear_cpp.gemv(v, lin.weight.detach()).shape == (136,)
    assert nvfp4_linear_cpp.batched_gemm(x, lin.weight.detach()).shape == (3, 50, 136)
    y3 = torch.ops.nvfp4_b200.linear(x, lin.weight.detach(), lin.bias.detach(), False)
    assert torch.equal(y3, y2)
    parts = torch.ops.nvfp4_b200.quantize(x)
    assert parts[0].numel() == x.numel() // 2 and parts[1].numel() == x.numel() // 16


def test_ragged_n_and_k_through_linear(nv, oracle):
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import nvfp4_linear_cpp
    x = randn_bf16((37, 80), 90)   # K = 80: multiple of 16, not of 32
    w = randn_bf16((20, 80), 91)   # N = 20: not a multiple of 8
    y = nvfp4_linear_cpp.gemm(x.cuda(), w.cuda())
    assert y.shape == (37, 20)
    ref = _oracle_gemm(oracle, x, w)
    assert rel_fro(y.float().cpu(), ref) <= TOL


def test_output_amax_fused_in_epilogue(nv):
    """max|D| from the GEMM epilogue equals the separate amax pass bit for bit, so the next
    quantizer produces the same bytes either way (ragged M and N, GELU)."""
    M, N, K = 777, 1032, 512
    a = nv.FP4Tensor.from_bfloat16(student_t_bf16((M, K), 95, device="cuda"))
    b = nv.FP4Tensor.from_bfloat16(outlier_weight_bf16((N, K), 96, device="cuda"))
    bias = randn_bf16((N,), 97, 0.5, device="cuda")
    amax = torch.full((1,), 123.0, dtype=torch.float32, device="cuda")  # the call zeroes it
    y = nv.fp4_gemm(a, b, bias=bias, gelu=True, out_amax=amax)
    nv.check_status()
    assert float(amax.item()) == float(y.abs().max().float().item())
    q = nv.FP4Tensor.from_bfloat16(y)
    assert float(q.global_amax().item()) == float(amax.item())


def test_residual_tiles_land_where_they_belong(nv, oracle):
    """Residual with ragged M and N over several tiles: the epilogue fetches each 32 x 64 piece
    of C by a tiled copy into the output slab, so a misplaced or mis-swizzled piece shows up per
    piece, not in the global norm.  The residual is large against the product."""
    M, N, K = 700, 776, 256
    x = randn_bf16((M, K), 31)
    w = randn_bf16((N, K), 32, 0.02)
    res = randn_bf16((M, N), 33, 4.0)
    a = nv.FP4Tensor.from_bfloat16(x.cuda())
    b = nv.FP4Tensor.from_bfloat16(w.cuda())
    y = nv.fp4_gemm(a, b, 1.0, 1.0, C=res.cuda()).float().cpu()
    nv.check_status()
    ref = _oracle_gemm(oracle, x, w, residual=res)
    assert rel_fro(y, ref) <= TOL
    for m0 in range(0, M, 32):
        for n0 in range(0, N, 64):
            assert rel_fro(y[m0:m0 + 32, n0:n0 + 64], ref[m0:m0 + 32, n0:n0 + 64]) <= 2 * TOL, (m0, n0)
    # and the plain product is what is left after taking the residual away again
    plain = nv.fp4_gemm(a, b).float().cpu()
    assert (y - res.float() - plain).abs().max() <= 0.15        # bf16 rounding at |y| up to 16+


def test_repeated_launches_are_bit_identical_at_full_size(nv):
    """Races in the tile hand-off show up as rare launches in which one 128 x 64 piece differs;
    the attention-out shape with gate and residual is the one that exposed a real one."""
    M, N, K = 27280, 3072, 3072
    a = nv.FP4Tensor.from_bfloat16(student_t_bf16((M, K), 41, device="cuda"), linear_scales=False)
    b = nv.FP4Tensor.from_bfloat16(outlier_weight_bf16((N, K), 42, device="cuda"), linear_scales=False)
    bias = randn_bf16((N,), 43, 0.01, device="cuda")
    gate = torch.randn(N, generator=torch.Generator().manual_seed(44)).cuda()
    res = student_t_bf16((M, N), 45, device="cuda")
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    ref = nv.fp4_gemm(a, b, 1.0, 1.0, bias=bias, gate=gate, C=res, out=out).clone()
    for i in range(150):
        y = nv.fp4_gemm(a, b, 1.0, 1.0, bias=bias, gate=gate, C=res, out=out)
        assert torch.equal(y, ref), i
    nv.check_status()


def test_short_k_many_tiles_repeatable(nv, oracle):
    """K of one pipeline stage: the main loop of a tile is shorter than its epilogue, the
    regime in which reuse of an accumulator has to wait for every warp that still reads it."""
    M, N, K = 4096, 2048, 128
    x = randn_bf16((M, K), 51)
    w = randn_bf16((N, K), 52, 0.05)
    res = randn_bf16((M, N), 53)
    a = nv.FP4Tensor.from_bfloat16(x.cuda())
    b = nv.FP4Tensor.from_bfloat16(w.cuda())
    rc = res.cuda()
    ref = nv.fp4_gemm(a, b, 1.0, 1.0, C=rc, gelu=True).clone()
    assert rel_fro(ref.float().cpu(), _oracle_gemm(oracle, x, w, act=1, residual=res)) <= TOL
    for i in range(100):
        assert torch.equal(nv.fp4_gemm(a, b, 1.0, 1.0, C=rc, gelu=True), ref), i
    nv.check_status()


@pytest.mark.parametrize("M,N,K", [(300, 3072, 512), (1100, 9216, 256), (513, 5120, 1024),
                                   (256, 448, 128), (257, 520, 96), (4095, 1536, 3072)])
def test_tilings_agree_bit_for_bit(M, N, K):
    """Uniform and alternating tilings compute every output element as the same sum over K, so
    their results are identical bits -- including ragged edges, the narrow tiles that start 64
    rows into a scale atom, and the fused epilogue."""
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import nvfp4
    a = nvfp4.FP4Tensor.from_bfloat16(student_t_bf16((M, K), 7 + M, device="cuda"), linear_scales=False)
    b = nvfp4.FP4Tensor.from_bfloat16(outlier_weight_bf16((N, K), 8 + N, device="cuda"), linear_scales=False)
    bias = randn_bf16((N,), 9, 0.01, device="cuda")
    gate = torch.randn(N, generator=torch.Generator().manual_seed(10)).cuda()
    res = randn_bf16((M, N), 11, device="cuda")
    outs = {}
    try:
        for mode in ("uniform", "alternating", "auto"):
            nvfp4.set_gemm_tiling(mode)
            amax = torch.zeros(1, device="cuda")
            outs[mode] = (nvfp4.fp4_gemm(a, b), nvfp4.fp4_gemm(a, b, 1.0, 1.0, bias=bias, gate=gate, C=res),
                          nvfp4.fp4_gemm(a, b, bias=bias, gelu=True, out_amax=amax), amax)
            nvfp4.check_status()
    finally:
        nvfp4.set_gemm_tiling("auto")
    for mode in ("alternating", "auto"):
        for got, want in zip(outs[mode], outs["uniform"]):
            assert torch.equal(got, want), mode


def test_stacked_weights_equal_separate_gemms():
    """Several weights stacked along N, each with its own tensor scale, in one launch: every
    slice equals the GEMM against that weight alone (the hoisted text K/V projections)."""
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import nvfp4
    from blackwell_diffusion_rtx6000_5090_i2v_b200.nvfp4 import StackedWeights
    M, K, rows, count = 512, 1024, 768, 5
    x = randn_bf16((M, K), 21, device="cuda")
    ws = [randn_bf16((rows, K), 30 + i, 0.02 * (1 + i), device="cuda") for i in range(count)]
    bs = [randn_bf16((rows,), 40 + i, 0.01, device="cuda") for i in range(count)]
    packed = [nvfp4.FP4Tensor.from_bfloat16(w, linear_scales=False) for w in ws]
    a = nvfp4.FP4Tensor.from_bfloat16(x, linear_scales=False)
    stack = StackedWeights(packed, bs)
    try:
        for mode in ("uniform", "alternating"):
            nvfp4.set_gemm_tiling(mode)
            y = stack.gemm(a)
            nvfp4.check_status()
            assert y.shape == (M, rows * count)
            for i in range(count):
                want = nvfp4.fp4_gemm(a, packed[i], bias=bs[i])
                assert torch.equal(y[:, i * rows:(i + 1) * rows], want), (mode, i)
    finally:
        nvfp4.set_gemm_tiling("auto")
