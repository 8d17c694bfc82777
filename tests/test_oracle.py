"""CPU tests of the oracle itself: converters against the CUDA toolkit's host
implementations, the scale recipe against hand-computed answers, and the
committed golden vectors."""
import ctypes as C
import os

import numpy as np
import pytest

from helpers import bits_of, randn_bf16

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "nvfp4_cases.npz")


def _many(fn, x):
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(x.size, np.uint8)
    fn(x.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p), x.size)
    return out


def _sample_floats():
    rng = np.random.default_rng(7)
    every_bf16 = (np.arange(65536, dtype=np.uint32) << 16).view(np.float32)
    wide = rng.standard_normal(200000).astype(np.float32) * np.float32(8.0)
    tiny = (rng.standard_normal(50000) * 2.0 ** -9).astype(np.float32)
    big = (rng.standard_normal(50000) * 300).astype(np.float32)
    # every representable value, its midpoints and their fp32 neighbours
    e2m1 = np.array([0, .5, 1, 1.5, 2, 3, 4, 6], np.float32)
    mids = (e2m1[:-1] + e2m1[1:]) / 2
    pts = np.concatenate([e2m1, mids])
    pts = np.concatenate([pts, np.nextafter(pts, np.float32(np.inf)),
                          np.nextafter(pts, np.float32(-np.inf))])
    return np.concatenate([every_bf16, wide, tiny, big, pts, -pts]).astype(np.float32)


def test_e2m1_matches_toolkit(oracle):
    xs = _sample_floats()
    tk = _many(oracle.toolkit().tk_f32_to_e2m1_many, xs)
    mine = np.array([oracle.lib().nvfp4_oracle_f32_to_e2m1(float(v)) for v in xs], np.uint8)
    assert np.array_equal(tk, mine)


def test_e4m3_matches_toolkit(oracle):
    xs = _sample_floats()
    tk = _many(oracle.toolkit().tk_f32_to_e4m3_many, xs)
    mine = np.array([oracle.lib().nvfp4_oracle_f32_to_e4m3(float(v)) for v in xs], np.uint8)
    assert np.array_equal(tk, mine)


def test_e4m3_decode_matches_toolkit(oracle):
    for b in range(256):
        u = oracle.lib().nvfp4_oracle_e4m3_to_f32(b)
        v = oracle.toolkit().tk_e4m3_to_f32(b)
        assert u == v or (u != u and v != v)


def test_pack_order_matches_toolkit(oracle):
    # first element of a pair lands in the low nibble (1.0 -> code 2, -6.0 -> code 0xF)
    assert oracle.toolkit().tk_f32x2_to_e2m1x2(1.0, -6.0) == 0xF2


def test_pack_order_value(oracle):
    x = np.zeros((1, 16), np.float32)
    x[0, 0], x[0, 1] = 1.0, -6.0
    packed, scales, amax = oracle.quantize(oracle.f32_to_bf16_bits(x))
    assert amax == 6.0
    assert scales[0, 0] == 0x7E  # 448
    assert packed[0, 0] == 0xF2


def test_constants_and_global_scale(oracle):
    # S_enc = 448*6/amax, per-tensor scale = amax/(6*448)
    assert oracle.global_encode_scale(1.0) == np.float32(2688.0)
    assert oracle.global_encode_scale(0.0) == 1.0
    assert oracle.global_encode_scale(float("inf")) == 1.0
    assert oracle.global_decode_scale(2688.0) == 1.0
    a = np.float32(3.75)
    assert oracle.global_encode_scale(float(a)) == np.float32(2688.0) / a


def test_zero_tensor(oracle):
    x = np.zeros((4, 64), np.uint16)
    packed, scales, amax = oracle.quantize(x)
    assert amax == 0.0 and not packed.any() and not scales.any()
    assert not oracle.dequantize_f32(packed, scales, amax).any()


def test_roundtrip_error_bound(oracle):
    # the reference's own bound: mean relative error < 0.3
    # (fx/src/s4/nvfp4/test_quantization.cpp:86-87)
    x = randn_bf16((128, 256), 42)
    xb = bits_of(x)
    packed, scales, amax = oracle.quantize(xb)
    xq = oracle.dequantize_f32(packed, scales, amax)
    xf = x.float().numpy()
    rel = np.abs(xq - xf).mean() / np.abs(xf).mean()
    assert rel < 0.3 and rel < 0.12


def test_bf16_max_is_finite(oracle):
    # extrema case of fx/src/s4/nvfp4/test_nvfp4_quantize_te.py:113-154
    x = np.full((2, 32), 0x7F7F, np.uint16)
    packed, scales, amax = oracle.quantize(x)
    xq = oracle.dequantize_f32(packed, scales, amax)
    assert np.isfinite(xq).all()
    assert np.all(packed == 0x77) and np.all(scales == 0x7E)


def test_golden_vectors(oracle):
    g = np.load(GOLDEN)
    names = sorted({k.split(".")[0] for k in g.files} - {"linear"})
    assert names
    for n in names:
        packed, scales, amax = oracle.quantize(g[f"{n}.x"])
        assert np.array_equal(packed, g[f"{n}.packed"]), n
        assert np.array_equal(scales, g[f"{n}.scales"]), n
        assert np.float32(amax) == g[f"{n}.amax"], n
        assert np.float32(oracle.global_decode_scale(amax)) == g[f"{n}.gscale"], n
        assert np.array_equal(oracle.dequantize_bf16(packed, scales, amax), g[f"{n}.dequant_bf16"]), n
    y = oracle.linear(g["linear.x"], g["linear.w"], g["linear.b"])
    assert np.array_equal(y, g["linear.y"])


REF_SCALES = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_te_scales.npz")


def test_block_scales_equal_the_reference_kernels(oracle):
    """The E4M3 block scales the reference's own kernel (block_1d_quantization_kernel_te,
    fx/src/s4/nvfp4/quantization_te.cu:92-135) produced on a B200 for the golden inputs
    (tests/golden/make_ref_scales.py) are byte for byte the oracle's."""
    g, r = np.load(GOLDEN), np.load(REF_SCALES)
    for name in ("normal", "student_t", "weights", "tiny_blocks", "edge"):
        assert float(r[f"{name}.amax"]) == float(g[f"{name}.amax"])
        _, scales, _ = oracle.quantize(g[f"{name}.x"], float(r[f"{name}.amax"]))
        assert np.array_equal(scales, r[f"{name}.scales"]), name


def test_golden_edge_codes(oracle):
    # row 4 of the edge case holds the E2M1 tie points; with amax 3.39e38 elsewhere the row's
    # own block scale decides, so check the block in isolation
    x = np.array([[0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0,
                   -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0]], np.float32)
    packed, scales, amax = oracle.quantize(oracle.f32_to_bf16_bits(x))
    codes = np.stack([packed[0] & 0xF, packed[0] >> 4], 1).reshape(-1)
    # ties go to the even code: .25->0, .75->1(code 2), 1.25->1(2), 1.75->2(4), 2.5->2(4),
    # 3.5->4(6), 5->4(6), 6->6(7)
    assert list(codes[:8]) == [0, 2, 2, 4, 4, 6, 6, 7]
    assert list(codes[8:]) == [8, 10, 10, 12, 12, 14, 14, 15]


def test_swizzle_layout(oracle):
    rows, cols = 300, 320  # ragged in both directions: 20 K-blocks, 3 row tiles of 128
    sc = (np.arange(rows * (cols // 16)) % 251).astype(np.uint8).reshape(rows, cols // 16)
    swz = oracle.swizzle_scales(sc, cols)
    k_atoms = 8  # 20 blocks -> padded to 32 -> 8 atoms
    assert swz.size == 4 * k_atoms * 512  # rows padded to 512 -> 4 tiles
    seen = np.zeros(swz.size, bool)
    for r in (0, 1, 31, 32, 127, 128, 299):
        for k in (0, 3, 4, 19):
            off = ((r // 128) * k_atoms + k // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + k % 4
            assert swz[off] == sc[r, k]
            seen[off] = True
    # padding is zero
    total = int(swz.astype(np.int64).sum())
    assert total == int(sc.astype(np.int64).sum())


def test_fp32_and_bf16_dequant_variants_agree(oracle):
    # dequantized operands kept in fp32 (the grading oracle) vs rounded to bf16 first (the
    # literal __float2bfloat16 of the reference's dequant kernel): bf16 rounding of every
    # operand costs about 2^-9 relative, so the two agree to a few 1e-3 relative Frobenius
    x = bits_of(randn_bf16((64, 512), 11))
    w = bits_of(randn_bf16((48, 512), 12, 0.02))
    px, sx, ax = oracle.quantize(x)
    pw, sw, aw = oracle.quantize(w)
    y32 = oracle.matmul_nt(oracle.dequantize_f32(px, sx, ax), oracle.dequantize_f32(pw, sw, aw),
                           want_f32=True)[1]
    xb = oracle.bf16_bits_to_f32(oracle.dequantize_bf16(px, sx, ax))
    wb = oracle.bf16_bits_to_f32(oracle.dequantize_bf16(pw, sw, aw))
    y16 = oracle.matmul_nt(xb, wb, want_f32=True)[1]
    assert np.linalg.norm(y32 - y16) / np.linalg.norm(y32) < 5e-3


def test_epilogue_terms(oracle):
    rng = np.random.default_rng(3)
    xq = rng.standard_normal((8, 32)).astype(np.float32)
    wq = rng.standard_normal((16, 32)).astype(np.float32)
    bias = oracle.f32_to_bf16_bits(rng.standard_normal(16).astype(np.float32))
    gate = rng.standard_normal(16).astype(np.float32)
    res = oracle.f32_to_bf16_bits(rng.standard_normal((8, 16)).astype(np.float32))
    _, y = oracle.matmul_nt(xq, wq, bias, act=1, gate=gate, residual_bits=res, want_f32=True)
    z = xq @ wq.T + oracle.bf16_bits_to_f32(bias)
    z = 0.5 * z * (1 + np.tanh(0.7978845608028654 * (z + 0.044715 * z ** 3)))
    z = z * gate + oracle.bf16_bits_to_f32(res)
    assert np.allclose(y, z, rtol=1e-4, atol=1e-4)


def test_fast_division_by_six_is_exact(oracle):
    """The kernels' three-operation x / 6 equals IEEE division on every bf16 value (the only
    inputs it ever sees: block maxima of bf16 tensors) and on a few million fp32 values."""
    import numpy as np
    lib = oracle.lib()
    bf16 = (np.arange(1 << 16, dtype=np.uint32) << 16).view(np.float32)
    rng = np.random.default_rng(6)
    fp32 = rng.integers(0, 1 << 32, size=4_000_000, dtype=np.uint64).astype(np.uint32).view(np.float32)
    for arr in (bf16, fp32):
        a = np.ascontiguousarray(arr)
        assert lib.nvfp4_oracle_div6_mismatches(a.ctypes.data, a.size) == 0
