"""The timed CPU baseline legs (oracle/cpu_baseline.py) at toy sizes: they run, agree with the
oracle's linear, and the transliterated reference loop keeps the reference's own rounding rule."""
import numpy as np
import torch


def test_block_linears_leg_matches_the_oracle_linear(oracle):
    from oracle import cpu_baseline as B
    assert B.use_all_cores() >= 1
    bl = B.BlockLinearsM4096(rows=8)
    assert [s.name for s in bl.specs] == ["qkv", "attn_out", "ffn_up", "ffn_down"]
    assert bl.flops == sum(2.0 * 8 * s.n * s.k for s in bl.specs)
    assert bl.prepare_weights() > 0
    assert bl.run(False) > 0 and bl.run(True) > 0
    # the leg's arithmetic (oracle quantize/dequantize + fp32 matmul + bias) against the oracle's
    # own whole-linear routine on the first linear: same bf16 output up to the summation order
    s = bl.specs[1]
    xq, wq = B._quant_dequant(bl.x[s.name]), bl.wq[s.name]
    y = B._finish(xq @ wq.t(), bl.b[s.name], s.gelu).float()
    ref_bits = oracle.linear(bl.x[s.name], bl.w[s.name], B._bits(bl.b[s.name]), act=0)
    ref = torch.from_numpy(oracle.bf16_bits_to_f32(ref_bits))
    assert float((y - ref).norm() / ref.norm()) < 5e-3


def test_literal_loop_keeps_the_reference_rounding():
    from oracle import cpu_baseline as B
    # ties go to the smaller magnitude (fx/src/s4/nvfp4/linear/nvfp4_linear.cpp:40-58), unlike
    # round-to-nearest-even E2M1 where 0.75 -> 1 and 3.5 -> 4
    assert B._round_like_the_reference(0.75) == 0.5
    assert B._round_like_the_reference(1.75) == 1.5
    assert B._round_like_the_reference(3.5) == 3.0
    assert B._round_like_the_reference(-2.5) == -2.0
    assert B._round_like_the_reference(7.0) == 6.0 and B._round_like_the_reference(-9.0) == -6.0
    r = B.literal_slice(rows=2, cols=64)
    assert r["slice"] == [2, 64] and r["seconds"] > 0
    assert abs(r["extrapolated_seconds_27280x3072"] - r["ns_per_element"] * 1e-9 * 27280 * 3072) < 1e-6


def test_config1_leg_reports_all_parts(monkeypatch):
    from oracle import cpu_baseline as B
    # the full configuration takes a second or two on a few cores: run it once and check the report
    r = B.config1_full()
    assert r["shape"] == [4096, 3072, 3072]
    assert abs(r["total_ms"] - (r["quantize_ms"] + r["dequantize_ms"] + r["matmul_ms"])) < 1e-6
    assert np.isfinite(r["tflops"]) and r["tflops"] > 0
