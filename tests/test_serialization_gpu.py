"""Pre-quantized weight files: what is loaded is byte-for-byte what was packed, and a GEMM on
the loaded weight equals a GEMM on the freshly quantized one."""
import pytest
import torch

from helpers import randn_bf16

pytestmark = pytest.mark.gpu


def test_save_load_round_trip(tmp_path):
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import nvfp4, nvfp4_serialization as ser
    w1 = randn_bf16((384, 512), 3, 0.02, device="cuda")
    w2 = randn_bf16((72, 96), 4, 0.5, device="cuda")
    bias = randn_bf16((384,), 5, 0.01, device="cuda")
    t1, t2 = nvfp4.FP4Tensor.from_bfloat16(w1), nvfp4.FP4Tensor.from_bfloat16(w2)
    path = str(tmp_path / "w.safetensors")
    ser.save_packed(path, {"blocks.0.ffn.weight": t1, "proj": t2}, extra={"blocks.0.ffn.bias": bias})
    packed, other = ser.load_packed(path)
    assert set(packed) == {"blocks.0.ffn.weight", "proj"} and set(other) == {"blocks.0.ffn.bias"}
    assert torch.equal(other["blocks.0.ffn.bias"], bias)
    for name, t in (("blocks.0.ffn.weight", t1), ("proj", t2)):
        u = packed[name]
        assert list(u.shape()) == list(t.shape())
        assert torch.equal(u.quantized_data(), t.quantized_data())
        assert torch.equal(u.scale_factors(), t.scale_factors())
        assert torch.equal(u.scale_factors_swizzled(), t.scale_factors_swizzled())
        assert float(u.global_scale()) == float(t.global_scale())
        assert torch.equal(u.to_bfloat16(), t.to_bfloat16())
    x = nvfp4.FP4Tensor.from_bfloat16(randn_bf16((200, 512), 6, device="cuda"))
    assert torch.equal(nvfp4.fp4_gemm(x, packed["blocks.0.ffn.weight"], bias=bias),
                       nvfp4.fp4_gemm(x, t1, bias=bias))
    nvfp4.check_status()


def test_reference_method_signatures():
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import nvfp4_serialization as ser
    q = ser.NVFP4Quantization()
    w = randn_bf16((64, 128), 9, device="cuda")
    data, meta = q.quantize_tensor(w, None, "w")
    assert data.dtype == torch.uint8 and tuple(data.shape) == (64, 64)
    h = meta.to_safetensors_header()
    assert h["shape"] == [64, 128] and h["quantization"]["type"] == "nvfp4"
    assert h["quantization"]["bits"] == 4 and h["quantization"]["group_size"] == 16
    back = q.dequantize_tensor(data, meta)
    assert back.shape == w.shape and back.dtype == torch.bfloat16
    rel = ((back.float() - w.float()).norm() / w.float().norm()).item()
    assert rel < 0.15
    with pytest.raises(RuntimeError):
        q.quantize_tensor(w.cpu())


def test_load_rejects_foreign_file(tmp_path):
    from safetensors.torch import save_file
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import nvfp4_serialization as ser
    path = str(tmp_path / "x.safetensors")
    save_file({"a": torch.zeros(4)}, path)
    with pytest.raises(RuntimeError):
        ser.load_packed(path)
