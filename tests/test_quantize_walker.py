"""``quantize_`` (the torchao-shaped module walker): which linears it converts and that the
converted modules carry the same parameters.  Runs on CPU: no forward pass is made."""
import torch
import torch.nn as nn


class _Block(nn.Module):
    def __init__(self):
        super().__init__()
        self.to_qkv = nn.Linear(64, 192)
        self.to_out = nn.ModuleList([nn.Linear(64, 64, bias=False), nn.Dropout(0.0)])
        self.odd = nn.Linear(60, 64)          # in_features % 32 != 0: stays
        self.tiny = nn.Linear(32, 8)
        self.norm = nn.LayerNorm(64)


def test_walker_replaces_eligible_linears():
    from blackwell_diffusion_rtx6000_5090_i2v_b200.nvfp4_linear_module import (
        NVFP4InferenceConfig, NVFP4Linear, quantize_)
    torch.manual_seed(0)
    model = nn.Sequential(_Block(), _Block())
    ref = {k: v.clone() for k, v in model.state_dict().items()}
    out = quantize_(model, NVFP4InferenceConfig(min_features=32, skip=("1.to_qkv",)))
    assert out is model
    b0, b1 = model[0], model[1]
    assert isinstance(b0.to_qkv, NVFP4Linear) and isinstance(b0.to_out[0], NVFP4Linear)
    assert type(b0.odd) is nn.Linear and type(b0.tiny) is nn.Linear and type(b0.norm) is nn.LayerNorm
    assert type(b1.to_qkv) is nn.Linear                      # skipped by path
    assert isinstance(b1.to_out[0], NVFP4Linear)
    q = b0.to_qkv
    assert (q.in_features, q.out_features) == (64, 192) and q.weight.dtype == torch.bfloat16
    assert torch.equal(q.weight, ref["0.to_qkv.weight"].to(torch.bfloat16))
    assert torch.equal(q.bias, ref["0.to_qkv.bias"].to(torch.bfloat16))
    assert b0.to_out[0].bias is None
    assert "format=nvfp4" in repr(q)


def test_filter_fn_and_root_linear():
    from blackwell_diffusion_rtx6000_5090_i2v_b200.nvfp4_linear_module import NVFP4Linear, quantize_
    lin = nn.Linear(128, 64)
    assert isinstance(quantize_(lin), NVFP4Linear)
    model = nn.Sequential(nn.Linear(64, 64), nn.Linear(64, 64))
    quantize_(model, filter_fn=lambda m, name: name == "1")
    assert type(model[0]) is nn.Linear and isinstance(model[1], NVFP4Linear)


import pytest  # noqa: E402


@pytest.mark.gpu
def test_converted_model_runs_close_to_the_float_model():
    from blackwell_diffusion_rtx6000_5090_i2v_b200.nvfp4_linear_module import quantize_
    torch.manual_seed(1)
    model = nn.Sequential(nn.Linear(256, 512), nn.GELU(approximate="tanh"), nn.Linear(512, 256)).cuda().bfloat16()
    x = torch.randn(100, 256, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        ref = model(x).float()
        y = quantize_(model)(x).float()
    assert y.shape == ref.shape
    assert ((y - ref).norm() / ref.norm()).item() < 0.2          # FP4 weights and activations
    assert torch.nn.functional.cosine_similarity(y.flatten(), ref.flatten(), dim=0).item() > 0.98
