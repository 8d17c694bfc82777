"""The ``te.Linear`` / ``fp8_autocast`` front end: the constructor and context-manager shapes
the reference's model files use (fx/src/s4/models/wan22/wan_transformer_megaupload.py:162-165,
fx/src/s4/models/wan22/bench_te_nvfp4.py:96-122), on CPU for the signatures and the bf16 path,
on the GPU for the NVFP4 path."""
import pytest
import torch


def test_constructor_and_context_shapes():
    import blackwell_diffusion_rtx6000_5090_i2v_b200.te_compat as te
    from blackwell_diffusion_rtx6000_5090_i2v_b200.te_compat import Format, NVFP4BlockScaling
    lin = te.Linear(64, 48)                                         # megaupload.py:46 form
    lin2 = te.Linear(64, 48, bias=True, params_dtype=torch.bfloat16)  # bench_te_nvfp4.py:120 form
    nob = te.Linear(64, 48, bias=False)
    assert lin.weight.shape == (48, 64) and lin.weight.dtype == torch.bfloat16
    assert lin2.bias is not None and nob.bias is None
    assert lin.in_features == 64 and lin.out_features == 48
    with pytest.raises(TypeError):
        te.Linear(64, 48, params_dtype=torch.float32)
    with pytest.raises(TypeError):
        te.Linear(64, 48, tp_size=2)
    recipe = NVFP4BlockScaling(fp4_format=Format.E2M1)
    assert recipe.fp4_format is Format.E2M1
    with pytest.raises(ValueError):
        NVFP4BlockScaling(fp4_format=Format.E4M3)
    # outside the context (and with enabled=False) the module is a plain bf16 linear
    x = torch.randn(2, 5, 64).to(torch.bfloat16)
    want = torch.nn.functional.linear(x, lin.weight, lin.bias)
    assert torch.equal(lin(x), want)
    with te.fp8_autocast(enabled=False, fp8_recipe=recipe):
        assert torch.equal(lin(x), want)
    # the context nests and restores
    assert te._active_recipe() is None
    with te.fp8_autocast(enabled=True, fp8_recipe=recipe):
        assert te._active_recipe() is recipe
        with te.fp8_autocast(enabled=False):
            assert te._active_recipe() is None
        assert te._active_recipe() is recipe
    assert te._active_recipe() is None
    with pytest.raises(NotImplementedError):
        with te.fp8_autocast(enabled=True, fp8_recipe=object()):
            pass


@pytest.mark.gpu
def test_autocast_runs_the_nvfp4_linear():
    import blackwell_diffusion_rtx6000_5090_i2v_b200.te_compat as te
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import nvfp4, nvfp4_linear_cpp
    from blackwell_diffusion_rtx6000_5090_i2v_b200.te_compat import Format, NVFP4BlockScaling
    torch.manual_seed(3)
    lin = te.Linear(768, 512, bias=True, params_dtype=torch.bfloat16).cuda()
    x = torch.randn(1, 128, 768, dtype=torch.bfloat16).cuda()
    with torch.no_grad():
        bf16 = lin(x)
        with te.fp8_autocast(enabled=True, fp8_recipe=NVFP4BlockScaling(fp4_format=Format.E2M1)):
            fp4 = lin(x)
        want = nvfp4_linear_cpp.linear(x, lin.weight, lin.bias)
    nvfp4.check_status()
    assert fp4.shape == (1, 128, 512) and torch.equal(fp4, want)
    assert not torch.equal(fp4, bf16)
    rel = float((fp4.float() - bf16.float()).norm() / bf16.float().norm())
    assert rel < 0.2, rel     # the reference's own bound for FP4 against bf16 (nvfp4_test.py:31)
