"""The preallocated block-linears runner: eager step against per-linear calls, and the same step
replayed from a CUDA graph."""
import pytest
import torch

from helpers import randn_bf16, student_t_bf16

pytestmark = pytest.mark.gpu


def _runner(tokens=700, dim=512, ffn=1536):
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import block_linears as bl
    specs = bl.wan_block_specs(dim, ffn)
    weights = {s.name: randn_bf16((s.n, s.k), 10 + i, 0.02, device="cuda") for i, s in enumerate(specs)}
    biases = {s.name: randn_bf16((s.n,), 20 + i, 0.01, device="cuda") for i, s in enumerate(specs)}
    runner = bl.WanBlockLinears(specs, tokens, weights, biases)
    inputs = {"qkv": student_t_bf16((tokens, dim), 1, device="cuda"),
              "attn_out": student_t_bf16((tokens, dim), 2, device="cuda"),
              "ffn_up": student_t_bf16((tokens, dim), 3, device="cuda")}
    return bl, runner, inputs, weights, biases


def test_step_equals_separate_linears():
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import nvfp4
    bl, runner, inputs, weights, biases = _runner()
    out = {k: v.clone() for k, v in runner.step(inputs).items()}
    nvfp4.check_status()
    for name in ("qkv", "attn_out"):
        ref = nvfp4.fp4_gemm(nvfp4.FP4Tensor.from_bfloat16(inputs[name]),
                             nvfp4.FP4Tensor.from_bfloat16(weights[name]), bias=biases[name])
        assert torch.equal(out[name], ref)
    hid = nvfp4.fp4_gemm(nvfp4.FP4Tensor.from_bfloat16(inputs["ffn_up"]),
                         nvfp4.FP4Tensor.from_bfloat16(weights["ffn_up"]), bias=biases["ffn_up"], gelu=True)
    assert torch.equal(out["ffn_up"], hid)
    down = nvfp4.fp4_gemm(nvfp4.FP4Tensor.from_bfloat16(hid),
                          nvfp4.FP4Tensor.from_bfloat16(weights["ffn_down"]), bias=biases["ffn_down"])
    assert torch.equal(out["ffn_down"], down)


def test_graph_replay_equals_eager():
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import nvfp4
    bl, runner, inputs, weights, biases = _runner()
    eager = {k: v.clone() for k, v in runner.step(inputs).items()}
    graph = runner.capture(inputs)
    for v in runner.out.values():
        v.zero_()
    graph.replay()
    torch.cuda.synchronize()
    nvfp4.check_status()
    for k, v in eager.items():
        assert torch.equal(runner.out[k], v), k
    # new contents in the same input tensors are picked up by a replay
    inputs["qkv"].copy_(student_t_bf16(tuple(inputs["qkv"].shape), 99, device="cuda"))
    graph.replay()
    torch.cuda.synchronize()
    ref = nvfp4.fp4_gemm(nvfp4.FP4Tensor.from_bfloat16(inputs["qkv"]),
                         nvfp4.FP4Tensor.from_bfloat16(weights["qkv"]), bias=biases["qkv"])
    assert torch.equal(runner.out["qkv"], ref)


def test_host_staged_steps_equal_direct_calls():
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import nvfp4
    bl, runner, inputs, weights, biases = _runner(tokens=333)
    specs = runner.specs
    host_in = {s.name: torch.empty(333, s.k, dtype=torch.bfloat16).pin_memory() for s in specs}
    host_out = {s.name: torch.empty(333, s.n, dtype=torch.bfloat16).pin_memory() for s in specs}
    staged = bl.HostStagedLinears(runner)
    for rnd in range(3):                      # back-to-back steps reuse the device buffers
        for i, s in enumerate(specs):
            host_in[s.name].copy_(student_t_bf16((333, s.k), 100 * rnd + i))
        staged.step(host_in, host_out)
        staged.wait()
        torch.cuda.synchronize()
        for s in specs:
            ref = nvfp4.fp4_gemm(nvfp4.FP4Tensor.from_bfloat16(host_in[s.name].cuda()),
                                 nvfp4.FP4Tensor.from_bfloat16(weights[s.name]), bias=biases[s.name],
                                 gelu=s.gelu)
            assert torch.equal(host_out[s.name].cuda(), ref), (rnd, s.name)
    nvfp4.check_status()
