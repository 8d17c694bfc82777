"""DiT step latency on the NVFP4 path: ``python -m blackwell_diffusion_rtx6000_5090_i2v_b200.dit_step``.

One denoising step of the Wan 2.2 shaped model (``dit.WanDiT``; random weights, seeded
synthetic latent and text) on one GPU, or token-sharded over the ranks of a ``torchrun``
launch with the Ulysses exchange around self-attention.  Prints one JSON line: step latency
(CUDA events, max over ranks), the per-component device time of rank 0, the linears'
aggregate TFLOP/s, and -- with ``--check`` -- the cosine of the step output against the same
model evaluated with dequantize-then-matmul linears (and, on several ranks, against the
unsharded model run on rank 0).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist

from . import dit, nvfp4

LATENTS = {"5b": (48, 31, 44, 80), "14b": (16, 21, 60, 104)}   # -> 27280 / 32760 tokens
CONFIGS = {"5b": dit.WAN22_TI2V_5B, "14b": dit.WAN22_A14B}


def _cos(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double().flatten(), b.double().flatten()
    return float(torch.dot(a, b) / (a.norm() * b.norm()))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--config", choices=sorted(CONFIGS), default="5b")
    ap.add_argument("--layers", type=int, default=None, help="blocks to build (default: all)")
    ap.add_argument("--frames", type=int, default=None, help="latent frames (default: the config's)")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--check", action="store_true", help="cosine against the dequant model")
    ap.add_argument("--sdpa", choices=["default", "flash", "cudnn"], default="default")
    ap.add_argument("--attention", choices=["library", "native"], default="library",
                    help="library: torch's scaled_dot_product_attention; native: the package's tcgen05 kernel")
    ap.add_argument("--graph", action="store_true",
                    help="also time the step replayed from a CUDA graph (single GPU, or sharded with "
                         "--exchange peer)")
    ap.add_argument("--exchange", choices=["nccl", "peer"], default="nccl",
                    help="head/sequence exchange: all-to-alls, or stores into peer memory")
    ap.add_argument("--amax-sync", action="store_true",
                    help="sharded runs: quantize every activation with the all-reduced (max) amax")
    args = ap.parse_args(argv)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        group = dist.group.WORLD
    nvfp4.init()

    cfg = CONFIGS[args.config]
    C, Fr, H, W = LATENTS[args.config]
    if args.frames:
        Fr = args.frames
    model = dit.WanDiT(cfg, device=f"cuda:{local}", seed=1234 + (3 if args.config == "5b" else 4),
                       layers=args.layers)
    g = torch.Generator(device="cuda").manual_seed(4321)
    latent = torch.randn(C, Fr, H, W, generator=g, device="cuda").to(torch.bfloat16)
    text = torch.randn(512, cfg.text_dim, generator=g, device="cuda").to(torch.bfloat16)
    tokens = Fr * (H // 2) * (W // 2)

    dit.ATTENTION_BACKEND = args.attention
    backends = None
    if args.sdpa != "default":
        from torch.nn.attention import SDPBackend
        backends = [SDPBackend.FLASH_ATTENTION if args.sdpa == "flash" else SDPBackend.CUDNN_ATTENTION]

    def step(mode="nvfp4", grp=group, exchange=args.exchange):
        kw = dict(mode=mode, group=grp, exchange=exchange, amax_sync=args.amax_sync and grp is not None)
        if backends is not None:
            from torch.nn.attention import sdpa_kernel
            with sdpa_kernel(backends):
                return model.forward(latent, 500.0, text, **kw)
        return model.forward(latent, 500.0, text, **kw)

    def fence():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.no_grad():
        for _ in range(args.warmup):
            y = step()
        times = []
        for _ in range(args.steps):
            fence()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            y = step()
            e1.record()
            fence()
            t = torch.tensor([e0.elapsed_time(e1)], device="cuda")
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            times.append(float(t))
        nvfp4.check_status()
        # one more step with the per-component marks on
        dit.TIMELINE = dit.Timeline()
        dit.TIMELINE.mark("start")
        step()
        dit.TIMELINE.mark("other")
        parts = dit.TIMELINE.totals_ms()
        dit.TIMELINE = None

        checks = {}
        if args.graph and (world == 1 or args.exchange == "peer") and not args.amax_sync:
            if world == 1:
                graph, gout = model.capture(latent, 500.0, text)
                finish = lambda: gout                                      # noqa: E731
            else:
                graph, gshard, ggrid = model.capture(latent, 500.0, text, group=group)
                finish = lambda: model.gather_tokens(gshard, ggrid, group)  # noqa: E731
            gtimes = []
            for _ in range(args.steps):
                fence()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                graph.replay()
                gy = finish()
                e1.record()
                fence()
                t = torch.tensor([e0.elapsed_time(e1)], device="cuda")
                if world > 1:
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                gtimes.append(float(t))
            nvfp4.check_status()
            checks["graph_replay_ms"] = round(statistics.median(gtimes), 3)
            checks["graph_replay_equals_eager"] = bool(torch.equal(gy, y))
        if args.check:
            ref = step(mode="dequant")
            checks["cosine_vs_dequant_model"] = _cos(y, ref)
            # control: the dequant model against itself with every GEMM's K sum in reverse order
            ctl = step(mode="dequant_reordered")
            checks["cosine_dequant_model_vs_itself_reordered_sums"] = _cos(ref, ctl)
            del ctl
            # The same two comparisons with the comparison model's activation quantizers using
            # the per-tensor amax the NVFP4 path had for the same tensor (its block scales and
            # elements still come from its own activations): isolates how much of the
            # free-running divergence enters through the FP32 tensor scale.
            dit.AMAX_RECORD = {}
            y_rec = step()
            pinned, dit.AMAX_RECORD = dit.AMAX_RECORD, None
            checks["recorded_step_equals_step"] = bool(torch.equal(y_rec, y))
            dit.AMAX_PIN = pinned
            ref_pin = step(mode="dequant")
            ctl_pin = step(mode="dequant_reordered")
            dit.AMAX_PIN = None
            checks["cosine_vs_dequant_model_pinned_amax"] = _cos(y, ref_pin)
            checks["cosine_pinned_dequant_model_vs_itself_reordered_sums"] = _cos(ref_pin, ctl_pin)
            del ref_pin, ctl_pin, y_rec
            # The comparison model fed, linear by linear, the packed activation the NVFP4 path
            # quantized (matmuls, epilogues, norms, attention and the residual stream stay its
            # own): the step-level statement of "same quantized inputs, independent arithmetic".
            dit.QUANT_RECORD = {}
            step()
            shared, dit.QUANT_RECORD = dit.QUANT_RECORD, None
            dit.QUANT_PIN = shared
            ref_shared = step(mode="dequant")
            dit.QUANT_PIN = None
            checks["cosine_vs_dequant_model_shared_packed_activations"] = _cos(y, ref_shared)
            del ref_shared
            # and where the free-running comparison model parts ways with the NVFP4 path: element
            # codes, block scales or tensor amax, for the first two blocks and the last
            dit.QUANT_RECORD = {}
            step(mode="dequant")
            free, dit.QUANT_RECORD = dit.QUANT_RECORD, None
            flips = dit.flip_stats(shared, free)
            keep = [n for n in flips if n.startswith(("blocks.0.", "blocks.1.", f"blocks.{len(model.blocks) - 1}."))]
            checks["packed_activation_differences"] = {n: {k: (round(v, 5) if isinstance(v, float) else v)
                                                           for k, v in flips[n].items()} for n in keep}
            del shared, free
            if world == 1:
                per_block = model.compare_blocks(latent, 500.0, text)
                checks["per_block_same_input_cosine_min"] = min(c for c, _ in per_block)
                checks["per_block_same_input_delta_cosine_min"] = min(d for _, d in per_block)
            if world > 1 and args.exchange == "peer":
                other = step(exchange="nccl")
                checks["peer_exchange_equals_nccl_exchange"] = bool(torch.equal(y, other))
                del other
            if world > 1:
                fence()
                if rank == 0:
                    full = step(grp=None)
                    checks["cosine_sharded_vs_single_gpu"] = _cos(y, full)
                fence()

    if rank == 0:
        ms = statistics.median(times)
        lin = model.linear_flops(tokens)
        att = model.attention_flops(tokens)
        gemm_ms = sum(v for k, v in parts.items() if k.startswith("gemm")) + parts.get("text_kv", 0.0)
        cfgm, nb = model.cfg, len(model.blocks)
        per_linear = {}
        for name, n_out, k_in in (("qkv", 3 * cfgm.dim, cfgm.dim), ("attn_out", cfgm.dim, cfgm.dim),
                                  ("cross_q", cfgm.dim, cfgm.dim), ("cross_out", cfgm.dim, cfgm.dim),
                                  ("ffn_up", cfgm.ffn, cfgm.dim), ("ffn_down", cfgm.dim, cfgm.ffn)):
            ms_l = parts.get("gemm_" + name)
            if ms_l:
                per_linear[name] = round(2.0 * (tokens // world) * n_out * k_in * nb / (ms_l * 1e-3) / 1e12, 1)
        line = {
            "metric": "dit_step_latency", "unit": "ms", "value": round(ms, 3),
            "higher_is_better": False, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "config": {"workload": f"wan2.2 {args.config} shape, {len(model.blocks)} blocks, "
                                   f"{tokens} tokens, text 512x{cfg.text_dim}",
                       "tokens_per_rank": tokens // world, "sdpa": args.sdpa,
                       "attention": args.attention,
                       "exchange": args.exchange if world > 1 else None,
                       "amax_sync": bool(args.amax_sync and world > 1),
                       "parallelism": f"ulysses{world}" if world > 1 else "single"},
            "all_ms": [round(t, 3) for t in times],
            "components_ms_rank0": {k: round(v, 3) for k, v in sorted(parts.items())},
            "linear_tflop": round(lin / 1e12, 2), "attention_tflop": round(att / 1e12, 2),
            "gemm_tflops_per_gpu": round(lin / world / (gemm_ms * 1e-3) / 1e12, 1) if gemm_ms else None,
            "gemm_tflops_per_linear_rank0": per_linear,
            "data": "synthetic", "dtype": "nvfp4 linears, bf16 attention",
        }
        line.update(checks)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
