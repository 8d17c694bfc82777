"""Two-GPU check of the head/sequence exchange: stores into peer memory fused into the q/k norm
+ RoPE kernel against the all-to-all form (same bits), on child processes over NCCL.  Skipped
on a single-GPU box; the layout logic is covered on CPU ranks in test_ulysses_cpu.py."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from blackwell_diffusion_rtx6000_5090_i2v_b200 import dit, nvfp4
        cfg = dit.WanDiTConfig(dim=512, heads=4, ffn=1024, layers=2, in_channels=16, out_channels=16,
                               text_dim=256)
        model = dit.WanDiT(cfg, device=f"cuda:{rank}", seed=11)
        g = torch.Generator(device="cuda").manual_seed(5)
        latent = torch.randn(16, 4, 8, 16, generator=g, device="cuda").to(torch.bfloat16)   # 128 tokens
        text = torch.randn(24, 256, generator=g, device="cuda").to(torch.bfloat16)
        grp = dist.group.WORLD
        a = model.forward(latent, 500.0, text, group=grp, exchange="nccl")
        b = model.forward(latent, 500.0, text, group=grp, exchange="peer")
        c = model.forward(latent, 500.0, text, group=grp, exchange="peer")   # second use of the buffers
        nvfp4.check_status()
        assert torch.isfinite(a.float()).all()
        assert torch.equal(a, b) and torch.equal(b, c)
        # every quantizer's amax all-reduced (max) over the shards: the sharded step quantizes
        # with the unsharded model's tensor scales and reproduces its output
        d = model.forward(latent, 500.0, text, group=grp, exchange="peer", amax_sync=True)
        full = model.forward(latent, 500.0, text)
        nvfp4.check_status()
        cos = torch.dot(d.double().flatten(), full.double().flatten()) / (d.double().norm() * full.double().norm())
        assert float(cos) >= 1 - 1e-9, float(cos)
        # the sharded step recorded into a CUDA graph: the flag waits' epochs live in device
        # memory, so each replay meets the peers' matching replay; same bits as the eager step
        graph, shard, grid = model.capture(latent, 500.0, text, group=grp)
        for _ in range(3):
            graph.replay()
            g = model.gather_tokens(shard, grid, grp)
            nvfp4.check_status()
            assert torch.equal(g, b)
        # and eager steps still work after replays (the epochs moved on consistently)
        assert torch.equal(model.forward(latent, 500.0, text, group=grp, exchange="peer"), b)
        out[rank] = 1
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_exchange_equals_all_to_all():
    import torch.multiprocessing as mp
    port = _free_port()
    out = mp.get_context("spawn").Manager().dict()
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    assert sorted(out.keys()) == [0, 1]
