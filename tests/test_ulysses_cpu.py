"""Ulysses head/sequence exchange on CPU ranks (gloo, world sizes 2 and 4): the exchange is
its own inverse, puts the right tokens and heads on each rank, and attention computed on the
head shards equals attention on the full tensor."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, L, H, D, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from blackwell_diffusion_rtx6000_5090_i2v_b200 import ulysses
        g = torch.Generator().manual_seed(7)
        q = torch.randn(L, H, D, generator=g)
        k = torch.randn(L, H, D, generator=g)
        v = torch.randn(L, H, D, generator=g)
        Lp, Hp = L // world, H // world
        sl = slice(rank * Lp, (rank + 1) * Lp)
        # token shard -> head shard
        qh = ulysses.seq_to_heads(q[sl].contiguous())
        assert qh.shape == (L, Hp, D)
        assert torch.equal(qh, q[:, rank * Hp:(rank + 1) * Hp])
        # packed q|k|v exchange as the block does it
        qkv = ulysses.seq_to_heads(torch.cat([q[sl], k[sl], v[sl]], dim=-1).contiguous())
        qh, kh, vh = qkv.split(D, dim=-1)
        assert torch.equal(kh, k[:, rank * Hp:(rank + 1) * Hp])
        # attention on my heads over the full sequence, then back to my tokens
        o = torch.nn.functional.scaled_dot_product_attention(
            qh.transpose(0, 1), kh.transpose(0, 1), vh.transpose(0, 1)).transpose(0, 1)
        o_local = ulysses.heads_to_seq(o.contiguous())
        assert o_local.shape == (Lp, H, D)
        ref = torch.nn.functional.scaled_dot_product_attention(
            q.transpose(0, 1), k.transpose(0, 1), v.transpose(0, 1)).transpose(0, 1)
        assert torch.allclose(o_local, ref[sl], atol=1e-5, rtol=1e-5)
        # round trip
        assert torch.equal(ulysses.heads_to_seq(ulysses.seq_to_heads(q[sl].contiguous())), q[sl])
        # the send buffer already grouped by destination rank (the layout the q/k norm + RoPE
        # kernel writes in its exchange form): one collective, no packing copy
        packed = torch.cat([q[sl], k[sl], v[sl]], dim=-1)                    # [Lp, H, 3D]
        send = packed.reshape(Lp, world, Hp, 3 * D).permute(1, 0, 2, 3).contiguous()
        assert torch.equal(ulysses.all_to_all_packed(send, dist.group.WORLD), qkv)
        # bad head count is refused before any communication
        try:
            ulysses.seq_to_heads(torch.zeros(Lp, H + 1, D))
            raised = False
        except ValueError:
            raised = True
        assert raised
        out[rank] = 1
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,L,H", [(2, 10, 4), (4, 24, 8)])
def test_exchange_and_attention(world, L, H):
    port = _free_port()
    out = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, L, H, 8, out), nprocs=world, join=True)
    assert sorted(out.keys()) == list(range(world))


def test_single_rank_is_identity():
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import ulysses
    x = torch.randn(6, 4, 8)
    assert ulysses.seq_to_heads(x) is x and ulysses.heads_to_seq(x) is x
    # A14B shape at 8 ranks: 4 tensors of 4095 tokens x 40 heads x 128 x 2 B, 7/8 of which leave
    assert ulysses.exchange_bytes_per_rank(32760, 40, 128, 8) == 4 * 4095 * 40 * 128 * 2 * 7 // 8


def _leaver(rank, world, port, out):
    """Rank 1 leaves between steps (no collective of its own in flight); rank 0's next exchange
    must end with an error inside the group's time limit instead of hanging."""
    import datetime
    import time
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import ulysses
    x = torch.randn(4, 4, 8)
    ulysses.seq_to_heads(x)                     # one healthy step on both ranks
    if rank == 1:
        out[1] = "left"
        os._exit(0)                             # gone: no goodbye, no destroy
    t0 = time.perf_counter()
    try:
        ulysses.seq_to_heads(x)
        out[0] = "no error"
    except Exception as e:                      # gloo reports the closed connection or the timeout
        out[0] = f"error after {time.perf_counter() - t0:.1f}s: {type(e).__name__}"
    os._exit(0)


def test_departed_rank_surfaces_as_error_not_a_hang():
    port = _free_port()
    out = mp.Manager().dict()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_leaver, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=60)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.kill()
    assert not alive, "a rank hung after its peer left"
    assert out.get(1) == "left"
    assert str(out.get(0, "")).startswith("error after"), out.get(0)
