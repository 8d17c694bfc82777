"""The flag-ordered exchange kernels on ONE GPU, through the C ABI: the ranks of a
sequence-parallel step are emulated as consecutive launches over separate buffers (every
producer has finished before a wait kernel starts, so no kernel ever waits for a later launch),
plus the bounded wait running out on a flag nobody raises."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr_array(tensors):
    return (C.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def _setup(world):
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import _native as N
    words = N.lib.nvfp4_exchange_sync_bytes() // 4
    sync = [torch.zeros(words, dtype=torch.int32, device="cuda") for _ in range(world)]
    return N, sync, _ptr_array(sync)


@pytest.mark.parametrize("world,L,Hp,D,transposed", [(2, 600, 3, 128, False), (4, 1024, 2, 64, True),
                                                      (1, 77, 5, 128, False), (8, 4096, 5, 128, True)])
def test_return_exchange_layout_amax_and_flags(world, L, Hp, D, transposed):
    """Every emulated rank's attention output lands in the right rows / head columns of every
    destination's buffer, the destination's wait kernel leaves max|assembled buffer| in the amax
    slot, and a second round (next epoch) works on the same sync blocks."""
    N, sync, sync_ptrs = _setup(world)
    H, Lp = Hp * world, L // world
    st = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = [torch.zeros(Lp, H, D, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    out_ptrs = _ptr_array(out)
    amax = [torch.full((1,), -1.0, device="cuda") for _ in range(world)]
    for rnd in range(2):
        g = torch.Generator(device="cuda").manual_seed(10 * rnd + world)
        o = []
        for r in range(world):
            t = torch.randn(Hp, L, D, generator=g, device="cuda") * (1 + r)
            t = t.to(torch.bfloat16)
            # attention kernels hand back either [L, Hp, D] memory or a transposed view of [Hp, L, D]
            o.append(t.transpose(0, 1) if transposed else t.transpose(0, 1).contiguous())
        for r in range(world):
            rc = N.lib.nvfp4_attn_return_exchange_bf16(o[r].data_ptr(), o[r].stride(0), o[r].stride(1), L,
                                                       Hp, D, out_ptrs, sync_ptrs, world, r, st)
            assert rc == 0, N.status_string(rc)
        for s in range(world):
            rc = N.lib.nvfp4_exchange_wait(sync[s].data_ptr(), 1, world, 50_000_000, amax[s].data_ptr(),
                                           status.data_ptr(), st)
            assert rc == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        for s in range(world):
            want = torch.cat([o[r][s * Lp:(s + 1) * Lp] for r in range(world)], dim=1)   # [Lp, H, D]
            assert torch.equal(out[s], want), (rnd, s)
            assert float(amax[s].item()) == float(want.float().abs().max().item()), (rnd, s)


@pytest.mark.parametrize("world,heads,Lp", [(2, 4, 150), (4, 8, 33), (8, 40, 9)])
def test_rope_exchange_raises_flags_and_wait_passes(world, heads, Lp):
    """The q/k norm + RoPE kernel in its exchange form with sync blocks, 2 / 4 / 8 emulated ranks
    (odd token counts per rank, five heads per rank as in the 8-GPU A14B run): the pieces equal
    the plain packed form's, and the kind-0 wait passes on every rank."""
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import dit
    D = 128
    N, sync, sync_ptrs = _setup(world)
    L, Hp, dim = world * Lp, heads // world, heads * D
    cfg = dit.WanDiTConfig(dim=dim, heads=heads, ffn=1024, layers=1, in_channels=16, out_channels=16)
    cos, sin = dit.rope_tables(cfg, (1, 1, L), "cuda")
    cs = dit.pack_rope_table(cos, sin)
    g = torch.Generator(device="cuda").manual_seed(3)
    qkv = (torch.randn(L, 3 * dim, generator=g, device="cuda") * 2).to(torch.bfloat16)
    gq = 1 + 0.1 * torch.randn(dim, generator=g, device="cuda")
    gk = 1 + 0.1 * torch.randn(dim, generator=g, device="cuda")
    want = dit.qk_norm_rope(qkv, heads, D, gq, gk, cfg.eps, cs, packed=True)       # [L, heads, 3D]
    bufs = [torch.zeros(L, Hp, 3 * D, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    buf_ptrs = _ptr_array(bufs)
    st = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for r in range(world):
        shard = qkv[r * Lp:(r + 1) * Lp].contiguous()
        table = cs[r * Lp:(r + 1) * Lp].contiguous()
        base = shard.data_ptr()
        rc = N.lib.nvfp4_qk_norm_rope_exchange_bf16(
            base, base + 2 * dim, base + 4 * dim, 3 * dim, Lp, heads, D, gq.data_ptr(), gk.data_ptr(),
            float(cfg.eps), table.data_ptr(), buf_ptrs, world, r * Lp,
            sync_ptrs, r, status.data_ptr(), st)
        assert rc == 0, N.status_string(rc)
        torch.cuda.synchronize()
    for s in range(world):
        assert N.lib.nvfp4_exchange_wait(sync[s].data_ptr(), 0, world, 50_000_000, None,
                                         status.data_ptr(), st) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for s in range(world):
        assert torch.equal(bufs[s], want[:, s * Hp:(s + 1) * Hp]), s


def test_wait_runs_out_and_reports_the_missing_rank():
    """A flag nobody raises: the wait kernel gives up after its limit (milliseconds), names the
    first missing rank in the status word and returns normally; the context stays usable and a
    later, properly signalled round passes again."""
    import time
    world = 2
    N, sync, sync_ptrs = _setup(world)
    st = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    rc = N.lib.nvfp4_exchange_wait(sync[0].data_ptr(), 0, world, 3_000_000, None, status.data_ptr(), st)
    assert rc == 0
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert int(status.item()) == 0xB00, hex(int(status.item()))      # rank 0's flag is the first missing
    assert 0.002 <= waited < 1.0, waited
    # only rank 1 missing: raise rank 0's flag by hand to the epoch the next wait expects (2)
    status.zero_()
    sync[0][0] = 2
    rc = N.lib.nvfp4_exchange_wait(sync[0].data_ptr(), 0, world, 3_000_000, None, status.data_ptr(), st)
    torch.cuda.synchronize()
    assert rc == 0 and int(status.item()) == 0xB01
    # while the status word stays set, a further wait on a missing flag returns at once
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    assert N.lib.nvfp4_exchange_wait(sync[0].data_ptr(), 0, world, 2_000_000_000, None,
                                     status.data_ptr(), st) == 0
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 0.5 and int(status.item()) == 0xB01
    # bad arguments are refused on the host
    assert N.lib.nvfp4_exchange_wait(None, 0, world, 1000, None, None, st) == 1
    assert N.lib.nvfp4_exchange_wait(sync[0].data_ptr(), 2, world, 1000, None, None, st) == 1
    assert N.lib.nvfp4_exchange_wait(sync[0].data_ptr(), 0, 9, 1000, None, None, st) == 1
    assert N.lib.nvfp4_exchange_wait(sync[0].data_ptr(), 0, world, 0, None, None, st) == 1
    # the device still works: a signalled round of the other kind passes
    status.zero_()
    Lp, Hp, D = 64, 2, 128
    o = [torch.randn(world * Lp, Hp, D, device="cuda").to(torch.bfloat16) for _ in range(world)]
    out = [torch.zeros(Lp, Hp * world, D, dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    out_ptrs = _ptr_array(out)
    for r in range(world):
        assert N.lib.nvfp4_attn_return_exchange_bf16(o[r].data_ptr(), o[r].stride(0), o[r].stride(1),
                                                     world * Lp, Hp, D, out_ptrs, sync_ptrs, world, r, st) == 0
    amax = torch.zeros(1, device="cuda")
    assert N.lib.nvfp4_exchange_wait(sync[1].data_ptr(), 1, world, 50_000_000, amax.data_ptr(),
                                     status.data_ptr(), st) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert float(amax.item()) == float(out[1].float().abs().max().item())
