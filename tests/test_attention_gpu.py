"""The package's tcgen05 attention kernel (``nvfp4_attention_bf16``) against an fp32 softmax(QK^T)V
and against the library kernel it can replace (the reference's call sites:
fx/src/s4/models/wan22/wan_transformer_fast.py:47-58, wan_transformer.py:126-129,164-167).

Tolerance: bf16 attention output.  The fp32 reference rounds nothing; both kernels round the
probabilities and the output to bf16, so the kernel must stay within twice the library's own
maximum error (and 1e-2 absolute as a floor for |o| of order one)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(q, k, v):
    qf, kf, vf = (t.float().transpose(0, 1) for t in (q, k, v))
    s = qf @ kf.transpose(1, 2) / q.shape[-1] ** 0.5
    return (torch.softmax(s, -1) @ vf).transpose(0, 1)


def _inputs(Lq, Lk, H, mag, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = (torch.randn(Lq, H, 128, generator=g, device="cuda") * mag).bfloat16()
    k = (torch.randn(Lk, H, 128, generator=g, device="cuda") * mag).bfloat16()
    v = torch.randn(Lk, H, 128, generator=g, device="cuda").bfloat16()
    return q, k, v


@pytest.mark.parametrize("Lq,Lk,H,mag", [
    (256, 128, 1, 1.0),       # one key tile
    (256, 256, 1, 1.0),       # two key tiles: the accumulate path
    (128, 512, 2, 1.0),       # second query tile entirely past the end
    (300, 1000, 3, 1.0),      # ragged queries and keys
    (1, 1, 1, 1.0),           # a single query and key
    (257, 129, 2, 1.0),       # one row / one key into the next tile
    (512, 2048, 4, 4.0),      # logits large enough that the running maximum is raised late
    (1000, 4000, 2, 8.0),
    (1024, 512, 24, 1.0),     # the cross-attention shape: 512 text tokens, 24 heads
])
def test_attention_matches_fp32(Lq, Lk, H, mag):
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import dit, nvfp4
    q, k, v = _inputs(Lq, Lk, H, mag, 100 + Lq + Lk)
    amax = torch.zeros(1, device="cuda")
    o = dit.attention_native(q, k, v, amax=amax)
    nvfp4.check_status()
    r = _ref(q, k, v)
    err = (o.float() - r).abs().max().item()
    old = dit.ATTENTION_BACKEND
    dit.ATTENTION_BACKEND = "library"
    try:
        err_lib = (dit.attention(q, k, v).float() - r).abs().max().item()
    finally:
        dit.ATTENTION_BACKEND = old
    assert err <= max(2 * err_lib, 1e-2), (err, err_lib)
    # the folded maximum is the maximum of the bf16 output, bit for bit
    assert amax.item() == o.float().abs().max().item()


def test_attention_on_fused_qkv_views():
    """q, k, v as column blocks of one [L, 3*H*128] projection output (no copy), o into a view."""
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import dit, nvfp4
    L, H = 700, 6
    g = torch.Generator(device="cuda").manual_seed(3)
    qkv = torch.randn(L, 3 * H * 128, generator=g, device="cuda").bfloat16()
    q, k, v = (t.view(L, H, 128) for t in qkv.split(H * 128, dim=-1))
    wide = torch.zeros(L, 2 * H * 128, dtype=torch.bfloat16, device="cuda")
    out = wide[:, H * 128:].view(L, H, 128)
    o = dit.attention_native(q, k, v, out=out)
    nvfp4.check_status()
    assert o.data_ptr() == out.data_ptr()
    assert torch.equal(o, dit.attention_native(q.contiguous(), k.contiguous(), v.contiguous()))
    assert (o.float() - _ref(q, k, v)).abs().max().item() <= 1e-2
    assert not wide[:, :H * 128].any()        # nothing written outside the view


def test_attention_repeatable_and_full_length():
    """The Wan 2.2 5B sequence (27280 tokens: 213 full key tiles and one of 16 keys) on two heads:
    bit-identical between launches and within bf16 of the library kernel."""
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import dit, nvfp4
    q, k, v = _inputs(27280, 27280, 2, 1.0, 7)
    a = dit.attention_native(q, k, v)
    b = dit.attention_native(q, k, v)
    nvfp4.check_status()
    assert torch.equal(a, b)
    old = dit.ATTENTION_BACKEND
    dit.ATTENTION_BACKEND = "library"
    try:
        lib = dit.attention(q, k, v)
    finally:
        dit.ATTENTION_BACKEND = old
    d = (a.float() - lib.float()).abs().max().item()
    cos = torch.nn.functional.cosine_similarity(a.flatten().double(), lib.flatten().double(), dim=0).item()
    assert d <= 2e-3 and cos >= 0.9999, (d, cos)


def test_attention_rejects_bad_arguments():
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import _native as N
    x = torch.zeros(256, 1, 128, dtype=torch.bfloat16, device="cuda")
    st = N.stream_ptr()

    def call(q=x, hd=128, lk=256, qs=128, scale=0.1, o=x):
        return N.lib.nvfp4_attention_bf16(q.data_ptr() if q is not None else None, qs, 128, x.data_ptr(), 128, 128,
                                          x.data_ptr(), 128, 128, 256, lk, 1, hd, scale,
                                          o.data_ptr() if o is not None else None, 128, 128, None, None, st)
    assert call() == 0
    assert call(hd=64) == 1            # only head dimension 128
    assert call(lk=0) == 1             # softmax over no keys
    assert call(q=None) == 1
    assert call(o=None) == 1
    assert call(scale=0.0) == 1
    assert call(qs=132) == 2           # token stride not a multiple of 16 bytes
    torch.cuda.synchronize()


def test_block_with_native_attention_matches_library():
    """A DiT block stack with the package's attention kernel (self-attention hands its folded
    max|o| to the attention-out quantizer, cross-attention runs through it too) against the
    same model on the library kernel: the two attention kernels differ by bf16 roundings only."""
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import dit, nvfp4
    cfg = dit.WanDiTConfig(dim=512, heads=4, ffn=1024, layers=2, in_channels=16, out_channels=16,
                           text_dim=256)
    model = dit.WanDiT(cfg, device="cuda", seed=11)
    g = torch.Generator(device="cuda").manual_seed(5)
    latent = torch.randn(16, 4, 16, 20, generator=g, device="cuda").to(torch.bfloat16)   # 320 tokens
    text = torch.randn(24, 256, generator=g, device="cuda").to(torch.bfloat16)
    old = dit.ATTENTION_BACKEND
    try:
        dit.ATTENTION_BACKEND = "library"
        a = model.forward(latent, 500.0, text)
        dit.ATTENTION_BACKEND = "native"
        b = model.forward(latent, 500.0, text)
    finally:
        dit.ATTENTION_BACKEND = old
    nvfp4.check_status()
    cos = torch.nn.functional.cosine_similarity(a.flatten().double(), b.flatten().double(), dim=0).item()
    assert cos >= 0.999, cos
