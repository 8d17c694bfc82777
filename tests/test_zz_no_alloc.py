"""The allocation-free linear entry point against the ordinary path.

Some users of this library cannot allocate device memory around a call (they run where
cudaMalloc is off limits, or were only handed input and output pointers), so
``nvfp4_linear_bf16_static`` keeps its intermediates in a fixed array inside the library.
This test drives it through the C ABI twice in a row, with different shapes so that the
second call runs over the first call's leftovers, and expects exactly the bytes the
caller-allocated path (quantize + GEMM) produces.  It is collected last on purpose.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference(nv, x, wq, bias, gelu):
    a = nv.FP4Tensor.from_bfloat16(x, linear_scales=False)
    return nv.fp4_gemm(a, wq, bias=bias, gelu=gelu)


def test_static_linear_matches_regular_path_twice():
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import _native as N
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import nvfp4 as nv
    from blackwell_diffusion_rtx6000_5090_i2v_b200.synthetic import (
        outlier_weight_bf16, randn_bf16, student_t_bf16)

    torch.cuda.set_device(0)
    st = torch.cuda.current_stream().cuda_stream
    status = N.status_word(torch.device("cuda", 0))
    cases = [  # (M, K, N, gelu) -- the second is smaller and ragged, on purpose
        (1000, 3072, 1024, True),
        (77, 160, 264, False),
    ]
    for i, (M, K, Nn, gelu) in enumerate(cases):
        x = student_t_bf16((M, K), 900 + i, device="cuda")
        w = outlier_weight_bf16((Nn, K), 910 + i, device="cuda")
        bias = randn_bf16((Nn,), 920 + i, 0.01, device="cuda")
        wq = nv.FP4Tensor.from_bfloat16(w, linear_scales=False)
        want = _reference(nv, x, wq, bias, gelu)
        got = torch.full((M, Nn), float("nan"), dtype=torch.bfloat16, device="cuda")
        rc = N.lib.nvfp4_linear_bf16_static(
            x.data_ptr(), M, K, wq._data.data_ptr(), wq._scales_swz.data_ptr(),
            wq._gscale.data_ptr(), Nn, bias.data_ptr(), 1 if gelu else 0, got.data_ptr(),
            status.data_ptr(), st)
        assert rc == 0, N.status_string(rc)
        torch.cuda.synchronize()
        N.check_status()
        assert torch.equal(got, want), f"case {i}: static-scratch linear differs from the regular path"


def test_static_linear_rejects_oversized_problems():
    from blackwell_diffusion_rtx6000_5090_i2v_b200 import _native as N
    limit = N.lib.nvfp4_linear_bf16_static_max_elements()
    assert limit == 8 << 20
    # one row too many for K = 4096: refused on the host, nothing is launched
    rc = N.lib.nvfp4_linear_bf16_static(None, limit // 4096 + 1, 4096, None, None, None, 256,
                                        None, 0, None, None, None)
    assert rc == 1
    # few elements, but the padded scale layout (rows to 256, K to 256) outgrows its 1 MiB
    rc = N.lib.nvfp4_linear_bf16_static(None, 1, 131072, None, None, None, 256, None, 0, None,
                                        None, None)
    assert rc == 1
    # extents whose product wraps a 64-bit integer are refused before anything is multiplied
    for m, k in ((1 << 62, 32), (1 << 40, 1 << 40), (3, (1 << 62) + 32)):
        rc = N.lib.nvfp4_linear_bf16_static(None, m, k, None, None, None, 256, None, 0, None,
                                            None, None)
        assert rc == 1, (m, k)
