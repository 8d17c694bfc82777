"""The four NVFP4 linears of one Wan 2.2 DiT block as one preallocated runner.

Call sites being accelerated: ``to_qkv`` / ``to_out`` of the self-attention
(fx/src/s4/models/wan22/wan_transformer.py:111,129) and the feed-forward
up (+GELU-tanh) / down projections (:185,220).  Weights are quantized once at
construction; every step quantizes the bf16 activations (amax pass + pack
pass) and runs the tcgen05 GEMM with bias (and GELU) fused in its epilogue.
All buffers are allocated up front, so a step launches kernels only.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from . import _native as N
from .nvfp4 import FP4Tensor
from .shapes import WAN22_A14B, WAN22_TI2V_5B, LinearSpec, wan_block_specs  # noqa: F401  (re-exported)


class _QuantScratch:
    """Reusable packed-activation buffers for an [m, k] bf16 input."""

    def __init__(self, m: int, k: int, device):
        self.m, self.k = m, k
        self.data = torch.empty(m * k // 2, dtype=torch.uint8, device=device)
        self.sf = torch.empty(N.lib.nvfp4_swizzled_scale_bytes(m, k), dtype=torch.uint8,
                              device=device)
        self.amax = torch.empty(1, dtype=torch.float32, device=device)
        self.gscale = torch.empty(1, dtype=torch.float32, device=device)


class WanBlockLinears:
    """Quantized weights + scratch for the block's linears at a fixed token count."""

    def __init__(self, specs: List[LinearSpec], tokens: int, weights: Dict[str, torch.Tensor],
                 biases: Optional[Dict[str, torch.Tensor]] = None, device="cuda"):
        self.specs = specs
        self.tokens = tokens
        self.device = torch.device(device)
        self.w: Dict[str, FP4Tensor] = {}
        self.bias: Dict[str, Optional[torch.Tensor]] = {}
        self.act: Dict[str, _QuantScratch] = {}
        self.out: Dict[str, torch.Tensor] = {}
        for s in specs:
            w = weights[s.name]
            assert tuple(w.shape) == (s.n, s.k) and w.dtype == torch.bfloat16
            self.w[s.name] = FP4Tensor.from_bfloat16(w.to(self.device), linear_scales=False)
            b = biases.get(s.name) if biases else None
            self.bias[s.name] = b.to(self.device).contiguous() if b is not None else None
            self.act[s.name] = _QuantScratch(tokens, s.k, self.device)
            self.out[s.name] = torch.empty(tokens, s.n, dtype=torch.bfloat16, device=self.device)
        self.status = N.status_word(self.device)
        self.flops_per_step = sum(2 * tokens * s.n * s.k for s in specs)
        self.quant_bytes_per_step = sum(2.5625 * tokens * s.k for s in specs)
        # amax + quantize + gemm per linear, minus the amax pass the ffn_up epilogue absorbs
        self.kernels_per_step = 3 * len(specs) - (1 if {"ffn_up", "ffn_down"} <= {s.name for s in specs} else 0)

    def quantize(self, name: str, x: torch.Tensor, stream: int) -> None:
        q = self.act[name]
        N.check(N.lib.nvfp4_amax_bf16(x.data_ptr(), q.m * q.k, q.amax.data_ptr(), stream), "amax")
        N.check(N.lib.nvfp4_quantize_bf16(x.data_ptr(), q.m, q.k, q.amax.data_ptr(),
                                          q.data.data_ptr(), None, q.sf.data_ptr(),
                                          q.gscale.data_ptr(), stream), "quantize")

    def quantize_with_amax(self, name: str, x: torch.Tensor, stream: int) -> None:
        """Pack ``x`` using the amax already sitting in the slot (left there by the GEMM that
        produced ``x``)."""
        q = self.act[name]
        N.check(N.lib.nvfp4_quantize_bf16(x.data_ptr(), q.m, q.k, q.amax.data_ptr(),
                                          q.data.data_ptr(), None, q.sf.data_ptr(),
                                          q.gscale.data_ptr(), stream), "quantize")

    def gemm(self, spec: LinearSpec, stream: int,
             out_amax: Optional[torch.Tensor] = None) -> torch.Tensor:
        q, w, out = self.act[spec.name], self.w[spec.name], self.out[spec.name]
        b = self.bias[spec.name]
        N.check(N.lib.nvfp4_gemm(q.data.data_ptr(), w._data.data_ptr(), q.sf.data_ptr(),
                                 w._scales_swz.data_ptr(), q.gscale.data_ptr(),
                                 w._gscale.data_ptr(), q.m, spec.n, spec.k, 1.0, 0.0, None,
                                 b.data_ptr() if b is not None else None, None,
                                 N.ACT_GELU_TANH if spec.gelu else N.ACT_NONE, out.data_ptr(),
                                 out_amax.data_ptr() if out_amax is not None else None,
                                 self.status.data_ptr(), stream), "gemm")
        return out

    def linear(self, name: str, x: torch.Tensor) -> torch.Tensor:
        """y = act(x @ W^T + b) for the named linear; x is bf16 [tokens, k] on the device."""
        spec = next(s for s in self.specs if s.name == name)
        assert x.shape == (self.tokens, spec.k) and x.dtype == torch.bfloat16 and x.is_contiguous()
        st = N.stream_ptr()
        self.quantize(name, x, st)
        return self.gemm(spec, st)

    def step(self, inputs: Dict[str, torch.Tensor],
             gemm_events: Optional[List[Tuple[torch.cuda.Event, torch.cuda.Event]]] = None
             ) -> Dict[str, torch.Tensor]:
        """One pass over the block's linears.  ``inputs`` maps a linear's name to its bf16
        activation; ``ffn_down`` consumes ``ffn_up``'s output when not given.  When
        ``gemm_events`` is a list, an event pair around every GEMM launch is appended."""
        st = N.stream_ptr()
        names = [s.name for s in self.specs]
        chained = "ffn_down" in names and "ffn_up" in names and inputs.get("ffn_down") is None
        for s in self.specs:
            x = inputs.get(s.name)
            if s.name == "ffn_down" and chained:
                # its amax came out of the ffn_up GEMM's epilogue: one pass over the hidden
                self.quantize_with_amax(s.name, self.out["ffn_up"], st)
            else:
                self.quantize(s.name, x, st)
            amax_next = self.act["ffn_down"].amax if (s.name == "ffn_up" and chained) else None
            if gemm_events is not None:
                e0 = torch.cuda.Event(enable_timing=True)
                e1 = torch.cuda.Event(enable_timing=True)
                e0.record()
                self.gemm(s, st, amax_next)
                e1.record()
                gemm_events.append((e0, e1))
            else:
                self.gemm(s, st, amax_next)
        return self.out

    def capture(self, inputs: Dict[str, torch.Tensor]) -> "torch.cuda.CUDAGraph":
        """Record one :meth:`step` over ``inputs`` into a CUDA graph (the static-shape capture of
        fx/src/s4/models/wan_22/wan_attention_static.py:566-630, for this path's launches).  The
        step allocates nothing and never synchronises with the host, so the graph holds exactly
        its kernels and memsets; ``graph.replay()`` re-runs them on whatever the input tensors
        then contain, results in ``self.out``."""
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            self.step(inputs)                       # warm-up outside the capture
        torch.cuda.current_stream(self.device).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.step(inputs)
        return graph


class HostStagedLinears:
    """The block's linears for activations that live in pinned HOST memory: copy in, compute,
    copy out, on three streams so that the PCIe transfers of one linear overlap the kernels of
    another and the two directions run at the same time.

    Per linear i:  H2D_i (copy-in stream) -> amax + quantize + GEMM_i (compute stream)
    -> D2H_i (copy-out stream), chained by events.  From one step to the next, H2D_i waits for
    the previous GEMM_i to have consumed the device input buffer and GEMM_i waits for the
    previous D2H_i to have drained the output buffer, so steps can be enqueued back to back.
    """

    def __init__(self, runner: WanBlockLinears):
        self.r = runner
        dev = runner.device
        self.s_in = torch.cuda.Stream(device=dev)
        self.s_run = torch.cuda.Stream(device=dev)
        self.s_out = torch.cuda.Stream(device=dev)
        self.dev_in = {s.name: torch.empty(runner.tokens, s.k, dtype=torch.bfloat16, device=dev)
                       for s in runner.specs}
        mk = lambda: {s.name: torch.cuda.Event() for s in runner.specs}  # noqa: E731
        self.loaded, self.computed, self.drained = mk(), mk(), mk()
        self._first = True

    def step(self, host_in: Dict[str, torch.Tensor], host_out: Dict[str, torch.Tensor]) -> None:
        """Enqueue one pass: ``host_in[name]`` bf16 ``[tokens, k]`` pinned -> ``host_out[name]``
        bf16 ``[tokens, n]`` pinned.  Returns at once; :meth:`wait` orders the caller's stream
        after everything enqueued so far."""
        r = self.r
        if self._first:
            cur = torch.cuda.current_stream(r.device)
            for s in (self.s_in, self.s_run, self.s_out):
                s.wait_stream(cur)
        for spec in r.specs:
            n = spec.name
            with torch.cuda.stream(self.s_in):
                if not self._first:
                    self.s_in.wait_event(self.computed[n])      # input buffer consumed
                self.dev_in[n].copy_(host_in[n], non_blocking=True)
                self.loaded[n].record(self.s_in)
            with torch.cuda.stream(self.s_run):
                self.s_run.wait_event(self.loaded[n])
                if not self._first:
                    self.s_run.wait_event(self.drained[n])      # output buffer copied out
                y = r.linear(n, self.dev_in[n])
                self.computed[n].record(self.s_run)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.computed[n])
                host_out[n].copy_(y, non_blocking=True)
                self.drained[n].record(self.s_out)
        self._first = False

    def wait(self) -> None:
        cur = torch.cuda.current_stream(self.r.device)
        for s in (self.s_in, self.s_run, self.s_out):
            cur.wait_stream(s)
