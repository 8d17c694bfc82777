"""Ulysses sequence-parallel exchange around self-attention.

Every linear, norm and quantize op of the DiT block is token-row independent,
so with P ranks each rank keeps ``L/P`` tokens and replicated weights and needs
no communication -- except self-attention, where every query must see every
key.  One all-to-all turns the token-sharded ``[L/P, H, D]`` tensors into
head-sharded ``[L, H/P, D]`` ones, attention runs on full sequences of the
local heads, and the inverse all-to-all restores token sharding.  The
reference has no distributed code at all; this is the exchange step of the
multi-GPU configuration (Wan2.2-A14B shape, 2/4/8 GPUs of one node).

The collectives are ``torch.distributed.all_to_all_single`` (NCCL over NVLink on
GPUs, gloo in the CPU tests); data always lands in the rank's own memory before
any kernel reads it.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


def _world(group) -> int:
    return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


def seq_to_heads(x: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """``[L/P, H, D]`` (this rank's tokens, all heads) -> ``[L, H/P, D]`` (all tokens, this
    rank's heads).  Rank r ends up with heads ``[r*H/P, (r+1)*H/P)``; tokens keep rank order."""
    P = _world(group)
    if P == 1:
        return x
    Lp, H, D = x.shape
    if H % P != 0:
        raise ValueError(f"heads ({H}) must divide by the world size ({P})")
    # group heads by destination rank: [P, L/P, H/P, D]
    send = x.reshape(Lp, P, H // P, D).permute(1, 0, 2, 3).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    # recv[s] holds source rank s's tokens for my heads: concatenate along tokens
    return recv.reshape(P * Lp, H // P, D)


def all_to_all_packed(send: torch.Tensor, group: dist.ProcessGroup) -> torch.Tensor:
    """``send[r]`` = this rank's ``[L/P, H/P, C]`` pieces for rank r (already grouped by
    destination, as ``nvfp4_qk_norm_rope_exchange_bf16`` writes them) -> ``[L, H/P, C]``: all
    tokens of this rank's heads, tokens in rank order.  One collective, no packing copies."""
    P, Lp, Hp, C = send.shape
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv.reshape(P * Lp, Hp, C)


def heads_to_seq(x: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Inverse of :func:`seq_to_heads`: ``[L, H/P, D]`` -> ``[L/P, H, D]``."""
    P = _world(group)
    if P == 1:
        return x
    L, Hp, D = x.shape
    if L % P != 0:
        raise ValueError(f"tokens ({L}) must divide by the world size ({P})")
    Lp = L // P
    send = x.reshape(P, Lp, Hp, D).contiguous()          # [dest rank, its tokens, my heads, D]
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    # recv[s] holds my tokens for source rank s's heads: interleave back to head order
    return recv.permute(1, 0, 2, 3).reshape(Lp, P * Hp, D)


def exchange_bytes_per_rank(tokens: int, heads: int, head_dim: int, world: int,
                            tensors: int = 4, elem_bytes: int = 2) -> int:
    """Bytes each rank sends per block: q, k, v out and the attention output back, of which
    (P-1)/P leaves the GPU."""
    per_tensor = tokens // world * heads * head_dim * elem_bytes
    return tensors * per_tensor * (world - 1) // world


class PeerExchange:
    """The two exchanges of a block done by stores into peer memory instead of all-to-alls.

    Every rank holds, in symmetric memory mapped by all ranks of the node, a packed
    ``[L, H/P, 3D]`` buffer (its heads of q | k | v for ALL tokens), an ``[L/P, H, D]`` buffer
    (all heads of the attention output for ITS tokens) and a small sync block.  The q/k norm +
    RoPE kernel of each rank stores its tokens' pieces straight into the owning ranks' packed
    buffers over NVLink (``nvfp4_qk_norm_rope_exchange_bf16``); after attention one kernel
    moves each rank's head columns into the owning ranks' output buffers and takes max|o| on
    the way (``nvfp4_attn_return_exchange_bf16``).  The last CTA of either kernel raises this
    rank's flag in every rank's sync block, and a one-warp kernel with a bounded wait
    (``nvfp4_exchange_wait``) holds the consumer's stream until all ranks' flags are up: no
    collective call is left in the block.  Two sets of buffers alternate from block to block:
    passing a wait means every peer has passed the previous one, so a rank never overwrites a
    buffer a peer still reads.

    Plain loads and stores only -- no multicast mapping is created or used.
    """

    def __init__(self, tokens_total: int, heads: int, head_dim: int, group: dist.ProcessGroup,
                 device: torch.device, wait_limit_s: float = 30.0):
        import ctypes
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        from . import _native as N
        P, r = dist.get_world_size(group), dist.get_rank(group)
        if heads % P or tokens_total % P:
            raise ValueError("heads and tokens must divide by the world size")
        self.group, self.P, self.rank = group, P, r
        self.L, self.Lp, self.H, self.Hp, self.D = tokens_total, tokens_total // P, heads, heads // P, head_dim
        self.wait_limit_ns = int(wait_limit_s * 1e9)
        self.qkv, self.o, self.qkv_ptrs, self.o_ptrs = [], [], [], []

        def ptr_array(handle):
            return (ctypes.c_void_p * P)(*[int(p) for p in handle.buffer_ptrs])

        for _ in range(2):
            t = symm.empty((self.L, self.Hp, 3 * head_dim), dtype=torch.bfloat16, device=device)
            self.qkv.append(t)
            self.qkv_ptrs.append(ptr_array(symm.rendezvous(t, group)))
            t = symm.empty((self.Lp, heads, head_dim), dtype=torch.bfloat16, device=device)
            self.o.append(t)
            self.o_ptrs.append(ptr_array(symm.rendezvous(t, group)))
        self.sync = symm.empty((N.lib.nvfp4_exchange_sync_bytes() // 4,), dtype=torch.int32, device=device)
        self.sync.zero_()
        self.sync_ptrs = ptr_array(symm.rendezvous(self.sync, group))
        self.amax = torch.zeros(1, dtype=torch.float32, device=device)   # of the assembled attention output
        self.turn = 0
        # every rank's sync block is zero before any peer can raise a flag in it
        torch.cuda.synchronize(device)
        dist.barrier(group)

    def wait(self, kind: int, amax_out: Optional[torch.Tensor] = None) -> None:
        """Hold the current stream until all ranks' producer kernels of this exchange are done
        (``kind`` 0: q|k|v pieces, 1: attention output)."""
        from . import _native as N
        N.check(N.lib.nvfp4_exchange_wait(self.sync.data_ptr(), kind, self.P, self.wait_limit_ns,
                                          N.ptr(amax_out), N.ptr(N.status_word(self.sync.device)),
                                          N.stream_ptr()), "exchange wait")

    def return_attention_output(self, o: torch.Tensor):
        """``o`` is ``[L, H/P, D]`` (my heads, all tokens).  Returns ``([L/P, H, D] buffer holding
        all heads of my tokens, its amax as a one-element device tensor)`` once every rank's
        stores have landed."""
        from . import _native as N
        if o.shape != (self.L, self.Hp, self.D) or o.dtype != torch.bfloat16 or o.stride(2) != 1:
            raise RuntimeError("return_attention_output: o must be bf16 [L, H/P, D] with unit inner stride")
        i = self.turn
        N.check(N.lib.nvfp4_attn_return_exchange_bf16(o.data_ptr(), o.stride(0), o.stride(1), self.L,
                                                      self.Hp, self.D, self.o_ptrs[i], self.sync_ptrs,
                                                      self.P, self.rank, N.stream_ptr()),
                "attention return exchange")
        self.wait(1, self.amax)
        self.turn ^= 1
        return self.o[i], self.amax
