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
    ``[L, H/P, 3D]`` buffer (its heads of q | k | v for ALL tokens) and an ``[L/P, H, D]`` buffer
    (all heads of the attention output for ITS tokens).  The q/k norm + RoPE kernel of each rank
    stores its tokens' pieces straight into the owning ranks' packed buffers over NVLink
    (``nvfp4_qk_norm_rope_exchange_bf16``), and after attention each rank copies its heads'
    output rows into the owning ranks' output buffers.  What remains of the collective is one
    tiny all-reduce after each set of stores, which orders the consumers on every rank after
    the producers on all ranks.  Two sets of buffers alternate from block to block: a rank can
    be at most one barrier ahead of a peer, so it never overwrites a buffer a peer still reads.

    Plain loads and stores only -- no multicast mapping is created or used.
    """

    def __init__(self, tokens_total: int, heads: int, head_dim: int, group: dist.ProcessGroup,
                 device: torch.device):
        import ctypes
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        P, r = dist.get_world_size(group), dist.get_rank(group)
        if heads % P or tokens_total % P:
            raise ValueError("heads and tokens must divide by the world size")
        self.group, self.P, self.rank = group, P, r
        self.L, self.Lp, self.H, self.Hp, self.D = tokens_total, tokens_total // P, heads, heads // P, head_dim
        self.qkv, self.o, self.qkv_ptrs, self.o_peer = [], [], [], []
        for _ in range(2):
            t = symm.empty((self.L, self.Hp, 3 * head_dim), dtype=torch.bfloat16, device=device)
            h = symm.rendezvous(t, group)
            self.qkv.append(t)
            self.qkv_ptrs.append((ctypes.c_void_p * P)(*[int(p) for p in h.buffer_ptrs]))
            t = symm.empty((self.Lp, heads, head_dim), dtype=torch.bfloat16, device=device)
            h = symm.rendezvous(t, group)
            self.o.append(t)
            self.o_peer.append([h.get_buffer(s, (self.Lp, heads, head_dim), torch.bfloat16)
                                for s in range(P)])
        self._flag = torch.zeros(1, dtype=torch.float32, device=device)
        self.turn = 0

    def barrier(self) -> None:
        """Stream-ordered: every rank's work enqueued before it is complete on every rank
        before anything enqueued after it starts."""
        dist.all_reduce(self._flag, group=self.group)

    def scatter_attention_output(self, o: torch.Tensor) -> torch.Tensor:
        """``o`` is ``[L, H/P, D]`` (my heads, all tokens).  Store each rank's token rows into its
        output buffer and return mine, ``[L/P, H, D]``, once every rank has done the same."""
        i, r, Lp, Hp = self.turn, self.rank, self.Lp, self.Hp
        for s in range(self.P):
            self.o_peer[i][s][:, r * Hp:(r + 1) * Hp, :].copy_(o[s * Lp:(s + 1) * Lp])
        self.barrier()
        out = self.o[i]
        self.turn ^= 1
        return out
