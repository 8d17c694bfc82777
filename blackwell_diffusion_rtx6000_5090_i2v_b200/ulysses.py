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
