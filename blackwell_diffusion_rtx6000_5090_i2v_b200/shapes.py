"""Shapes of the benchmark configurations (plain data: importing this module loads neither
torch nor the CUDA library, so CPU-only tools can share it)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List


@dataclass(frozen=True)
class LinearSpec:
    name: str
    n: int      # out features
    k: int      # in features
    gelu: bool = False


def wan_block_specs(dim: int, ffn: int) -> List[LinearSpec]:
    """The four linears of a DiT block the block-linears benchmark runs: ``to_qkv`` / ``to_out``
    (fx/src/s4/models/wan22/wan_transformer.py:111,129) and the feed-forward up (+GELU-tanh) /
    down projections (:185,220)."""
    return [LinearSpec("qkv", 3 * dim, dim), LinearSpec("attn_out", dim, dim),
            LinearSpec("ffn_up", ffn, dim, gelu=True), LinearSpec("ffn_down", dim, ffn)]


WAN22_TI2V_5B = dict(dim=3072, ffn=14336, tokens=27280)   # 1280x704, 121 frames
WAN22_A14B = dict(dim=5120, ffn=13824, tokens=32760)      # 832x480, 81 frames
