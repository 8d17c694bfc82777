"""Pre-quantized NVFP4 weights on disk: pack once offline, load packed.

Fills the stubs the reference leaves open, ``NVFP4Quantization.quantize_tensor`` /
``dequantize_tensor`` (fx/src/s4/models/wan_22/wan_serialization.py:204-239), and its
safetensors layout for quantized tensors (``TensorMetadata.to_safetensors_header``, :112-129;
``save_to_safetensors`` / ``load_from_safetensors``, :450-560), so that weight quantization
leaves the step entirely.  Per weight ``name`` the file holds

    name                  uint8  [N, K/2]   E2M1 codes, even element in the low nibble
    name.scales           uint8  [N, K/16]  E4M3 block scales, linear row-major
    name.global_scale     fp32   [1]        amax / (6 * 448)
    name.amax             fp32   [1]        tensor amax (dequantize forms float(sf) / S_enc from it)

and the file's metadata carries, per tensor, the reference's quantization header
(``type: nvfp4, bits: 4, group_size: 16, scale: <global scale>``) with the original shape and
dtype.  The tensor-core (swizzled) scale layout is derived on load, never stored.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

import torch

from .nvfp4 import FP4Tensor

FORMAT = "nvfp4-b200/1"


@dataclass
class TensorMetadata:
    """The reference's per-tensor record (wan_serialization.py:86-129), quantization part."""
    name: str
    shape: Tuple[int, ...]
    dtype: str
    quantized: bool = False
    quant_type: Optional[str] = None
    quant_bits: Optional[int] = None
    quant_scale: Optional[float] = None
    quant_zero_point: Optional[float] = None
    quant_group_size: Optional[int] = None
    # the packed tensor the nibbles belong to (not serialised by to_safetensors_header)
    packed: Optional[FP4Tensor] = None

    def to_safetensors_header(self) -> Dict[str, Any]:
        header: Dict[str, Any] = {"dtype": self.dtype, "shape": list(self.shape)}
        if self.quantized:
            header["quantization"] = {"type": self.quant_type, "bits": self.quant_bits,
                                      "scale": self.quant_scale, "zero_point": self.quant_zero_point,
                                      "group_size": self.quant_group_size}
        return header


class NVFP4Quantization:
    """``quantize_tensor`` / ``dequantize_tensor`` with the reference's signatures."""

    def quantize_tensor(self, tensor: torch.Tensor, config: Any = None,
                        tensor_name: str = "") -> Tuple[torch.Tensor, TensorMetadata]:
        """bf16 (or fp16/fp32, cast to bf16) CUDA tensor with a last dimension % 16 == 0 ->
        (packed nibbles as uint8 ``[..., K/2]``, metadata).  The metadata's ``packed`` field is
        the full :class:`FP4Tensor` (scales, tensor scale)."""
        if not tensor.is_cuda:
            raise RuntimeError("[s4] [nvfp4] [tensor] Input must be on CUDA device")
        t = FP4Tensor.from_bfloat16(tensor.to(torch.bfloat16).contiguous(), linear_scales=True,
                                    swizzled_scales=False)
        shape = tuple(tensor.shape)
        meta = TensorMetadata(name=tensor_name, shape=shape, dtype=str(tensor.dtype).replace("torch.", ""),
                              quantized=True, quant_type="nvfp4", quant_bits=4,
                              quant_scale=float(t.global_scale().item()), quant_zero_point=None,
                              quant_group_size=16, packed=t)
        return t.quantized_data().view(*shape[:-1], shape[-1] // 2), meta

    def dequantize_tensor(self, quantized_tensor: torch.Tensor, metadata: TensorMetadata) -> torch.Tensor:
        if metadata.packed is None or metadata.packed.quantized_data().data_ptr() != quantized_tensor.data_ptr():
            raise RuntimeError("[s4] [nvfp4] [tensor] metadata does not belong to this packed tensor")
        return metadata.packed.to_bfloat16()


def save_packed(path: str, tensors: Dict[str, FP4Tensor],
                extra: Optional[Dict[str, torch.Tensor]] = None) -> None:
    """Write packed weights (and ``extra`` unquantized tensors such as biases) to a safetensors
    file."""
    from safetensors.torch import save_file
    blobs: Dict[str, torch.Tensor] = {}
    header: Dict[str, Any] = {}
    for name, t in tensors.items():
        shape = list(t.shape())
        blobs[name] = t.quantized_data().view(*shape[:-1], shape[-1] // 2).cpu()
        blobs[name + ".scales"] = t.scale_factors().view(*shape[:-1], shape[-1] // 16).cpu()
        blobs[name + ".global_scale"] = t.global_scale().cpu()
        blobs[name + ".amax"] = t.global_amax().cpu()
        header[name] = TensorMetadata(name, tuple(shape), "bfloat16", True, "nvfp4", 4,
                                      float(t.global_scale().item()), None, 16).to_safetensors_header()
    for name, t in (extra or {}).items():
        if name in blobs:
            raise ValueError(f"duplicate tensor name {name}")
        blobs[name] = t.detach().cpu().contiguous()
    save_file(blobs, path, metadata={"format": FORMAT, "tensors": json.dumps(header)})


def load_packed(path: str, device="cuda") -> Tuple[Dict[str, FP4Tensor], Dict[str, torch.Tensor]]:
    """Read a file written by :func:`save_packed`: (packed weights, other tensors), on ``device``."""
    from safetensors import safe_open
    packed: Dict[str, FP4Tensor] = {}
    other: Dict[str, torch.Tensor] = {}
    with safe_open(path, framework="pt", device="cpu") as f:
        meta = f.metadata() or {}
        if meta.get("format") != FORMAT:
            raise RuntimeError(f"{path}: not an {FORMAT} file")
        header = json.loads(meta["tensors"])
        consumed = set()
        for name, h in header.items():
            q = h.get("quantization") or {}
            if q.get("type") != "nvfp4" or q.get("bits") != 4 or q.get("group_size") != 16:
                raise RuntimeError(f"{path}: {name} is not NVFP4 block-16")
            parts = [f.get_tensor(name + sfx).to(device) for sfx in ("", ".scales", ".amax", ".global_scale")]
            packed[name] = FP4Tensor.from_packed(parts[0], parts[1], parts[2], parts[3], h["shape"])
            consumed.update(name + sfx for sfx in ("", ".scales", ".amax", ".global_scale"))
        for key in f.keys():
            if key not in consumed:
                other[key] = f.get_tensor(key).to(device)
    return packed, other
