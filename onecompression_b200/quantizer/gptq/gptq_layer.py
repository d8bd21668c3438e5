"""AutoGPTQ int32 packing on the GPU and the g_idx rule of the inference layer
(reference: onecomp/quantizer/gptq/gptq_layer.py:36-245, 423-433).

Function names and shapes are the reference's; tensors must be CUDA tensors and the
results stay on their device.
"""

from __future__ import annotations

from typing import Optional, Tuple, Union

import torch

from ... import kernels

PACKABLE_WBITS = (2, 3, 4, 8)


def _normalize_wbits(wbits: int) -> int:
    if isinstance(wbits, bool):
        raise ValueError(f"wbits must be an integer value, got {wbits!r}.")
    if isinstance(wbits, int):
        return int(wbits)
    if isinstance(wbits, float) and wbits.is_integer():
        return int(wbits)
    raise ValueError(f"wbits must be an integer value, got {wbits!r}.")


def is_packable_wbits(wbits: int) -> bool:
    return wbits in PACKABLE_WBITS


def pack_int_weights(weights: torch.Tensor, wbits: int) -> torch.Tensor:
    """(out_features, in_features) codes → packed int32 (in_features·wbits/32, out_features)."""
    return kernels.pack_qweight(weights, wbits)


def unpack_int_weights(packed: torch.Tensor, wbits: int,
                       original_shape: Union[torch.Size, Tuple[int, ...]]) -> torch.Tensor:
    return kernels.unpack_qweight(packed, wbits, original_shape)


def pack_zeros(zeros: torch.Tensor, wbits: int) -> torch.Tensor:
    """(num_groups, out_features) integer zero points → packed int32
    (num_groups, out_features·wbits/32); values are masked to ``wbits`` first."""
    return kernels.pack_qzeros(zeros, wbits, add=0)


def unpack_zeros(packed_zeros: torch.Tensor, wbits: int, out_features: int) -> torch.Tensor:
    return kernels.unpack_qzeros(packed_zeros, wbits, out_features, add=0)


def normalize_scale_zero(tensor: torch.Tensor, out_features: int) -> torch.Tensor:
    """(out,), (out,1) or (G,out) → (G,out)."""
    if tensor.dim() == 1:
        return tensor.unsqueeze(0)
    if tensor.dim() == 2 and tensor.shape == (out_features, 1):
        return tensor.t()
    return tensor


def make_g_idx(perm: Optional[torch.Tensor], groupsize: int, in_features: int, device=None) -> torch.Tensor:
    """g_idx of the inference layer: argsort(perm)//groupsize with act-order,
    arange//groupsize without, zeros for per-channel (int32)."""
    if groupsize == -1:
        return torch.zeros(in_features, dtype=torch.int32, device=device)
    base = torch.arange(in_features, device=device) // groupsize
    if perm is None:
        return base.to(torch.int32)
    g = torch.empty(in_features, dtype=torch.long, device=device)
    g[perm.to(device=device, dtype=torch.long)] = base
    return g.to(torch.int32)
