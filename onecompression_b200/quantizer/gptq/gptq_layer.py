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


class GPTQLinear(torch.nn.Module):
    """Inference layer over a GPTQ result in the AutoGPTQ (v1) tensor layout - the consumer of
    what the column loop packs (reference: GPTQLinear, onecomp/quantizer/gptq/gptq_layer.py:247-714).

    Buffers (the safetensors keys of a saved model): ``qweight`` int32 (in·bits/32, out),
    ``qzeros`` int32 (G, out·bits/32) holding (zero − 1) & mask, ``scales`` fp16 (G, out),
    ``g_idx`` int32 (in,), optional ``bias`` fp16.  Bit widths without a packed layout keep
    ``qweight`` (out, in) and ``qzeros`` (G, out) as plain integers.  ``forward`` dequantizes on
    the GPU (one kernel for the packed layout) and applies the linear map.
    """

    def __init__(self, in_features, out_features, wbits, groupsize, actorder, quantized_weight, scale,
                 zero, perm=None, bias=None, device="cuda", pack_weights=True, use_gemlite=None,
                 input_weight_is_packed=False, input_zero_is_packed=False):
        super().__init__()
        del use_gemlite  # no GemLite path here
        wbits = _normalize_wbits(wbits)
        self.in_features, self.out_features = in_features, out_features
        self.wbits, self.groupsize, self.actorder = wbits, groupsize, actorder
        self.checkpoint_format = "gptq"
        device = torch.device(device)
        mask = (1 << wbits) - 1
        pack = bool(pack_weights and is_packable_wbits(wbits))

        qw = quantized_weight.to(device=device, dtype=torch.int32)
        if input_weight_is_packed and not pack:
            qw = unpack_int_weights(qw, wbits, (out_features, in_features))
        elif pack and not input_weight_is_packed:
            qw = pack_int_weights(qw, wbits)
        self.register_buffer("qweight", qw.contiguous())

        self.register_buffer(
            "scales", normalize_scale_zero(scale, out_features).to(device=device, dtype=torch.float16).contiguous())

        if input_zero_is_packed:
            qz = zero.to(device=device, dtype=torch.int32)
            if not pack:
                qz = unpack_zeros(qz, wbits, out_features)
        else:
            raw = normalize_scale_zero(zero, out_features).to(device)
            stored = raw.float().round().to(torch.int32) - 1          # v1: stored = zero - 1
            qz = pack_zeros(stored.contiguous(), wbits) if pack else stored
        self.register_buffer("qzeros", qz.contiguous())

        if bias is not None:
            self.register_buffer("bias", bias.detach().to(device=device, dtype=torch.float16))
        else:
            self.bias = None
        self.register_buffer("g_idx", make_g_idx(perm if actorder else None, groupsize, in_features, device=device))
        self._weight_is_packed = pack
        self._mask = mask

    @classmethod
    def from_quantization_result(cls, result, bias=None, device="cuda", pack_weights=True, use_gemlite=None):
        shape = getattr(result, "qweight_original_shape", None)
        out_features, in_features = shape if shape is not None else tuple(result.qweight.shape)
        return cls(
            in_features=in_features, out_features=out_features, wbits=result.wbits,
            groupsize=result.groupsize, actorder=result.actorder, quantized_weight=result.qweight,
            scale=result.scales, zero=result.qzeros, perm=result.perm, bias=bias, device=device,
            pack_weights=pack_weights, use_gemlite=use_gemlite,
            input_weight_is_packed=bool(getattr(result, "qweight_is_packed", False)),
            input_zero_is_packed=bool(getattr(result, "qzeros_is_packed", False)),
        )

    def dequantized_weight(self) -> torch.Tensor:
        """fp16 (out, in) weight: scale·(q − zero) with zero = (stored + 1) & mask."""
        if self._weight_is_packed:
            return kernels.dequantize_packed(self.qweight, self.qzeros, self.scales, self.g_idx, self.wbits,
                                             (self.out_features, self.in_features))
        zeros = (self.qzeros + 1) & self._mask
        g = self.g_idx.long()
        w = self.scales[g, :].T.float() * (self.qweight.float() - zeros[g, :].T.float())
        return w.to(torch.float16)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w = self.dequantized_weight().to(x.dtype)
        b = self.bias.to(x.dtype) if self.bias is not None else None
        return torch.nn.functional.linear(x, w, b)

    def unpack_in_place(self) -> None:
        if not self._weight_is_packed:
            return
        self.register_buffer("qweight", unpack_int_weights(self.qweight, self.wbits, (self.out_features, self.in_features)))
        self.register_buffer("qzeros", unpack_zeros(self.qzeros, self.wbits, self.out_features))
        self._weight_is_packed = False

    def pack_in_place(self) -> None:
        if self._weight_is_packed or not is_packable_wbits(self.wbits):
            return
        self.register_buffer("qweight", pack_int_weights(self.qweight.to(torch.int32), self.wbits))
        self.register_buffer("qzeros", pack_zeros(self.qzeros.to(torch.int32).contiguous(), self.wbits))
        self._weight_is_packed = True
