"""Saving a quantized model in the layout its consumers read (reference: Runner.save_quantized_model,
onecomp/runner.py:2238-2438; per-layer keys onecomp/quantizer/gptq/gptq_layer.py:395-433).

Every quantized ``nn.Linear`` becomes a ``GPTQLinear`` whose buffers are the safetensors keys
``<name>.qweight`` (int32, in·bits/32 × out), ``<name>.qzeros`` (int32, G × out·bits/32, v1 offset),
``<name>.scales`` (fp16, G × out), ``<name>.g_idx`` (int32, in) and optionally ``<name>.bias``;
``config.json`` gains ``quantization_config`` (``quant_method`` gptq / mixed_gptq, ``bits``,
``group_size``, ``desc_act``, ``sym``, ``checkpoint_format`` "gptq", ``quantization_bits`` per layer).
Layers kept unpacked in memory are packed in the exported dict only.
"""

from __future__ import annotations

import json
import os
from typing import Optional

import torch

from ..quantizer.gptq.gptq_layer import GPTQLinear, is_packable_wbits, pack_int_weights, pack_zeros


def build_quantization_config(model, quantizer) -> dict:
    """``quantization_config`` for ``config.json`` (reference runner.py:1641-1700)."""
    cfg = quantizer.get_quant_config()
    names = sorted(quantizer.results)
    num_layers = getattr(getattr(model, "config", None), "num_hidden_layers", None)
    if num_layers is None:
        num_layers = 1 + max((int(p) for n in names for a, p in zip(n.split("."), n.split(".")[1:]) if a == "layers" and p.isdigit()),
                             default=-1)
    cfg = quantizer.finalize_quant_config_for_save(cfg, names, num_hidden_layers=num_layers)
    cfg.setdefault("modules_in_block_to_quantize", None)
    return cfg


def quantized_state_dict(model) -> dict:
    """The model's state dict with every ``GPTQLinear`` in the packed layout (the in-memory layers
    are not modified)."""
    state = {k: v for k, v in model.state_dict().items()}
    for name, layer in model.named_modules():
        if not isinstance(layer, GPTQLinear) or layer._weight_is_packed or not is_packable_wbits(layer.wbits):
            continue
        state[f"{name}.qweight"] = pack_int_weights(layer.qweight.to(torch.int32), layer.wbits)
        state[f"{name}.qzeros"] = pack_zeros(layer.qzeros.to(torch.int32).contiguous(), layer.wbits)
    return state


def save_quantized_model(model, quantizer, save_directory: str, pack_weights: bool = True,
                         filename: str = "model.safetensors") -> str:
    """Replace the quantized layers by ``GPTQLinear`` (``quantizer.apply_results_to_model``), write
    the tensors to ``<save_directory>/<filename>`` and the configuration to ``config.json``."""
    from safetensors.torch import save_file

    if not quantizer.results:
        raise RuntimeError("save_quantized_model: the quantizer holds no results; run the quantization first")
    os.makedirs(save_directory, exist_ok=True)
    device = next(model.parameters()).device
    quantizer.apply_results_to_model(model, pack_weights=pack_weights, device=device)
    qcfg = build_quantization_config(model, quantizer)
    state = quantized_state_dict(model)
    seen, tensors = {}, {}
    for key, t in state.items():  # tied tensors are written once
        ptr = (t.data_ptr(), tuple(t.shape), t.dtype)
        if t.numel() and ptr in seen:
            continue
        seen[ptr] = key
        tensors[key] = t.detach().contiguous().cpu()
    save_file(tensors, os.path.join(save_directory, filename), metadata={"format": "pt"})
    config = getattr(model, "config", None)
    cfg_dict = config.to_dict() if config is not None and hasattr(config, "to_dict") else {}
    cfg_dict["quantization_config"] = qcfg
    with open(os.path.join(save_directory, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg_dict, f, indent=2, sort_keys=True, default=str)
    return save_directory


def load_quantized_layers(model, save_directory: str, device: Optional[str] = None,
                          filename: str = "model.safetensors"):
    """Rebuild the ``GPTQLinear`` layers of ``model`` (a freshly constructed, unquantized model of the
    same architecture) from a directory written by ``save_quantized_model`` and load all tensors
    (reference: load_quantized_model, onecomp/runner.py:2996-3028 for the per-layer rule)."""
    from safetensors.torch import load_file

    with open(os.path.join(save_directory, "config.json"), encoding="utf-8") as f:
        qcfg = json.load(f)["quantization_config"]
    tensors = load_file(os.path.join(save_directory, filename))
    device = device or str(next(model.parameters()).device)
    from ..quantizer.gptq._gptq import GPTQ

    for key in [k for k in tensors if k.endswith(".qweight")]:
        name = key[: -len(".qweight")]
        bits = GPTQ.resolve_bits(name, qcfg.get("bits", 4), qcfg.get("mlp_wbits"), qcfg.get("module_wbits"))
        gs = GPTQ.resolve_groupsize(name, qcfg.get("group_size", -1), qcfg.get("mlp_groupsize"))
        *parents, attr = name.split(".")
        parent = model
        for p in parents:
            parent = getattr(parent, p)
        old = getattr(parent, attr)
        g_idx = tensors[name + ".g_idx"]
        layer = GPTQLinear(
            in_features=old.in_features, out_features=old.out_features, wbits=bits, groupsize=gs,
            actorder=False, quantized_weight=tensors[key], scale=tensors[name + ".scales"],
            zero=tensors[name + ".qzeros"], bias=tensors.get(name + ".bias"), device=device,
            input_weight_is_packed=is_packable_wbits(bits), input_zero_is_packed=is_packable_wbits(bits),
        )
        layer.actorder = bool(qcfg.get("desc_act", False))
        layer.g_idx.copy_(g_idx.to(layer.g_idx.device))
        setattr(parent, attr, layer)
    missing = model.load_state_dict({k: v for k, v in tensors.items()}, strict=False)
    return model, missing
