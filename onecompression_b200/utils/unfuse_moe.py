"""Per-expert ``nn.Linear`` layers for mixtures whose experts are stored as fused 3-D tensors.

GPTQ and the QEP driver work on ``nn.Linear`` modules, one Hessian per layer; GPT-OSS keeps the
weights of all experts of a layer in two parameters (``gate_up_proj`` [E, hidden, 2·inter] with gate
and up interleaved along the last axis, ``down_proj`` [E, inter, hidden], plus biases).
``unfuse_moe_experts`` swaps every such module for ``RoutedExperts``: E sub-modules with
``gate_proj`` / ``up_proj`` / ``down_proj`` linears that are called with the tokens routed to them
only, so that each expert's Hessian comes from its own tokens (reference:
onecomp/utils/unfuse_moe.py:20-116, 380-466, 639-675).  ``fuse_moe_experts`` is the way back for
the save path: loaders of GPT-OSS checkpoints expect the fused ``gate_up_proj`` / ``down_proj``
keys, so the (dequantized) per-expert weights are written back into fused tensors (reference
:499-574, 677-729).
"""

from __future__ import annotations

import torch
from torch import nn


class Expert(nn.Module):
    """One expert: gate, up and down projections (with bias)."""

    def __init__(self, gate_proj: nn.Linear, up_proj: nn.Linear, down_proj: nn.Linear):
        super().__init__()
        self.gate_proj, self.up_proj, self.down_proj = gate_proj, up_proj, down_proj


def gpt_oss_glu(alpha: float, limit: float):
    """(gate, up) -> hidden of GPT-OSS: clamped gate·sigmoid(alpha·gate) times (up + 1)."""

    def combine(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        gate = gate.clamp(max=limit)
        up = up.clamp(min=-limit, max=limit)
        return (up + 1) * (gate * torch.sigmoid(gate * alpha))

    return combine


class RoutedExperts(nn.Module):
    """Drop-in for a fused experts module: same call signature, per-expert linears inside."""

    def __init__(self, experts, combine, origin=None):
        super().__init__()
        self.experts = nn.ModuleList(experts)
        self.combine = combine
        # (class, config, alpha, limit) of the fused module this one replaced, for the way back
        self.origin = origin

    def __len__(self):
        return len(self.experts)

    def __getitem__(self, idx):
        return self.experts[int(idx)]

    def forward(self, hidden_states, router_indices=None, routing_weights=None, top_k_index=None,
                top_k_weights=None):
        indices = router_indices if router_indices is not None else top_k_index
        weights = routing_weights if routing_weights is not None else top_k_weights
        out = torch.zeros_like(hidden_states)
        for e, expert in enumerate(self.experts):
            token_idx, slot = torch.where(indices == e)
            if token_idx.numel() == 0:
                continue                     # an expert without tokens is not called at all
            x = hidden_states[token_idx]
            y = expert.down_proj(self.combine(expert.gate_proj(x), expert.up_proj(x)))
            out.index_add_(0, token_idx, (y * weights[token_idx, slot, None]).to(out.dtype))
        return out


def _is_gpt_oss_style(module: nn.Module) -> bool:
    gu, dn = getattr(module, "gate_up_proj", None), getattr(module, "down_proj", None)
    return (isinstance(gu, torch.Tensor) and isinstance(dn, torch.Tensor) and gu.dim() == 3 and dn.dim() == 3
            and gu.shape[0] == dn.shape[0] and gu.shape[2] == 2 * dn.shape[1] and gu.shape[1] == dn.shape[2]
            and hasattr(module, "gate_up_proj_bias") and hasattr(module, "down_proj_bias"))


def _linear(weight: torch.Tensor, bias: torch.Tensor) -> nn.Linear:
    lin = nn.Linear(weight.shape[1], weight.shape[0], bias=True, device=weight.device, dtype=weight.dtype)
    lin.weight = nn.Parameter(weight.contiguous(), requires_grad=False)
    lin.bias = nn.Parameter(bias.contiguous(), requires_grad=False)
    return lin


def unfuse_one(module: nn.Module) -> RoutedExperts:
    gu, gub = module.gate_up_proj.data, module.gate_up_proj_bias.data
    dn, dnb = module.down_proj.data, module.down_proj_bias.data
    experts = []
    for e in range(gu.shape[0]):
        experts.append(Expert(
            _linear(gu[e, :, 0::2].t(), gub[e, 0::2]),      # gate: even columns
            _linear(gu[e, :, 1::2].t(), gub[e, 1::2]),      # up: odd columns
            _linear(dn[e].t(), dnb[e]),
        ))
    alpha, limit = float(getattr(module, "alpha", 1.702)), float(getattr(module, "limit", 7.0))
    return RoutedExperts(experts, gpt_oss_glu(alpha, limit),
                         origin=(type(module), getattr(module, "config", None), alpha, limit))


def unfuse_moe_experts(model: nn.Module) -> int:
    """Replace every fused experts module of ``model`` in place; returns how many were replaced."""
    todo = [(name, mod) for name, mod in model.named_modules() if _is_gpt_oss_style(mod)]
    for name, mod in todo:
        parent = model
        *path, leaf = name.split(".")
        for p in path:
            parent = getattr(parent, p)
        setattr(parent, leaf, unfuse_one(mod))
    return len(todo)


def _dense_weight_bias(linear: nn.Module):
    """(weight [out, in], bias or None) of an expert layer: a plain Linear (which, after
    quantization, holds the dequantized weight) or a packed GPTQLinear (dequantized here)."""
    weight = getattr(linear, "weight", None)
    if isinstance(weight, torch.Tensor):
        return weight.data, (linear.bias.data if getattr(linear, "bias", None) is not None else None)
    if hasattr(linear, "dequantized_weight"):
        return linear.dequantized_weight(), (linear.bias.data if getattr(linear, "bias", None) is not None else None)
    raise TypeError(f"Cannot fuse expert layer without weight: {type(linear)}")


def fuse_one(routed: RoutedExperts, like: nn.Module = None, dtype=None) -> nn.Module:
    """A fused experts module with the layout of GPT-OSS from per-expert layers: gate and up
    interleaved along the last axis of ``gate_up_proj`` [E, hidden, 2*inter], ``down_proj``
    [E, inter, hidden], biases [E, 2*inter] / [E, hidden].  ``like``: a fused module to fill (its
    class and attributes are kept); otherwise transformers' GptOssExperts is instantiated."""
    e0 = routed[0]
    gate_w0, _ = _dense_weight_bias(e0.gate_proj)
    inter, hidden = gate_w0.shape
    n = len(routed)
    dtype = dtype or gate_w0.dtype
    dev = gate_w0.device
    gate_up = torch.empty((n, hidden, 2 * inter), dtype=dtype, device=dev)
    gate_up_b = torch.zeros((n, 2 * inter), dtype=dtype, device=dev)
    down = torch.empty((n, inter, hidden), dtype=dtype, device=dev)
    down_b = torch.zeros((n, hidden), dtype=dtype, device=dev)
    for i in range(n):
        ex = routed[i]
        gw, gb = _dense_weight_bias(ex.gate_proj)
        uw, ub = _dense_weight_bias(ex.up_proj)
        dw, db = _dense_weight_bias(ex.down_proj)
        gate_up[i, :, 0::2] = gw.t().to(dtype)
        gate_up[i, :, 1::2] = uw.t().to(dtype)
        down[i] = dw.t().to(dtype)
        if gb is not None:
            gate_up_b[i, 0::2] = gb.to(dtype)
        if ub is not None:
            gate_up_b[i, 1::2] = ub.to(dtype)
        if db is not None:
            down_b[i] = db.to(dtype)
    if like is None:
        cls, config, alpha, limit = routed.origin if routed.origin is not None else (None, None, None, None)
        if cls is None:
            from transformers.models.gpt_oss.modeling_gpt_oss import GptOssExperts as cls
        if config is None:
            from types import SimpleNamespace

            config = SimpleNamespace(intermediate_size=inter, num_local_experts=n, hidden_size=hidden,
                                     _experts_implementation="eager")
        like = cls(config)
        if alpha is not None:
            like.alpha, like.limit = alpha, limit
    for name, value in (("gate_up_proj", gate_up), ("gate_up_proj_bias", gate_up_b), ("down_proj", down),
                        ("down_proj_bias", down_b)):
        setattr(like, name, nn.Parameter(value.contiguous(), requires_grad=False))
    return like


def fuse_moe_experts(model: nn.Module, dtype=None) -> int:
    """Replace every ``RoutedExperts`` of ``model`` by a fused experts module (in place); returns how
    many were replaced.  A module made by ``unfuse_moe_experts`` remembers the class, configuration
    and activation constants of the fused module it replaced."""
    todo = [(name, mod) for name, mod in model.named_modules() if isinstance(mod, RoutedExperts)]
    for name, mod in todo:
        parent = model
        *path, leaf = name.split(".")
        for p_ in path:
            parent = getattr(parent, p_)
        setattr(parent, leaf, fuse_one(mod, dtype=dtype))
    return len(todo)
