"""Per-expert ``nn.Linear`` layers for mixtures whose experts are stored as fused 3-D tensors.

GPTQ and the QEP driver work on ``nn.Linear`` modules, one Hessian per layer; GPT-OSS keeps the
weights of all experts of a layer in two parameters (``gate_up_proj`` [E, hidden, 2·inter] with gate
and up interleaved along the last axis, ``down_proj`` [E, inter, hidden], plus biases).
``unfuse_moe_experts`` swaps every such module for ``RoutedExperts``: E sub-modules with
``gate_proj`` / ``up_proj`` / ``down_proj`` linears that are called with the tokens routed to them
only, so that each expert's Hessian comes from its own tokens (reference:
onecomp/utils/unfuse_moe.py:20-116, 380-466, 639-675).
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

    def __init__(self, experts, combine):
        super().__init__()
        self.experts = nn.ModuleList(experts)
        self.combine = combine

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
    return RoutedExperts(experts, gpt_oss_glu(float(getattr(module, "alpha", 1.702)),
                                              float(getattr(module, "limit", 7.0))))


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
