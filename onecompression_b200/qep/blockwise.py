"""Decoder-block utilities for the block-wise drivers (behaviour of
onecomp/utils/blockwise.py:19-93, 150-285, 364-400, 501-555 for plain decoder stacks:
Llama / Qwen3 / GPT-OSS style blocks that take ``hidden_states`` plus keyword
arguments captured once).  Per-layer embeddings and mixed attention types of other
families are not handled here.
"""

from __future__ import annotations

import torch
from torch import nn


class StopForward(Exception):
    """Raised from a hook to end a forward pass as soon as what was needed is captured."""


def get_blocks(model: nn.Module) -> nn.ModuleList:
    """The decoder blocks: the first ModuleList whose items are transformer layers.
    With a ``language_model`` / ``text_model`` sub-module only that one is searched."""
    try:
        from transformers.modeling_layers import GradientCheckpointingLayer as _Layer
    except ImportError:  # pragma: no cover
        _Layer = nn.Module
    root = model
    for name, mod in model.named_modules():
        if name.endswith(("language_model", "text_model")):
            root = mod
            break
    for module in root.modules():
        if isinstance(module, nn.ModuleList) and len(module) > 0 and isinstance(module[0], _Layer):
            return module
    raise RuntimeError("Transformer blocks not found.")


class _Catcher(nn.Module):
    def __init__(self, module):
        super().__init__()
        self.module = module
        self.inp = None
        self.kwargs = {}

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self.module, name)

    def forward(self, inp, *args, **kwargs):
        self.inp = inp
        self.kwargs.update(kwargs)
        raise StopForward()


@torch.no_grad()
def get_blocks_and_inputs(model, model_inputs, batch_size, store_device=None):
    """(blocks, first-block inputs [N, S, hidden], block kwargs captured with one sample).

    The model runs where it lives; the captured hidden states are stored on
    ``store_device`` (default: where they were produced)."""
    blocks = get_blocks(model)
    ids = model_inputs["input_ids"]
    extra = {k: v for k, v in model_inputs.items() if k != "input_ids"}
    extra["use_cache"] = False
    catcher = _Catcher(blocks[0])
    blocks[0] = catcher
    try:
        one = {k: (v[:1] if isinstance(v, torch.Tensor) and v.dim() >= 1 else v) for k, v in extra.items()}
        try:
            model(ids[:1], **one)
        except StopForward:
            pass
        kwargs = dict(catcher.kwargs)
        chunks = []
        for first in range(0, ids.shape[0], batch_size):
            part = {
                k: (v[first : first + batch_size] if isinstance(v, torch.Tensor) and v.dim() >= 1 else v)
                for k, v in extra.items()
            }
            try:
                model(ids[first : first + batch_size], **part)
            except StopForward:
                x = catcher.inp
                chunks.append(x.to(store_device) if store_device is not None else x.clone())
    finally:
        blocks[0] = catcher.module
    return blocks, torch.cat(chunks), kwargs


def move_to_device(x, device):
    if isinstance(x, torch.Tensor):
        return x.to(device)
    if isinstance(x, dict):
        return {k: move_to_device(v, device) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return type(x)(move_to_device(v, device) for v in x)
    return x


def expand_batch(kwargs, batch_size):
    """Tensors captured with batch 1 become views of the wanted batch size."""
    def grow(v):
        if isinstance(v, torch.Tensor) and v.dim() >= 1 and v.shape[0] == 1 and batch_size > 1:
            return v.expand(batch_size, *v.shape[1:])
        if isinstance(v, (list, tuple)):
            return type(v)(grow(t) for t in v)
        if isinstance(v, dict):
            return {k: grow(t) for k, t in v.items()}
        return v

    return {k: grow(v) for k, v in kwargs.items()}


def call_block(block, x, kwargs):
    out = block(x, **expand_batch(kwargs, x.shape[0]))
    return out[0] if isinstance(out, tuple) else out


@torch.no_grad()
def forward_input(inps, block, kwargs, batch_size, device, out=None):
    """Block outputs for all samples, ``batch_size`` sequences at a time."""
    outs = []
    for first in range(0, inps.shape[0], batch_size):
        y = call_block(block, inps[first : first + batch_size].to(device), kwargs)
        if out is not None:
            out[first : first + batch_size].copy_(y)
        else:
            outs.append(y.to(inps.device))
    return out if out is not None else torch.cat(outs)
