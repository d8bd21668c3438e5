"""Small seeded models for the block-driver fixtures and tests.

Used on both sides of ``tests/golden/driver_*.npz``: ``tests/golden/make_golden.py`` runs the
reference's block-wise QEP driver on them (CPU), the GPU tests run this package's driver on the
same weights and token ids.  Test infrastructure only.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn
from transformers.modeling_layers import GradientCheckpointingLayer

LLAMA_KW = dict(
    hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
    num_key_value_heads=2, head_dim=16, vocab_size=128, max_position_embeddings=64,
    rms_norm_eps=1e-5, tie_word_embeddings=False, attention_bias=False, mlp_bias=False,
)
LLAMA_N_SEQ, LLAMA_SEQ = 20, 24          # 20 sequences: chunks of 16 + 4 in the drivers


def tiny_llama(seed: int = 0, dtype=torch.float16):
    """A 2-layer LlamaForCausalLM (hidden 64, 4 q / 2 kv heads of 16, intermediate 128), random
    init, eager attention (the same operator sequence on CPU and GPU)."""
    from transformers import LlamaConfig, LlamaForCausalLM

    cfg = LlamaConfig(**LLAMA_KW)
    cfg._attn_implementation = "eager"        # pylint: disable=protected-access
    torch.manual_seed(seed)
    model = LlamaForCausalLM(cfg)
    # wider weights than the 0.02 default so that a 64-wide layer has something to quantize
    g = torch.Generator().manual_seed(seed + 1)
    for name, p in model.named_parameters():
        if p.dim() == 2 and "embed" not in name and "lm_head" not in name:
            p.data = torch.randn(p.shape, generator=g) * 0.08
    return model.to(dtype).eval()


def llama_ids(seed: int = 0):
    g = torch.Generator().manual_seed(seed + 100)
    return torch.randint(0, LLAMA_KW["vocab_size"], (LLAMA_N_SEQ, LLAMA_SEQ), generator=g)


# ---- a hard-routed mixture-of-experts stack ------------------------------------------------
MOE_HIDDEN, MOE_INTER, MOE_EXPERTS, MOE_VOCAB = 32, 64, 4, 48
MOE_N_SEQ, MOE_SEQ = 18, 40


class _Expert(nn.Module):
    def __init__(self):
        super().__init__()
        self.gate_proj = nn.Linear(MOE_HIDDEN, MOE_INTER, bias=False)
        self.up_proj = nn.Linear(MOE_HIDDEN, MOE_INTER, bias=False)
        self.down_proj = nn.Linear(MOE_INTER, MOE_HIDDEN, bias=False)

    def forward(self, x):
        return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))


class _RoutedMLP(nn.Module):
    """Top-1 routing on the first MOE_EXPERTS channels; an expert runs only on the tokens routed to
    it (so an expert without tokens never sees a forward call)."""

    def __init__(self):
        super().__init__()
        self.router = nn.Linear(MOE_HIDDEN, MOE_EXPERTS, bias=False)
        self.experts = nn.ModuleList([_Expert() for _ in range(MOE_EXPERTS)])

    def forward(self, x):
        shape = x.shape
        flat = x.reshape(-1, shape[-1])
        choice = self.router(flat).float().argmax(dim=-1)
        out = torch.zeros_like(flat)
        for e, expert in enumerate(self.experts):
            rows = torch.nonzero(choice == e).flatten()
            if rows.numel():
                out[rows] = expert(flat[rows]) * 0.25
        return out.reshape(shape)


class _RoutedBlock(GradientCheckpointingLayer):
    def __init__(self):
        super().__init__()
        self.pre = nn.Linear(MOE_HIDDEN, MOE_HIDDEN, bias=False)      # a regular (non-expert) layer
        self.mlp = _RoutedMLP()

    def forward(self, hidden_states, **_kwargs):
        h = hidden_states + 0.25 * self.pre(hidden_states)
        return h + self.mlp(h)


class _Stack(nn.Module):
    def __init__(self, n_blocks):
        super().__init__()
        self.layers = nn.ModuleList([_RoutedBlock() for _ in range(n_blocks)])


class RoutedMoE(nn.Module):
    """embed -> two routed blocks.  Channel c < MOE_EXPERTS of a token's embedding is large for
    c = token % MOE_EXPERTS and zero otherwise, and the routers (and ``pre``) leave those channels
    alone, so token t always goes to expert t % MOE_EXPERTS in every block and on every device."""

    def __init__(self, seed: int = 0, n_blocks: int = 2):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        self.embed = nn.Embedding(MOE_VOCAB, MOE_HIDDEN)
        emb = torch.randn(MOE_VOCAB, MOE_HIDDEN, generator=g)
        emb[:, :MOE_EXPERTS] = 0
        emb[torch.arange(MOE_VOCAB), torch.arange(MOE_VOCAB) % MOE_EXPERTS] = 8.0
        self.embed.weight.data = emb
        self.model = _Stack(n_blocks)
        for blk in self.model.layers:
            for name, p in blk.named_parameters():
                p.data = torch.randn(p.shape, generator=g) * (0.18 if "router" not in name else 0.0)
            r = torch.zeros(MOE_EXPERTS, MOE_HIDDEN)
            r[torch.arange(MOE_EXPERTS), torch.arange(MOE_EXPERTS)] = 4.0
            blk.mlp.router.weight.data = r
            # nothing writes into the routing channels
            blk.pre.weight.data[:MOE_EXPERTS] = 0
            for ex in blk.mlp.experts:
                ex.down_proj.weight.data[:MOE_EXPERTS] = 0

    def forward(self, input_ids, **kwargs):
        h = self.embed(input_ids)
        for blk in self.model.layers:
            h = blk(h, **kwargs)
        return h


def routed_moe(seed: int = 0, dtype=torch.float16):
    return RoutedMoE(seed).to(dtype).eval()


def moe_ids(seed: int = 0):
    """Sequence 0 (the one the drivers group with) only holds tokens of expert 0; the other
    sequences mix experts 0, 1 and 2; no token of expert 3 exists."""
    g = torch.Generator().manual_seed(seed + 200)
    ids = torch.randint(0, MOE_VOCAB, (MOE_N_SEQ, MOE_SEQ), generator=g)
    ids = ids - (ids % MOE_EXPERTS == 3).long()             # expert 3 -> expert 2
    ids[0] = ids[0] - ids[0] % MOE_EXPERTS                   # sequence 0 -> expert 0 only
    return ids
