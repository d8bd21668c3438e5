"""Seeded synthetic workloads with the shapes of the benchmark configurations.

They stand in for real checkpoints and the C4 calibration set (neither can be
present offline): random-init decoder blocks with N(0, 0.02²) fp16 weights and
calibration tokens drawn uniformly from the vocabulary and pushed through a random
embedding table.  Tests and the benchmark feed the same tensors to this package and
to the CPU checker of the test-suite.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

LLAMA3_8B = dict(hidden_size=4096, intermediate_size=14336, num_attention_heads=32,
                 num_key_value_heads=8, head_dim=128, vocab_size=128256, num_hidden_layers=32,
                 rms_norm_eps=1e-5, rope_theta=500000.0, max_position_embeddings=8192)
QWEN3_14B = dict(hidden_size=5120, intermediate_size=17408, num_attention_heads=40,
                 num_key_value_heads=8, head_dim=128, vocab_size=151936, num_hidden_layers=40,
                 rms_norm_eps=1e-6, rope_theta=1000000.0, max_position_embeddings=8192)


def single_linear_case(seed: int, out: int, d: int, n_seq: int, seq: int, outliers: int = 8):
    """Config-1 style layer: W ~ N(0, 0.02²) fp16 [out, d]; X ~ N(0,1) fp16
    [n_seq, seq, d] with ``outliers`` seeded channels scaled by 20 (CPU tensors)."""
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(out, d, generator=g) * 0.02).half()
    x = torch.randn(n_seq, seq, d, generator=g)
    x[..., torch.randperm(d, generator=g)[:outliers]] *= 20
    return w, x.half()


def llama_config(shape: dict, num_layers: int):
    from transformers import LlamaConfig

    cfg = LlamaConfig(**{**shape, "num_hidden_layers": num_layers})
    cfg._attn_implementation = "sdpa"
    return cfg


@dataclass
class DecoderStack:
    """Random-init decoder blocks plus what a block forward needs."""

    blocks: list
    kwargs: dict
    config: object


def _init_block_(block, seed, std=0.02):
    g = torch.Generator(device=block.input_layernorm.weight.device).manual_seed(seed)
    for name, p in block.named_parameters():
        if p.dim() >= 2:
            p.data.normal_(0.0, std, generator=g)
        elif "norm" in name:
            p.data.fill_(1.0)
        else:
            p.data.zero_()


def llama_blocks(shape: dict, num_layers: int, seq_len: int, device, seed: int = 0,
                 dtype=torch.float16) -> DecoderStack:
    """``num_layers`` LlamaDecoderLayer modules (transformers) on ``device`` with seeded
    N(0, 0.02²) weights, and the rotary position embeddings for ``seq_len``."""
    from transformers.models.llama.modeling_llama import LlamaDecoderLayer, LlamaRotaryEmbedding

    cfg = llama_config(shape, num_layers)
    blocks = []
    with torch.device(device):
        for i in range(num_layers):
            blk = LlamaDecoderLayer(cfg, layer_idx=i).to(dtype)
            _init_block_(blk, seed * 1000 + i)
            blk.eval()
            blocks.append(blk)
        rot = LlamaRotaryEmbedding(cfg)
        pos = torch.arange(seq_len).unsqueeze(0)
        cos, sin = rot(torch.zeros(1, seq_len, cfg.hidden_size, dtype=dtype), pos)
    kwargs = {"position_embeddings": (cos, sin), "position_ids": pos, "attention_mask": None,
              "use_cache": False}
    return DecoderStack(blocks, kwargs, cfg)


def embedded_tokens(vocab: int, hidden: int, n_seq: int, seq_len: int, device, seed: int = 0,
                    dtype=torch.float16, row_range=None):
    """First-block inputs: uniform token ids in [0, vocab) looked up in a seeded
    N(0, 0.02²) embedding table.  ``row_range`` (first, last) returns only those
    sequences (token sharding) while drawing the same ids as the full set."""
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, vocab, (n_seq, seq_len), generator=g)
    if row_range is not None:
        ids = ids[row_range[0] : row_range[1]]
    gd = torch.Generator(device=device).manual_seed(seed + 1)
    table = torch.empty((vocab, hidden), dtype=dtype, device=device).normal_(0.0, 0.02, generator=gd)
    return table[ids.to(device)]
