"""Host logic of the fused block operators: which modules / functions are recognised (by source),
that unrecognised formulations are left alone, and that the patches are undone."""

import sys

import torch

from onecompression_b200.qep._quantize_with_qep_arch import _FusedOps


def _blocks():
    from transformers import LlamaConfig, Qwen3Config
    from transformers.models.llama.modeling_llama import LlamaDecoderLayer
    from transformers.models.qwen3.modeling_qwen3 import Qwen3DecoderLayer

    out = []
    for cfg_cls, layer_cls in ((LlamaConfig, LlamaDecoderLayer), (Qwen3Config, Qwen3DecoderLayer)):
        cfg = cfg_cls(hidden_size=64, intermediate_size=128, num_attention_heads=4, num_key_value_heads=2,
                      num_hidden_layers=1, vocab_size=64, head_dim=16)
        out.append(layer_cls(cfg, 0).half())
    return out


def test_recognised_modules_and_restoration():
    llama, qwen = _blocks()
    for blk, n_norms in ((llama, 2), (qwen, 4)):          # Qwen3 adds q_norm and k_norm
        ns = sys.modules[type(blk.self_attn).__module__]
        original = ns.apply_rotary_pos_emb
        ops = _FusedOps([blk])
        assert len(ops.norm_mods) == n_norms and len(ops.mlp_mods) == 1 and len(ops.rope_spaces) == 1
        with ops:
            assert ns.apply_rotary_pos_emb is not original
            assert "forward" in blk.mlp.__dict__ and "forward" in blk.input_layernorm.__dict__
            # CPU tensors are not taken by the kernels: the patched callables fall back to the model code
            x = torch.randn(2, 3, 64).half()
            assert torch.equal(blk.input_layernorm(x), type(blk.input_layernorm).forward(blk.input_layernorm, x))
        assert ns.apply_rotary_pos_emb is original
        assert "forward" not in blk.mlp.__dict__ and "forward" not in blk.input_layernorm.__dict__


def test_other_formulations_are_left_alone():
    llama, _ = _blocks()

    class OtherNorm(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.weight = torch.nn.Parameter(torch.ones(64).half())
            self.variance_epsilon = 1e-6

        def forward(self, x):
            return x * self.weight              # not the RMSNorm formula

    class OtherMLP(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.gate_proj = torch.nn.Linear(64, 128)
            self.up_proj = torch.nn.Linear(64, 128)
            self.down_proj = torch.nn.Linear(128, 64)
            self.act_fn = torch.nn.GELU()       # gated, but not SiLU

        def forward(self, x):
            down_proj = self.down_proj(self.act_fn(self.gate_proj(x)) * self.up_proj(x))
            return down_proj

    llama.input_layernorm = OtherNorm()
    llama.mlp = OtherMLP()
    ops = _FusedOps([llama])
    assert len(ops.norm_mods) == 1 and len(ops.mlp_mods) == 0       # only post_attention_layernorm is left
    assert len(_FusedOps([llama], norms=False, elementwise=False).norm_mods) == 0


def test_unrecognised_modules_are_reported_once(caplog):
    """A module that looks like a fusable operator but whose code differs (another formulation, or a
    library release that rewords a forward) is named in the log once, so the extra kernels of the
    model's own operators do not go unnoticed."""
    import logging

    from onecompression_b200.qep import _quantize_with_qep_arch as arch

    llama, _ = _blocks()

    class ReworkedRMSNorm(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.weight = torch.nn.Parameter(torch.ones(64).half())
            self.variance_epsilon = 1e-6

        def forward(self, x):
            v = x.float().pow(2).mean(-1, keepdim=True)
            return (self.weight * (x.float() * torch.rsqrt(v + self.variance_epsilon))).to(x.dtype)

    llama.input_layernorm = ReworkedRMSNorm()
    arch._declined_logged.clear()
    with caplog.at_level(logging.INFO, logger=arch.logger.name):
        first = _FusedOps([llama])
        _FusedOps([llama])
    assert len(first.norm_mods) == 1
    lines = [r.getMessage() for r in caplog.records if "ReworkedRMSNorm" in r.getMessage()]
    assert len(lines) == 1 and "model's own operators" in lines[0]
