"""Un-fusing GPT-OSS style experts: same function, per-expert linears that only see their own tokens."""

import torch

from onecompression_b200.utils import RoutedExperts, unfuse_moe_experts


def _tiny_gpt_oss():
    from transformers import GptOssConfig
    from transformers.models.gpt_oss.modeling_gpt_oss import GptOssDecoderLayer

    torch.manual_seed(0)
    cfg = GptOssConfig(hidden_size=64, intermediate_size=64, num_local_experts=4, num_experts_per_tok=2,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=16, num_hidden_layers=1,
                       vocab_size=128, max_position_embeddings=64, layer_types=["full_attention"])
    layer = GptOssDecoderLayer(cfg, 0).float().eval()
    for p in layer.parameters():
        p.data.normal_(0, 0.2)
    return cfg, layer


def test_unfused_experts_compute_the_same_function():
    _cfg, layer = _tiny_gpt_oss()
    fused = layer.mlp.experts
    x = torch.randn(40, 64)
    idx = torch.stack([torch.randperm(4)[:2] for _ in range(40)])
    idx[idx == 3] = 0                       # expert 3 never gets a token
    w = torch.rand(40, 2)
    with torch.no_grad():
        want = fused(x, router_indices=idx, routing_weights=w)
    assert unfuse_moe_experts(layer) == 1
    routed = layer.mlp.experts
    assert isinstance(routed, RoutedExperts) and len(routed) == 4
    assert routed[0].gate_proj.weight.shape == (64, 64) and routed[0].down_proj.bias.shape == (64,)
    calls = []
    hooks = [routed[e].up_proj.register_forward_hook(lambda m, i, o, e=e: calls.append((e, i[0].shape[0])))
             for e in range(4)]
    with torch.no_grad():
        got = routed(x, router_indices=idx, routing_weights=w)
    for h in hooks:
        h.remove()
    assert torch.allclose(got, want, rtol=1e-5, atol=1e-5)
    assert sorted(e for e, _ in calls) == [0, 1, 2]                 # the unrouted expert is not called
    assert sum(n for _, n in calls) == 80                           # every (token, slot) pair exactly once
    names = [n for n, m in layer.named_modules() if isinstance(m, torch.nn.Linear) and "experts" in n]
    assert len(names) == 12 and "mlp.experts.experts.2.down_proj" in names
