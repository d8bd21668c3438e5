"""Un-fusing GPT-OSS style experts: same function, per-expert linears that only see their own tokens."""

import torch

from onecompression_b200.utils import RoutedExperts, fuse_moe_experts, unfuse_moe_experts


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


def test_fusing_back_restores_the_fused_layout():
    """un-fuse -> fuse gives back the very tensors (layout of the reference's _fuse_gpt_oss_one,
    onecomp/utils/unfuse_moe.py:499-574: gate / up interleaved, down transposed) and the same
    function; a changed expert weight lands at its place in the fused tensors."""
    _cfg, layer = _tiny_gpt_oss()
    fused = layer.mlp.experts
    before = {k: getattr(fused, k).data.clone() for k in
              ("gate_up_proj", "gate_up_proj_bias", "down_proj", "down_proj_bias")}
    x = torch.randn(24, 64)
    idx = torch.stack([torch.randperm(4)[:2] for _ in range(24)])
    w = torch.rand(24, 2)
    with torch.no_grad():
        want = fused(x, router_indices=idx, routing_weights=w)
    assert unfuse_moe_experts(layer) == 1
    layer.mlp.experts[2].up_proj.weight.data[5, 7] = 3.0          # stands for a quantized weight
    assert fuse_moe_experts(layer) == 1
    again = layer.mlp.experts
    assert type(again).__name__ == "GptOssExperts"
    assert sorted(k for k, _ in again.named_parameters()) == sorted(before)
    for k, v in before.items():
        got = getattr(again, k).data
        assert got.shape == v.shape and got.dtype == v.dtype
        if k == "gate_up_proj":
            assert got[2, 7, 2 * 5 + 1] == 3.0                    # up = odd columns; [expert, in, 2*out+1]
            got = got.clone()
            got[2, 7, 2 * 5 + 1] = v[2, 7, 2 * 5 + 1]
        assert torch.equal(got, v), k
    layer.mlp.experts.gate_up_proj.data[2, 7, 11] = before["gate_up_proj"][2, 7, 11]
    with torch.no_grad():
        got = layer.mlp.experts(x, router_indices=idx, routing_weights=w)
    assert torch.allclose(got, want, rtol=1e-5, atol=1e-5)
    assert fuse_moe_experts(layer) == 0
