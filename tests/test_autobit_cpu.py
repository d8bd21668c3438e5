"""The bit-assignment solver on CPU: optimality against brute force, fused ties, budgets."""

import itertools
import random

import pytest

from onecompression_b200.quantizer.autobit import effective_bits_per_param, solve_assignment


def _brute(errors, params, eff, target, fused):
    n, nb = len(errors), len(errors[0])
    budget = target * sum(params)
    best, arg = float("inf"), None
    for choice in itertools.product(range(nb), repeat=n):
        if any(len({choice[m] for m in g}) > 1 for g in fused):
            continue
        cost = sum(eff[m][choice[m]] * params[m] for m in range(n))
        if cost > budget * (1 + 1e-12):
            continue
        e = sum(errors[m][choice[m]] for m in range(n))
        if e < best:
            best, arg = e, choice
    return best, arg


@pytest.mark.parametrize("seed", range(8))
def test_solver_is_optimal_on_small_instances(seed):
    rnd = random.Random(seed)
    n, bits = 7, (2, 3, 4)
    params = [rnd.choice([4096 * 4096, 1024 * 4096, 14336 * 4096]) for _ in range(n)]
    errors = [sorted((rnd.random() * p / 1e6 for _ in bits), reverse=True) for p in params]
    eff = [[effective_bits_per_param(b, 128) for b in bits] for _ in range(n)]
    fused = [[0, 1, 2], [4, 5]]
    for target in (2.2, 2.9, 3.3, 3.8, 4.2):
        want, arg = _brute(errors, params, eff, target, fused)
        chosen, thinned = solve_assignment(errors, params, eff, target, fused)
        assert not thinned
        got = sum(errors[m][chosen[m]] for m in range(n))
        assert abs(got - want) <= 1e-9 * max(1.0, want), (chosen, arg)
        assert sum(eff[m][chosen[m]] * params[m] for m in range(n)) <= target * sum(params) * (1 + 1e-12)
        assert chosen[0] == chosen[1] == chosen[2] and chosen[4] == chosen[5]


def test_solver_reports_infeasible_budget():
    with pytest.raises(RuntimeError, match="infeasible"):
        solve_assignment([[1.0, 0.5]], [100], [[2.1, 4.1]], 1.5)


def test_effective_bits_formula():
    assert effective_bits_per_param(4, 128) == 4 + 20 / 128
    assert effective_bits_per_param(3, -1, in_features=4096) == 3 + 19 / 4096
    assert effective_bits_per_param(2, -1) == 2.0


def test_model_scale_instance_solves_fast():
    """280 layers x 3 candidates (the Qwen3-14B size of config 4) stays exact and quick."""
    import time

    rnd = random.Random(0)
    shapes = [5120 * 5120, 1024 * 5120, 1024 * 5120, 5120 * 5120, 17408 * 5120, 17408 * 5120, 5120 * 17408]
    params = shapes * 40
    errors = [[p * (0.5 + rnd.random()) * s for s in (16.0, 4.0, 1.0)] for p in params]
    eff = [[effective_bits_per_param(b, 128) for b in (2, 3, 4)] for _ in params]
    fused = [[7 * l, 7 * l + 1, 7 * l + 2] for l in range(40)] + [[7 * l + 4, 7 * l + 5] for l in range(40)]
    t = time.time()
    chosen, thinned = solve_assignment(errors, params, eff, 3.5 + 19.5 / 128, fused)
    assert time.time() - t < 60
    used = sum(eff[m][chosen[m]] * params[m] for m in range(len(params))) / sum(params)
    assert used <= 3.5 + 19.5 / 128 + 1e-9 and used > 3.3
    assert len(set(chosen)) > 1


def test_activation_stats_on_cpu_model():
    """a = E[x²] per input channel and b = E[(dL/dy)²] per output channel, against a direct
    computation on a tiny fp32 Llama (no GPU involved: hooks and autograd only)."""
    import torch
    from transformers import LlamaConfig, LlamaForCausalLM

    from onecompression_b200.quantizer.autobit import collect_activation_stats

    torch.manual_seed(0)
    cfg = LlamaConfig(hidden_size=32, intermediate_size=64, num_attention_heads=2, num_key_value_heads=2,
                      num_hidden_layers=1, vocab_size=64, max_position_embeddings=32)
    model = LlamaForCausalLM(cfg).eval()
    ids = torch.randint(0, 64, (5, 12))
    cands = [(n, m) for n, m in model.named_modules() if isinstance(m, torch.nn.Linear) and "lm_head" not in n]
    a, b = collect_activation_stats(model, ids, cands, batch_size=2)
    assert len(a) == 7 and all(not p.requires_grad or True for p in model.parameters())
    name, mod = cands[3]        # o_proj
    xs, gs = [], []
    h1 = mod.register_forward_hook(lambda m, i, o: xs.append(i[0].detach()))
    h2 = mod.register_full_backward_hook(lambda m, gi, go: gs.append(go[0].detach()))
    for p in model.parameters():
        p.requires_grad_(True)
    for i in range(5):          # one sequence at a time, each with its own mean loss
        out = model(input_ids=ids[i:i + 1], labels=ids[i:i + 1])
        out.loss.backward()
        model.zero_grad()
    h1.remove(); h2.remove()
    x = torch.cat([t.reshape(-1, t.shape[-1]) for t in xs]); g = torch.cat([t.reshape(-1, t.shape[-1]) for t in gs])
    assert torch.allclose(a[name], x.pow(2).mean(0), rtol=1e-4, atol=1e-8)
    assert torch.allclose(b[name], g.pow(2).mean(0), rtol=1e-3, atol=1e-12)
    a2, b2 = collect_activation_stats(model, ids, cands, batch_size=5, use_curvature_b=False)
    assert all(v is None for v in b2.values()) and torch.allclose(a2[name], a[name], rtol=1e-5)
