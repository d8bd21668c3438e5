"""The multi-rank host logic on CPU: two gloo ranks shard tokens for the moments and
weight rows for the quantization; the assembled result must equal the unsharded one
(rows are independent given the inverse-Hessian factor)."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import gptq_oracle as orc


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_row_slab_partition():
    from onecompression_b200.sharding import row_slab, seq_shard

    for out in (32, 96, 1024, 4096, 14336, 2880, 100):
        for world in (1, 2, 3, 4, 8):
            slabs = [row_slab(out, r, world) for r in range(world)]
            assert slabs[0][0] == 0 and slabs[-1][1] == out
            for (a, b), (c, d) in zip(slabs, slabs[1:]):
                assert b == c and a <= b
            assert all(a % 32 == 0 for a, b in slabs if b > a)
    for n in (128, 7, 16):
        for world in (1, 2, 4, 8):
            parts = [seq_shard(n, r, world) for r in range(world)]
            assert parts[0][0] == 0 and parts[-1][1] == n
            assert all(p[1] == q[0] for p, q in zip(parts, parts[1:]))


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    from onecompression_b200 import GPTQ, QEPConfig
    from onecompression_b200.sharding import ShardedContext, row_slab, seq_shard

    ctx = ShardedContext()
    g = torch.Generator().manual_seed(1)
    n_seq, seq, d, out = 6, 32, 64, 96
    xq = torch.randn(n_seq, seq, d, generator=g).half()
    xf = (xq.float() * (1 + 0.05 * torch.randn(n_seq, seq, d, generator=g))).half()
    w = (torch.randn(out, d, generator=g) * 0.02).half()

    # tokens: per-rank running means -> global means
    a, b = seq_shard(n_seq, rank, world)
    h_loc, c_loc, n_loc = orc.hessian_and_crossterm([xq[a:b]], [xf[a:b]])
    h, c, n = ctx.reduce_moments(h_loc.clone(), c_loc.clone(), n_loc)
    h_all, c_all, n_all = orc.hessian_and_crossterm([xq], [xf])
    assert n == n_all
    assert torch.allclose(h, h_all, rtol=1e-5, atol=1e-6) and torch.allclose(c, c_all, rtol=1e-4, atol=1e-6)
    # the cross term reduced in the background while the caller works on H: same values after the wait
    h2, c2, n2 = ctx.reduce_moments(h_loc.clone(), c_loc.clone(), n_loc, defer_cross=True)
    assert torch.equal(h2, h) and n2 == n
    ctx.wait_cross()
    assert torch.equal(c2, c)
    ctx.wait_cross()                      # nothing pending: a no-op

    # rows: every rank quantizes its slab with the oracle standing in for the kernels
    u = orc.inverse_hessian_upper(h_all.clone(), 0.01)
    lin = torch.nn.Linear(d, out, bias=False).half()
    lin.weight.data = w.clone()
    q = GPTQ(wbits=4, groupsize=32, sym=False)
    q.module_to_name = {lin: "layer"}

    def compute(w_slab, cross):
        wa = orc.qep_adjust_weight(w_slab, h_all, cross, 0.01, 0.5)
        r = orc.gptq_quantize(wa, h_all.clone(), wbits=4, groupsize=32, sym=False, u_override=u)
        qw, qz = orc.pack_result(r["qweight"].numpy(), r["qzeros"].numpy(), 4)
        deq = orc.dequantize_result(qw, r["scales"], qz, None, 4, 32, wa.shape)
        return {"qweight": torch.from_numpy(qw), "qzeros": torch.from_numpy(qz), "scales": r["scales"],
                "zeros": r["qzeros"], "dequantized": deq}

    class F:  # stands in for the device factor
        perm = None

    res = ctx.quantize_rows(q, lin, h_all, c_all, QEPConfig(), F(), compute=compute)
    whole = compute(w, c_all)
    assert np.array_equal(res.qweight.numpy(), whole["qweight"].numpy())
    assert np.array_equal(res.qzeros.numpy(), whole["qzeros"].numpy())
    assert torch.equal(res.scales, whole["scales"])
    assert torch.equal(res.__dict__["_device_dequantized"], whole["dequantized"])
    assert q.results["layer"] is res

    # two layers with one input, stacked: the stacked rows are split over the ranks and the gathered
    # result is cut back per layer; slabs may straddle the boundary between the layers
    w2 = (torch.randn(64, d, generator=g) * 0.02).half()
    lin_a, lin_b = torch.nn.Linear(d, out, bias=False).half(), torch.nn.Linear(d, 64, bias=False).half()
    lin_a.weight.data, lin_b.weight.data = w.clone(), w2.clone()
    q2 = GPTQ(wbits=4, groupsize=32, sym=False)
    q2.module_to_name = {lin_a: "a", lin_b: "b"}
    both = ctx.quantize_rows_stacked(q2, [lin_a, lin_b], h_all, c_all, QEPConfig(), F(), compute=compute)
    for lin_x, w_x, key in ((lin_a, w, "a"), (lin_b, w2, "b")):
        alone = compute(w_x, c_all)
        r = both[lin_x]
        assert q2.results[key] is r and r.qweight_original_shape == (w_x.shape[0], d)
        assert np.array_equal(r.qweight.numpy(), alone["qweight"].numpy())
        assert np.array_equal(r.qzeros.numpy(), alone["qzeros"].numpy())
        assert torch.equal(r.scales, alone["scales"])
        assert torch.equal(r.__dict__["_device_dequantized"], alone["dequantized"])

    # a quantizer that does not pack (bit widths without a packed layout): integer codes and raw
    # zero points are gathered instead, with the flags of the single-GPU result
    q5 = GPTQ(wbits=5, groupsize=32, sym=False, bitpack_on_quantize=False)
    lin5 = torch.nn.Linear(d, out, bias=False).half()
    lin5.weight.data = w.clone()
    q5.module_to_name = {lin5: "layer5"}

    def compute_unpacked(w_slab, cross):
        r = orc.gptq_quantize(w_slab, h_all.clone(), wbits=5, groupsize=32, sym=False, u_override=u)
        deq = (r["scales"].float().T.repeat_interleave(32, 1)
               * (r["qweight"].float() - r["qzeros"].float().T.repeat_interleave(32, 1))).half()
        return {"codes": r["qweight"], "zeros": r["qzeros"], "scales": r["scales"], "dequantized": deq}

    res5 = ctx.quantize_rows(q5, lin5, h_all, None, QEPConfig(), F(), compute=compute_unpacked)
    whole5 = compute_unpacked(w, None)
    assert not res5.qweight_is_packed and not res5.qzeros_is_packed
    assert res5.qweight.shape == (out, d) and torch.equal(res5.qweight, whole5["codes"])
    assert torch.equal(res5.qzeros, whole5["zeros"]) and torch.equal(res5.scales, whole5["scales"])

    # independent layers (experts): dealt round-robin, results broadcast from their owners
    experts, items = [], []
    q3 = GPTQ(wbits=4, groupsize=32, sym=False)
    for e in range(5):
        lin_e = torch.nn.Linear(d, 64, bias=False).half()
        lin_e.weight.data = (torch.randn(64, d, generator=g) * 0.02).half()
        h_e = h_all * (1.0 + 0.1 * e)
        q3.module_to_name[lin_e] = f"expert{e}"
        experts.append(lin_e)
        items.append((lin_e, h_e))
    calls = []

    def compute_whole(weight, hessian):
        calls.append(1)
        r = orc.gptq_quantize(weight, hessian.clone(), wbits=4, groupsize=32, sym=False)
        qw, qz = orc.pack_result(r["qweight"].numpy(), r["qzeros"].numpy(), 4)
        deq = orc.dequantize_result(qw, r["scales"], qz, None, 4, 32, weight.shape)
        return {"qweight": torch.from_numpy(qw), "qzeros": torch.from_numpy(qz), "scales": r["scales"],
                "dequantized": deq}

    done = ctx.quantize_independent(q3, items, compute=compute_whole)
    assert len(calls) == len([i for i in range(5) if i % world == rank])      # only the owned layers
    for lin_e, h_e in items:
        alone = compute_whole(lin_e.weight.data, h_e)
        r = done[lin_e]
        assert np.array_equal(r.qweight.numpy(), alone["qweight"].numpy())
        assert np.array_equal(r.qzeros.numpy(), alone["qzeros"].numpy())
        assert torch.equal(r.scales, alone["scales"])
        assert torch.equal(r.__dict__["_device_dequantized"], alone["dequantized"])
        assert q3.results[q3.module_to_name[lin_e]] is r
    open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_token_and_row_sharding_two_ranks(tmp_path, world):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_correction_factor_rule(monkeypatch):
    """The QEP correction may borrow the column loop's factor only if that factor was built with the
    correction's damping and needed no retry (reference adjust_weight, _quantizer.py:396-428, damps
    and retries by its own rule); otherwise the Hessian is factored again, without act-order and
    with the correction's shift sequence.  One GPU and the row-sharded path share this rule."""
    from onecompression_b200 import kernels
    from onecompression_b200.kernels import HessianFactor
    from onecompression_b200.quantizer import _quantizer as qmod

    calls = []

    def fake_factor(h, percdamp, actorder, max_retries=5, shifts=None):
        calls.append((percdamp, actorder, shifts is not None))
        return "fresh"

    monkeypatch.setattr(kernels, "factor_hessian", fake_factor)
    z = torch.zeros(1)

    def fac(percdamp, attempts, actorder=False):
        return HessianFactor(z, z, z, z, z, actorder, percdamp, 1.0, attempts)

    same = fac(0.01, 1)
    assert qmod.qep_factor(None, same, 0.01) is same and not calls
    act = fac(0.01, 1, actorder=True)
    assert qmod.qep_factor(None, act, 0.01) is act and not calls          # the kernels apply P
    assert qmod.qep_factor(None, fac(0.05, 1), 0.01) == "fresh"            # other damping
    assert qmod.qep_factor(None, fac(0.01, 2), 0.01) == "fresh"            # a retried factor
    assert qmod.qep_factor(None, None, 0.01) == "fresh"
    assert calls == [(0.01, False, True)] * 3

    # the shift sequence of the retry rule, in units of the first damp, against the reference's loop:
    # damp_k = percdamp * mean(diag) of the matrix as damped so far; after the k-th failure
    # 10^k * damp_k more is added
    def reference_totals(percdamp, attempts, mean=1.0):
        total, out, mult = 0.0, [], 1.0
        for k in range(attempts):
            damp = percdamp * (mean + total)
            total += damp
            out.append(total / (percdamp * mean))
            mult *= 10.0
            total += mult * damp          # what the except branch adds before the next attempt
        return out

    rule = qmod._qep_shift_rule()
    got = [rule(k, 0.01) for k in range(4)]
    want = reference_totals(0.01, 4)
    assert got[0] == 1.0
    for k in range(4):
        assert abs(got[k] - want[k]) <= 1e-12 * want[k], (k, got, want)
