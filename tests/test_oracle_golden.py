"""The CPU oracle against outputs of the reference itself (tests/golden)."""

import numpy as np
import pytest
import torch

from conftest import f16, gptq_case_names, load_golden
from oracle import gptq_oracle as orc


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
def test_pack_matches_reference(bits):
    g = load_golden("pack.npz")
    codes, zeros = g[f"codes{bits}"], g[f"zeros{bits}"]
    assert np.array_equal(orc.pack_qweight(codes, bits), g[f"qweight{bits}"])
    assert np.array_equal(orc.pack_qzeros(zeros - 1, bits), g[f"qzeros{bits}"])
    assert np.array_equal(orc.unpack_qweight(g[f"qweight{bits}"], bits, codes.shape), codes)
    z = orc.unpack_qzeros(g[f"qzeros{bits}"], bits, zeros.shape[1])
    assert np.array_equal((z + 1) & ((1 << bits) - 1), zeros)


def test_pack_rejects_unaligned():
    with pytest.raises(AssertionError):
        orc.pack_rows(np.zeros((7, 4), dtype=np.int32), 4)
    with pytest.raises(AssertionError):
        orc.pack_rows(np.zeros((16, 4), dtype=np.int32), 3)


@pytest.mark.parametrize("bits", [2, 3, 4, 8])
@pytest.mark.parametrize("sym", [False, True])
def test_find_params_matches_reference(bits, sym):
    g = load_golden("find_params.npz")
    x = torch.from_numpy(g["x"])
    s, z = orc.find_params(x, bits, sym)
    assert np.array_equal(s.numpy(), g[f"scale_b{bits}_s{int(sym)}"])
    assert np.array_equal(z.numpy(), g[f"zero_b{bits}_s{int(sym)}"])
    q = orc.quantize_codes(x, s, z, bits)
    assert np.array_equal(q.numpy(), g[f"q_b{bits}_s{int(sym)}"])
    assert np.array_equal(orc.dequantize_codes(q, s, z).numpy(), g[f"dq_b{bits}_s{int(sym)}"])


def test_find_params_mse_matches_reference():
    g = load_golden("find_params.npz")
    s, z = orc.find_params(torch.from_numpy(g["x"]), 4, False, mse=True, norm=2.4, grid=100)
    assert np.array_equal(s.numpy(), g["scale_mse"])
    assert np.array_equal(z.numpy(), g["zero_mse"])


def test_moments_match_reference():
    torch.set_num_threads(1)
    g = load_golden("moments.npz")
    xq, xf = f16(g["xq"]), f16(g["xf"])
    h, n = orc.hessian_running_mean(xq)
    assert n == int(g["n"])
    assert np.array_equal(h.numpy(), g["H"])
    assert np.array_equal(orc.delta_hatx_running_mean(xq, xf).numpy(), g["C_generic"])
    chunk = int(g["arch_chunk"])
    hq, cq, nq = orc.hessian_and_crossterm(xq.split(chunk), xf.split(chunk))
    assert nq == int(g["n_arch"])
    assert np.array_equal(hq.numpy(), g["H_arch"])
    assert np.array_equal(cq.numpy(), g["C_arch"])


def test_expert_rule_no_tokens():
    h, c, n = orc.hessian_and_crossterm([torch.zeros(0, 8).half(), torch.zeros(0, 8).half()])
    assert h is None and n == 0
    x = torch.randn(5, 8).half()
    h1, _, n1 = orc.hessian_and_crossterm([torch.zeros(0, 8).half(), x])
    h2, _ = orc.hessian_running_mean(x)
    assert n1 == 5 and torch.equal(h1, h2)


@pytest.mark.parametrize("name", gptq_case_names())
def test_gptq_matches_reference(name):
    torch.set_num_threads(1)
    g = load_golden(f"gptq_{name}.npz")
    w = f16(g["W"])
    bits, gs = int(g["wbits"]), int(g["groupsize"])
    r = orc.gptq_quantize(
        w, torch.from_numpy(g["H"].copy()), blocksize=int(g["blocksize"]), percdamp=0.01,
        wbits=bits, groupsize=gs, actorder=bool(g["actorder"]), sym=bool(g["sym"]),
        mse=bool(g.get("mse", 0)),
    )
    assert np.array_equal(r["u"].numpy(), g["U"])
    assert np.array_equal(r["qweight"].numpy(), g["codes"])
    assert np.array_equal(r["scales"].numpy().view(np.uint16), g["scales"])
    assert np.array_equal(r["qzeros"].numpy(), g["qzeros"])
    if bool(g["actorder"]):
        assert np.array_equal(r["perm"].numpy(), g["perm"])
    else:
        assert r["perm"] is None
    qw, qz = orc.pack_result(r["qweight"].numpy(), r["qzeros"].numpy(), bits)
    assert np.array_equal(qw, g["qweight_packed"])
    assert np.array_equal(qz, g["qzeros_packed"])
    deq = orc.dequantize_result(
        qw, r["scales"], qz, None if r["perm"] is None else r["perm"].numpy(), bits, gs, w.shape
    )
    assert np.array_equal(deq.numpy().view(np.uint16), g["dequantized"])


def test_qep_adjust_matches_reference():
    torch.set_num_threads(1)
    g = load_golden("qep_adjust.npz")
    w = f16(g["W"])
    h, c = torch.from_numpy(g["H"]), torch.from_numpy(g["C"])
    adj = orc.qep_adjust_weight(w, h, c, 0.01, 0.5)
    assert np.array_equal(adj.numpy().view(np.uint16), g["adjusted"])
    r = orc.gptq_quantize(adj, h.clone(), wbits=4, groupsize=128, sym=False)
    qw, qz = orc.pack_result(r["qweight"].numpy(), r["qzeros"].numpy(), 4)
    assert np.array_equal(qw, g["qweight_packed"])
    assert np.array_equal(qz, g["qzeros_packed"])
    assert np.array_equal(r["scales"].numpy().view(np.uint16), g["scales"])


def test_cholesky_retry_then_failure():
    h = -torch.eye(8)
    with pytest.raises(RuntimeError):
        orc.inverse_hessian_upper(h, 0.01)
    # a rank-deficient PSD matrix succeeds once damping is added
    v = torch.randn(8, 2)
    u = orc.inverse_hessian_upper(v @ v.t(), 0.01)
    assert torch.isfinite(u).all()


def test_group_index_rule():
    perm = np.array([3, 0, 2, 1, 5, 4, 7, 6])
    gi = orc.group_index(perm, 4, 8)
    assert gi.dtype == np.int32
    assert np.array_equal(gi, np.argsort(perm) // 4)
    assert np.array_equal(orc.group_index(None, 4, 8), np.arange(8) // 4)
    assert np.array_equal(orc.group_index(None, -1, 8), np.zeros(8))


@pytest.mark.parametrize("bits,gs,sym", [(4, 32, False), (4, 32, True), (3, -1, False), (2, 64, True)])
def test_rtn_matches_reference(bits, gs, sym):
    g = load_golden("rtn.npz")
    key = f"b{bits}_g{gs}_s{int(sym)}"
    r = orc.rtn_quantize(f16(g["W"]), bits, gs, sym)
    assert np.array_equal(r["quantized_weight"].numpy(), g[f"codes_{key}"])
    assert np.array_equal(r["scale"].numpy().view(np.uint16), g[f"scale_{key}"])
    assert np.array_equal(r["zero"].numpy().view(np.uint16), g[f"zero_{key}"])
    assert np.array_equal(r["dequantized_weight"].numpy().view(np.uint16), g[f"deq_{key}"])
    with pytest.raises(ValueError):
        orc.rtn_quantize(f16(g["W"]), 4, 48, False)


def test_bf16_module_matches_reference():
    """bfloat16 weights and activations: moments, correction written back in bf16, GPTQ and RTN."""
    from conftest import bf16, bits16

    torch.set_num_threads(1)
    g = load_golden("bf16.npz")
    w, xq, xf = bf16(g["W"]), bf16(g["xq"]), bf16(g["xf"])
    h, n = orc.hessian_running_mean(xq.unsqueeze(0))
    assert n == int(g["n"]) and np.array_equal(h.numpy(), g["H"])
    c = orc.delta_hatx_running_mean(xq.unsqueeze(0), xf.unsqueeze(0))
    assert np.array_equal(c.numpy(), g["C"])
    r = orc.gptq_quantize(w, h.clone(), wbits=4, groupsize=64, sym=False)
    assert np.array_equal(r["qweight"].numpy(), g["codes"])
    assert np.array_equal(r["scales"].numpy().view(np.uint16), g["scales"])
    assert np.array_equal(r["qzeros"].numpy(), g["qzeros"])
    adj = orc.qep_adjust_weight(w, h, c, 0.01, 0.5)
    assert adj.dtype == torch.bfloat16 and np.array_equal(bits16(adj), g["adjusted"])
    r2 = orc.gptq_quantize(adj, h.clone(), wbits=4, groupsize=64, sym=False)
    qw, qz = orc.pack_result(r2["qweight"].numpy(), r2["qzeros"].numpy(), 4)
    assert np.array_equal(qw, g["qep_qweight_packed"]) and np.array_equal(qz, g["qep_qzeros_packed"])
    assert np.array_equal(r2["scales"].numpy().view(np.uint16), g["qep_scales"])
    deq = orc.dequantize_result(qw, r2["scales"], qz, None, 4, 64, (32, 256))
    assert np.array_equal(bits16(deq), g["qep_dequantized"])
    assert np.array_equal(bits16(deq.to(torch.bfloat16)), g["qep_installed"])
    rt = orc.rtn_quantize(w, 4, 32, False)
    assert np.array_equal(rt["quantized_weight"].numpy(), g["rtn_codes"])
    assert rt["dequantized_weight"].dtype == torch.bfloat16 and int(g["rtn_deq_is_bf16"]) == 1
    assert np.array_equal(bits16(rt["dequantized_weight"]), g["rtn_deq"])
