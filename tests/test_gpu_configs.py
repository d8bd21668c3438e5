"""Parity on the benchmark configurations themselves (or their shapes): config 1 at full
size against the CPU oracle with the north-star tolerances, the MoE-expert shapes of
config 5 (d = 2880, group 32, skewed routing), and a two-GPU run of the sharded path."""

import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from conftest import ROOT
from oracle import gptq_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_config1_single_linear_full_size():
    """W 4096x4096 fp16 ~ N(0, 0.02^2); X 32 x 2048 x 4096 fp16 N(0,1) with 8 outlier channels x20;
    4-bit asymmetric, group 128, damp 0.01, block 128, no act-order."""
    from onecompression_b200 import GPTQ, synthetic

    torch.set_num_threads(max(1, os.cpu_count() or 1))
    w, x = synthetic.single_linear_case(seed=1, out=4096, d=4096, n_seq=32, seq=2048)
    lin = torch.nn.Linear(4096, 4096, bias=False).half()
    lin.weight.data = w.clone()
    lin = lin.to(DEV)
    q = GPTQ(wbits=4, groupsize=128, sym=False, percdamp=0.01, blocksize=128)
    q.module_to_name = {lin: "layer"}
    h, n = q.calculate_hessian(lin, x.to(DEV))
    res = q.quantize_layer(lin, None, hessian=h)

    h_ref, n_ref = orc.hessian_running_mean(x)
    assert n == n_ref == 65536
    rel_h = ((h.cpu().double() - h_ref.double()).norm() / h_ref.double().norm()).item()
    assert rel_h < 1e-5, rel_h                                   # H within 1e-5 relative Frobenius
    ref = orc.gptq_quantize(w, h_ref.clone(), blocksize=128, percdamp=0.01, wbits=4, groupsize=128, sym=False)

    codes = orc.unpack_qweight(res.qweight.numpy(), 4, (4096, 4096))
    same = (codes == ref["qweight"].numpy()).mean()
    assert same >= 0.999, same                                   # >= 99.9 % identical integer codes
    s = res.scales.numpy().view(np.uint16).astype(np.int64)
    sref = ref["scales"].numpy().view(np.uint16).astype(np.int64)
    # scales: one fp16 ulp is the 1e-3 relative bar; a group downstream of one of the rare
    # differing codes can move further, so the bar applies to 99.9 % of the scales
    assert (np.abs(s - sref) <= 1).mean() >= 0.999
    assert (s == sref).mean() > 0.99
    rel_s = np.abs(res.scales.float().numpy() - ref["scales"].float().numpy()) / ref["scales"].float().numpy()
    assert rel_s.max() < 0.05
    # packed layout is bit-exact for the codes and zeros it encodes
    zeros = (orc.unpack_qzeros(res.qzeros.numpy(), 4, 4096) + 1) & 15
    qw, qz = orc.pack_result(codes, zeros, 4)
    assert np.array_equal(qw, res.qweight.numpy()) and np.array_equal(qz, res.qzeros.numpy())
    # reconstruction error within 0.5 % of the reference's
    qw_r, qz_r = orc.pack_result(ref["qweight"].numpy(), ref["qzeros"].numpy(), 4)
    deq_ref = orc.dequantize_result(qw_r, ref["scales"], qz_r, None, 4, 128, (4096, 4096))
    e_ref = orc.reconstruction_error(w, deq_ref, h_ref, n)
    e_got = orc.reconstruction_error(w, res.compute_dequantized_weight(), h_ref, n)
    assert abs(e_got - e_ref) <= 0.005 * e_ref, (e_got, e_ref)


def test_config5_expert_shapes_group32():
    """GPT-OSS-20B expert shape: d = 2880 (22 blocks of 128 + one of 64), group 32 (groups that
    start inside a block are fitted on stale columns), Hessians from routed tokens only with
    skewed counts, one expert without tokens."""
    from onecompression_b200 import kernels as K

    g = torch.Generator().manual_seed(9)
    d, out = 2880, 256
    counts = [12000, 3000, 64, 0]
    w = (torch.randn(out, d, generator=g) * 0.02).half()
    for t in counts:
        chunks = [torch.randn(t // 2, d, generator=g).half(), torch.randn(t - t // 2, d, generator=g).half()]
        acc = K.MomentAccumulator(d, DEV)
        for c in chunks:
            if c.shape[0]:
                acc.add(c.to(DEV))
        h, _, n = acc.finalize()
        h_ref, _, n_ref = orc.hessian_and_crossterm(chunks)
        assert n == n_ref == t
        if t == 0:
            assert h_ref is None          # the driver skips (or RTN-quantizes) such an expert
            continue
        assert ((h.cpu().double() - h_ref.double()).norm() / h_ref.double().norm()).item() < 1e-5
        fac = K.factor_hessian(h, 0.01, False)
        got = K.gptq_quantize(w.to(DEV), fac, wbits=4, groupsize=32, sym=False, want_codes=True)
        ref = orc.gptq_quantize(w, h_ref.clone(), wbits=4, groupsize=32, sym=False)
        equal = got["codes"].cpu().numpy() == ref["qweight"].numpy()
        same = equal.mean()
        if t >= 4 * d:
            assert same >= 0.999, (t, same)
        elif t >= d:
            assert same >= 0.99, (t, same)      # barely determined Hessian: ill-conditioned on both sides
        else:
            # 64 tokens for 2880 columns: H is rank deficient, U rests on the damping alone and
            # both sides amplify rounding; agreement is looser there
            assert same >= 0.98, (t, same)
        s = got["scales"].cpu().numpy().view(np.uint16).astype(np.int64)
        sref = ref["scales"].numpy().view(np.uint16).astype(np.int64)
        close = np.abs(s - sref) <= 1
        assert close.mean() >= (0.999 if t >= 4 * d else 0.95)
        # groups fitted before their row's first differing code are untouched by code differences:
        # there the scales agree to one fp16 ulp whatever the conditioning
        first_bad = np.where(equal.all(axis=1), d, np.argmin(equal, axis=1))
        clean = (np.arange(close.shape[0])[:, None] * 32) <= first_bad[None, :]
        assert close[clean].mean() >= 0.999, (t, close[clean].mean())


def test_config4_qwen3_shapes_mixed_bits():
    """Qwen3-14B k_proj shape (1024 x 5120), group 128, one layer per candidate bit width of the
    mixed-precision configuration, against the oracle on the same Hessian."""
    from onecompression_b200 import kernels as K

    torch.set_num_threads(max(1, os.cpu_count() or 1))
    g = torch.Generator().manual_seed(4)
    d, out, n_seq, seq = 5120, 1024, 12, 2048
    w = (torch.randn(out, d, generator=g) * 0.02).half()
    x = torch.randn(n_seq, seq, d, generator=g).half()
    x[..., torch.randperm(d, generator=g)[:8]] *= 20
    acc = K.MomentAccumulator(d, DEV)
    for i in range(0, n_seq, 4):
        acc.add(x[i:i + 4].reshape(-1, d).to(DEV))
    h, _, n = acc.finalize()
    h_ref, n_ref = orc.hessian_running_mean(x)
    assert n == n_ref
    assert ((h.cpu().double() - h_ref.double()).norm() / h_ref.double().norm()).item() < 1e-5
    fac = K.factor_hessian(h, 0.01, False)
    for bits in (2, 3, 4):
        got = K.gptq_quantize(w.to(DEV), fac, wbits=bits, groupsize=128, sym=True, want_codes=True)
        ref = orc.gptq_quantize(w, h_ref.clone(), wbits=bits, groupsize=128, sym=True)
        equal = got["codes"].cpu().numpy() == ref["qweight"].numpy()
        assert equal.mean() >= 0.999, (bits, equal.mean())
        s = got["scales"].cpu().numpy().view(np.uint16).astype(np.int64)
        sref = ref["scales"].numpy().view(np.uint16).astype(np.int64)
        close = np.abs(s - sref) <= 1                               # [G, out], one fp16 ulp = 1e-3 relative
        # a differing code moves every later column of its row (at 2-3 bits by more than an ulp
        # of the group maximum), so the one-ulp bar is for groups fitted before the row's first
        # differing code; all groups together still agree almost everywhere
        first_bad = np.where(equal.all(axis=1), d, np.argmin(equal, axis=1))        # [out]
        clean = (np.arange(d // 128)[:, None] * 128) <= first_bad[None, :]
        assert close[clean].mean() >= 0.9995, (bits, close[clean].mean())
        assert close.mean() >= 0.99, (bits, close.mean())
        qw, qz = orc.pack_result(got["codes"].cpu().numpy(), got["zeros"].cpu().numpy().astype(np.int64), bits)
        assert np.array_equal(qw, got["qweight"].cpu().numpy()) and np.array_equal(qz, got["qzeros"].cpu().numpy())


def test_largest_layer_shape_properties():
    """Qwen3-14B down_proj (5120 x 17408, 136 column blocks): too large for the CPU oracle, so the
    checks are size-independent properties: the packed result decodes to exactly the propagated
    weight, codes stay in range, and the Hessian-weighted error is below round-to-nearest's."""
    from onecompression_b200 import kernels as K

    g = torch.Generator(device=DEV).manual_seed(7)
    d, out, tokens = 17408, 5120, 32768
    w = (torch.randn(out, d, generator=g, device=DEV) * 0.02).half()
    x = torch.randn(tokens, d, generator=g, device=DEV)
    x += torch.randn(tokens, 256, generator=g, device=DEV) @ torch.randn(256, d, generator=g, device=DEV) * 0.2
    x = x.half()           # correlated channels, so that error feedback has something to use
    x[:, ::2176] *= 10
    acc = K.MomentAccumulator(d, DEV)
    for i in range(0, tokens, 8192):
        acc.add(x[i:i + 8192])
    h, _, n = acc.finalize()
    assert n == tokens
    fac = K.factor_hessian(h, 0.01, False)
    got = K.gptq_quantize(w, fac, wbits=3, groupsize=128, sym=True, want_codes=True)
    codes = got["codes"]
    assert int(codes.min()) >= 0 and int(codes.max()) <= 7
    g_idx = (torch.arange(d, device=DEV) // 128).to(torch.int32)
    deq = K.dequantize_packed(got["qweight"], got["qzeros"], got["scales"], g_idx, 3, (out, d))
    assert torch.equal(deq, got["dequantized"])
    unpacked = K.unpack_qweight(got["qweight"], 3, (out, d))
    assert torch.equal(unpacked.to(codes.dtype), codes)
    rtn = K.rtn_quantize(w, 3, 128, True)["dequantized"]

    def weighted_error(w_hat):
        total = 0.0
        for r in range(0, out, 1024):
            dw = (w[r:r + 1024].float() - w_hat[r:r + 1024].float())
            total += float(((dw @ h) * dw).sum())
        return total

    e_gptq, e_rtn = weighted_error(got["dequantized"]), weighted_error(rtn)
    assert e_gptq < 0.95 * e_rtn, (e_gptq, e_rtn)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_sharded_run_matches_single_gpu(tmp_path):
    """Tokens and rows sharded over two ranks (NCCL) against the single-GPU result."""
    script = os.path.join(ROOT, "tests", "_two_gpu_worker.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29533", script, str(tmp_path)]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert (tmp_path / "ok").exists()
