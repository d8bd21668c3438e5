"""The widest layers of the benchmark configurations against the CPU oracle.

Llama-3-8B's down_proj has 14336 input channels (112 column blocks, 28 groups of four blocks) and
Qwen3-14B's 17408 (136 blocks).  Rows of W are independent given the Hessian (every step of
run_gptq, onecomp/quantizer/gptq/_gptq.py:720-765, is per row or a right-multiplication by U), so
the oracle quantizes a slab of rows against the full Hessian - one CPU Cholesky chain and a column
loop over a few hundred rows - and the same rows of the full-size GPU result are compared with it.

What can be asked at this width.  A row's codes are a chaotic function of the arithmetic over
14336 sequential columns: one differing code changes every later code of its row, so any two
correct fp32 computations that differ in the last bit somewhere (another BLAS, another summation
order in the trailing update, another factorisation) lose whole row tails.  99.9 % identical codes
is therefore not reachable by the reference against itself on such a layer, and the test measures
that instead of assuming it: the oracle is run again (a) with its own factor perturbed by one fp32
ulp per entry and (b) with the exactly rounded float64 factor, and its agreement with its first
run gives the floor for (a) the column loop alone and (b) factor + column loop.  Also, the damped
Hessian's condition number times the fp32 epsilon is about 1e-4 here: the reference's fp32 factor
is that far from the exact one, and so is this build's.  The bars:
  * U as close to the float64 factor as the reference's chain is (within a factor of two);
  * the column loop alone, fed the reference's U: code agreement no worse than floor (a) minus
    half a point, at least 99 %;
  * factor + column loop: code agreement no worse than floor (b) minus two points;
  * in both: fp16 scales within one ulp for every group fitted before its row's first differing
    code, packed layout bit-exact, and - the criterion that does not depend on positions - the
    slab's reconstruction error within 0.5 % of the reference's.
Covered: 3-bit symmetric (the headline configuration), 4-bit asymmetric with act-order
(configuration 2), and two bit widths of the mixed-precision configuration at Qwen3's width.
"""

import os

import numpy as np
import pytest
import torch

from oracle import gptq_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOKENS = 16384
SLAB = (1024, 1024 + 192)        # rows handed to the oracle

_cache = {}


def _problem(d, out):
    """Seeded W [out, d] and H from TOKENS tokens with outlier channels and correlated channels
    (so that error feedback and act-order have something to work with)."""
    if d not in _cache:
        _cache.clear()
        from onecompression_b200 import kernels as K

        g = torch.Generator(device=DEV).manual_seed(d)
        w = (torch.randn(out, d, generator=g, device=DEV) * 0.02).half()
        x = torch.randn(TOKENS, d, generator=g, device=DEV)
        x += torch.randn(TOKENS, 64, generator=g, device=DEV) @ torch.randn(64, d, generator=g, device=DEV) * 0.3
        x *= (0.5 + torch.rand(d, generator=g, device=DEV))          # distinct channel scales
        x[:, torch.randperm(d, generator=g, device=DEV)[:8]] *= 20
        x = x.half()
        acc = K.MomentAccumulator(d, DEV)
        for part in x.split(4096):
            acc.add(part)
        h, _, n = acc.finalize()
        assert n == TOKENS
        # independent check of the moment kernel at this width: float64 on the same device
        rows = slice(5000, 5256)
        want = (2.0 / TOKENS) * (x[:, rows].double().t() @ x.double())
        rel = ((h[rows].double() - want).norm() / want.norm()).item()
        assert rel < 1e-5, rel
        del x, want
        _cache[d] = (w, h, h.cpu())
    return _cache[d]


@pytest.mark.parametrize("d,out,bits,sym,actorder", [
    (14336, 4096, 3, True, False),
    (14336, 4096, 4, False, True),
    (17408, 5120, 4, True, False),
    (17408, 5120, 2, True, True),
])
def test_row_slab_of_a_wide_layer_matches_oracle(d, out, bits, sym, actorder):
    from onecompression_b200 import kernels as K

    torch.set_num_threads(max(1, os.cpu_count() or 1))
    w, h, h_cpu = _problem(d, out)
    fac = K.factor_hessian(h, 0.01, actorder)
    assert fac.attempts == 1
    got = K.gptq_quantize(w, fac, wbits=bits, groupsize=128, sym=sym, want_codes=True, want_scales_f32=True)
    r0, r1 = SLAB
    w_slab = w[r0:r1].cpu()
    perm = None
    if actorder:
        # Among this many fp32 diagonal entries a few are exactly equal, and torch.argsort (which the
        # reference uses, _gptq.py:699) is not stable: tied columns may come in either order.  The
        # order found here must be a descending sort too (the same key sequence); the oracle then
        # runs with this order so that codes are comparable position by position.
        diag = torch.diag(h_cpu)
        perm_ref = torch.argsort(diag, descending=True)
        perm = fac.perm.cpu().long()
        assert torch.equal(torch.sort(perm).values, torch.arange(d))
        assert torch.equal(diag[perm], diag[perm_ref])
        n_diff = int((perm != perm_ref).sum())
        print(f"[wide d={d}] {n_diff} positions of the column order differ from torch.argsort's (ties)")
        assert n_diff <= 64
    ref = orc.gptq_quantize(w_slab, h_cpu.clone(), blocksize=128, percdamp=0.01, wbits=bits, groupsize=128,
                            sym=sym, actorder=actorder, perm_override=perm)
    # The factor.  At this width fp32 rounding alone moves U by about 1e-4 (the damped Hessian's
    # condition number times the fp32 epsilon), so two fp32 computations agree with each other no
    # better than each agrees with the exact factor.  Reference point: the same chain in float64.
    a64 = h.double()
    idx = torch.arange(d, device=DEV)
    damp32 = torch.tensor(0.01, dtype=torch.float32, device=DEV) * torch.mean(torch.diag(h))
    a64[idx, idx] = (torch.diag(h) + damp32).double()           # the fp32 matrix both sides factor
    if actorder:
        pd = perm.to(DEV)
        a64 = a64[pd][:, pd]
    low = torch.linalg.cholesky(a64)
    del a64
    u64 = torch.linalg.cholesky(torch.cholesky_inverse(low), upper=True)
    del low
    nrm = u64.norm().item()
    err_got = ((fac.u.double() - u64).norm().item()) / nrm
    u_ref = ref["u"].to(DEV).double()
    err_ref = ((u_ref - u64).norm().item()) / nrm
    rel_u = ((fac.u.double() - u_ref).norm().item()) / u_ref.norm().item()
    u64_f32 = u64.float().cpu()
    del u64, u_ref
    torch.cuda.empty_cache()
    print(f"[wide d={d} act={actorder}] U against float64: this build {err_got:.2e}, reference chain {err_ref:.2e}; "
          f"against each other {rel_u:.2e}")
    assert err_got <= max(2e-5, 2.0 * err_ref), (err_got, err_ref)
    assert rel_u <= max(2e-5, 2.5 * max(err_got, err_ref)), rel_u
    # the reference's sensitivity (b) to its own factor's rounding: its column loop with the exactly
    # rounded factor against its column loop with its fp32 factor
    kw_o = dict(blocksize=128, percdamp=0.01, wbits=bits, groupsize=128, sym=sym, actorder=actorder,
                perm_override=perm)
    exact = orc.gptq_quantize(w_slab, h_cpu.clone(), u_override=u64_f32, **kw_o)
    floor_factor = (exact["qweight"].numpy() == ref["qweight"].numpy()).mean()
    del exact, u64_f32
    # ... and (a) to last-bit noise: its own factor with every entry moved by about one fp32 ulp
    gen = torch.Generator().manual_seed(d + bits)
    noisy = ref["u"] * (1 + 6e-8 * torch.randn(ref["u"].shape, generator=gen))
    jitter = orc.gptq_quantize(w_slab, h_cpu.clone(), u_override=noisy, **kw_o)
    floor_ulp = (jitter["qweight"].numpy() == ref["qweight"].numpy()).mean()
    del jitter, noisy
    # the column loop alone: this build's kernels with the reference's factor
    import copy

    fac_ref = copy.copy(fac)
    fac_ref.u = ref["u"].to(DEV).contiguous()
    alone = K.gptq_quantize(w[r0:r1].contiguous(), fac_ref, wbits=bits, groupsize=128, sym=sym, want_codes=True)
    eq_alone = alone["codes"].cpu().numpy() == ref["qweight"].numpy()
    s_alone = alone["scales"].cpu().numpy().view(np.uint16).astype(np.int64)
    sref = ref["scales"].numpy().view(np.uint16).astype(np.int64)
    close_alone = np.abs(s_alone - sref) <= 1
    print(f"[wide d={d} b{bits} act={actorder}] column loop with the reference's U: identical codes "
          f"{eq_alone.mean():.6f}; the reference against itself with one-ulp noise in U: {floor_ulp:.6f}")
    assert eq_alone.mean() >= max(0.99, floor_ulp - 0.005), (eq_alone.mean(), floor_ulp)
    if not actorder:
        first_bad = np.where(eq_alone.all(axis=1), d, np.argmin(eq_alone, axis=1))
        clean = (np.arange(d // 128)[:, None] * 128) <= first_bad[None, :]
        assert close_alone[clean].mean() >= 0.9999, close_alone[clean].mean()
    del alone, fac_ref
    # codes of the slab
    codes = got["codes"][r0:r1].cpu().numpy()
    equal = codes == ref["qweight"].numpy()
    print(f"[wide d={d} b{bits} act={actorder}] factor + column loop: identical codes {equal.mean():.6f}; "
          f"the reference against itself with an exactly rounded factor: {floor_factor:.6f}")
    assert equal.mean() >= floor_factor - 0.02 and equal.mean() >= 0.93, (equal.mean(), floor_factor)
    # scales: one fp16 ulp (the 1e-3 relative bar) for every group fitted before its row's first
    # differing code
    s = got["scales"][:, r0:r1].cpu().numpy().view(np.uint16).astype(np.int64)
    close = np.abs(s - sref) <= 1
    if not actorder:
        first_bad = np.where(equal.all(axis=1), d, np.argmin(equal, axis=1))
        clean = (np.arange(d // 128)[:, None] * 128) <= first_bad[None, :]
        assert close[clean].mean() >= 0.999, close[clean].mean()
    # packed layout is bit-exact for the codes and zero points it encodes
    zeros = got["zeros"][:, r0:r1].cpu().numpy().astype(np.int64)
    qw, qz = orc.pack_result(codes, zeros, bits)
    assert np.array_equal(qw, got["qweight"][:, r0:r1].cpu().numpy())
    assert np.array_equal(qz, got["qzeros"][:, r0 * bits // 32:r1 * bits // 32].cpu().numpy())
    # reconstruction error of the slab within 0.5 % of the reference's
    perm_np = perm.numpy() if actorder else None
    qw_r, qz_r = orc.pack_result(ref["qweight"].numpy(), ref["qzeros"].numpy(), bits)
    deq_ref = orc.dequantize_result(qw_r, ref["scales"], qz_r, perm_np, bits, 128, w_slab.shape)
    e_ref = orc.reconstruction_error(w_slab, deq_ref, h_cpu, TOKENS)
    e_got = orc.reconstruction_error(w_slab, got["dequantized"][r0:r1].cpu(), h_cpu, TOKENS)
    assert abs(e_got - e_ref) <= 0.005 * e_ref, (e_got, e_ref)
    print(f"[wide d={d} b{bits} act={actorder}] scales within one ulp {close.mean():.6f}, "
          f"reconstruction error {e_got:.5e} vs {e_ref:.5e} ({(e_got - e_ref) / e_ref:+.3%})")
