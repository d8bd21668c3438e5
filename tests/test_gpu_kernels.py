"""GPU parity tests of the individual kernels against the CPU oracle and the golden
vectors produced by the reference.  Every call goes through the C ABI."""

import numpy as np
import pytest
import torch

from conftest import f16, gptq_case_names, load_golden
from oracle import gptq_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from onecompression_b200 import kernels

    return kernels


def dev():
    return torch.device("cuda:0")


# ---- fp32 GEMM engine ------------------------------------------------------------

@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (300, 260, 77), (64, 1000, 130), (513, 129, 16)])
def test_gemm_matches_torch_fp32(K, ta, tb, m, n, k):
    g = torch.Generator().manual_seed(m * 7 + n * 3 + k)
    a = torch.randn((k, m) if ta else (m, k), generator=g)
    b = torch.randn((n, k) if tb else (k, n), generator=g)
    c0 = torch.randn(m, n, generator=g)
    want = 0.5 * c0.double() - 1.5 * ((a.t() if ta else a).double() @ (b.t() if tb else b).double())
    c = c0.clone().to(dev())
    K.gemm_f32(a.to(dev()), b.to(dev()), c, alpha=-1.5, beta=0.5, trans_a=ta, trans_b=tb)
    got = c.cpu().double()
    assert ((got - want).norm() / want.norm()).item() < 2e-6


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("m,n,k", [(256, 384, 512), (1000, 520, 260), (128, 128, 32), (72, 4096, 128), (640, 200, 1028)])
def test_gemm_tensor_core_engine(K, ta, tb, m, n, k):
    """3xTF32 engine (aligned operands) against float64 and against the FMA engine."""
    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randn((k, m) if ta else (m, k), generator=g)
    b = torch.randn((n, k) if tb else (k, n), generator=g)
    c0 = torch.randn(m, n, generator=g)
    want = 0.25 * c0.double() + 2.0 * ((a.t() if ta else a).double() @ (b.t() if tb else b).double())
    ad, bd = a.to(dev()), b.to(dev())
    assert K.set_gemm_engine(0) in (0, 1)
    c_tc = K.gemm_f32(ad, bd, c0.clone().to(dev()), alpha=2.0, beta=0.25, trans_a=ta, trans_b=tb).cpu()
    K.set_gemm_engine(1)
    try:
        c_fma = K.gemm_f32(ad, bd, c0.clone().to(dev()), alpha=2.0, beta=0.25, trans_a=ta, trans_b=tb).cpu()
    finally:
        K.set_gemm_engine(0)
    assert K.gemm_tc_status() == 0
    e_tc = ((c_tc.double() - want).norm() / want.norm()).item()
    e_fma = ((c_fma.double() - want).norm() / want.norm()).item()
    assert e_fma < 1e-6
    assert e_tc < 2e-6, (e_tc, e_fma)


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("m,n,k", [(256, 512, 96), (200, 300, 72), (128, 256, 16), (384, 1000, 520), (4096, 2560, 264), (300, 200, 64), (64, 136, 24)])
def test_gemm_tile_shapes_give_the_same_bits(K, ta, tb, m, n, k):
    """128 x 128 and 128 x 256 output tiles cut k into the same accumulation chains, so a plain
    product does not depend on the shape the engine picks (which depends on M, i.e. on how many
    rows a rank holds); the last size lets the engine choose wide tiles by itself."""
    g = torch.Generator().manual_seed(m + 3 * n + 7 * k)
    a = torch.randn((k, m) if ta else (m, k), generator=g).to(dev())
    b = torch.randn((n, k) if tb else (k, n), generator=g).to(dev())
    c0 = torch.randn(m, n, generator=g).to(dev())
    want = 0.5 * c0.double() + 1.5 * ((a.t() if ta else a).double() @ (b.t() if tb else b).double())
    out = {}
    try:
        for shape in (1, 2, 0):
            K.set_gemm_tile_shape(shape)
            out[shape] = K.gemm_f32(a, b, c0.clone(), alpha=1.5, beta=0.5, trans_a=ta, trans_b=tb)
    finally:
        K.set_gemm_tile_shape(0)
    assert K.gemm_tc_status() == 0
    assert torch.equal(out[1], out[2]) and torch.equal(out[1], out[0])
    assert ((out[2].double() - want).norm() / want.norm()).item() < 2e-6


@pytest.mark.parametrize("n,k", [(1024, 160), (1152, 512), (640, 48)])
def test_gemm_lower_tiles_only_with_wide_tiles(K, n, k):
    """Symmetric rank-k update that skips the 128 x 128 tiles above the diagonal (flag 1): a wide
    tile that straddles the diagonal computes and writes only its lower 128 columns, so the result
    and the untouched tiles are those of the narrow shape, bit for bit."""
    g = torch.Generator().manual_seed(n + k)
    p = torch.randn(n, k, generator=g).to(dev())
    c0 = torch.randn(n, n, generator=g).to(dev())
    out = {}
    try:
        for shape in (1, 2):
            K.set_gemm_tile_shape(shape)
            out[shape] = K.gemm_f32(p, p, c0.clone(), alpha=-1.0, beta=1.0, trans_b=True, flags=1)
    finally:
        K.set_gemm_tile_shape(0)
    assert K.gemm_tc_status() == 0
    assert torch.equal(out[1], out[2])
    want = c0.double() - p.double() @ p.double().t()
    low = torch.tril(torch.ones(n, n, device=dev(), dtype=torch.bool))
    assert ((out[2].double() - want)[low].norm() / want[low].norm()).item() < 2e-6
    # tiles strictly above the diagonal were skipped: C is unchanged there
    blk = torch.arange(n, device=dev()) // 128
    above = blk[None, :] > blk[:, None]
    assert torch.equal(out[2][above], c0[above])


@pytest.mark.parametrize("flag", [2, 8, 4, 16])
def test_gemm_triangular_ranges_with_wide_tiles(K, flag):
    """The k-range flags with 128 x 256 tiles: a wide tile runs the union of its halves' ranges, i.e.
    a few more exact zeros of the triangular operand, and gives the bits of the narrow shape."""
    g = torch.Generator().manual_seed(flag)
    n, m = 1152, 520
    tri = torch.randn(n, n, generator=g)
    tri = torch.tril(tri) if flag in (2, 4) else torch.triu(tri)
    other = torch.randn(m, n, generator=g)
    if flag in (2, 8):                       # B triangular: C = other @ tri
        a, b, want = other, tri, other.double() @ tri.double()
    else:                                    # A triangular: C = tri @ other^T
        a, b, want = tri, other.t().contiguous(), tri.double() @ other.double().t()
    out = {}
    try:
        for shape in (1, 2):
            K.set_gemm_tile_shape(shape)
            out[shape] = K.gemm_f32(a.to(dev()), b.to(dev()), flags=flag)
    finally:
        K.set_gemm_tile_shape(0)
    assert K.gemm_tc_status() == 0
    assert torch.equal(out[1], out[2])
    assert ((out[2].cpu().double() - want).norm() / want.norm()).item() < 2e-6


def test_gemm_tensor_core_long_k_same_sign(K):
    """All-positive operands and K = 8192: the chunked drain keeps the truncation bias of the
    tensor-core accumulator out of the result."""
    g = torch.Generator().manual_seed(1)
    a = torch.rand(256, 8192, generator=g) + 0.5
    b = torch.rand(8192, 256, generator=g) + 0.5
    want = a.double() @ b.double()
    got = K.gemm_f32(a.to(dev()), b.to(dev())).cpu().double()
    rel = ((got - want).abs() / want).max().item()
    assert rel < 5e-6, rel


def test_gemm_triangular_flags(K):
    g = torch.Generator().manual_seed(5)
    n = 384
    low = torch.tril(torch.randn(n, n, generator=g))
    up = torch.triu(torch.randn(n, n, generator=g))
    a = torch.randn(200, n, generator=g)
    # B lower triangular: k range starts at the tile's first column (flag 2)
    got = K.gemm_f32(a.to(dev()), low.to(dev()), flags=2).cpu()
    assert torch.allclose(got, a @ low, rtol=1e-4, atol=1e-4)
    # B upper triangular: k range ends at the tile's last column (flag 8)
    got = K.gemm_f32(a.to(dev()), up.to(dev()), flags=8).cpu()
    assert torch.allclose(got, a @ up, rtol=1e-4, atol=1e-4)
    # A lower triangular (flag 4)
    b = torch.randn(n, 150, generator=g)
    got = K.gemm_f32(low.to(dev()), b.to(dev()), flags=4).cpu()
    assert torch.allclose(got, low @ b, rtol=1e-4, atol=1e-4)
    # symmetric rank-k update, lower tiles only (flag 1)
    p = torch.randn(n, 96, generator=g)
    c = torch.zeros(n, n).to(dev())
    K.gemm_f32(p.to(dev()), p.to(dev()), c, trans_b=True, flags=1)
    want = p @ p.t()
    assert torch.allclose(torch.tril(c.cpu()), torch.tril(want), rtol=1e-4, atol=1e-4)


# ---- packing -------------------------------------------------------------------------

@pytest.mark.parametrize("bits", [2, 3, 4, 8])
def test_pack_matches_reference_vectors(K, bits):
    g = load_golden("pack.npz")
    codes = torch.from_numpy(g[f"codes{bits}"]).to(dev())
    zeros = torch.from_numpy(g[f"zeros{bits}"]).to(dev())
    qw = K.pack_qweight(codes, bits)
    assert np.array_equal(qw.cpu().numpy(), g[f"qweight{bits}"])
    qz = K.pack_qzeros(zeros, bits, add=-1)
    assert np.array_equal(qz.cpu().numpy(), g[f"qzeros{bits}"])
    assert torch.equal(K.unpack_qweight(qw, bits, codes.shape), codes)
    assert torch.equal(K.unpack_qzeros(qz, bits, zeros.shape[1], add=1), zeros)


def test_pack_rejects_unaligned(K):
    with pytest.raises(AssertionError):
        K.pack_qweight(torch.zeros(8, 7, dtype=torch.int32, device=dev()), 4)
    with pytest.raises(AssertionError):
        K.pack_qweight(torch.zeros(8, 16, dtype=torch.int32, device=dev()), 3)


# ---- second moments --------------------------------------------------------------------

def _rel(a, b):
    a, b = a.double(), b.double()
    return ((a - b).norm() / b.norm()).item()


@pytest.mark.parametrize("simt", [True, False])
def test_moments_match_reference_vectors(K, simt):
    g = load_golden("moments.npz")
    xq, xf = f16(g["xq"]).to(dev()), f16(g["xf"]).to(dev())
    acc = K.MomentAccumulator(64, dev(), cross=True, force_simt=simt)
    chunk = int(g["arch_chunk"])
    for a, b in zip(xq.split(chunk), xf.split(chunk)):
        acc.add(a, b)
    h, c, n = acc.finalize()
    assert n == int(g["n_arch"])
    assert _rel(h.cpu(), torch.from_numpy(g["H_arch"])) < 1e-5   # north-star tolerance for H
    assert _rel(c.cpu(), torch.from_numpy(g["C_arch"])) < 1e-4
    h2, n2 = K.hessian_from_activations(xq, force_simt=simt)
    assert n2 == int(g["n"]) and _rel(h2.cpu(), torch.from_numpy(g["H"])) < 1e-5
    assert torch.equal(h2, h2.t())


@pytest.mark.parametrize("engine", ["single", "pair"])
@pytest.mark.parametrize("d,ntok,chunk", [(512, 8192, 0), (2880, 4096, 1024), (1000, 3000, 0), (264, 100, 0)])
def test_hessian_tensor_core_vs_float64(K, d, ntok, chunk, engine):
    g = torch.Generator().manual_seed(d)
    x = torch.randn(ntok, d, generator=g)
    x[:, torch.randperm(d, generator=g)[:8]] *= 20
    x = x.half()
    want = (2.0 / ntok) * (x.double().t() @ x.double())
    acc = K.MomentAccumulator(d, dev(), chunk_tokens=chunk, engine=engine)
    for part in x.to(dev()).split(ntok // 2 + 7):
        acc.add(part)
    h, _, n = acc.finalize()
    assert n == ntok
    assert _rel(h.cpu(), want) < 1e-5
    assert torch.equal(h, h.t())


def test_pair_engine_equals_single_engine_bit_for_bit(K):
    """Both tensor-core engines add the same products in the same order (512-token chains, fp32
    sums of the chains), so their results are identical."""
    g = torch.Generator().manual_seed(11)
    d, ntok = 1536, 5000
    xf = torch.randn(ntok, d, generator=g).half().to(dev())
    xq = (xf.float() * 1.01).half()
    out = {}
    for engine in ("single", "pair"):
        acc = K.MomentAccumulator(d, dev(), cross=True, engine=engine)
        for a, b in zip(xq.split(2048), xf.split(2048)):
            acc.add(a, b)
        out[engine] = acc.finalize()
    assert torch.equal(out["single"][0], out["pair"][0]) and torch.equal(out["single"][1], out["pair"][1])


@pytest.mark.parametrize("engine", ["single", "pair"])
def test_cross_term_tensor_core_vs_float64(K, engine):
    g = torch.Generator().manual_seed(3)
    d, ntok = 768, 4096
    xf = torch.randn(ntok, d, generator=g).half()
    xq = (xf.float() * (1 + 0.03 * torch.randn(ntok, d, generator=g))).half()
    want_c = (2.0 / ntok) * ((xf.double() - xq.double()).t() @ xq.double())
    want_h = (2.0 / ntok) * (xq.double().t() @ xq.double())
    acc = K.MomentAccumulator(d, dev(), cross=True, engine=engine)
    acc.add(xq.to(dev()), xf.to(dev()))
    h, c, _ = acc.finalize()
    assert _rel(h.cpu(), want_h) < 1e-5
    assert _rel(c.cpu(), want_c) < 1e-4


@pytest.mark.parametrize("engine", ["single", "pair", "simt"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_cross_term_when_the_activations_have_drifted_apart(K, engine, dtype):
    """After many quantized blocks Xq is no small perturbation of Xf: half the magnitude off, signs
    flipped, tiny entries next to large ones.  fp16(Xf - Xq) alone then carries 2^-11 relative
    error per element; the kernel carries the difference as two 16-bit terms, so C still meets the
    bar of H (1e-5 relative Frobenius against float64) for fp16.  bf16 has 8-bit terms: two of
    them hold 16 bits, which bounds the error at 2^-17 per element."""
    g = torch.Generator().manual_seed(17)
    d, ntok = 640, 6000
    xf = torch.randn(ntok, d, generator=g)
    xf[:, 100:164] *= 1e-3                                   # a block of tiny entries
    xf[:, 7] *= 30                                           # an outlier channel
    xq = xf * (1 + 0.5 * torch.randn(ntok, d, generator=g))
    flip = torch.rand(ntok, d, generator=g) < 0.1
    xq = torch.where(flip, -xq, xq)
    xf, xq = xf.to(dtype), xq.to(dtype)
    want_c = (2.0 / ntok) * ((xf.double() - xq.double()).t() @ xq.double())
    want_h = (2.0 / ntok) * (xq.double().t() @ xq.double())
    acc = K.MomentAccumulator(d, dev(), cross=True, engine=engine)
    for a, b in zip(xq.to(dev()).split(2500), xf.to(dev()).split(2500)):
        acc.add(a, b)
    h, c, n = acc.finalize()
    assert n == ntok
    assert _rel(h.cpu(), want_h) < 1e-5
    bar = 1e-5 if dtype == torch.float16 else 3e-5
    assert _rel(c.cpu(), want_c) < bar, _rel(c.cpu(), want_c)
    # C is dominated by its diagonal here (Xf - Xq correlates with Xq), which hides rounding errors
    # of the difference in a whole-matrix norm; the off-diagonal entries show them.  One 16-bit term
    # leaves 2e-4 (fp16) / 2e-3 (bf16) there, two terms leave the accumulation error only.
    off = ~torch.eye(d, dtype=torch.bool)
    one_term = (2.0 / ntok) * ((xf.float() - xq.float()).to(dtype).double().t() @ xq.double())
    e_one = _rel(one_term[off], want_c[off])
    e_two = _rel(c.cpu().double()[off], want_c[off])
    print(f"[cross {engine} {dtype}] off-diagonal error: two terms {e_two:.2e}, one term would leave {e_one:.2e}")
    assert e_one > 1e-4
    assert e_two < 0.1 * e_one and e_two < 3e-5, (e_two, e_one)


@pytest.mark.parametrize("cross", [False, True])
def test_moments_from_strided_activations(K, cross):
    """Column slices of a wider buffer (row stride 2d) and differently strided Xf / Xq: the result is
    that of contiguous copies, and nothing beyond the slices is read or written (canaries)."""
    g = torch.Generator().manual_seed(23)
    d, ntok = 256, 3000
    big_q = torch.randn(ntok, 2 * d, generator=g).half().to(dev())
    big_f = (big_q.float() * (1 + 0.05 * torch.randn(ntok, 2 * d, generator=g).to(dev()))).half()
    xq = big_q[:, :d]                      # stride 2d, kept as a view by the accumulator
    xf = big_f[:, d:]                      # stride 2d at a column offset
    xf_c = xf.contiguous()                 # stride d: differs from xq's
    guard = big_q[:, d:].clone()
    want = K.MomentAccumulator(d, dev(), cross=cross)
    want.add(xq.contiguous(), xf_c if cross else None)
    h0, c0, _ = want.finalize()
    for xf_in in ((xf, xf_c) if cross else (None,)):
        acc = K.MomentAccumulator(d, dev(), cross=cross)
        acc.add(xq, xf_in)
        h, c, n = acc.finalize()
        assert n == ntok and torch.equal(h, h0)
        if cross:
            assert torch.equal(c, c0)
    assert torch.equal(big_q[:, d:], guard)
    ref_h = (2.0 / ntok) * (xq.double().t() @ xq.double())
    assert _rel(h0.cpu(), ref_h.cpu()) < 1e-5
    if cross:
        ref_c = (2.0 / ntok) * ((xf.double() - xq.double()).t() @ xq.double())
        assert _rel(c0.cpu(), ref_c.cpu()) < 1e-5


# ---- inverse-Hessian factor ---------------------------------------------------------------

@pytest.mark.parametrize("name", gptq_case_names())
def test_factor_matches_reference_u(K, name):
    g = load_golden(f"gptq_{name}.npz")
    h = torch.from_numpy(g["H"]).to(dev())
    fac = K.factor_hessian(h, 0.01, bool(g["actorder"]))
    assert fac.attempts == 1
    if bool(g["actorder"]):
        assert np.array_equal(fac.perm.cpu().numpy().astype(np.int64), g["perm"])
    assert _rel(fac.u.cpu(), torch.from_numpy(g["U"])) < 2e-5
    assert torch.equal(fac.u, torch.triu(fac.u))


@pytest.mark.parametrize("n", [100, 129, 300, 1024])
def test_factor_identity_property(K, n):
    g = torch.Generator().manual_seed(n)
    x = torch.randn(4 * n, n, generator=g)
    h = (2.0 / (4 * n)) * (x.t() @ x)
    fac = K.factor_hessian(h.to(dev()), 0.01, actorder=True)
    u = fac.u.cpu().double()
    p = fac.perm.cpu().long()
    hp = h.double()[p][:, p] + float(fac.damp[0].item()) * torch.eye(n, dtype=torch.float64)
    ident = u @ hp @ u.t()          # U Hp U^T = I  when U^T U = Hp^-1
    assert (ident - torch.eye(n, dtype=torch.float64)).abs().max().item() < 5e-4


def test_factor_retries_and_fails_like_reference(K):
    h = -torch.eye(64)
    with pytest.raises(RuntimeError, match="Cholesky decomposition failed after 5"):
        K.factor_hessian(h.to(dev()), 0.01, False)
    # PSD but rank deficient: the first damping already repairs it
    v = torch.randn(64, 3)
    fac = K.factor_hessian((v @ v.t()).to(dev()), 0.01, False)
    assert fac.attempts == 1 and torch.isfinite(fac.u).all()
    # indefinite: needs the escalating retries; diag mean 1 -> damp .01; total after k fails 0.01*(1+10+100..)
    m = torch.eye(64)
    m[0, 0] = -0.5
    m[1, 1] = 2.5 - 0.0     # keeps the mean of the diagonal at about 1
    fac = K.factor_hessian(m.to(dev()), 0.01, False)
    assert fac.attempts == 3        # 0.01, 0.11 fail; 1.11 > 0.5 works


# ---- column loop --------------------------------------------------------------------------------

def _run_case(K, g, use_reference_u):
    w = f16(g["W"]).to(dev())
    bits, gs = int(g["wbits"]), int(g["groupsize"])
    act = bool(g["actorder"])
    h = torch.from_numpy(g["H"]).to(dev())
    fac = K.factor_hessian(h, 0.01, act)
    if use_reference_u:
        fac.u = torch.from_numpy(g["U"]).to(dev()).contiguous()
        if act:
            perm = torch.from_numpy(g["perm"]).to(dev())
            fac.perm = perm.to(torch.int32)
            fac.invperm = torch.argsort(perm).to(torch.int32)
    return K.gptq_quantize(
        w, fac, wbits=bits, groupsize=gs, sym=bool(g["sym"]), blocksize=int(g["blocksize"]),
        pack=True, want_codes=True, want_dequantized=True, want_scales_f32=True,
        mse=bool(g.get("mse", 0)),
    ), fac


@pytest.mark.parametrize("name", gptq_case_names())
def test_column_loop_with_reference_factor(K, name):
    """Same U as the reference: codes, zeros and fp16 scales must agree almost everywhere
    (the trailing fp32 GEMM sums in another order than the reference's BLAS)."""
    g = load_golden(f"gptq_{name}.npz")
    out, _ = _run_case(K, g, use_reference_u=True)
    bits, gs = int(g["wbits"]), int(g["groupsize"])
    codes = out["codes"].cpu().numpy()
    same = (codes == g["codes"]).mean()
    assert same >= 0.999, f"{same:.5f} identical codes"
    zeros = out["zeros"].cpu().numpy()
    zref = g["qzeros"] if gs != -1 else g["qzeros"].reshape(1, -1)
    assert (zeros == zref).mean() >= 0.999
    s = out["scales"].cpu().numpy().view(np.uint16).astype(np.int64)
    sref = (g["scales"] if gs != -1 else g["scales"].reshape(1, -1)).astype(np.int64)
    assert (np.abs(s - sref) <= 1).all(), "fp16 scales differ by more than one ulp"
    if same == 1.0 and (zeros == zref).all() and (s == sref).all():
        assert np.array_equal(out["qweight"].cpu().numpy(), g["qweight_packed"])
        assert np.array_equal(out["qzeros"].cpu().numpy(), g["qzeros_packed"])
        assert np.array_equal(out["dequantized"].cpu().numpy().view(np.uint16), g["dequantized"])


@pytest.mark.parametrize("name", gptq_case_names())
def test_full_layer_against_reference(K, name):
    """Own factor + column loop: north-star tolerances (codes >= 99.9 %, scales 1e-3 before
    the fp16 cast i.e. <= 1 fp16 ulp after it, reconstruction error within 0.5 %)."""
    g = load_golden(f"gptq_{name}.npz")
    out, fac = _run_case(K, g, use_reference_u=False)
    bits, gs = int(g["wbits"]), int(g["groupsize"])
    if bool(g["actorder"]):
        assert np.array_equal(fac.perm.cpu().numpy().astype(np.int64), g["perm"])
    codes = out["codes"].cpu().numpy()
    assert (codes == g["codes"]).mean() >= 0.999
    s = out["scales"].cpu().numpy().view(np.uint16).astype(np.int64)
    sref = (g["scales"] if gs != -1 else g["scales"].reshape(1, -1)).astype(np.int64)
    assert (np.abs(s - sref) <= 1).all()
    # packed tensors are self-consistent with the codes (bit-exact layout)
    qw, qz = orc.pack_result(codes, out["zeros"].cpu().numpy(), bits)
    assert np.array_equal(out["qweight"].cpu().numpy(), qw)
    assert np.array_equal(out["qzeros"].cpu().numpy(), qz)
    # dequantised weight equals the reference formula applied to our own result
    perm = fac.perm.cpu().numpy().astype(np.int64) if bool(g["actorder"]) else None
    sc = out["scales"].cpu() if gs != -1 else out["scales"].cpu().reshape(-1, 1)
    deq = orc.dequantize_result(qw, sc, qz, perm, bits, gs, codes.shape)
    assert np.array_equal(out["dequantized"].cpu().numpy().view(np.uint16), deq.numpy().view(np.uint16))
    # reconstruction error within 0.5 % of the reference's
    w = f16(g["W"])
    h = torch.from_numpy(g["H"])
    e_ref = orc.reconstruction_error(w, f16(g["dequantized"]), h, int(g["n"]))
    e_got = orc.reconstruction_error(w, out["dequantized"].cpu(), h, int(g["n"]))
    assert abs(e_got - e_ref) <= 0.005 * e_ref


def test_unpacked_bit_widths(K):
    """wbits without a packed layout (here 5) still quantize; packing is refused."""
    g = load_golden("gptq_b4_g128_asym.npz")
    w = f16(g["W"]).to(dev())
    fac = K.factor_hessian(torch.from_numpy(g["H"]).to(dev()), 0.01, False)
    out = K.gptq_quantize(w, fac, wbits=5, groupsize=128, sym=False, pack=False, want_codes=True)
    ref = orc.gptq_quantize(f16(g["W"]), torch.from_numpy(g["H"].copy()), wbits=5, groupsize=128, sym=False)
    assert (out["codes"].cpu().numpy() == ref["qweight"].numpy()).mean() >= 0.999
    with pytest.raises(ValueError):
        K.gptq_quantize(w, fac, wbits=5, groupsize=128, sym=False, pack=True)


# ---- QEP correction ---------------------------------------------------------------------------------

def test_qep_adjust_matches_reference(K):
    g = load_golden("qep_adjust.npz")
    w = f16(g["W"]).to(dev()).contiguous()
    h, c = torch.from_numpy(g["H"]).to(dev()), torch.from_numpy(g["C"]).to(dev())
    for act in (False, True):
        fac = K.factor_hessian(h, 0.01, act)
        wa = w.clone()
        K.qep_adjust(wa, c, fac, 0.5)
        got = wa.cpu().numpy().view(np.uint16).astype(np.int64)
        want = g["adjusted"].astype(np.int64)
        assert (got == want).mean() >= 0.995          # fp16 rounding boundaries
        assert np.abs(got - want).max() <= 1          # never more than one fp16 ulp


# ---- RTN fallback -------------------------------------------------------------------------------------

@pytest.mark.parametrize("bits,gs,sym", [(4, 32, False), (4, 32, True), (3, -1, False), (2, 64, True)])
def test_rtn_matches_reference_vectors(K, bits, gs, sym):
    g = load_golden("rtn.npz")
    key = f"b{bits}_g{gs}_s{int(sym)}"
    r = K.rtn_quantize(f16(g["W"]).to(dev()), bits, gs, sym)
    assert np.array_equal(r["codes"].cpu().numpy(), g[f"codes_{key}"])
    assert np.array_equal(r["scales"].half().cpu().numpy().view(np.uint16), g[f"scale_{key}"])
    assert np.array_equal(r["zeros"].half().cpu().numpy().view(np.uint16), g[f"zero_{key}"])
    assert np.array_equal(r["dequantized"].cpu().numpy().view(np.uint16), g[f"deq_{key}"])
    with pytest.raises(ValueError):
        K.rtn_quantize(f16(g["W"]).to(dev()), 4, 48, False)


# ---- fused RMSNorm of the block passes ------------------------------------------------------------------

@pytest.mark.parametrize("rows,d", [(64, 4096), (33, 2880), (5, 100)])
def test_rmsnorm_matches_module_formula(K, rows, d):
    from transformers.models.llama.modeling_llama import LlamaRMSNorm

    g = torch.Generator().manual_seed(d)
    x = (torch.randn(rows, d, generator=g) * 3).half().to(dev())
    mod = LlamaRMSNorm(d, eps=1e-5).half().to(dev())
    mod.weight.data = (1 + 0.1 * torch.randn(d, generator=g)).half().to(dev())
    with torch.no_grad():
        want = mod(x)
        got = K.rmsnorm_f16(x, mod.weight.data, mod.variance_epsilon)
    a = got.cpu().numpy().view(np.uint16).astype(np.int64)
    b = want.cpu().numpy().view(np.uint16).astype(np.int64)
    assert np.abs(a - b).max() <= 1                 # same rounding points; the row sum is ordered differently
    assert (a == b).mean() > 0.999


# ---- fused rotary embedding and SwiGLU of the block passes -------------------------------------------------

@pytest.mark.parametrize("b,h,s,d,bcast", [(3, 8, 64, 128, True), (2, 4, 33, 64, False), (1, 2, 7, 32, True)])
def test_rope_is_bit_identical_to_the_model_code(K, b, h, s, d, bcast):
    from transformers.models.llama.modeling_llama import apply_rotary_pos_emb

    g = torch.Generator().manual_seed(b * 100 + d)
    proj = (torch.randn(b, s, h * d, generator=g) * 2).half().to(dev())
    q = proj.view(b, s, h, d).transpose(1, 2)                       # the layout attention code produces
    ang = torch.rand(1 if bcast else b, s, d, generator=g) * 6.28
    cos, sin = ang.cos().half().to(dev()), ang.sin().half().to(dev())
    want, _ = apply_rotary_pos_emb(q, q, cos, sin)
    assert K.rope_supported(q, cos, sin)
    got = K.rope_f16(q, cos, sin)
    assert got.stride() == want.stride() == q.stride()
    assert torch.equal(got, want)
    qc = q.contiguous()                                             # a different memory order
    assert torch.equal(K.rope_f16(qc, cos, sin), want)
    assert not K.rope_supported(q.float(), cos, sin) and not K.rope_supported(q[..., :24], cos[..., :24], sin[..., :24])


@pytest.mark.parametrize("shape", [(4, 64, 1024), (3, 5, 250), (1, 1, 7)])
def test_swiglu_is_bit_identical_to_the_model_code(K, shape):
    g = torch.Generator().manual_seed(shape[-1])
    gate = (torch.randn(*shape, generator=g) * 4).half().to(dev())
    up = (torch.randn(*shape, generator=g) * 2).half().to(dev())
    gate.view(-1)[:4] = torch.tensor([0.0, -0.0, 65504.0, -65504.0], dtype=torch.float16)
    want = torch.nn.functional.silu(gate) * up
    assert torch.equal(K.swiglu_f16(gate, up), want)
    g2 = gate.clone()
    assert K.swiglu_f16(g2, up, inplace=True).data_ptr() == g2.data_ptr() and torch.equal(g2, want)


# ---- bfloat16 modules --------------------------------------------------------------------------------

@pytest.mark.parametrize("engine", ["single", "pair", "simt"])
def test_bf16_moments_match_reference_vectors(K, engine):
    from conftest import bf16

    g = load_golden("bf16.npz")
    xq, xf = bf16(g["xq"]).to(dev()), bf16(g["xf"]).to(dev())
    acc = K.MomentAccumulator(256, dev(), cross=True, engine=engine)
    for a, b in zip(xq.split(8 * 64), xf.split(8 * 64)):     # the reference's slices of 8 "sequences"
        acc.add(a, b)
    h, c, n = acc.finalize()
    assert n == int(g["n"])
    assert _rel(h.cpu(), torch.from_numpy(g["H"])) < 1e-5
    assert _rel(c.cpu(), torch.from_numpy(g["C"])) < 1e-4


def test_bf16_layer_matches_reference_vectors(K):
    """GPTQ, QEP correction (written back in bf16), installed weight and RTN on a bf16 module."""
    from conftest import bf16, bits16

    g = load_golden("bf16.npz")
    w = bf16(g["W"]).to(dev())
    h, c = torch.from_numpy(g["H"]).to(dev()), torch.from_numpy(g["C"]).to(dev())
    fac = K.factor_hessian(h, 0.01, False)
    got = K.gptq_quantize(w, fac, wbits=4, groupsize=64, sym=False, want_codes=True)
    assert (got["codes"].cpu().numpy() == g["codes"]).mean() >= 0.999
    assert np.abs(bits16(got["scales"]).astype(np.int64) - g["scales"].astype(np.int64)).max() <= 1
    adj = w.clone()
    K.qep_adjust(adj, c, fac, 0.5)
    assert adj.dtype == torch.bfloat16
    d_adj = np.abs(bits16(adj).astype(np.int64) - g["adjusted"].astype(np.int64))
    assert d_adj.max() <= 1 and (d_adj == 0).mean() > 0.99
    # from the reference's own corrected weight, the packed result and the weight the driver installs
    from conftest import bf16 as _b

    adj_ref = _b(g["adjusted"]).to(dev())
    q2 = K.gptq_quantize(adj_ref, fac, wbits=4, groupsize=64, sym=False, want_codes=True)
    same = q2["qweight"].cpu().numpy() == g["qep_qweight_packed"]
    assert same.mean() >= 0.995
    if same.all() and np.array_equal(bits16(q2["scales"]), g["qep_scales"]):
        assert q2["dequantized"].dtype == torch.bfloat16
        assert np.array_equal(bits16(q2["dequantized"]), g["qep_installed"])
    rt = K.rtn_quantize(w, 4, 32, False)
    assert np.array_equal(rt["codes"].cpu().numpy(), g["rtn_codes"])
    assert rt["dequantized"].dtype == torch.bfloat16 and np.array_equal(bits16(rt["dequantized"]), g["rtn_deq"])


def test_all_zero_weight_rows_through_the_column_loop(K):
    """Rows of W that are entirely zero (pruned outputs): find_params gives them the range (-1, +1)
    (reference _gptq.py:914-917), every code is the zero point, the dequantized row is zero."""
    g = load_golden("gptq_b4_g128_asym.npz")
    w = f16(g["W"]).clone()
    w[3] = 0
    w[17] = 0
    h = torch.from_numpy(g["H"])
    for sym in (False, True):
        fac = K.factor_hessian(h.to(dev()), 0.01, False)
        out = K.gptq_quantize(w.to(dev()), fac, wbits=4, groupsize=128, sym=sym, want_codes=True,
                              want_scales_f32=True)
        ref = orc.gptq_quantize(w, h.clone(), wbits=4, groupsize=128, sym=sym)
        codes = out["codes"].cpu().numpy()
        assert (codes == ref["qweight"].numpy()).mean() >= 0.999
        for r in (3, 17):
            assert np.array_equal(codes[r], ref["qweight"].numpy()[r])
            assert np.array_equal(out["zeros"].cpu().numpy()[:, r], ref["qzeros"].numpy()[:, r])
            assert torch.equal(out["scales"].cpu()[:, r], ref["scales"][:, r])
            assert torch.all(out["scales_f32"].cpu()[:, r] == 2.0 / 15.0)
            assert not out["dequantized"][r].any()


def test_column_loop_does_not_depend_on_rows_per_cta(K):
    """The kernel picks 32, 64, 128 or 256 rows per CTA from the layer's row count, and CTAs with few
    rows hand work to helper threads; a row's result must not depend on any of that (this is what
    makes stacked layers, batched experts and row slabs on several GPUs bit-identical to the plain
    call).  19200 rows run with 256 rows per CTA, their halves with 128, a 4096-row slab with 32."""
    g = torch.Generator(device=dev()).manual_seed(77)
    d, out = 512, 19200
    x = torch.randn(4096, d, generator=g, device=dev()).half()
    x[:, ::37] *= 6
    h, _ = K.hessian_from_activations(x)
    w = (torch.randn(out, d, generator=g, device=dev()) * 0.02).half()
    for act, gs in ((False, 128), (True, 32)):
        fac = K.factor_hessian(h, 0.01, act)
        whole = K.gptq_quantize(w, fac, wbits=3, groupsize=gs, sym=False, want_codes=True)
        for r0, r1 in ((0, 9600), (9600, 19200), (1024, 5120), (7000 // 32 * 32, 7000 // 32 * 32 + 64)):
            part = K.gptq_quantize(w[r0:r1].contiguous(), fac, wbits=3, groupsize=gs, sym=False, want_codes=True)
            assert torch.equal(part["codes"], whole["codes"][r0:r1]), (act, r0, r1)
            assert torch.equal(part["scales"], whole["scales"][:, r0:r1])
            assert torch.equal(part["dequantized"], whole["dequantized"][r0:r1])
            assert torch.equal(part["qweight"], whole["qweight"][:, r0:r1])
