"""CPU restatement of the reference's GPTQ / QEP layer-quantization path.

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by
the CPU legs of the benchmark.  The product never imports it.

Every function names the reference code it follows (paths are relative to the
OneComp source tree, v1.4.0).  Float math is torch-on-CPU fp32 with the same
operation order as the reference so that, on CPU, results are bit-identical to
it; integer packing is numpy.

Parity is pinned by ``tests/test_oracle_golden.py`` against fixtures that were
produced by the reference's own functions (see ``tests/golden/make_golden.py``).
"""

from __future__ import annotations

import math
from typing import Iterable, Optional

import numpy as np
import torch

# --------------------------------------------------------------------------
# Moments: Hessian and QEP cross term
# --------------------------------------------------------------------------


def hessian_running_mean(x: torch.Tensor, seqs_per_slice: int = 8):
    """H = (2/N) XᵀX accumulated as a running mean over slices of sequences.

    Follows ``Quantizer.calculate_hessian``
    (onecomp/quantizer/_quantizer.py:764-832): slices of at most
    ``seqs_per_slice`` sequences; per slice the old mean is rescaled by
    n/(n+t) and the slice, pre-scaled by sqrt(2/n_new) in fp32, is added.

    x: [batch, seq, d] (or [tokens, d]) fp16/fp32.  Returns (H fp32 [d,d], N).
    """
    if x.dim() == 2:
        x = x.unsqueeze(0)
    assert x.dim() == 3
    d = x.shape[-1]
    h = torch.zeros((d, d), dtype=torch.float32)
    n = 0
    step = min(x.shape[0], seqs_per_slice)
    for s in range(0, x.shape[0], step):
        xs = x[s : s + step].float().reshape(-1, d)
        t = xs.shape[0]
        h *= n / (n + t)
        n += t
        xt = math.sqrt(2 / n) * xs.t()
        h += xt.matmul(xt.t())
    return h, n


def delta_hatx_running_mean(xq: torch.Tensor, xf: torch.Tensor, seqs_per_slice: int = 8):
    """C = (2/N)(X_f − X_q)ᵀ X_q as a running mean.

    Follows ``Quantizer.calculate_delta_hatX``
    (onecomp/quantizer/_quantizer.py:834-895).
    """
    if xq.dim() == 2:
        xq = xq.unsqueeze(0)
        xf = xf.unsqueeze(0)
    d = xq.shape[-1]
    c = torch.zeros((d, d), dtype=torch.float32)
    n = 0
    step = min(xq.shape[0], seqs_per_slice)
    for s in range(0, xq.shape[0], step):
        q = xq[s : s + step].float()
        f = xf[s : s + step].float()
        delta = (f - q).reshape(-1, d).t()
        q = q.reshape(-1, d).t()
        t = delta.shape[1]
        c *= n / (n + t)
        n += t
        c += (math.sqrt(2 / n) * delta).matmul((math.sqrt(2 / n) * q).t())
    return c


def hessian_and_crossterm(
    chunks_q: Iterable[torch.Tensor], chunks_f: Optional[Iterable[torch.Tensor]] = None
):
    """H and C from per-chunk activations of the quantized / full-precision block.

    Follows ``compute_hessian_and_crossterm``
    (onecomp/qep/_quantize_with_qep_arch.py:118-201): per chunk
    x_q, x_f are flattened to [T,d] fp32, both moments are rescaled by
    n/(n+T), the chunk is scaled by sqrt(2/n_new) and
    H += x_qᵀx_q, C += (x_f − x_q)ᵀ x_q.

    With ``chunks_f`` None only H is produced, which is the per-expert rule of
    ``_compute_per_module_hessians`` (same file, :204-272): chunks with zero
    tokens are skipped and a module that saw no token at all yields None.
    """
    h = c = None
    n = 0
    it_f = iter(chunks_f) if chunks_f is not None else None
    for xq in chunks_q:
        xf = next(it_f) if it_f is not None else None
        d = xq.shape[-1]
        xq = xq.reshape(-1, d).float()
        t = xq.shape[0]
        if h is None:
            h = torch.zeros((d, d), dtype=torch.float32)
            c = torch.zeros((d, d), dtype=torch.float32) if it_f is not None else None
        if t == 0:
            continue
        h *= n / (n + t)
        if c is not None:
            c *= n / (n + t)
        n += t
        xqs = math.sqrt(2 / n) * xq
        h += xqs.t() @ xqs
        if c is not None:
            xfs = math.sqrt(2 / n) * xf.reshape(-1, d).float()
            c += (xfs - xqs).t() @ xqs
    if n == 0:
        return None, None, 0
    return h, c, n


# --------------------------------------------------------------------------
# Scale / zero fitting, quantize, dequantize
# --------------------------------------------------------------------------


def find_params(x: torch.Tensor, wbits: int, sym: bool, mse: bool = False,
                norm: float = 2.4, grid: int = 100, maxshrink: float = 0.8):
    """Per-row scale and zero over the given columns.

    Follows ``GPTQExcecutor.find_params`` with ``perchannel=True, weight=True``
    (onecomp/quantizer/gptq/_gptq.py:886-972): the range always contains 0;
    symmetric mode mirrors the larger magnitude but flips xmin only where it is
    negative; all-zero rows get (−1, +1); scale=(xmax−xmin)/maxq;
    zero=round(−xmin/scale) or (maxq+1)/2.  Optional ``mse`` shrink search
    (:928-950).

    x: [rows, cols] fp32.  Returns (scale [rows,1], zero [rows,1]) fp32.
    """
    maxq = torch.tensor(2**wbits - 1)
    x = x.flatten(1)
    zeros = torch.zeros(x.shape[0])
    xmin = torch.minimum(x.min(1)[0], zeros)
    xmax = torch.maximum(x.max(1)[0], zeros)
    if sym:
        xmax = torch.maximum(torch.abs(xmin), xmax)
        neg = xmin < 0
        if torch.any(neg):
            xmin[neg] = -xmax[neg]
    flat = (xmin == 0) & (xmax == 0)
    xmin[flat] = -1
    xmax[flat] = +1
    scale = (xmax - xmin) / maxq
    if sym:
        zero = torch.full_like(scale, (maxq + 1) / 2)
    else:
        zero = torch.round(-xmin / scale)
    if mse:
        best = torch.full([x.shape[0]], float("inf"))
        for i in range(int(maxshrink * grid)):
            p = 1 - i / grid
            xmin1 = p * xmin
            xmax1 = p * xmax
            scale1 = (xmax1 - xmin1) / maxq
            zero1 = torch.round(-xmin1 / scale1) if not sym else zero
            q = quantize_codes(x, scale1.unsqueeze(1), zero1.unsqueeze(1), wbits)
            r = dequantize_codes(q, scale1.unsqueeze(1), zero1.unsqueeze(1))
            r -= x
            r.abs_()
            r.pow_(norm)
            err = torch.sum(r, 1)
            better = err < best
            if torch.any(better):
                best[better] = err[better]
                scale[better] = scale1[better]
                zero[better] = zero1[better]
    return scale.reshape(-1, 1), zero.reshape(-1, 1)


def quantize_codes(x, scale, zero, wbits: int):
    """clamp(round(x/scale)+zero, 0, maxq) as int32 (…/gptq/_gptq.py:800-820).
    ``round`` is round-half-to-even and the divide is a true fp32 divide."""
    return torch.clamp(torch.round(x / scale) + zero, 0, 2**wbits - 1).int()


def dequantize_codes(q, scale, zero):
    """scale·(q − zero) in fp32 (…/gptq/_gptq.py:823-840)."""
    return scale * (q.float() - zero)


def rtn_quantize(weight: torch.Tensor, wbits: int, groupsize: int, sym: bool):
    """Round-to-nearest group quantization used for experts without calibration tokens.

    Follows ``run_rtn`` / ``pseudo_quantize_tensor`` (onecomp/quantizer/rtn/rtn_impl.py:22-102,
    onecomp/quantizer/rtn/quantizer.py:64-181, mse off): per group the range contains 0,
    symmetric mode mirrors it on both sides, all-zero groups get (-1, +1),
    scale = max((max-min)/q_max, 1e-5), zero = round(-min/scale) or (q_max+1)/2,
    dequantized = (q - zero) * scale in the weight's dtype.
    Returns dict(quantized_weight int32 [out,d], scale fp16 [out,G], zero fp16 [out,G],
    dequantized_weight)."""
    w = weight.clone().float()
    shape = w.shape
    if groupsize > 0:
        if w.shape[-1] % groupsize != 0:
            raise ValueError(f"Tensor shape {w.shape[-1]} must be divisible by group size {groupsize}")
        w = w.reshape(-1, w.shape[-1] // groupsize, groupsize)
    else:
        w = w.reshape(-1, 1, w.shape[-1])
    q_max = 2**wbits - 1
    zero_t = torch.zeros(1)
    w_max = torch.maximum(w.amax(dim=-1, keepdim=True), zero_t)
    w_min = torch.minimum(w.amin(dim=-1, keepdim=True), zero_t)
    if sym:
        w_max = torch.maximum(torch.abs(w_min), w_max)
        w_min = -w_max
    flat = (w_min == 0) & (w_max == 0)
    w_min[flat] = -1
    w_max[flat] = +1
    scale = ((w_max - w_min) / q_max).clamp(min=1e-5)
    zero = torch.full_like(scale, (q_max + 1) / 2) if sym else torch.round(-w_min / scale)
    q = torch.clamp(torch.round(w / scale) + zero, 0, q_max).int()
    deq = (q.float() - zero) * scale
    return {
        "quantized_weight": q.reshape(shape),
        "scale": scale.squeeze(-1).to(torch.float16),
        "zero": zero.squeeze(-1).to(torch.float16),
        "dequantized_weight": deq.reshape(shape).to(weight.dtype),
    }


# --------------------------------------------------------------------------
# Inverse-Hessian factor
# --------------------------------------------------------------------------


class CholeskyFailed(RuntimeError):
    pass


def inverse_hessian_upper(h: torch.Tensor, percdamp: float, max_retries: int = 5):
    """Upper Cholesky factor U of (H + damp·I)⁻¹, so that UᵀU = H⁻¹.

    Follows ``_compute_inverse_hessian`` (…/gptq/_gptq.py:594-643):
    damp = percdamp·mean(diag H) added in place; L = chol(H); on failure add
    10ᵏ·damp cumulatively (k = 1…), at most ``max_retries`` attempts, then
    RuntimeError; U = chol(cholesky_inverse(L), upper).
    """
    damp = percdamp * torch.mean(torch.diag(h))
    idx = torch.arange(h.shape[0])
    h[idx, idx] += damp
    mult = 1.0
    for _ in range(max_retries):
        try:
            low = torch.linalg.cholesky(h)
            break
        except torch._C._LinAlgError:  # pylint: disable=protected-access
            mult *= 10.0
            h[idx, idx] += mult * damp
    else:
        raise CholeskyFailed(
            "Cholesky decomposition failed after %d damping attempts." % max_retries
        )
    return torch.linalg.cholesky(torch.cholesky_inverse(low), upper=True)


# --------------------------------------------------------------------------
# GPTQ column loop
# --------------------------------------------------------------------------


def gptq_quantize(
    weight: torch.Tensor,
    h: torch.Tensor,
    blocksize: int = 128,
    percdamp: float = 0.01,
    wbits: int = 4,
    groupsize: int = -1,
    actorder: bool = False,
    sym: bool = True,
    mse: bool = False,
    q_grid: int = 600,
    q_norm: float = 2.4,
    u_override: Optional[torch.Tensor] = None,
    perm_override: Optional[torch.Tensor] = None,
):
    """GPTQ for one Linear weight [out, d]; ``h`` [d,d] fp32 is modified in place.

    Follows ``run_gptq`` (onecomp/quantizer/gptq/_gptq.py:646-794):

    * per-channel params are fitted on the whole row before dead columns are
      zeroed (:690-695);
    * dead columns (diag H == 0) get H=1, W=0;
    * act-order sorts columns by descending diag H (:697-702);
    * U from ``inverse_hessian_upper``;
    * per block of ``blocksize`` columns a copy W1 of the block is quantized
      column by column; err=(w−ŵ)/U[i,i]; W1[:, i:] −= err ⊗ U[i, i:] (:759-761);
    * group params at a group's first column are fitted on the *block-entry*
      matrix columns c … c+groupsize (:737-745), i.e. they see the previous
      blocks' lazy updates but none of the current block's in-block updates;
    * after the block W[:, i2:] −= Err · U[i1:i2, i2:] (:765);
    * codes are returned in original column order (:767-768).

    Returns dict(qweight int32 [out,d], scales fp16 [G,out] or [out,1],
    qzeros int32 [G,out] or [out,1], perm int64 [d] or None, scales_f32 (the
    pre-cast fp32 scales, for tolerance checks), u (the factor used)).
    ``u_override`` lets a test feed a given U instead of factorising ``h``;
    ``perm_override`` a given act-order column order instead of torch.argsort's (which
    is not stable: columns with exactly equal diagonal entries may come in either order,
    and do on another device or build; a test that found such ties hands over the order
    it wants both sides to use).
    """
    w = weight.clone().float()
    out, d = w.shape
    scale, zero = find_params(w, wbits, sym, mse, q_norm, q_grid)

    dead = torch.diag(h) == 0
    h[dead, dead] = 1
    w[:, dead] = 0

    perm = None
    if actorder:
        perm = torch.argsort(torch.diag(h), descending=True)
        if perm_override is not None:
            perm = perm_override.to(perm.dtype)
        w = w[:, perm]
        h = h[perm][:, perm]
        invperm = torch.argsort(perm)

    codes = torch.zeros((out, d), dtype=torch.int32)
    u = inverse_hessian_upper(h, percdamp) if u_override is None else u_override

    if groupsize != -1:
        ngroups = (d + groupsize - 1) // groupsize
        all_scales = torch.zeros(out, ngroups, dtype=torch.float32)
        all_zeros = torch.zeros(out, ngroups, dtype=torch.float32)

    for i1 in range(0, d, blocksize):
        i2 = min(i1 + blocksize, d)
        count = i2 - i1
        w1 = w[:, i1:i2].clone()
        q1 = torch.zeros_like(w1, dtype=torch.int32)
        err1 = torch.zeros_like(w1)
        u1 = u[i1:i2, i1:i2]
        for i in range(count):
            col = w1[:, i]
            diag = u1[i, i]
            if groupsize != -1 and (i1 + i) % groupsize == 0:
                scale, zero = find_params(
                    w[:, (i1 + i) : (i1 + i + groupsize)], wbits, sym, mse, q_norm, q_grid
                )
                g = (i1 + i) // groupsize
                all_scales[:, g] = scale.squeeze(-1)
                all_zeros[:, g] = zero.squeeze(-1)
            qi = quantize_codes(col.unsqueeze(1), scale, zero, wbits)
            deq = dequantize_codes(qi, scale, zero).flatten()
            q1[:, i] = qi.flatten()
            e = (col - deq) / diag
            w1[:, i:] -= e.unsqueeze(1).matmul(u1[i, i:].unsqueeze(0))
            err1[:, i] = e
        codes[:, i1:i2] = q1
        w[:, i2:] -= err1.matmul(u[i1:i2, i2:])

    if actorder:
        codes = codes[:, invperm]

    if groupsize != -1:
        scales_f32 = all_scales.T.contiguous()
        qzeros = all_zeros.to(torch.int32).T.contiguous()
    else:
        scales_f32 = scale.clone()
        qzeros = zero.to(torch.int32)
    return {
        "qweight": codes,
        "scales": scales_f32.to(torch.float16),
        "qzeros": qzeros,
        "perm": perm,
        "scales_f32": scales_f32,
        "u": u,
    }


# --------------------------------------------------------------------------
# Packing (AutoGPTQ int32 layout), numpy integer arithmetic
# --------------------------------------------------------------------------


def pack_rows(matrix: np.ndarray, wbits: int) -> np.ndarray:
    """Pack integer values along axis 0 into int32 words.

    Follows ``_pack_rows`` (onecomp/quantizer/gptq/gptq_layer.py:36-83).
    2/4/8 bit: word r holds rows r·f … r·f+f−1 (f = 32/bits), value k at bit
    k·bits.  3 bit: 32 values form one little-endian 96-bit stream stored in 3
    consecutive words.  Inputs are masked to ``wbits`` first, so a stored −1
    becomes the all-ones code.
    """
    rows, cols = matrix.shape
    vals = matrix.astype(np.int64) & ((1 << wbits) - 1)
    if wbits in (2, 4, 8):
        f = 32 // wbits
        assert rows % f == 0, f"rows ({rows}) must be divisible by pack_factor ({f})"
        v = vals.reshape(rows // f, f, cols).astype(np.uint64)
        word = np.zeros((rows // f, cols), dtype=np.uint64)
        for k in range(f):
            word |= v[:, k, :] << np.uint64(k * wbits)
        return word.astype(np.uint32).view(np.int32)
    if wbits == 3:
        assert rows % 32 == 0, f"rows ({rows}) must be divisible by 32 for 3-bit packing"
        nb = rows // 32
        v = vals.reshape(nb, 32, cols)
        words = np.zeros((nb, 3, cols), dtype=np.uint64)
        for k in range(32):
            bit = 3 * k
            wi, off = divmod(bit, 32)
            val = v[:, k, :].astype(np.uint64)
            words[:, wi, :] |= (val << np.uint64(off)) & np.uint64(0xFFFFFFFF)
            if off + 3 > 32:
                words[:, wi + 1, :] |= val >> np.uint64(32 - off)
        return words.reshape(nb * 3, cols).astype(np.uint32).view(np.int32)
    raise ValueError(f"Unsupported wbits for packing: {wbits}")


def unpack_rows(packed: np.ndarray, wbits: int, num_rows: int) -> np.ndarray:
    """Inverse of :func:`pack_rows` (…/gptq_layer.py:86-126)."""
    prow, cols = packed.shape
    p = packed.view(np.uint32).astype(np.uint64)
    mask = np.uint64((1 << wbits) - 1)
    if wbits in (2, 4, 8):
        f = 32 // wbits
        out = np.zeros((prow, f, cols), dtype=np.int32)
        for k in range(f):
            out[:, k, :] = ((p >> np.uint64(k * wbits)) & mask).astype(np.int32)
        return out.reshape(prow * f, cols)[:num_rows]
    if wbits == 3:
        nb = prow // 3
        p3 = p.reshape(nb, 3, cols)
        out = np.zeros((nb, 32, cols), dtype=np.int32)
        for k in range(32):
            wi, off = divmod(3 * k, 32)
            v = p3[:, wi, :] >> np.uint64(off)
            if off + 3 > 32:
                v = v | (p3[:, wi + 1, :] << np.uint64(32 - off))
            out[:, k, :] = (v & mask).astype(np.int32)
        return out.reshape(nb * 32, cols)[:num_rows]
    raise ValueError(f"Unsupported wbits for unpacking: {wbits}")


def pack_qweight(codes: np.ndarray, wbits: int) -> np.ndarray:
    """codes [out, in] → int32 [in·bits/32, out] (``pack_int_weights``, :129-139)."""
    return pack_rows(np.ascontiguousarray(codes.T), wbits)


def unpack_qweight(packed: np.ndarray, wbits: int, shape) -> np.ndarray:
    return np.ascontiguousarray(unpack_rows(packed, wbits, shape[1]).T)


def pack_qzeros(zeros: np.ndarray, wbits: int) -> np.ndarray:
    """zeros [G, out] → int32 [G, out·bits/32] (``pack_zeros``, :160-170)."""
    return np.ascontiguousarray(pack_rows(np.ascontiguousarray(zeros.T), wbits).T)


def unpack_qzeros(packed: np.ndarray, wbits: int, out_features: int) -> np.ndarray:
    return np.ascontiguousarray(
        unpack_rows(np.ascontiguousarray(packed.T), wbits, out_features).T
    )


def normalize_zeros(zeros: np.ndarray, out_features: int) -> np.ndarray:
    """(out,), (out,1) or (G,out) → (G,out) (``normalize_scale_zero``, :187-205)."""
    if zeros.ndim == 1:
        return zeros[None, :]
    if zeros.ndim == 2 and zeros.shape == (out_features, 1):
        return zeros.T
    return zeros


def pack_result(codes: np.ndarray, qzeros: np.ndarray, wbits: int):
    """What ``GPTQ.quantize_layer`` stores when ``bitpack_on_quantize`` is on
    (onecomp/quantizer/gptq/_gptq.py:445-464): packed codes, and zeros
    normalised to [G,out], minus one (the v1 checkpoint offset), masked, packed."""
    out = codes.shape[0]
    z = normalize_zeros(qzeros, out).astype(np.int32) - 1
    return pack_qweight(codes.astype(np.int32), wbits), pack_qzeros(z, wbits)


def group_index(perm: Optional[np.ndarray], groupsize: int, d: int) -> np.ndarray:
    """g_idx of the inference layer (…/gptq_layer.py:423-433; result docstring
    …/_gptq.py:55-58): g_idx[perm[i]] = i // groupsize, identity without perm,
    zeros for per-channel."""
    if groupsize == -1:
        return np.zeros(d, dtype=np.int32)
    base = np.arange(d) // groupsize
    if perm is None:
        return base.astype(np.int32)
    g = np.empty(d, dtype=np.int64)
    g[np.asarray(perm)] = base
    return g.astype(np.int32)


def dequantize_result(qweight_packed, scales_f16, qzeros_packed, perm, wbits, groupsize, shape):
    """Ŵ fp16 [out,d] used for QEP propagation.

    Follows ``GPTQResult.compute_dequantized_weight``
    (onecomp/quantizer/gptq/_gptq.py:84-168): unpack, zeros=(stored+1)&mask,
    gather fp16 scales/zeros by g_idx, fp32 scale·(q − zero), cast to fp16.
    """
    out, d = shape
    q = torch.from_numpy(unpack_qweight(np.asarray(qweight_packed), wbits, shape).astype(np.int32))
    z = unpack_qzeros(np.asarray(qzeros_packed), wbits, out)
    z = torch.from_numpy(((z + 1) & ((1 << wbits) - 1)).astype(np.int32))
    s = torch.as_tensor(scales_f16)
    if groupsize == -1:
        if s.ndim == 1:
            s = s.unsqueeze(1)
        zz = z.T if z.shape == (1, out) else z
        return dequantize_codes(q, s, zz.float()).to(torch.float16)
    g = torch.from_numpy(group_index(None if perm is None else np.asarray(perm), groupsize, d)).long()
    se = s[g, :].T.to(torch.float16)
    ze = z[g, :].T.to(torch.float16)
    return dequantize_codes(q, se, ze).to(torch.float16).contiguous()


# --------------------------------------------------------------------------
# QEP weight correction
# --------------------------------------------------------------------------


def qep_adjust_weight(weight: torch.Tensor, h: torch.Tensor, c: torch.Tensor,
                      percdamp: float = 0.01, perccorr: float = 0.5):
    """W ← fp16( W + perccorr · (W·C)·(H + damp·I)⁻¹ ).

    Follows ``Quantizer.adjust_weight``
    (onecomp/quantizer/_quantizer.py:362-432): works on clones of H and C; dead
    columns get H=1, W=0; inside each attempt damp = percdamp·mean(diag H) of the
    *current* (already damped) H is added; the solve is potrf + potrs on
    (W·C)ᵀ; on failure 10ᵏ·damp more is added and the attempt repeats (≤5).
    """
    w = weight.clone().float()
    h = h.clone()
    c = c.clone()
    dead = torch.diag(h) == 0
    h[dead, dead] = 1
    w[:, dead] = 0
    idx = torch.arange(h.shape[0])
    mult = 1.0
    for _ in range(5):
        try:
            damp = percdamp * torch.mean(torch.diag(h))
            h[idx, idx] += damp
            rhs = w @ c
            low = torch.linalg.cholesky(h)
            delta = torch.cholesky_solve(rhs.t(), low).t()
            w = w + (perccorr * delta)
            break
        except torch._C._LinAlgError:  # pylint: disable=protected-access
            mult *= 10.0
            h[idx, idx] += mult * damp
    else:
        raise CholeskyFailed("Cholesky decomposition failed after 5 damping attempts.")
    return w.to(weight.dtype)


# --------------------------------------------------------------------------
# Error measure used by the parity criteria
# --------------------------------------------------------------------------


def reconstruction_error(weight, w_hat, h, nsamples: int) -> float:
    """‖WX − ŴX‖²_F from the second moment: tr(Δ (N/2·H) Δᵀ) in float64, where
    H=(2/N)XᵀX is the *undamped* Hessian (cf. the output error of
    onecomp/quantizer/_quantizer.py:961-1031, which forms the products directly)."""
    delta = (weight.double() - w_hat.double())
    return float(torch.sum((delta @ h.double()) * delta).item() * nsamples / 2)
