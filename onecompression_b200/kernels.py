"""Tensor-level wrappers over the C ABI (``include/onecomp_b200.h``).

torch supplies device memory and the current stream; all arithmetic happens in
the CUDA library.  Nothing here falls back to torch or to the CPU: a missing
library or a CPU tensor raises.
"""

from __future__ import annotations

import logging
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib
from ._lib import call, ptr, stream_handle

logger = logging.getLogger(__name__)

PACKABLE_WBITS = (2, 3, 4, 8)
MAX_BLOCKSIZE = 128

_sm_count_cache: dict[int, int] = {}


def sm_count(device) -> int:
    idx = torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    if idx not in _sm_count_cache:
        _sm_count_cache[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _sm_count_cache[idx]


def _require_cuda(t: torch.Tensor, what: str):
    if not t.is_cuda:
        raise RuntimeError(
            f"{what} must be a CUDA tensor: onecompression_b200 runs on the GPU only (no CPU path)"
        )


# ---------------------------------------------------------------------------
# second moments
# ---------------------------------------------------------------------------


# 16-bit element types the kernels read and write (the C ABI's OC_DTYPE_* codes)
_DTYPES = {torch.float16: 0, torch.bfloat16: 1}


class MomentAccumulator:
    """Running-mean Hessian H = (2/N) XqᵀXq and, optionally, the QEP cross term
    C = (2/N)(Xf − Xq)ᵀXq, accumulated chunk by chunk on the GPU.

    Same update rule as the reference (onecomp/quantizer/_quantizer.py:824-830,
    onecomp/qep/_quantize_with_qep_arch.py:182-196): before a chunk of t tokens
    the moments are scaled by n/(n+t), then the chunk enters with weight 2/(n+t).
    """

    ENGINES = {"auto": 0, "simt": 1, "single": 2, "pair": 3}

    def __init__(self, d: int, device, cross: bool = False, chunk_tokens: int = 0,
                 force_simt: bool = False, engine: str = "auto"):
        self.d = d
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("MomentAccumulator needs a CUDA device (no CPU path)")
        self.H = torch.zeros((d, d), dtype=torch.float32, device=self.device)
        self.C = torch.zeros((d, d), dtype=torch.float32, device=self.device) if cross else None
        self.nsamples = 0
        self.chunk_tokens = chunk_tokens
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        # the tensor-core kernel needs 16-byte rows; decide once so that every chunk of
        # one accumulation takes the same path
        self.force_simt = bool(force_simt) or d % 8 != 0 or engine == "simt"
        self.engine = 1 if self.force_simt else self.ENGINES[engine]
        self._scratch = None
        self._needs_mirror = False

    def add(self, xq: torch.Tensor, xf: Optional[torch.Tensor] = None):
        """Fold a chunk of activations ([..., d], fp16) into the moments."""
        if xq.shape[-1] != self.d:
            raise ValueError(f"activation width {xq.shape[-1]} != {self.d}")
        xq = self._as_rows(xq)
        t = xq.shape[0]
        if t == 0:
            return
        cross = self.C is not None
        if cross:
            if xf is None:
                raise ValueError("this accumulator also builds the cross term: pass xf")
            xf = self._as_rows(xf)
            if xf.shape != xq.shape:
                raise ValueError("xf and xq differ in shape")
            if xf.dtype != xq.dtype:
                xf = xf.to(xq.dtype)
            if xf.stride(0) != xq.stride(0):
                # the kernels read both with one row stride
                xq, xf = xq.contiguous(), xf.contiguous()
        n = self.nsamples
        a_old = n / (n + t)
        a_new = 2.0 / (n + t)
        self.nsamples = n + t
        scratch = None
        if cross and not self.force_simt:
            # Xf - Xq as two 16-bit terms, rows packed: [2, t, d]
            need = 2 * t * self.d
            if self._scratch is None or self._scratch.numel() < need or self._scratch.dtype != xq.dtype:
                self._scratch = torch.empty(need, dtype=xq.dtype, device=self.device)
            scratch = self._scratch
        with torch.cuda.device(self.device):
            call(
                "oc_moment_accum", ptr(xq), ptr(xf) if cross else None, ptr(scratch), t, self.d,
                xq.stride(0), ptr(self.H), ptr(self.C), self.d, a_old, a_new, self.chunk_tokens,
                sm_count(self.device), self.engine, _DTYPES[xq.dtype], ptr(self.status), stream_handle(),
            )
        self._needs_mirror = not self.force_simt

    def _as_rows(self, x: torch.Tensor) -> torch.Tensor:
        _require_cuda(x, "activations")
        if x.dtype not in _DTYPES:
            x = x.to(torch.float16)
        x = x.reshape(-1, self.d)
        if x.stride(1) != 1 or x.stride(0) % 8 != 0 or x.data_ptr() % 16 != 0:
            x = x.contiguous()
        return x

    def finalize(self, check: bool = True):
        """Complete H (mirror the upper triangle) and return (H, C, nsamples)."""
        if self._needs_mirror:
            with torch.cuda.device(self.device):
                call("oc_mirror_upper", ptr(self.H), self.d, self.d, stream_handle())
            self._needs_mirror = False
        if check:
            code = int(self.status.item())
            if code != 0:
                raise RuntimeError(f"moment kernel: a bounded pipeline wait expired (code {code})")
        self._scratch = None
        return self.H, self.C, self.nsamples


def hessian_from_activations(x: torch.Tensor, seqs_per_slice: int = 8, **kw):
    """(H, N) for activations [batch, seq, d], folding ``seqs_per_slice`` sequences at a
    time as Quantizer.calculate_hessian does (onecomp/quantizer/_quantizer.py:811-830)."""
    if x.dim() == 2:
        x = x.unsqueeze(0)
    acc = MomentAccumulator(x.shape[-1], x.device, cross=False, **kw)
    step = min(x.shape[0], seqs_per_slice)
    for s in range(0, x.shape[0], step):
        acc.add(x[s : s + step])
    h, _, n = acc.finalize()
    return h, n


# ---------------------------------------------------------------------------
# inverse-Hessian factor
# ---------------------------------------------------------------------------


@dataclass
class HessianFactor:
    """U with UᵀU = (P H Pᵀ + damp·I)⁻¹ plus what the column loop needs with it."""

    u: torch.Tensor            # [d, d] fp32, upper triangular
    perm: torch.Tensor         # int32 [d]
    invperm: torch.Tensor      # int32 [d]
    dead: torch.Tensor         # uint8 [d], original column order
    damp: torch.Tensor         # float32 [2]: percdamp*mean(diag), mean(diag)
    actorder: bool
    percdamp: float
    rel_shift: float           # multiple of damp that was added to the diagonal
    attempts: int


_ws_cache: dict = {}


def _workspace(nbytes: int, device) -> torch.Tensor:
    """A reusable scratch buffer per device (grown on demand)."""
    key = (torch.device(device).index, torch.cuda.current_stream(device).cuda_stream)
    buf = _ws_cache.get(key)
    if buf is None or buf.numel() < nbytes:
        _ws_cache.pop(key, None)
        buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _ws_cache[key] = buf
    return buf


def release_workspaces():
    _ws_cache.clear()


def factor_hessian(h: torch.Tensor, percdamp: float, actorder: bool, max_retries: int = 5,
                   shifts=None) -> HessianFactor:
    """Factor a Hessian for GPTQ with the reference's retry rule: when the Cholesky
    factorisation meets a non-positive pivot, 10ᵏ·damp more is added to the diagonal
    (k = 1, 2, …) and it is tried again, ``max_retries`` attempts in all
    (onecomp/quantizer/gptq/_gptq.py:618-641).  ``h`` is not modified.

    ``shifts`` optionally gives the diagonal shift of each attempt as a multiple of
    damp (used by the QEP correction, whose rule differs on retries).
    """
    _require_cuda(h, "hessian")
    if h.dtype != torch.float32:
        h = h.float()
    if h.stride(1) != 1:
        h = h.contiguous()
    d = h.shape[0]
    dev = h.device
    u = torch.empty((d, d), dtype=torch.float32, device=dev)
    perm = torch.empty(d, dtype=torch.int32, device=dev)
    invperm = torch.empty(d, dtype=torch.int32, device=dev)
    dead = torch.empty(d, dtype=torch.uint8, device=dev)
    damp = torch.empty(2, dtype=torch.float32, device=dev)
    status = torch.empty(1, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        nbytes = _lib.load().oc_hinv_workspace_bytes(d)
        ws = _workspace(nbytes, dev)
        rel, mult = 1.0, 1.0
        for attempt in range(max_retries):
            if shifts is not None:
                rel = shifts(attempt, float(percdamp))
            call(
                "oc_hinv_factor", ptr(h), h.stride(0), d, float(percdamp), float(rel),
                1 if actorder else 0, 1 if attempt > 0 else 0, ptr(u), d, ptr(perm), ptr(invperm),
                ptr(dead), ptr(damp), ptr(status), ptr(ws), ws.numel(), stream_handle(),
            )
            if int(status.item()) == 0:
                check_gemm_status()
                return HessianFactor(u, perm, invperm, dead, damp, bool(actorder), float(percdamp),
                                     rel, attempt + 1)
            mult *= 10.0
            extra = mult * float(damp[0].item())
            rel += mult
            logger.warning(
                "Cholesky failed (attempt %d/%d); adding extra damping %.2e",
                attempt + 1, max_retries, extra,
            )
    raise RuntimeError(
        "Cholesky decomposition failed after %d damping attempts. "
        "The Hessian may be severely ill-conditioned." % max_retries
    )


def factor_hessians_batched(hs: torch.Tensor, percdamp: float, actorder: bool) -> dict:
    """First attempt of the factorisation for a batch of Hessians ``hs`` [B, n, n] (fp32, contiguous),
    enqueued without waiting: dict(u [B,n,n], perm, invperm int32 [B,n], dead uint8 [B,n], damp
    [B,2], status int32 [B]).  A non-zero status means that problem needs the retry rule of
    ``factor_hessian``."""
    _require_cuda(hs, "hessians")
    if hs.dtype != torch.float32 or hs.dim() != 3 or hs.shape[1] != hs.shape[2] or not hs.is_contiguous():
        raise TypeError("factor_hessians_batched expects a contiguous fp32 [B, n, n] tensor")
    batch, n, _ = hs.shape
    dev = hs.device
    out = {"u": torch.empty((batch, n, n), dtype=torch.float32, device=dev),
           "perm": torch.empty((batch, n), dtype=torch.int32, device=dev),
           "invperm": torch.empty((batch, n), dtype=torch.int32, device=dev),
           "dead": torch.empty((batch, n), dtype=torch.uint8, device=dev),
           "damp": torch.empty((batch, 2), dtype=torch.float32, device=dev),
           "status": torch.empty(batch, dtype=torch.int32, device=dev)}
    with torch.cuda.device(dev):
        ws = _workspace(_lib.load().oc_hinv_workspace_bytes(n) * batch, dev)
        call("oc_hinv_factor_batched", batch, ptr(hs), n, float(percdamp), 1 if actorder else 0, ptr(out["u"]),
             ptr(out["perm"]), ptr(out["invperm"]), ptr(out["dead"]), ptr(out["damp"]), ptr(out["status"]),
             ptr(ws), ws.numel(), stream_handle())
    return out


def factor_hessian_launch(h: torch.Tensor, percdamp: float, actorder: bool, buffers: Optional[dict] = None) -> dict:
    """First attempt of ``factor_hessian`` enqueued on the current stream without waiting for its
    status: lets several small factorisations run side by side on different streams.  Finish
    with ``factor_hessian_resolve``."""
    _require_cuda(h, "hessian")
    if h.dtype != torch.float32:
        h = h.float()
    if h.stride(1) != 1:
        h = h.contiguous()
    d = h.shape[0]
    dev = h.device
    buffers = buffers or {}       # contiguous views to write into (e.g. slices of batched arrays)
    out = {
        "h": h, "u": buffers.get("u", None) if buffers.get("u", None) is not None else torch.empty((d, d), dtype=torch.float32, device=dev),
        "perm": buffers["perm"] if "perm" in buffers else torch.empty(d, dtype=torch.int32, device=dev),
        "invperm": buffers["invperm"] if "invperm" in buffers else torch.empty(d, dtype=torch.int32, device=dev),
        "dead": buffers["dead"] if "dead" in buffers else torch.empty(d, dtype=torch.uint8, device=dev),
        "damp": torch.empty(2, dtype=torch.float32, device=dev),
        "status": torch.empty(1, dtype=torch.int32, device=dev),
        "percdamp": float(percdamp), "actorder": bool(actorder),
    }
    with torch.cuda.device(dev):
        ws = _workspace(_lib.load().oc_hinv_workspace_bytes(d), dev)
        call("oc_hinv_factor", ptr(h), h.stride(0), d, float(percdamp), 1.0, 1 if actorder else 0, 0,
             ptr(out["u"]), d, ptr(out["perm"]), ptr(out["invperm"]), ptr(out["dead"]), ptr(out["damp"]),
             ptr(out["status"]), ptr(ws), ws.numel(), stream_handle())
    return out


def factor_hessian_resolve(pending: dict, max_retries: int = 5) -> HessianFactor:
    """Waits for a launched factorisation; a failed first attempt goes through the retry rule of
    ``factor_hessian`` on the current stream."""
    if int(pending["status"].item()) == 0:
        return HessianFactor(pending["u"], pending["perm"], pending["invperm"], pending["dead"], pending["damp"],
                             pending["actorder"], pending["percdamp"], 1.0, 1)
    return factor_hessian(pending["h"], pending["percdamp"], pending["actorder"], max_retries)


# ---------------------------------------------------------------------------
# GPTQ column loop
# ---------------------------------------------------------------------------


def gptq_quantize(
    weight: torch.Tensor,
    factor: HessianFactor,
    wbits: int,
    groupsize: int,
    sym: bool,
    blocksize: int = 128,
    pack: bool = True,
    want_codes: bool = False,
    want_dequantized: bool = True,
    want_scales_f32: bool = False,
    outputs: Optional[dict] = None,
    ld_out: Optional[int] = None,
    mse: bool = False,
    q_grid: int = 600,
    q_norm: float = 2.4,
):
    """Run the column loop on ``weight`` [out, d] fp16 (CUDA) with a ready factor.

    Returns a dict of CUDA tensors: qweight / qzeros (packed, when ``pack``), scales
    (fp16 [G, out]), zeros (int32 [G, out]), optionally codes (int32 [out, d]),
    dequantized (fp16 [out, d]), scales_f32.  ``outputs`` may provide pre-allocated
    views (row slabs of full-layer buffers) under the same keys together with
    ``ld_out``, the row count of the full layer.
    """
    _require_cuda(weight, "weight")
    if weight.dtype not in _DTYPES:
        raise TypeError("gptq_quantize expects an fp16 or bf16 weight")
    if weight.dim() != 2:
        raise ValueError("weight must be 2-D [out_features, in_features]")
    if weight.stride(1) != 1:
        weight = weight.contiguous()
    out, d = weight.shape
    dev = weight.device
    if factor.u.shape[0] != d:
        raise ValueError("factor and weight disagree on in_features")
    if not 1 <= blocksize <= MAX_BLOCKSIZE:
        raise NotImplementedError(
            f"blocksize {blocksize}: the CUDA column kernel handles 1..{MAX_BLOCKSIZE}"
        )
    groups = 1 if groupsize == -1 else (d + groupsize - 1) // groupsize
    outputs = dict(outputs or {})
    ld = ld_out if ld_out is not None else out
    if pack:
        if wbits not in PACKABLE_WBITS:
            raise ValueError(f"packing supports wbits in {PACKABLE_WBITS}; got {wbits}")
        f = 32 if wbits == 3 else 32 // wbits
        # same assertions (and wording) as the reference packer, gptq_layer.py:55-66
        if wbits == 3:
            assert d % 32 == 0, f"rows ({d}) must be divisible by 32 for 3-bit packing"
            assert out % 32 == 0, f"rows ({out}) must be divisible by 32 for 3-bit packing"
        else:
            assert d % f == 0, f"rows ({d}) must be divisible by pack_factor ({f})"
            assert out % f == 0, f"rows ({out}) must be divisible by pack_factor ({f})"
        if "qweight" not in outputs:
            outputs["qweight"] = torch.empty((d * wbits // 32, out), dtype=torch.int32, device=dev)
        if "qzeros" not in outputs:
            outputs["qzeros"] = torch.empty((groups, out * wbits // 32), dtype=torch.int32, device=dev)
    if "scales" not in outputs:
        outputs["scales"] = torch.empty((groups, out), dtype=torch.float16, device=dev)
    if "zeros" not in outputs:
        outputs["zeros"] = torch.empty((groups, out), dtype=torch.int32, device=dev)
    if want_scales_f32 and "scales_f32" not in outputs:
        outputs["scales_f32"] = torch.empty((groups, out), dtype=torch.float32, device=dev)
    if want_codes and "codes" not in outputs:
        outputs["codes"] = torch.empty((out, d), dtype=torch.int32, device=dev)
    if want_dequantized and "dequantized" not in outputs:
        outputs["dequantized"] = torch.empty((out, d), dtype=weight.dtype, device=dev)
    deq = outputs.get("dequantized")
    with torch.cuda.device(dev):
        nbytes = _lib.load().oc_gptq_workspace_bytes(out, d, groupsize)
        ws = _workspace(nbytes, dev)
        call(
            "oc_gptq_quantize", ptr(weight), weight.stride(0), out, d, ptr(factor.u),
            factor.u.stride(0), ptr(factor.perm) if factor.actorder else None,
            ptr(factor.invperm) if factor.actorder else None, ptr(factor.dead), wbits, groupsize,
            1 if sym else 0, blocksize, 1 if mse else 0, int(q_grid), float(q_norm), sm_count(dev),
            ptr(outputs.get("qweight")),
            ptr(outputs.get("qzeros")), ptr(outputs["scales"]), ptr(outputs.get("scales_f32")),
            ptr(outputs["zeros"]), ld, ptr(outputs.get("codes")), ptr(deq),
            deq.stride(0) if deq is not None else d, _DTYPES[weight.dtype], ptr(ws), ws.numel(), stream_handle(),
        )
    return outputs


def gptq_quantize_batched(weights: torch.Tensor, u: torch.Tensor, dead: torch.Tensor, wbits: int,
                          groupsize: int, sym: bool, perm: Optional[torch.Tensor] = None,
                          invperm: Optional[torch.Tensor] = None, blocksize: int = 128, pack: bool = True,
                          mse: bool = False, q_grid: int = 600, q_norm: float = 2.4):
    """The column loop for a batch of equally shaped problems, each with its own factor: ``weights``
    [B, out, d] fp16 / bf16, ``u`` [B, d, d] fp32, ``dead`` [B, d] uint8, for act-order ``perm`` and
    ``invperm`` [B, d] int32.  One chain of launches for all problems.  Returns a dict of batched
    outputs: qweight / qzeros (packed) or codes / zeros, scales (fp16 [B, G, out]), dequantized
    [B, out, d]."""
    _require_cuda(weights, "weights")
    if weights.dtype not in _DTYPES or weights.dim() != 3 or not weights.is_contiguous():
        raise TypeError("gptq_quantize_batched expects a contiguous [B, out, d] fp16 or bf16 tensor")
    batch, out, d = weights.shape
    dev = weights.device
    if u.shape != (batch, d, d) or u.dtype != torch.float32 or not u.is_contiguous():
        raise ValueError("u must be a contiguous fp32 [B, d, d] tensor")
    groups = 1 if groupsize == -1 else (d + groupsize - 1) // groupsize
    res = {"scales": torch.empty((batch, groups, out), dtype=torch.float16, device=dev),
           "zeros": torch.empty((batch, groups, out), dtype=torch.int32, device=dev),
           "dequantized": torch.empty((batch, out, d), dtype=weights.dtype, device=dev)}
    if pack:
        if wbits not in PACKABLE_WBITS:
            raise ValueError(f"packing supports wbits in {PACKABLE_WBITS}; got {wbits}")
        f = 32 if wbits == 3 else 32 // wbits
        assert d % f == 0 and out % f == 0, "shapes must be divisible by the pack factor"
        res["qweight"] = torch.empty((batch, d * wbits // 32, out), dtype=torch.int32, device=dev)
        res["qzeros"] = torch.empty((batch, groups, out * wbits // 32), dtype=torch.int32, device=dev)
    else:
        res["codes"] = torch.empty((batch, out, d), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        nbytes = _lib.load().oc_gptq_workspace_bytes(out, d, groupsize) * batch
        ws = _workspace(nbytes, dev)
        call("oc_gptq_quantize_batched", batch, ptr(weights), d, out, d, ptr(u), d, ptr(perm), ptr(invperm),
             ptr(dead), wbits, groupsize, 1 if sym else 0, blocksize, 1 if mse else 0, int(q_grid), float(q_norm),
             sm_count(dev), ptr(res.get("qweight")), ptr(res.get("qzeros")), ptr(res["scales"]), None,
             ptr(res["zeros"]), ptr(res.get("codes")), ptr(res["dequantized"]), _DTYPES[weights.dtype], ptr(ws),
             ws.numel(), stream_handle())
    return res


# ---------------------------------------------------------------------------
# QEP weight correction
# ---------------------------------------------------------------------------


def qep_adjust(weight: torch.Tensor, c: torch.Tensor, factor: HessianFactor, perccorr: float):
    """In place: weight ← round16(Wz + perccorr·(Wz·C)·(H+damp·I)⁻¹) for an fp16 or bf16 CUDA weight."""
    _require_cuda(weight, "weight")
    if weight.dtype not in _DTYPES or weight.dim() != 2 or weight.stride(1) != 1:
        raise TypeError("qep_adjust expects a 2-D fp16 or bf16 weight with contiguous rows")
    if c.dtype != torch.float32 or c.stride(1) != 1:
        c = c.float().contiguous()
    out, d = weight.shape
    dev = weight.device
    with torch.cuda.device(dev):
        for r0 in range(0, out, 65535 // 32 * 32):
            rows = min(65535 // 32 * 32, out - r0)
            nbytes = _lib.load().oc_qep_workspace_bytes(rows, d)
            ws = _workspace(nbytes, dev)
            slab = weight[r0 : r0 + rows]
            call(
                "oc_qep_adjust", ptr(slab), slab.stride(0), rows, d, ptr(c), c.stride(0),
                ptr(factor.u), factor.u.stride(0), ptr(factor.perm) if factor.actorder else None,
                ptr(factor.dead), float(perccorr), _DTYPES[weight.dtype], ptr(ws), ws.numel(), stream_handle(),
            )
    return weight


def rtn_quantize(weight: torch.Tensor, wbits: int, groupsize: int, sym: bool):
    """Round-to-nearest group quantization (no Hessian).  Returns dict(codes int32 [out,d],
    scales fp32 [out,G], zeros fp32 [out,G], dequantized [out,d] in the weight's dtype) on the device."""
    _require_cuda(weight, "weight")
    if weight.dtype not in _DTYPES or weight.dim() != 2:
        raise TypeError("rtn_quantize expects a 2-D fp16 or bf16 weight")
    if weight.stride(1) != 1:
        weight = weight.contiguous()
    out, d = weight.shape
    gs = d if groupsize == -1 else groupsize
    if d % gs != 0:
        raise ValueError(f"Tensor shape {d} must be divisible by group size {groupsize}")
    groups = d // gs
    dev = weight.device
    res = {
        "codes": torch.empty((out, d), dtype=torch.int32, device=dev),
        "scales": torch.empty((out, groups), dtype=torch.float32, device=dev),
        "zeros": torch.empty((out, groups), dtype=torch.float32, device=dev),
        "dequantized": torch.empty((out, d), dtype=weight.dtype, device=dev),
    }
    with torch.cuda.device(dev):
        call("oc_rtn_quantize", ptr(weight), weight.stride(0), out, d, wbits, groupsize, 1 if sym else 0,
             ptr(res["scales"]), ptr(res["zeros"]), ptr(res["codes"]), ptr(res["dequantized"]),
             _DTYPES[weight.dtype], stream_handle())
    return res


# ---------------------------------------------------------------------------
# packed layout utilities
# ---------------------------------------------------------------------------


def _pack_factor(wbits: int) -> int:
    if wbits not in PACKABLE_WBITS:
        raise ValueError(f"Unsupported wbits for packing: {wbits}")
    return 32 if wbits == 3 else 32 // wbits


def pack_qweight(codes: torch.Tensor, wbits: int) -> torch.Tensor:
    _require_cuda(codes, "codes")
    f = _pack_factor(wbits)
    out, d = codes.shape
    if wbits == 3:
        assert d % 32 == 0, f"rows ({d}) must be divisible by 32 for 3-bit packing"
    else:
        assert d % f == 0, f"rows ({d}) must be divisible by pack_factor ({f})"
    codes = codes.to(torch.int32).contiguous()
    q = torch.empty((d * wbits // 32, out), dtype=torch.int32, device=codes.device)
    with torch.cuda.device(codes.device):
        call("oc_pack_qweight", ptr(codes), out, d, wbits, ptr(q), stream_handle())
    return q


def unpack_qweight(qweight: torch.Tensor, wbits: int, shape) -> torch.Tensor:
    _require_cuda(qweight, "qweight")
    _pack_factor(wbits)
    out, d = int(shape[0]), int(shape[1])
    qweight = qweight.to(torch.int32).contiguous()
    codes = torch.empty((out, d), dtype=torch.int32, device=qweight.device)
    with torch.cuda.device(qweight.device):
        call("oc_unpack_qweight", ptr(qweight), out, d, wbits, ptr(codes), stream_handle())
    return codes


def pack_qzeros(zeros: torch.Tensor, wbits: int, add: int = 0) -> torch.Tensor:
    _require_cuda(zeros, "zeros")
    f = _pack_factor(wbits)
    groups, out = zeros.shape
    if wbits == 3:
        assert out % 32 == 0, f"rows ({out}) must be divisible by 32 for 3-bit packing"
    else:
        assert out % f == 0, f"rows ({out}) must be divisible by pack_factor ({f})"
    zeros = zeros.to(torch.int32).contiguous()
    q = torch.empty((groups, out * wbits // 32), dtype=torch.int32, device=zeros.device)
    with torch.cuda.device(zeros.device):
        call("oc_pack_qzeros", ptr(zeros), groups, out, wbits, add, ptr(q), stream_handle())
    return q


def unpack_qzeros(qzeros: torch.Tensor, wbits: int, out_features: int, add: int = 0) -> torch.Tensor:
    _require_cuda(qzeros, "qzeros")
    _pack_factor(wbits)
    qzeros = qzeros.to(torch.int32).contiguous()
    groups = qzeros.shape[0]
    z = torch.empty((groups, out_features), dtype=torch.int32, device=qzeros.device)
    with torch.cuda.device(qzeros.device):
        call("oc_unpack_qzeros", ptr(qzeros), groups, out_features, wbits, add, ptr(z), stream_handle())
    return z


def dequantize_packed(qweight, qzeros, scales, g_idx, wbits: int, shape) -> torch.Tensor:
    _require_cuda(qweight, "qweight")
    out, d = int(shape[0]), int(shape[1])
    dev = qweight.device
    qweight = qweight.to(torch.int32).contiguous()
    qzeros = qzeros.to(device=dev, dtype=torch.int32).contiguous()
    scales = scales.to(device=dev, dtype=torch.float16).contiguous()
    if g_idx is not None:
        g_idx = g_idx.to(device=dev, dtype=torch.int32).contiguous()
    w = torch.empty((out, d), dtype=torch.float16, device=dev)
    with torch.cuda.device(dev):
        call("oc_dequantize_packed", ptr(qweight), ptr(qzeros), ptr(scales), ptr(g_idx), out, d,
             wbits, ptr(w), d, stream_handle())
    return w


def rmsnorm_f16(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """weight * fp16(float(x) * rsqrt(mean(float(x)²) + eps)) over the last dimension (fp16)."""
    _require_cuda(x, "x")
    d = x.shape[-1]
    if x.dtype != torch.float16 or weight.dtype != torch.float16:
        raise TypeError("rmsnorm_f16 expects fp16 input and weight")
    x2 = x.reshape(-1, d)
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    y = torch.empty((x2.shape[0], d), dtype=torch.float16, device=x.device)
    with torch.cuda.device(x.device):
        call("oc_rmsnorm_f16", ptr(x2), x2.stride(0), ptr(weight), float(eps), x2.shape[0], d, ptr(y), d,
             stream_handle())
    return y.view(x.shape)


def _dense(x: torch.Tensor) -> bool:
    """True if x's elements occupy one gap-free block of memory without overlap (any dim order)."""
    expect = 1
    for size, stride in sorted(((sz, st) for sz, st in zip(x.shape, x.stride()) if sz != 1), key=lambda p: p[1]):
        if stride != expect:
            return False
        expect *= size
    return True


def rope_supported(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> bool:
    """Whether ``rope_f16`` takes these tensors: fp16 CUDA, x [B, H, S, D] with unit last stride
    and no overlap, cos / sin [B or 1, S, D] of equal strides, D a multiple of 16."""
    if not (x.is_cuda and x.dtype == torch.float16 and x.dim() == 4 and x.stride(3) == 1):
        return False
    if cos.dim() != 3 or sin.shape != cos.shape or cos.dtype != torch.float16 or sin.dtype != torch.float16:
        return False
    if cos.stride() != sin.stride() or cos.stride(2) != 1 or cos.device != x.device or sin.device != x.device:
        return False
    b, _, s_len, d = x.shape
    return (d % 16 == 0 and cos.shape[1] == s_len and cos.shape[2] == d and cos.shape[0] in (1, b)
            and x.numel() > 0 and _dense(x))


def rope_f16(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x*cos + rotate_half(x)*sin for x [B, H, S, D] (any dense layout) and cos / sin [B|1, S, D],
    every operator rounded to fp16 like the unfused torch expression; the result has x's strides."""
    if not rope_supported(x, cos, sin):
        raise TypeError("rope_f16: unsupported tensors (see rope_supported)")
    y = torch.empty_like(x)          # preserve_format: x's strides
    if y.stride() != x.stride():
        raise TypeError("rope_f16: could not allocate an output with the input's layout")
    b, h, s_len, d = x.shape
    cb = 0 if cos.shape[0] == 1 else cos.stride(0)
    with torch.cuda.device(x.device):
        call("oc_rope_f16", ptr(x), ptr(y), ptr(cos), ptr(sin), b, h, s_len, d, x.stride(0), x.stride(1),
             x.stride(2), y.stride(0), y.stride(1), y.stride(2), cb, cos.stride(1), sm_count(x.device),
             stream_handle())
    return y


def swiglu_f16(gate: torch.Tensor, up: torch.Tensor, inplace: bool = False) -> torch.Tensor:
    """fp16(fp16(silu(gate)) * up) for two contiguous fp16 tensors of equal shape; with
    ``inplace`` the result overwrites ``gate``."""
    _require_cuda(gate, "gate")
    if (gate.dtype != torch.float16 or up.dtype != torch.float16 or gate.shape != up.shape
            or not gate.is_contiguous() or not up.is_contiguous() or up.device != gate.device):
        raise TypeError("swiglu_f16 expects two contiguous fp16 tensors of equal shape on one device")
    y = gate if inplace else torch.empty_like(gate)
    with torch.cuda.device(gate.device):
        call("oc_swiglu_f16", ptr(gate), ptr(up), ptr(y), gate.numel(), sm_count(gate.device), stream_handle())
    return y


class _HostCopier:
    """Device -> host copies of result tensors through two reusable page-locked staging buffers.

    A layer's results are a handful of small tensors: copied one by one into pageable memory each
    costs a device synchronisation and runs at a fraction of the link speed, and page-locking fresh
    memory for every result is slower still.  So the tensors are packed into a staging buffer with
    asynchronous copies, and a worker thread moves them on into ordinary host tensors once the
    copies have landed.  In deferred mode the caller does not wait for that: it gets the
    destination tensors at once and calls ``finish`` before anyone reads them."""

    def __init__(self):
        import queue
        import threading

        self._bufs = [None, None]
        self._busy = [None, None]        # threading.Event of the job that last used each buffer
        self._next = 0
        self._jobs = queue.Queue()
        self._pending = []
        self._error = None
        self._thread = None
        self._threading = threading
        self.deferred = False

    def _worker(self):
        while True:
            job = self._jobs.get()
            if job is None:
                return
            event, pairs, done = job
            try:
                event.synchronize()
                for dst, src in pairs:
                    dst.copy_(src)
            except Exception as exc:  # noqa: BLE001 - handed to the caller in finish()
                self._error = exc
            finally:
                done.set()

    def submit(self, tensors):
        todo = [(i, t) for i, t in enumerate(tensors) if t is not None and t.is_cuda]
        outs = list(tensors)
        if not todo:
            return outs
        if any(t.device != todo[0][1].device for _i, t in todo):
            raise ValueError("to_host: the tensors of one call must live on one device")
        if self._thread is None or not self._thread.is_alive():
            self._thread = self._threading.Thread(target=self._worker, daemon=True)
            self._thread.start()
        sizes = [(t.numel() * t.element_size() + 255) // 256 * 256 for _, t in todo]
        total = sum(sizes)
        slot = self._next
        self._next ^= 1
        if self._busy[slot] is not None:
            self._busy[slot].wait()      # the job that used this staging buffer before has drained it
        buf = self._bufs[slot]
        if buf is None or buf.numel() < total:
            buf = torch.empty(max(total, 64 << 20), dtype=torch.uint8, pin_memory=True)
            self._bufs[slot] = buf
        pairs, off = [], 0
        # the copies and the event that guards them go to the tensors' own device
        with torch.cuda.device(todo[0][1].device):
            for (i, t), sz in zip(todo, sizes):
                nbytes = t.numel() * t.element_size()
                view = buf[off : off + nbytes].view(t.dtype).view(t.shape)
                view.copy_(t.contiguous(), non_blocking=True)
                dst = torch.empty(t.shape, dtype=t.dtype)
                pairs.append((dst, view))
                outs[i] = dst
                off += sz
            event = torch.cuda.Event()
            event.record()
        done = self._threading.Event()
        self._busy[slot] = done
        self._pending.append(done)
        self._jobs.put((event, pairs, done))
        if not self.deferred:
            self.finish()
        return outs

    def finish(self):
        for done in self._pending:
            done.wait()
        self._pending = []
        if self._error is not None:
            exc, self._error = self._error, None
            raise exc


_copier = _HostCopier()


class LayerTimer:
    """Device time of a layer's kernels for ``QuantizationResult.quantization_time`` without stopping
    the host: events bracket the work on the current stream.  Outside a ``deferred_host_copies``
    block ``stop`` waits and fills the results at once; inside, the results are filled when the
    block ends (with the host copies)."""

    def __init__(self, device):
        self.device = torch.device(device)
        with torch.cuda.device(self.device):
            self.begin = torch.cuda.Event(enable_timing=True)
            self.begin.record()

    def stop(self, shares):
        """``shares``: [(result, fraction of the elapsed time that belongs to it)]."""
        with torch.cuda.device(self.device):
            end = torch.cuda.Event(enable_timing=True)
            end.record()
        entry = (self.begin, end, list(shares))
        if _copier.deferred:
            _pending_timers.append(entry)
        else:
            _resolve_timer(entry)


_pending_timers: list = []


def _resolve_timer(entry):
    begin, end, shares = entry
    end.synchronize()
    seconds = begin.elapsed_time(end) / 1e3
    for result, fraction in shares:
        result.quantization_time = seconds * fraction


def to_host(tensors):
    """Copy device tensors to ordinary host tensors (None entries pass through).  Outside a
    ``deferred_host_copies`` block the returned tensors are complete; inside, they are filled in the
    background and complete when the block ends (or after ``finish_host_copies``)."""
    return _copier.submit(tensors)


def finish_host_copies():
    _copier.finish()
    while _pending_timers:
        _resolve_timer(_pending_timers.pop(0))


class deferred_host_copies:
    """Context manager: ``to_host`` calls inside return at once; everything is complete on exit."""

    def __enter__(self):
        self._previous = _copier.deferred
        _copier.deferred = True
        return self

    def __exit__(self, *exc):
        _copier.deferred = self._previous
        if not _copier.deferred:
            finish_host_copies()
        return False


def set_gemm_engine(mode: int) -> int:
    """0: fp32 products run on the tensor cores as 3xTF32 when their operands are 16-byte
    aligned (default); 1: always the fp32 FMA kernel.  Returns the previous mode."""
    return _lib.load().oc_set_gemm_engine(int(mode))


def set_gemm_tile_shape(mode: int) -> int:
    """Output tile of the tensor-core engine for plain products: 0 chosen per product (default),
    1 always 128 x 128, 2 always 128 x 256.  Returns the previous setting."""
    return _lib.load().oc_set_gemm_tile_shape(int(mode))


def gemm_tc_status() -> int:
    return _lib.load().oc_gemm_tc_status()


def check_gemm_status():
    """Raise if a tensor-core product on the current device gave up on a bounded pipeline wait
    (its result, and everything computed from it, is invalid).  Reads one device word, so call it
    where the host has synchronised anyway."""
    code = gemm_tc_status()
    if code != 0:
        raise RuntimeError(f"fp32 tensor-core product: a bounded pipeline wait expired (code {code})")


def gemm_f32(a, b, c=None, alpha=1.0, beta=0.0, trans_a=False, trans_b=False, flags=0):
    """fp32 GEMM engine, exposed for tests: C = beta·C + alpha·op(A)·op(B)."""
    _require_cuda(a, "a")
    m = a.shape[1] if trans_a else a.shape[0]
    k = a.shape[0] if trans_a else a.shape[1]
    n = b.shape[0] if trans_b else b.shape[1]
    if c is None:
        c = torch.zeros((m, n), dtype=torch.float32, device=a.device)
    with torch.cuda.device(a.device):
        call("oc_gemm_f32", ptr(a), a.stride(0), ptr(b), b.stride(0), ptr(c), c.stride(0), m, n, k,
             float(alpha), float(beta), int(trans_a), int(trans_b), int(flags), stream_handle())
    return c
