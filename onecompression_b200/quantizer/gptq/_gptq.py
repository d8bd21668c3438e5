"""GPTQ quantizer with OneComp's API, computing on B200 through the CUDA library
(reference: onecomp/quantizer/gptq/_gptq.py).

``GPTQ``, ``GPTQResult`` and ``run_gptq`` keep the reference's names, fields,
defaults, validation messages and result layout (CPU tensors with the reference's
dtypes), so the drivers and the save path can use them unchanged.
"""

from __future__ import annotations

import logging
import re
from dataclasses import dataclass
from typing import Any, Optional

import torch
from torch import nn

from ... import kernels
from .._quantizer import QuantizationResult, Quantizer
from .gptq_layer import PACKABLE_WBITS, is_packable_wbits, make_g_idx

logger = logging.getLogger(__name__)

GPTQ_MAX_BITS = 15


@dataclass
class GPTQResult(QuantizationResult):
    """Result of one layer (fields as the reference's GPTQResult, _gptq.py:29-82).

    qweight: int32, packed (in·bits/32, out) when ``qweight_is_packed`` else (out, in);
    scales: fp16 (G, out) or (out, 1) per channel; qzeros: int32, packed
    (G, out·bits/32) holding (zero − 1) & mask when ``qzeros_is_packed`` else raw
    (G, out) / (out, 1); perm: int64 (in,) with act-order.  All on the CPU.
    """

    wbits: int = None
    groupsize: int = None
    actorder: bool = None
    sym: bool = None
    qweight: Optional[torch.Tensor] = None
    scales: Optional[torch.Tensor] = None
    qzeros: Optional[torch.Tensor] = None
    perm: Optional[torch.Tensor] = None
    qweight_is_packed: bool = False
    qzeros_is_packed: bool = False
    qweight_original_shape: Optional[tuple[int, int]] = None

    def __getstate__(self):
        # device-side caches (keys starting with "_device") are not part of a saved result
        return {k: v for k, v in self.__dict__.items() if not k.startswith("_device")}

    def compute_dequantized_weight(self, device=None) -> torch.Tensor:
        """Ŵ = fp16(scale·(q − zero)) as an fp16 CPU tensor (reference :84-168).

        Computed on the GPU (``device`` or the current CUDA device)."""
        if self.qweight is None or self.scales is None or self.qzeros is None:
            raise ValueError(
                "Quantized weights, scales, and zero points must be provided to compute dequantized weight."
            )
        dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        if dev.type != "cuda":
            dev = torch.device("cuda", torch.cuda.current_device())
        return self.dequantized_on(dev).cpu()

    def dequantized_on(self, dev) -> torch.Tensor:
        """The same weight, left on the CUDA device ``dev``."""
        bits = self.wbits
        packed_w = bool(getattr(self, "qweight_is_packed", False))
        packed_z = bool(getattr(self, "qzeros_is_packed", False))
        shape = getattr(self, "qweight_original_shape", None)
        qweight = self.qweight.to(dev)
        if packed_w:
            if shape is None:
                raise ValueError("qweight_original_shape is required to unpack packed GPTQ qweight.")
        else:
            shape = tuple(qweight.shape)
        out, d = int(shape[0]), int(shape[1])
        scales = self.scales.to(dev)
        qzeros = self.qzeros.to(dev)
        if self.groupsize == -1:
            scales = scales.reshape(1, out)
            if not packed_z:
                qzeros = qzeros.reshape(1, out)
            g_idx = None
        else:
            groups = (d + self.groupsize - 1) // self.groupsize
            if scales.shape == (out, groups) and out != groups:
                scales = scales.T
            if not packed_z and qzeros.shape == (out, groups) and out != groups:
                qzeros = qzeros.T
            if self.actorder and self.perm is not None and self.perm.numel() != d:
                raise ValueError(f"Invalid perm length: {self.perm.numel()}; expected {d}.")
            g_idx = make_g_idx(self.perm if self.actorder else None, self.groupsize, d, device=dev)
        if not is_packable_wbits(bits) or d % (32 if bits == 3 else 32 // bits) or out % (32 if bits == 3 else 32 // bits):
            return _dequantize_unpacked(
                qweight if not packed_w else kernels.unpack_qweight(qweight, bits, shape),
                scales, qzeros if not packed_z else (kernels.unpack_qzeros(qzeros, bits, out, add=1)),
                g_idx,
            )
        if not packed_w:
            qweight = kernels.pack_qweight(qweight.to(torch.int32), bits)
        if not packed_z:
            qzeros = kernels.pack_qzeros(qzeros.to(torch.int32).contiguous(), bits, add=-1)
        return kernels.dequantize_packed(qweight, qzeros, scales.contiguous(), g_idx, bits, (out, d))


def _dequantize_unpacked(codes, scales, zeros, g_idx):
    """Bit widths or shapes without a packed layout: the same formula through the
    packed kernel is not available, so gather on the device with index ops (plumbing,
    not a hot path: only results that were never packed reach it)."""
    out, d = codes.shape
    if g_idx is None:
        g_idx = torch.zeros(d, dtype=torch.long, device=codes.device)
    g = g_idx.long()
    s = scales[g, :].T.to(torch.float16).float()
    z = zeros[g, :].T.float()
    return (s * (codes.float() - z)).to(torch.float16).contiguous()


@dataclass
class GPTQ(Quantizer):
    """GPTQ quantizer (fields and defaults as the reference, _gptq.py:212-229).

    blocksize ≤ 128 is what the CUDA column kernel implements (larger values raise at
    ``setup``).  Modules must live on a CUDA device.
    """

    flag_calibration: bool = True
    flag_hessian: bool = True

    blocksize: int = 128
    percdamp: float = 0.01
    wbits: int = 4
    groupsize: int = -1
    actorder: bool = False
    mse: bool = False
    sym: bool = True
    q_grid: int = 600
    q_norm: float = 2.4
    mlp_wbits: Optional[int] = None
    mlp_groupsize: Optional[int] = None
    module_wbits: Optional[dict[str, int]] = None
    bitpack_on_quantize: bool = True

    @staticmethod
    def resolve_bits(layer_name, default_bits, mlp_bits=None, module_bits=None) -> int:
        """module_wbits[name] > mlp_wbits (name contains "mlp") > default."""
        if module_bits and layer_name is not None:
            b = module_bits.get(layer_name)
            if b is not None:
                return b
        if mlp_bits is not None and layer_name is not None and "mlp" in layer_name:
            return mlp_bits
        return default_bits

    @staticmethod
    def resolve_groupsize(layer_name, default_groupsize, mlp_groupsize=None) -> int:
        if mlp_groupsize is not None and layer_name is not None and "mlp" in layer_name:
            return mlp_groupsize
        return default_groupsize

    def __post_init__(self):
        if self.name is None:
            self.name = f"GPTQ_{self.wbits}bit"
        self.name += "_perchannel" if self.groupsize == -1 else f"_gs{self.groupsize}"
        super().__post_init__()

    def validate_params(self):
        """Same checks and messages as the reference (:271-383), all failures joined by '; '."""
        bad = []
        is_int = lambda v: isinstance(v, int)  # noqa: E731
        if not (is_int(self.blocksize) and self.blocksize >= 1):
            bad.append(f"Invalid GPTQ parameter 'blocksize': {self.blocksize!r} (expected int >= 1).")
        elif self.blocksize > kernels.MAX_BLOCKSIZE:
            bad.append(
                f"Invalid GPTQ parameter 'blocksize': {self.blocksize!r} "
                f"(the CUDA column kernel handles 1..{kernels.MAX_BLOCKSIZE})."
            )
        if not (isinstance(self.percdamp, (int, float)) and self.percdamp >= 3.95e-4):
            bad.append(
                f"Invalid GPTQ parameter 'percdamp': {self.percdamp!r} (expected numeric >= 3.95e-4)."
            )
        if not (is_int(self.wbits) and 1 <= self.wbits <= GPTQ_MAX_BITS):
            bad.append(
                f"Invalid GPTQ parameter 'wbits': {self.wbits!r} (expected int in 1..{GPTQ_MAX_BITS})."
            )
        if not (is_int(self.groupsize) and (self.groupsize == -1 or self.groupsize >= 1)):
            bad.append(
                f"Invalid GPTQ parameter 'groupsize': {self.groupsize!r} "
                f"(expected int: -1 for no grouping, or >= 1)."
            )
        if self.mse:
            if not (is_int(self.q_grid) and self.q_grid >= 1):
                bad.append(
                    f"Invalid GPTQ parameter 'q_grid': {self.q_grid!r} (expected int >= 1 when mse=True)."
                )
            if not (isinstance(self.q_norm, (int, float)) and self.q_norm > 0):
                bad.append(
                    f"Invalid GPTQ parameter 'q_norm': {self.q_norm!r} (expected numeric > 0 when mse=True)."
                )
        if self.mlp_wbits is not None and not (is_int(self.mlp_wbits) and 1 <= self.mlp_wbits <= GPTQ_MAX_BITS):
            bad.append(
                f"Invalid GPTQ parameter 'mlp_wbits': {self.mlp_wbits!r} (expected int in 1..{GPTQ_MAX_BITS})"
            )
        if self.mlp_groupsize is not None and not (
            is_int(self.mlp_groupsize)
            and (self.mlp_groupsize == -1 or (1 <= self.mlp_groupsize <= self.blocksize))
        ):
            bad.append(
                f"Invalid GPTQ parameter 'mlp_groupsize': {self.mlp_groupsize!r} (expected int -1 or 1..blocksize)"
            )
        if self.module_wbits is not None:
            if not isinstance(self.module_wbits, dict):
                bad.append(
                    "Invalid GPTQ parameter 'module_wbits': must be a dict[str, int], "
                    f"got {type(self.module_wbits).__name__!r}"
                )
            else:
                for layer_name, bits in self.module_wbits.items():
                    if not isinstance(layer_name, str):
                        bad.append("Invalid GPTQ parameter 'module_wbits': keys must be layer name strings.")
                    elif not (is_int(bits) and 1 <= bits <= GPTQ_MAX_BITS):
                        bad.append(
                            f"Invalid GPTQ parameter 'module_wbits[{layer_name!r}]': "
                            f"{bits!r} (expected int in 1..{GPTQ_MAX_BITS})"
                        )
        if not isinstance(self.bitpack_on_quantize, bool):
            bad.append(
                f"Invalid GPTQ parameter 'bitpack_on_quantize': {self.bitpack_on_quantize!r} (expected bool)."
            )
        elif self.bitpack_on_quantize:
            supported = sorted(PACKABLE_WBITS)

            def check(param, bits):
                if is_int(bits) and 1 <= bits <= GPTQ_MAX_BITS and not is_packable_wbits(bits):
                    bad.append(
                        f"Invalid GPTQ parameter '{param}': {bits!r} cannot be used "
                        f"with bitpack_on_quantize=True (expected one of {supported})."
                    )

            check("wbits", self.wbits)
            if self.mlp_wbits is not None:
                check("mlp_wbits", self.mlp_wbits)
            if isinstance(self.module_wbits, dict):
                for layer_name, bits in self.module_wbits.items():
                    if isinstance(layer_name, str):
                        check(f"module_wbits[{layer_name!r}]", bits)
        if bad:
            raise ValueError("; ".join(bad))

    # ------------------------------------------------------------------ one layer

    def quantize_layer(self, module, input=None, hessian=None, factor=None):  # pylint: disable=redefined-builtin
        """Quantize one layer from its Hessian; returns a GPTQResult with CPU tensors
        (reference :385-478).  ``factor`` optionally supplies a ready inverse-Hessian
        factor of ``hessian`` (see ``kernels.factor_hessian``)."""
        layer_name = self.module_to_name.get(module)
        bits = GPTQ.resolve_bits(layer_name, self.wbits, self.mlp_wbits, self.module_wbits)
        gs = GPTQ.resolve_groupsize(layer_name, self.groupsize, self.mlp_groupsize)
        if not (isinstance(bits, int) and 1 <= bits <= GPTQ_MAX_BITS):
            raise ValueError(
                f"Invalid GPTQ resolved wbits for layer {layer_name!r}: {bits!r} "
                f"(expected int in 1..{GPTQ_MAX_BITS})."
            )
        if self.bitpack_on_quantize and not is_packable_wbits(bits):
            raise ValueError(
                f"bitpack_on_quantize=True supports only wbits in {tuple(sorted(PACKABLE_WBITS))}; "
                f"got {bits}. Use bitpack_on_quantize=False for unpacked GPTQ results."
            )
        dev_out = _gptq_device(
            hessian, module, blocksize=self.blocksize, percdamp=self.percdamp, wbits=bits,
            groupsize=gs, actorder=self.actorder, mse=self.mse, sym=self.sym, q_grid=self.q_grid,
            q_norm=self.q_norm, pack=self.bitpack_on_quantize, factor=factor,
        )
        out_features, in_features = dev_out["shape"]
        perm = dev_out["perm"]
        packed = self.bitpack_on_quantize
        qweight, qzeros, scales, perm_host = kernels.to_host([
            dev_out["qweight"] if packed else dev_out["codes"],
            dev_out["qzeros"] if packed else dev_out["zeros"],
            dev_out["scales"], perm,
        ])
        if gs == -1:
            scales = scales.reshape(out_features, 1)
            if not packed:
                qzeros = qzeros.reshape(out_features, 1)
        result = GPTQResult(
            wbits=bits, groupsize=gs, actorder=self.actorder, sym=self.sym, qweight=qweight,
            scales=scales, qzeros=qzeros, perm=perm_host,
            qweight_is_packed=self.bitpack_on_quantize, qzeros_is_packed=self.bitpack_on_quantize,
            qweight_original_shape=(out_features, in_features),
        )
        # fp16 Ŵ left on the device for drivers that propagate it (not pickled)
        result.__dict__["_device_dequantized"] = dev_out["dequantized"]
        return result

    # ------------------------------------------------------------------ several layers, one input

    def stack_key(self, module):
        """Layers with equal keys (and one shared input, hence one Hessian) may be quantized as one
        stacked weight matrix: rows never interact in GPTQ or in the QEP correction, so stacking
        changes no result.  None when the layer cannot take part."""
        if (type(self).quantize_with_qep is not Quantizer.quantize_with_qep
                or type(self).quantize_layer is not GPTQ.quantize_layer):
            return None          # a subclass that hooks the per-layer calls gets per-layer calls
        name = self.module_to_name.get(module)
        w = getattr(module, "weight", None)
        if (name is None or type(module) is not torch.nn.Linear or w is None or not w.is_cuda
                or w.dtype not in (torch.float16, torch.bfloat16) or w.shape[0] % 32 != 0
                or self.calc_quant_error):
            return None
        bits = GPTQ.resolve_bits(name, self.wbits, self.mlp_wbits, self.module_wbits)
        gs = GPTQ.resolve_groupsize(name, self.groupsize, self.mlp_groupsize)
        if self.bitpack_on_quantize and not is_packable_wbits(bits):
            return None
        return (id(self), bits, gs, w.shape[1], w.device, w.dtype)

    def quantize_stacked(self, modules, hessian, factor, delta_hatX=None, percdamp=0.01, perccorr=0.5):
        """``quantize_with_qep`` for several layers that share ``hessian`` (equal ``stack_key``):
        one correction and one column loop over the row-wise concatenation of their weights.
        Returns {module: GPTQResult}; results are identical to the per-layer calls."""
        first = modules[0]
        timer = kernels.LayerTimer(first.weight.device)
        name0 = self.module_to_name[first]
        bits = GPTQ.resolve_bits(name0, self.wbits, self.mlp_wbits, self.module_wbits)
        gs = GPTQ.resolve_groupsize(name0, self.groupsize, self.mlp_groupsize)
        stacked = torch.cat([m.weight.data for m in modules], dim=0)
        rows = [m.weight.shape[0] for m in modules]
        if delta_hatX is not None:
            from .._quantizer import qep_factor

            fac = qep_factor(hessian, factor, percdamp)
            kernels.qep_adjust(stacked, delta_hatX.to(stacked.device), fac, perccorr)
            r0 = 0
            for m, r in zip(modules, rows):        # the corrected weight is the module's weight now
                m.weight.data.copy_(stacked[r0:r0 + r])
                r0 += r
        packed = self.bitpack_on_quantize
        out = kernels.gptq_quantize(
            stacked, factor, wbits=bits, groupsize=gs, sym=self.sym, blocksize=self.blocksize, pack=packed,
            want_codes=not packed, want_dequantized=True, mse=bool(self.mse), q_grid=self.q_grid,
            q_norm=self.q_norm,
        )
        d = stacked.shape[1]
        perm = factor.perm.to(torch.int64) if self.actorder else None
        pieces, r0 = [], 0
        for r in rows:
            if packed:
                pieces += [out["qweight"][:, r0:r0 + r], out["qzeros"][:, r0 * bits // 32:(r0 + r) * bits // 32]]
            else:
                pieces += [out["codes"][r0:r0 + r], out["zeros"][:, r0:r0 + r]]
            pieces.append(out["scales"][:, r0:r0 + r])
            r0 += r
        host = kernels.to_host(pieces + [perm] * len(rows))     # may still be in flight: do not read here
        results, r0 = {}, 0
        for i, (m, r) in enumerate(zip(modules, rows)):
            qweight, qzeros, scales = host[3 * i], host[3 * i + 1], host[3 * i + 2]
            if gs == -1:
                scales = scales.reshape(r, 1)
                if not packed:
                    qzeros = qzeros.reshape(r, 1)
            res = GPTQResult(
                wbits=bits, groupsize=gs, actorder=self.actorder, sym=self.sym, qweight=qweight, scales=scales,
                qzeros=qzeros, perm=host[3 * len(rows) + i],
                qweight_is_packed=packed, qzeros_is_packed=packed, qweight_original_shape=(r, d),
            )
            res.__dict__["_device_dequantized"] = out["dequantized"][r0:r0 + r]
            results[m] = res
            r0 += r
        # device time of the stacked call, shared out by rows (filled with the host copies when the
        # caller defers those)
        timer.stop([(results[m], r / sum(rows)) for m, r in zip(modules, rows)])
        return results

    # ------------------------------------------------------------------ many small layers, own Hessians

    def independent_on_device(self, items):
        """Factor and quantize layers that each come with a Hessian of their own (``items`` =
        [(module, hessian)], no weight correction).  Layers of equal shape and settings are batched:
        one chain of factorisation launches (``kernels.factor_hessians_batched``) and one chain of
        column-loop launches (``kernels.gptq_quantize_batched``) serve all of them, with a single
        device synchronisation for the statuses of the factorisations.  Returns, in the order of ``items``, dicts with the device
        outputs (qweight / qzeros or codes / zeros, scales, dequantized) plus ``perm`` (int64 or
        None), ``bits``, ``gs``, ``seconds``; everything is complete on return."""
        if not items:
            return []
        dev = items[0][0].weight.device
        packed = self.bitpack_on_quantize
        groups = {}
        for idx, (module, _h) in enumerate(items):
            name = self.module_to_name.get(module)
            bits = GPTQ.resolve_bits(name, self.wbits, self.mlp_wbits, self.module_wbits)
            gs = GPTQ.resolve_groupsize(name, self.groupsize, self.mlp_groupsize)
            if packed and not is_packable_wbits(bits):
                raise ValueError(
                    f"bitpack_on_quantize=True supports only wbits in {tuple(sorted(PACKABLE_WBITS))}; "
                    f"got {bits}. Use bitpack_on_quantize=False for unpacked GPTQ results.")
            w = _weight_matrix(module)
            groups.setdefault((tuple(w.shape), w.dtype, bits, gs), []).append(idx)
        done = [None] * len(items)
        for (shape, _dtype, bits, gs), idxs in groups.items():
            out_features, d = shape
            batch = len(idxs)
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
            weights = torch.stack([_weight_matrix(items[i][0]) for i in idxs]).contiguous()
            hs = torch.stack([items[i][1].to(device=dev, dtype=torch.float32) for i in idxs]).contiguous()
            fact = kernels.factor_hessians_batched(hs, self.percdamp, self.actorder)
            u, perm, invperm, dead = fact["u"], fact["perm"], fact["invperm"], fact["dead"]
            status = fact["status"].cpu()                                   # the one synchronisation
            for b in torch.nonzero(status).flatten().tolist():
                fac = kernels.factor_hessian(hs[b], self.percdamp, self.actorder)   # retry rule
                u[b].copy_(fac.u)
                perm[b].copy_(fac.perm)
                invperm[b].copy_(fac.invperm)
                dead[b].copy_(fac.dead)
            out = kernels.gptq_quantize_batched(
                weights, u, dead, bits, gs, self.sym, perm if self.actorder else None,
                invperm if self.actorder else None, blocksize=self.blocksize, pack=packed, mse=bool(self.mse),
                q_grid=self.q_grid, q_norm=self.q_norm)
            ev1.record()
            torch.cuda.synchronize(dev)
            seconds = ev0.elapsed_time(ev1) / 1e3 / batch
            for b, i in enumerate(idxs):
                one = {k: v[b] for k, v in out.items()}
                one.update(perm=perm[b].to(torch.int64) if self.actorder else None, bits=bits, gs=gs,
                           seconds=seconds)
                done[i] = one
        return done

    def quantize_independent(self, items):
        """``independent_on_device`` plus the results: {module: GPTQResult} with CPU tensors, the
        propagated weight left on the device, per-layer ``quantization_time``."""
        results = {}
        packed = self.bitpack_on_quantize
        for (module, _h), out in zip(items, self.independent_on_device(items)):
            out_features, in_features = module.weight.shape[0], module.weight.numel() // module.weight.shape[0]
            host = kernels.to_host([out["qweight"] if packed else out["codes"],
                                    out["qzeros"] if packed else out["zeros"], out["scales"], out["perm"]])
            scales, qzeros = host[2], host[1]
            if out["gs"] == -1:
                scales = scales.reshape(out_features, 1)
                if not packed:
                    qzeros = qzeros.reshape(out_features, 1)
            res = GPTQResult(
                wbits=out["bits"], groupsize=out["gs"], actorder=self.actorder, sym=self.sym, qweight=host[0],
                scales=scales, qzeros=qzeros, perm=host[3], qweight_is_packed=packed, qzeros_is_packed=packed,
                qweight_original_shape=(out_features, in_features))
            res.__dict__["_device_dequantized"] = out["dequantized"]
            res.quantization_time = out["seconds"]
            results[module] = res
        return results

    # ------------------------------------------------------------------ save-side metadata

    def get_quant_config(self) -> dict:
        """quantization_config for saved checkpoints (reference :480-517): v1 zero
        offset (``checkpoint_format`` "gptq"), ``mixed_gptq`` when any override exists."""
        mixed = self.module_wbits or self.mlp_wbits or self.mlp_groupsize is not None
        cfg: dict[str, Any] = {
            "quant_method": "mixed_gptq" if mixed else "gptq",
            "bits": self.wbits,
            "groupsize": self.groupsize,
            "actorder": self.actorder,
            "group_size": self.groupsize,
            "desc_act": self.actorder,
            "sym": self.sym,
            "checkpoint_format": "gptq",
        }
        if self.mlp_wbits is not None:
            cfg["mlp_wbits"] = self.mlp_wbits
        if self.mlp_groupsize is not None:
            cfg["mlp_groupsize"] = self.mlp_groupsize
        if self.module_wbits:
            cfg["module_wbits"] = dict(self.module_wbits)
        return cfg

    @staticmethod
    def _build_quantization_bits(quantized_names, quant_config, num_layers):
        pat = re.compile(r"\.layers\.(\d+)\.(.*)")
        default_bits = quant_config.get("bits", quant_config.get("wbits", 4))
        mlp_bits = quant_config.get("mlp_wbits")
        module_bits = quant_config.get("module_wbits") or {}
        default_gs = quant_config.get("group_size", quant_config.get("groupsize", -1))
        mlp_gs = quant_config.get("mlp_groupsize")
        per_layer: dict[int, dict[str, Any]] = {}
        for name in quantized_names:
            m = pat.search(name)
            if m is None:
                continue
            per_layer.setdefault(int(m.group(1)), {})[m.group(2)] = {
                "bits": GPTQ.resolve_bits(name, default_bits, mlp_bits, module_bits),
                "method": "gptq",
                "params": {"group_size": GPTQ.resolve_groupsize(name, default_gs, mlp_gs)},
            }
        if not per_layer:
            return []
        return [per_layer.get(i, {}) for i in range(num_layers)]

    def finalize_quant_config_for_save(self, quant_config, quantized_layer_names, num_hidden_layers=None):
        if num_hidden_layers is None:
            raise ValueError(
                "num_hidden_layers is required for GPTQ quantization_bits "
                "(Runner passes model.config.num_hidden_layers)"
            )
        quant_config["quantization_bits"] = GPTQ._build_quantization_bits(
            quantized_layer_names, quant_config, num_hidden_layers
        )
        return quant_config


def _create_inference_layer(self, result, linear_module, **kwargs):
    """Build a GPTQLinear from a GPTQResult (reference :568-591)."""
    from .gptq_layer import GPTQLinear

    pack_weights = kwargs.get("pack_weights", True)
    if pack_weights and not is_packable_wbits(result.wbits):
        raise ValueError(
            f"pack_weights=True supports only GPTQ wbits in {tuple(sorted(PACKABLE_WBITS))}; "
            f"got {result.wbits}. Use pack_weights=False for unpacked GPTQ results."
        )
    bias = getattr(linear_module, "bias", None)
    return GPTQLinear.from_quantization_result(
        result=result, bias=bias, device=linear_module.weight.device, pack_weights=pack_weights,
        use_gemlite=kwargs.get("use_gemlite"),
    )


GPTQ.create_inference_layer = _create_inference_layer


def _weight_matrix(layer) -> torch.Tensor:
    """2-D [out, in] view of the layer's weight (Conv2d flattened, Conv1D transposed)."""
    w = layer.weight.data
    if isinstance(layer, nn.Conv2d):
        w = w.flatten(1)
    try:
        from transformers import Conv1D  # optional

        if isinstance(layer, Conv1D):
            w = w.t()
    except ImportError:  # pragma: no cover
        pass
    return w


def _gptq_device(hessian, layer, blocksize, percdamp, wbits, groupsize, actorder, mse, sym, q_grid,
                 q_norm, pack, factor=None):
    """The whole layer on the GPU; returns device tensors."""
    w = _weight_matrix(layer)
    if not w.is_cuda:
        raise RuntimeError("GPTQ: the layer must live on a CUDA device (this build has no CPU path)")
    if w.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError(f"GPTQ: fp16 or bf16 weights expected, got {w.dtype}")
    if factor is None:
        if hessian is None:
            raise ValueError("GPTQ needs the layer's Hessian")
        factor = kernels.factor_hessian(hessian.to(w.device), percdamp, actorder)
    out = kernels.gptq_quantize(
        w, factor, wbits=wbits, groupsize=groupsize, sym=sym, blocksize=blocksize, pack=pack,
        want_codes=not pack, want_dequantized=True, mse=bool(mse), q_grid=q_grid, q_norm=q_norm,
    )
    out["shape"] = (w.shape[0], w.shape[1])
    out["perm"] = factor.perm.to(torch.int64) if actorder else None
    return out


def run_gptq(hessian, layer, blocksize=128, percdamp=0.01, wbits=GPTQ_MAX_BITS, groupsize=-1,
             actorder=False, mse=False, sym=True, q_grid=600, q_norm=2.4):
    """Functional form with the reference's signature and return value (:646-794):
    dict(qweight int32 [out,in] CPU, scales fp16 [G,out] or [out,1], qzeros int32
    [G,out] or [out,1], perm int64 or None).  ``hessian`` is left unchanged."""
    dev = _gptq_device(hessian, layer, blocksize, percdamp, wbits, groupsize, actorder, mse, sym,
                       q_grid, q_norm, pack=False)
    out_features = dev["shape"][0]
    scales, zeros = dev["scales"].cpu(), dev["zeros"].cpu()
    if groupsize == -1:
        scales, zeros = scales.reshape(out_features, 1), zeros.reshape(out_features, 1)
    codes = dev["codes"].cpu()
    try:
        from transformers import Conv1D

        if isinstance(layer, Conv1D):
            codes = codes.t()
    except ImportError:  # pragma: no cover
        pass
    return {
        "qweight": codes.reshape(layer.weight.shape),
        "scales": scales,
        "qzeros": zeros,
        "perm": dev["perm"].cpu() if dev["perm"] is not None else None,
    }
