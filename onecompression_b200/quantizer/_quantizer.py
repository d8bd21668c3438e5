"""Quantizer base class: the drop-in mirror of OneComp's ``Quantizer`` protocol for
the GPTQ / QEP path (reference: onecomp/quantizer/_quantizer.py:35-1031).

Same dataclass fields, method names, argument meaning and error behaviour; the
arithmetic behind ``calculate_hessian``, ``calculate_delta_hatX`` and
``adjust_weight`` runs in the CUDA library instead of torch ops.
"""

from __future__ import annotations

import time
from abc import ABCMeta, abstractmethod
from dataclasses import dataclass, field
from logging import getLogger
from typing import Any, Optional, Union

import torch
from torch.nn import Conv1d, Conv2d, Linear

from .. import kernels


@dataclass
class QuantizationResult:
    """Per-layer result record (reference fields, _quantizer.py:35-103)."""

    dequantized_weight: torch.Tensor = None
    quantization_time: float = None
    output_squared_error: float = None
    mean_output_squared_error: float = None
    weight_squared_error: float = None
    mean_weight_squared_error: float = None
    relative_output_squared_error: float = None
    relative_weight_squared_error: float = None

    def compute_dequantized_weight(self, device: torch.device = None) -> torch.Tensor:
        if self.dequantized_weight is None:
            raise NotImplementedError(
                "compute_dequantized_weight() is not implemented. "
                "Subclasses must override this method or set dequantized_weight."
            )
        return self.dequantized_weight.to(torch.float16).cpu()

    def get_statistics(self) -> dict:
        keys = (
            "quantization_time", "output_squared_error", "mean_output_squared_error",
            "weight_squared_error", "mean_weight_squared_error",
            "relative_output_squared_error", "relative_weight_squared_error",
        )
        return {k: getattr(self, k) for k in keys}


def _qep_shift_rule(percdamp_mean_ratio=None):
    """Diagonal shift per attempt of the QEP correction, as a multiple of
    damp₁ = percdamp·mean(diag H).  The reference (adjust_weight,
    _quantizer.py:403-428) recomputes damp from the already damped matrix at every
    attempt and adds 10ᵏ times the latest damp after the k-th failure."""
    state = {"total": 0.0, "last": 0.0, "mult": 1.0}

    def rule(attempt: int, percdamp: float) -> float:
        if attempt > 0:
            state["mult"] *= 10.0
            state["total"] += state["mult"] * state["last"]
        # damp_k = percdamp * (mean + total_so_far) = damp1 * (1 + percdamp * total/damp1 ...)
        # in units of damp1: last = 1 + percdamp * total
        state["last"] = 1.0 + percdamp * state["total"]
        state["total"] += state["last"]
        return state["total"]

    return rule


def qep_factor(hessian, factor, percdamp):
    """The inverse-Hessian factor the QEP correction may use.  The correction damps with its own
    ``percdamp`` and has its own retry rule (reference adjust_weight, _quantizer.py:396-428), so a
    factor made for the column loop serves only if it was built with the same damping and
    succeeded at the first attempt; otherwise the Hessian is factored again under the correction's
    rule."""
    usable = (factor is not None and factor.attempts == 1
              and abs(factor.percdamp - percdamp) < 1e-12)
    if usable:
        return factor
    return kernels.factor_hessian(hessian, percdamp, actorder=False, shifts=_qep_shift_rule())


@dataclass
class Quantizer(metaclass=ABCMeta):
    """Abstract quantizer (fields and defaults as _quantizer.py:171-201).

    Layer selection priority: ``target_layer_types`` → ``include_layer_names`` →
    ``include_layer_keywords`` → ``exclude_layer_names`` → ``exclude_layer_keywords``
    → ``num_layers``.
    """

    name: str = None
    num_layers: int = None
    calc_quant_error: bool = False
    bitpack_on_quantize: bool = False
    include_layer_names: list[str] = None
    exclude_layer_names: list[str] = field(default_factory=lambda: ["lm_head"])
    include_layer_keywords: list[str] = None
    exclude_layer_keywords: list[str] = field(default_factory=lambda: ["per_layer_model_projection"])
    target_layer_types: tuple = field(default_factory=lambda: (Linear,))
    hessian_dtype: torch.dtype = torch.float32
    module_to_name: dict = field(default_factory=dict)
    results: dict = field(default_factory=dict)
    flag_calibration: bool = False
    flag_hessian: bool = False
    flag_xtx: bool = False
    flag_nsamples: bool = False
    flag_qep_supported: bool = True

    def __post_init__(self):
        if self.name is None:
            self.name = type(self).__name__
        self.logger = getLogger(__name__)

    def validate_params(self):
        """Overridden where parameters need checking; called once from setup()."""

    # ------------------------------------------------------------------ drivers' entry points

    def quantize(self, module, input, output, hessian=None, nsamples=None):  # pylint: disable=redefined-builtin
        """Forward-hook entry (register_forward_hook signature; reference :219-257)."""
        name = self.module_to_name[module]
        self.logger.debug("Quantizing layer: %s", name)
        timer = self._start_timer(module)
        if hessian is None and self.flag_hessian:
            hessian, nsamples = self.calculate_hessian(module, input)
        extra = {"nsamples": nsamples} if self.flag_nsamples else {}
        result = self.quantize_layer(module, input, hessian=hessian, **extra)
        if isinstance(result, torch.Tensor):
            result = QuantizationResult(dequantized_weight=result)
        self._stop_timer(timer, result)
        self.results[name] = result
        if self.calc_quant_error:
            self._record_quantization_error(module, name, input, result)

    def quantize_with_qep(self, module, quant_input_activation, original_input_activation=None,
                          percdamp=0.01, perccorr=0.5, hessian=None, delta_hatX=None, nsamples=None,
                          factor=None):
        """Correct the weight for upstream quantization error, then quantize
        (reference :259-333).  ``factor`` optionally carries a ready inverse-Hessian
        factor of ``hessian`` so that layers sharing one input share one factorisation."""
        name = self.module_to_name[module]
        timer = self._start_timer(module)
        if hessian is None and self.flag_hessian:
            hessian, nsamples = self.calculate_hessian(module, quant_input_activation)
        if delta_hatX is not None or original_input_activation is not None:
            self.logger.debug("Adjusting the weight of the layer: %s", name)
            self.adjust_weight(
                module, quant_input_activation, original_input_activation,
                original_hessian=hessian, original_delta_hatX=delta_hatX,
                percdamp=percdamp, perccorr=perccorr, factor=factor,
            )
        self.logger.debug("Quantizing layer: %s", name)
        extra = {"nsamples": nsamples} if self.flag_nsamples else {}
        if factor is not None:
            extra["factor"] = factor
        result = self.quantize_layer(module, quant_input_activation, hessian=hessian, **extra)
        if isinstance(result, torch.Tensor):
            result = QuantizationResult(dequantized_weight=result)
        self._stop_timer(timer, result)
        self.results[name] = result
        if self.calc_quant_error:
            self._record_quantization_error(module, name, quant_input_activation, result)

    @staticmethod
    def _start_timer(module):
        """quantization_time is the device time of the layer's kernels on a CUDA module (events, so
        that a driver which defers the host copies is not stopped per layer), wall time otherwise."""
        if module.weight.is_cuda:
            return kernels.LayerTimer(module.weight.device)
        return time.time()

    @staticmethod
    def _stop_timer(timer, result):
        if isinstance(timer, kernels.LayerTimer):
            timer.stop([(result, 1.0)])
        else:
            result.quantization_time = time.time() - timer

    def _record_quantization_error(self, module, name, input, result):  # pylint: disable=redefined-builtin
        deq = result.compute_dequantized_weight()
        (result.output_squared_error, result.mean_output_squared_error,
         result.relative_output_squared_error) = self.calculate_output_quantization_error(module, input, deq)
        (result.weight_squared_error, result.mean_weight_squared_error,
         result.relative_weight_squared_error) = self.calculate_weight_quantization_error(module, deq)

    # ------------------------------------------------------------------ QEP weight correction

    def adjust_weight(self, module, quant_input_activation, original_input_activation,
                      original_hessian=None, original_delta_hatX=None, percdamp=0.01, perccorr=0.5,
                      factor=None):
        """W ← W + perccorr·(W·C)(H+damp·I)⁻¹, written back in the module's dtype
        (reference :362-432).  The given Hessian / cross term are not modified."""
        if isinstance(module, (Conv2d, Conv1d)):
            raise NotImplementedError("QEP weight correction is implemented for Linear layers")
        if original_hessian is None:
            hessian, _ = self.calculate_hessian(module, quant_input_activation)
        else:
            hessian = original_hessian
        if original_delta_hatX is None:
            delta_hatx = self.calculate_delta_hatX(module, quant_input_activation, original_input_activation)
        else:
            delta_hatx = original_delta_hatX
        weight = module.weight.data
        if not weight.is_cuda:
            raise RuntimeError("adjust_weight: the module must live on a CUDA device (no CPU path)")
        hessian = hessian.to(weight.device)
        delta_hatx = delta_hatx.to(weight.device)
        factor = qep_factor(hessian, factor, percdamp)
        w16 = weight if weight.dtype in (torch.float16, torch.bfloat16) else weight.to(torch.float16)
        w16 = w16.contiguous() if w16.stride(-1) != 1 else w16
        kernels.qep_adjust(w16, delta_hatx, factor, perccorr)
        if w16.data_ptr() != weight.data_ptr():
            module.weight.data = w16.to(weight.dtype)

    @abstractmethod
    def quantize_layer(self, module, input=None, hessian=None) -> Union[torch.Tensor, QuantizationResult]:  # pylint: disable=redefined-builtin
        raise NotImplementedError("quantize_layer method is not implemented")

    # ------------------------------------------------------------------ layer selection

    def _should_quantize_layer(self, name: str, module) -> bool:
        if not isinstance(module, self.target_layer_types):
            return False
        if self.include_layer_names is not None and name not in self.include_layer_names:
            return False
        if self.include_layer_keywords is not None and not any(
            k in name for k in self.include_layer_keywords
        ):
            return False
        if name in self.exclude_layer_names:
            return False
        if self.exclude_layer_keywords is not None and any(
            k in name for k in self.exclude_layer_keywords
        ):
            return False
        return True

    _VLM_TEXT_SUFFIXES = ("language_model", "text_model")

    def _get_text_search_root(self, model):
        for name, mod in model.named_modules():
            if any(name.endswith(s) for s in self._VLM_TEXT_SUFFIXES):
                return mod, name + "."
        return model, ""

    def setup(self, model):
        """Validate parameters and register the target layers (reference :521-562).
        Fused 3-D MoE expert tensors are not split here; pass a model whose experts
        are ``nn.Linear`` modules."""
        self.validate_params()
        assert len(self.module_to_name) == 0
        root, prefix = self._get_text_search_root(model)
        for name, module in root.named_modules():
            full = prefix + name if prefix else name
            if self._should_quantize_layer(full, module):
                self.module_to_name[module] = full
            if self.num_layers is not None and len(self.module_to_name) >= self.num_layers:
                break
        if self.num_layers is not None:
            assert len(self.module_to_name) == self.num_layers, (
                f"Expected {self.num_layers} layers to quantize, "
                f"but found {len(self.module_to_name)}"
            )

    def execute_post_processing(self):
        self.module_to_name = {}

    # ------------------------------------------------------------------ save / inference hooks

    def get_quant_config(self) -> dict:
        raise NotImplementedError(
            f"{type(self).__name__} does not support save_quantized_model. "
            "Override get_quant_config() and create_inference_layer() to enable saving."
        )

    def create_inference_layer(self, result, linear_module, **kwargs):
        raise NotImplementedError(
            f"{type(self).__name__} does not support save_quantized_model. "
            "Override create_inference_layer() to enable saving."
        )

    def apply_results_to_model(self, model, **kwargs):
        for name in list(self.results):
            *parents, attr = name.split(".")
            parent = model
            for p in parents:
                parent = getattr(parent, p)
            layer = self.create_inference_layer(
                result=self.results[name], linear_module=getattr(parent, attr), **kwargs
            )
            setattr(parent, attr, layer)

    def finalize_quant_config_for_save(self, quant_config: dict[str, Any],
                                       quantized_layer_names: list[str],
                                       num_hidden_layers: Optional[int] = None) -> dict[str, Any]:
        return quant_config

    def save_results(self, filepath):
        torch.save(self.results, filepath)
        self.logger.info("Saved quantization results to %s", filepath)

    def load_results(self, filepath, *, weights_only=False, allow_unsafe_deserialization=False):
        if not weights_only and not allow_unsafe_deserialization:
            raise ValueError(
                f"Refusing to load '{filepath}': loading with weights_only=False "
                "deserializes arbitrary Python objects via pickle and can execute "
                "code embedded in a malicious file (CWE-502). Only load result "
                "files from a fully trusted source, then pass "
                "allow_unsafe_deserialization=True to acknowledge this risk, or "
                "use weights_only=True for the safe (tensors-only) path."
            )
        self.results = torch.load(filepath, weights_only=weights_only)
        return self.results

    # ------------------------------------------------------------------ moments

    def calculate_hessian(self, module, input):  # pylint: disable=redefined-builtin
        """(H, nsamples) with H = (2/N)·XᵀX on the module's device (reference :764-832)."""
        x = input[0].detach() if isinstance(input, tuple) else input.detach()
        assert isinstance(module, Linear)
        if x.dim() == 2:
            x = x.unsqueeze(0)
        assert len(x.shape) == 3
        assert x.shape[-1] == module.weight.shape[1]
        device = module.weight.device
        if device.type != "cuda":
            raise RuntimeError("calculate_hessian: the module must live on a CUDA device (no CPU path)")
        acc = kernels.MomentAccumulator(x.shape[-1], device, cross=False)
        step = min(x.shape[0], 8)
        for s in range(0, x.shape[0], step):
            acc.add(x[s : s + step].to(device, non_blocking=True))
        h, _, n = acc.finalize()
        return h, n

    def calculate_delta_hatX(self, module, quant_input_activation, original_input_activation):
        """C = (2/N)(X_f − X_q)ᵀX_q (reference :834-895)."""
        assert isinstance(module, Linear)
        xq, xf = quant_input_activation, original_input_activation
        if xq.dim() == 2:
            xq, xf = xq.unsqueeze(0), xf.unsqueeze(0)
        assert len(xq.shape) == 3 and xq.shape == xf.shape
        assert xq.shape[-1] == module.weight.shape[1]
        device = module.weight.device
        if device.type != "cuda":
            raise RuntimeError("calculate_delta_hatX: the module must live on a CUDA device (no CPU path)")
        acc = kernels.MomentAccumulator(xq.shape[-1], device, cross=True)
        step = min(xq.shape[0], 8)
        for s in range(0, xq.shape[0], step):
            acc.add(xq[s : s + step].to(device, non_blocking=True),
                    xf[s : s + step].to(device, non_blocking=True))
        _, c, _ = acc.finalize()
        return c

    # ------------------------------------------------------------------ error metrics (:897-1031)

    def calculate_weight_quantization_error(self, module, dequantized_weight):
        w = module.weight.data.detach()
        w_hat = dequantized_weight.to(w.device)
        norm2 = torch.sum(w.double().pow(2)).item()
        diff = (w - w_hat).double()
        err = torch.sum(diff * diff).item()
        return err, err / diff.numel(), (err / norm2 if norm2 > 0 else None)

    def calculate_output_quantization_error(self, module, input, dequantized_weight):  # pylint: disable=redefined-builtin
        if input is None:
            return None, None, None
        x = input[0].detach() if isinstance(input, tuple) else input.detach()
        assert len(x.shape) == 3
        w = module.weight.data.detach()
        w_hat = dequantized_weight.to(w.device)
        flat = x.reshape(-1, x.shape[-1])
        step = min(flat.shape[0], 512)
        err = norm2 = 0.0
        count = 0
        for s in range(0, flat.shape[0], step):
            xt = flat[s : s + step].T.to(w.device)
            ref = w @ xt
            norm2 += torch.sum(ref.double().pow(2)).item()
            diff = (ref - w_hat @ xt).double()
            err += torch.sum(diff * diff).item()
            count += diff.numel()
        return err, err / count, (err / norm2 if norm2 > 0 else None)


class ResultLoader:
    """Read a file written by ``Quantizer.save_results`` (reference :1034-1091)."""

    def __init__(self, filepath, *, allow_unsafe_deserialization=False):
        if not allow_unsafe_deserialization:
            raise ValueError(
                f"Refusing to load '{filepath}': result files are pickles; pass "
                "allow_unsafe_deserialization=True for files from a trusted source."
            )
        self.results = torch.load(filepath, weights_only=False)

    def get_layer_names(self):
        return list(self.results)

    def get_result(self, name):
        return self.results[name]
