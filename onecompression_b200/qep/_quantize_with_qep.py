"""Generic (architecture-independent) QEP driver (reference: onecomp/qep/_quantize_with_qep.py:35-133).

Layer by layer, in the order the quantizer registered them: the input of the layer in the partly
quantized model is captured with a forward pass, the layer is corrected against the input it has
in the original model, quantized, and replaced by its dequantized weight.  Each layer computes its
own Hessian and cross term from the captured activations (``Quantizer.calculate_hessian`` /
``calculate_delta_hatX``, slices of eight sequences), so this path needs nothing from the model but
``model(**inputs)``; it costs one forward pass per layer and is the slow, general alternative to
the block-wise driver.

The passes run ``batch_size`` sequences at a time and stop at the captured layer; activations are
kept on ``store_device`` (the host by default, as in the reference, since all layers' original
inputs are held at once).
"""

from __future__ import annotations

from logging import getLogger
from typing import Optional

import torch

from ..quantizer._quantizer import Quantizer
from ._qep_config import QEPConfig
from .blockwise import StopForward

logger = getLogger(__name__)


def _chunks(inputs: dict, batch_size: int):
    n = next(v.shape[0] for v in inputs.values() if isinstance(v, torch.Tensor) and v.dim() >= 1)
    for first in range(0, n, batch_size):
        yield {k: (v[first : first + batch_size] if isinstance(v, torch.Tensor) and v.dim() >= 1 else v)
               for k, v in inputs.items()}


@torch.no_grad()
def capture_input_activations(model, inputs, module_to_name, exclude_layer_keywords=None, batch_size=16,
                              store_device="cpu", stop_after_last=False):
    """{name: input activations [N, S, d] on ``store_device``} of the given layers over the whole
    calibration set (reference onecomp/utils/activation_capture.py:17-110).  With
    ``stop_after_last`` a pass ends as soon as every wanted layer has been seen."""
    exclude = exclude_layer_keywords or []
    wanted = {m: n for m, n in module_to_name.items() if not any(k in n for k in exclude)}
    parts = {n: [] for n in wanted.values()}
    seen = set()

    def hook(module, args):
        x = args[0] if isinstance(args, tuple) else args
        parts[wanted[module]].append(x.detach().to(store_device))
        seen.add(module)
        if stop_after_last and len(seen) == len(wanted):
            raise StopForward()

    handles = [m.register_forward_pre_hook(hook) for m in wanted]
    device = next(model.parameters()).device
    try:
        for chunk in _chunks(inputs, batch_size):
            seen.clear()
            chunk = {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in chunk.items()}
            try:
                model(**chunk)
            except StopForward:
                pass
    finally:
        for h in handles:
            h.remove()
    return {n: torch.cat(p) for n, p in parts.items() if p}


@torch.no_grad()
def run_quantize_with_qep(model_config, quantizer: Quantizer, qep_config: QEPConfig, calibration_config=None, *,
                          report_progress: bool = True, model=None, model_inputs: Optional[dict] = None,
                          batch_size: int = 16, store_device="cpu"):
    """Quantize every target layer of ``model`` with QEP, one layer at a time.

    ``model`` (on a CUDA device) and ``model_inputs`` ({"input_ids": ..., ...}) can be given directly;
    otherwise ``model_config.load_model()`` and ``calibration_config.model_inputs`` supply them.
    Results land in ``quantizer.results``; the model ends up holding the dequantized weights."""
    if model is None:
        model = model_config.load_model()
    if model_inputs is None:
        model_inputs = getattr(calibration_config, "model_inputs", None)
        if model_inputs is None:
            raise ValueError("pass model_inputs (or a calibration_config that carries them)")
    if next(model.parameters()).device.type != "cuda":
        raise RuntimeError("run_quantize_with_qep computes on a CUDA device only: move the model there")
    inputs = dict(model_inputs)
    inputs.setdefault("use_cache", False)

    quantizer.setup(model)
    # 1. inputs of every corrected layer in the original model
    original = capture_input_activations(model, inputs, quantizer.module_to_name,
                                         exclude_layer_keywords=qep_config.exclude_layer_keywords,
                                         batch_size=batch_size, store_device=store_device)
    logger.info("Quantizing the model using %s", quantizer.name)
    total = len(quantizer.module_to_name)
    # 2. layer by layer
    for k, (module, name) in enumerate(list(quantizer.module_to_name.items())):
        xq = capture_input_activations(model, inputs, {module: name}, batch_size=batch_size,
                                       store_device=store_device, stop_after_last=True)[name]
        quantizer.quantize_with_qep(module, xq, original_input_activation=original.pop(name, None),
                                    percdamp=qep_config.percdamp, perccorr=qep_config.perccorr)
        result = quantizer.results[name]
        w_hat = result.__dict__.pop("_device_dequantized", None)
        if w_hat is None:
            w_hat = result.compute_dequantized_weight().to(module.weight.device)
        module.weight.data = w_hat.to(module.weight.dtype).reshape(module.weight.shape)
        del xq
        if report_progress:
            logger.info("[progress] QEP quantization (general, per layer) %d/%d %s", k + 1, total, name)
    quantizer.execute_post_processing()
