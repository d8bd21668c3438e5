"""Calibration in chunks without error propagation (reference:
onecomp/runner_methods/chunked_quantization.py:48-334).

The model runs over the calibration set ``batch_size`` sequences at a time; forward hooks
fold each target layer's input into its Hessian on the GPU; then every layer is quantized
from its Hessian.  The reference accumulates XᵀX in fp64 per layer and forms
H = (2/n)·XᵀX; here H comes from the tensor-core moment kernel (exact fp16 products, fp32
sums in bounded chains, measured 2e-6 from the exact moment), and layers that receive the very
same input tensor (q/k/v, gate/up) share one accumulation.
"""

from __future__ import annotations

from logging import getLogger
from typing import List, Optional

import torch

from .. import kernels
from ..quantizer._quantizer import Quantizer

logger = getLogger(__name__)


@torch.no_grad()
def accumulate_moments(model, inputs, group, batch_size: int, device=None):
    """{module: (H, nsamples)} for the (module, name) pairs of ``group``."""
    ids = inputs["input_ids"]
    extra = {k: v for k, v in inputs.items() if k != "input_ids"}
    device = device or next(model.parameters()).device
    modules = [m for m, _ in group]
    seen = []

    def hook(module, inp, _out):
        seen.append((module, inp[0] if isinstance(inp, tuple) else inp))

    handles = [m.register_forward_hook(hook) for m in modules]
    accs, owner = {}, {}
    try:
        for first in range(0, ids.shape[0], batch_size):
            part = {k: (v[first : first + batch_size].to(device) if isinstance(v, torch.Tensor) and v.dim() >= 1 else v)
                    for k, v in extra.items()}
            model(ids[first : first + batch_size].to(device), use_cache=False, **part)
            by_tensor = {}
            for module, x in seen:
                by_tensor.setdefault(id(x), (x, []))[1].append(module)
            for x, mods in by_tensor.values():
                # layers fed by the same tensor object share one accumulation; the sharing
                # pattern is fixed by the first chunk
                lead = owner.setdefault(mods[0], mods[0])
                for m in mods:
                    if owner.setdefault(m, lead) is not lead:
                        raise RuntimeError("input sharing between layers changed from one chunk to the next")
                if lead not in accs:
                    accs[lead] = kernels.MomentAccumulator(x.shape[-1], x.device)
                accs[lead].add(x)
            seen.clear()
    finally:
        for h in handles:
            h.remove()
    finished = {lead: acc.finalize() for lead, acc in accs.items()}
    out = {}
    for m in modules:
        lead = owner.get(m)
        if lead is None:
            continue
        h, _c, n = finished[lead]
        out[m] = (h, n)
    return out


def quantize_group(quantizer: Quantizer, group, moments):
    """Quantize every layer of ``group`` from its Hessian (reference :280-334)."""
    factors = {}
    for module, name in group:
        if module not in moments:
            logger.warning("Layer %s received no calibration input; skipped", name)
            continue
        h, n = moments[module]
        extra = {}
        # layers that share one Hessian share its factorisation
        if hasattr(quantizer, "percdamp") and hasattr(quantizer, "actorder"):
            key = h.data_ptr()
            if key not in factors:
                factors[key] = kernels.factor_hessian(h, quantizer.percdamp, quantizer.actorder)
            extra["factor"] = factors[key]
        import time

        t0 = time.time()
        result = quantizer.quantize_layer(module, None, hessian=h, **extra)
        if module.weight.is_cuda:
            torch.cuda.synchronize(module.weight.device)
        result.quantization_time = time.time() - t0
        quantizer.results[name] = result


@torch.no_grad()
def run_chunked_quantization(model_config, quantizers: List[Quantizer], calibration_config=None, *,
                             report_progress: bool = True, model=None, model_inputs=None,
                             batch_size: Optional[int] = None, num_layers_per_group: Optional[int] = None):
    """Quantize with every quantizer of ``quantizers`` from shared Hessians.

    ``model`` (on a CUDA device) and ``model_inputs`` ({"input_ids": …}) may be passed directly;
    otherwise ``model_config.load_model()`` and ``calibration_config.model_inputs`` supply them.
    ``batch_size`` / ``num_layers_per_group`` default to the calibration config's values."""
    if model is None:
        model = model_config.load_model()
    if model_inputs is None:
        model_inputs = getattr(calibration_config, "model_inputs", None)
        if model_inputs is None:
            raise ValueError("pass model_inputs (or a calibration_config that carries them)")
    batch_size = batch_size or getattr(calibration_config, "batch_size", None) or 8
    per_group = num_layers_per_group or getattr(calibration_config, "num_layers_per_group", None) or 7
    for q in quantizers:
        q.setup(model)
    names = [list(q.module_to_name.values()) for q in quantizers]
    if not all(n == names[0] for n in names[1:]):
        raise ValueError(
            "All quantizers must target the same layers. Got:\n"
            + "\n".join(f"  {q.name}: {n}" for q, n in zip(quantizers, names))
        )
    layers = list(quantizers[0].module_to_name.items())
    n_groups = (len(layers) + per_group - 1) // per_group
    for gi, start in enumerate(range(0, len(layers), per_group)):
        group = layers[start : start + per_group]
        moments = accumulate_moments(model, model_inputs, group, batch_size)
        for q in quantizers:
            # every quantizer has its own module -> name map over the same modules
            own = [(m, q.module_to_name[m]) for m, _ in group]
            quantize_group(q, own, moments)
        if report_progress:
            logger.info("[progress] Chunked quantization %d/%d", gi + 1, n_groups)
    for q in quantizers:
        q.execute_post_processing()
