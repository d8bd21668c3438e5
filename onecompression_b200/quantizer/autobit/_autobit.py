"""Mixed-precision assignment for GPTQ: which candidate quantizer each layer gets under an
average bits-per-weight budget (reference: onecomp/quantizer/autobit/_autobit.py:45-706,
onecomp/quantizer/autobit/ilp.py:19-355).

Same problem statement as the reference: one candidate per layer, layers that an inference engine
fuses (q/k/v, gate/up) share a candidate, Σ effective-bits·params ≤ target·Σ params, minimise the
sum of per-layer round-to-nearest errors (optionally weighted by the input second moments).  The
reference hands this multiple-choice knapsack to OR-Tools' SCIP; this module solves it exactly
with a Pareto dynamic programme (the candidate costs are integers once multiplied by the group
sizes), so it needs no solver package.  The RTN errors are computed on the GPU.

``collect_activation_stats`` gathers the two diagonals of the activation-aware cost with forward
and backward hooks.  Not covered here: the DBF fallback for budgets below 2 bits.
"""

from __future__ import annotations

import re
from dataclasses import dataclass, field
from typing import Union

import torch

from ... import kernels
from .._quantizer import QuantizationResult, Quantizer
from ..gptq._gptq import GPTQ
from ..gptq.gptq_layer import PACKABLE_WBITS


def effective_bits_per_param(wbits, group_size=128, scale_bits=16, zero_bits=None, in_features=None):
    """Bits per weight including the fp16 scale and the packed zero of every group
    (reference onecomp/utils/vram_estimator.py:16-44)."""
    if zero_bits is None:
        zero_bits = wbits
    meta = scale_bits + zero_bits
    if group_size > 0:
        return wbits + meta / group_size
    if in_features is not None and in_features > 0:
        return wbits + meta / in_features
    return float(wbits)


def collect_activation_stats(model, input_ids, candidates, batch_size=4, use_curvature_b=True):
    """Diagonal statistics of the activation-aware cost (reference
    onecomp/quantizer/autobit/activation_stats.py:75-282): for every candidate layer
    a[name] = E_tokens[x_p²] over its input channels and, with ``use_curvature_b``,
    b[name] = E_tokens[(∂L/∂y_q)²] over its output channels, L being the mean next-token
    cross-entropy of each calibration sequence taken on its own.

    ``candidates`` is a list of (name, module); ``input_ids`` [n_seq, seq] lives on the model's
    device.  The whole model is differentiated at once (the reference walks block by block to fit
    large models in memory; the statistics are the same).  Returns (a, b) dicts of fp32 tensors on
    the CPU; b[name] is None without curvature."""
    import torch.nn.functional as F

    a_acc = {n: torch.zeros(m.weight.shape[1], dtype=torch.float64) for n, m in candidates}
    b_acc = {n: torch.zeros(m.weight.shape[0], dtype=torch.float64) for n, m in candidates}
    counts = {n: 0 for n, _ in candidates}
    hooks = []

    def fwd(name):
        def hook(_m, inp, _out):
            x = inp[0].detach().float().reshape(-1, inp[0].shape[-1])
            a_acc[name] += x.pow(2).sum(0).double().cpu()
            counts[name] += x.shape[0]
        return hook

    def bwd(name):
        def hook(_m, _gin, gout):
            if gout[0] is not None:
                g = gout[0].detach().float().reshape(-1, gout[0].shape[-1])
                b_acc[name] += g.pow(2).sum(0).double().cpu()
        return hook

    for name, module in candidates:
        hooks.append(module.register_forward_hook(fwd(name)))
        if use_curvature_b:
            hooks.append(module.register_full_backward_hook(bwd(name)))
    flags = {p: p.requires_grad for p in model.parameters()}
    try:
        for p in flags:
            p.requires_grad_(use_curvature_b)
        for first in range(0, input_ids.shape[0], batch_size):
            ids = input_ids[first:first + batch_size]
            with torch.set_grad_enabled(use_curvature_b):
                logits = model(input_ids=ids).logits
                if use_curvature_b:
                    per_tok = F.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]).float(),
                                              ids[:, 1:].reshape(-1), reduction="none")
                    per_tok.view(ids.shape[0], -1).mean(1).sum().backward()
            model.zero_grad(set_to_none=True)
    finally:
        for h in hooks:
            h.remove()
        for p, f in flags.items():
            p.requires_grad_(f)
    a = {n: (a_acc[n] / max(counts[n], 1)).float() for n in a_acc}
    b = {n: ((b_acc[n] / max(counts[n], 1)).float() if use_curvature_b else None) for n in b_acc}
    return a, b


def solve_assignment(errors, params, eff_bits, target_bit, fused_groups=None, max_states=400000):
    """Exact multiple-choice knapsack: returns the chosen candidate index per module.

    errors[m][b], eff_bits[m][b]: error and effective bits per weight of candidate b for module m;
    params[m]: weights in module m; fused_groups: lists of module indices that must agree.
    Minimises Σ errors subject to Σ eff_bits·params ≤ target_bit·Σ params (reference ilp.py:263-355).
    States are (cost, error) pairs kept Pareto-optimal; if their number ever exceeded
    ``max_states`` the costs of neighbouring states would be merged (not exact any more); the
    return value's second element tells whether that happened.
    """
    n = len(errors)
    nb = len(errors[0]) if n else 0
    budget = target_bit * sum(params)
    # tie fused modules into one item
    owner = list(range(n))
    for group in fused_groups or []:
        for m in group[1:]:
            owner[m] = owner[group[0]]
    items = {}
    for m in range(n):
        items.setdefault(owner[m], []).append(m)
    order = sorted(items)
    # Pareto front after each item: arrays cost, err, and back-pointers
    cost = torch.zeros(1, dtype=torch.float64)
    err = torch.zeros(1, dtype=torch.float64)
    back = []
    thinned = False
    scale = max(max(max(e) for e in errors), 1e-300) if n else 1.0
    for key in order:
        mods = items[key]
        c_b = torch.tensor([sum(eff_bits[m][b] * params[m] for m in mods) for b in range(nb)], dtype=torch.float64)
        e_b = torch.tensor([sum(errors[m][b] for m in mods) / scale for b in range(nb)], dtype=torch.float64)
        nc = (cost[:, None] + c_b[None, :]).reshape(-1)
        ne = (err[:, None] + e_b[None, :]).reshape(-1)
        src = torch.arange(cost.numel()).repeat_interleave(nb)
        ch = torch.arange(nb).repeat(cost.numel())
        keep = nc <= budget * (1 + 1e-12)
        nc, ne, src, ch = nc[keep], ne[keep], src[keep], ch[keep]
        if nc.numel() == 0:
            raise RuntimeError(
                f"bit assignment is infeasible: target_bit={target_bit} is below every candidate")
        # Pareto filter: sort by cost, keep strictly decreasing error
        idx = torch.argsort(nc, stable=True)
        nc, ne, src, ch = nc[idx], ne[idx], src[idx], ch[idx]
        run_min = torch.cummin(ne, 0).values
        prev = torch.cat([torch.tensor([float("inf")], dtype=torch.float64), run_min[:-1]])
        good = ne < prev
        nc, ne, src, ch = nc[good], ne[good], src[good], ch[good]
        if nc.numel() > max_states:
            pick = torch.linspace(0, nc.numel() - 1, max_states).long().unique()
            nc, ne, src, ch = nc[pick], ne[pick], src[pick], ch[pick]
            thinned = True
        back.append((src, ch))
        cost, err = nc, ne
    state = int(torch.argmin(err))
    chosen_items = {}
    for key, (src, ch) in zip(reversed(order), reversed(back)):
        chosen_items[key] = int(ch[state])
        state = int(src[state])
    return [chosen_items[owner[m]] for m in range(n)], thinned


@dataclass
class AutoBitQuantizer(Quantizer):
    """Assigns every target layer to one of ``quantizers`` (GPTQ candidates) under ``target_bit``
    and dispatches ``quantize_layer`` to the assigned candidate.

    assignment_strategy: "ilp" (RTN error Σ ΔW²), "activation_aware" (Σ b_q·a_p·ΔW_qp² with
    ``input_moments`` {layer name: a [in]} and ``output_curvature`` {layer name: b [out]} supplied
    by the caller; as in the reference the weighting applies only when both are present), or
    "manual" (each candidate's own include/exclude rules decide).
    target_bit: average bits per weight; raw bit-widths are converted to the effective budget of
    the uniform baseline (scale and zero overhead included) unless ``target_bit_is_effective``.
    """

    quantizers: list = field(default_factory=list)
    assignment_strategy: str = "ilp"
    target_bit: float = None
    target_bit_is_effective: bool = False
    input_moments: dict = None
    output_curvature: dict = None
    calibration_input_ids: torch.Tensor = None     # used to collect the two statistics when absent
    use_curvature_b: bool = True
    stats_batch_size: int = 4
    bitpack_on_quantize: bool = True
    fused_groups: list = field(default_factory=lambda: [
        ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"],
        ["mlp.gate_proj", "mlp.up_proj"],
    ])
    enable_fused_groups: bool = True
    _module_to_quantizer: dict = field(default_factory=dict, repr=False, init=False)
    _name_to_quantizer: dict = field(default_factory=dict, repr=False, init=False)

    def __post_init__(self):
        super().__post_init__()
        if not self.quantizers:
            raise ValueError("quantizers must be provided")
        if self.assignment_strategy not in ("ilp", "activation_aware", "manual"):
            raise ValueError(f"unknown assignment_strategy {self.assignment_strategy!r}")
        self.flag_calibration = any(q.flag_calibration for q in self.quantizers)
        self.flag_hessian = any(q.flag_hessian for q in self.quantizers)
        self.flag_qep_supported = all(q.flag_qep_supported for q in self.quantizers)

    # attributes the block driver reads on a GPTQ-like quantizer
    @property
    def percdamp(self):
        return self.quantizers[0].percdamp

    @property
    def actorder(self):
        return self.quantizers[0].actorder

    def validate_params(self):
        bad = []
        if self.target_bit is not None and (
            not isinstance(self.target_bit, (int, float)) or self.target_bit <= 0
        ):
            bad.append(f"Invalid parameter 'target_bit': {self.target_bit!r} (expected positive number or None)")
        for i, q in enumerate(self.quantizers):
            if not isinstance(q, GPTQ):
                bad.append(f"quantizers[{i}] ({type(q).__name__}): candidates must be GPTQ quantizers")
            elif self.enable_fused_groups and q.wbits not in PACKABLE_WBITS:
                bad.append(
                    f"quantizers[{i}] (GPTQ wbits={q.wbits}): "
                    f"vLLM only supports GPTQ bit-widths {sorted(PACKABLE_WBITS)}")
        if self.assignment_strategy != "manual" and self.target_bit is None:
            bad.append("target_bit must be set when using the ILP strategy. "
                       "Example: AutoBitQuantizer(..., target_bit=4.0)")
        if bad:
            raise ValueError("; ".join(bad))
        for q in self.quantizers:
            q.bitpack_on_quantize = self.bitpack_on_quantize
            q.validate_params()

    # ---- assignment ------------------------------------------------------------------
    def _candidates(self, model):
        root, prefix = self._get_text_search_root(model)
        out = []
        for name, module in root.named_modules():
            full = prefix + name if prefix else name
            if self._should_quantize_layer(full, module):
                out.append((full, module))
            if self.num_layers is not None and len(out) >= self.num_layers:
                break
        return out

    def _effective_target(self, cands):
        """Raw target → effective budget of the uniform baseline, averaged over the candidates'
        group sizes (reference _autobit.py:390-432)."""
        gss = [q.groupsize or -1 for q in self.quantizers]
        total = sum(m.weight.numel() for _, m in cands)
        bits = 0.0
        for _, m in cands:
            eff = [effective_bits_per_param(self.target_bit, gs, in_features=m.weight.shape[1]) for gs in gss]
            bits += sum(eff) / len(eff) * m.weight.numel()
        return bits / total

    def _rtn_errors(self, name, module):
        """Σ(ΔW)² (optionally Σ a_p ΔW_qp²) of asymmetric RTN for every candidate
        (reference ilp.py:218-260)."""
        w = module.weight.data
        if not w.is_cuda:
            raise RuntimeError("AutoBit evaluates its RTN errors on the GPU: move the model to a CUDA device")
        w16 = w if w.dtype in (torch.float16, torch.bfloat16) else w.half()
        a = b = None
        if (self.assignment_strategy == "activation_aware" and self.input_moments is not None
                and self.output_curvature is not None):
            a = self.input_moments[name].to(w.device).float()
            b = self.output_curvature[name].to(w.device).float()
        errs = []
        for q in self.quantizers:
            d = w16.shape[1]
            gs = q.groupsize if (q.groupsize == -1 or d % q.groupsize == 0) else -1
            deq = kernels.rtn_quantize(w16, q.wbits, gs, sym=False)["dequantized"]
            dw2 = (w16.float() - deq.float()).pow(2)
            errs.append(float(b @ (dw2 @ a) if a is not None else dw2.sum()))
        return errs

    def _fused_index_groups(self, cands):
        pat = re.compile(r"\.layers\.(\d+)\.(.*)")
        groups = {}
        for i, (name, _) in enumerate(cands):
            m = pat.search(name)
            if m is None:
                continue
            for gi, suffixes in enumerate(self.fused_groups):
                if m.group(2) in suffixes:
                    groups.setdefault((int(m.group(1)), gi), []).append(i)
                    break
        return [g for g in groups.values() if len(g) >= 2]

    def setup(self, model):
        self.validate_params()
        assert len(self.module_to_name) == 0
        self._module_to_quantizer, self._name_to_quantizer, self.results = {}, {}, {}
        if self.assignment_strategy == "manual":
            pairs = []
            for name, module in self._candidates(model):
                for q in self.quantizers:
                    if q._should_quantize_layer(name, module):
                        pairs.append((name, module, q))
                        break
        else:
            cands = self._candidates(model)
            if (self.assignment_strategy == "activation_aware" and self.input_moments is None
                    and self.calibration_input_ids is not None):
                self.input_moments, self.output_curvature = collect_activation_stats(
                    model, self.calibration_input_ids, cands, self.stats_batch_size, self.use_curvature_b)
                if not self.use_curvature_b:
                    self.output_curvature = None
            target = self.target_bit if self.target_bit_is_effective else self._effective_target(cands)
            self.effective_target_bit = target
            errors = [self._rtn_errors(n, m) for n, m in cands]
            params = [m.weight.numel() for _, m in cands]
            eff = [[effective_bits_per_param(q.wbits, q.groupsize or -1, in_features=m.weight.shape[1])
                    for q in self.quantizers] for _, m in cands]
            fused = self._fused_index_groups(cands) if self.enable_fused_groups else []
            chosen, thinned = solve_assignment(errors, params, eff, target, fused)
            if thinned:
                self.logger.warning("bit assignment: state set was thinned; the result may be slightly sub-optimal")
            pairs = [(n, m, self.quantizers[b]) for (n, m), b in zip(cands, chosen)]
            total = sum(params)
            used = sum(eff[i][b] * params[i] for i, b in enumerate(chosen)) / total
            self.logger.info("AutoBit: %.4f effective bpw (target %.4f)", used, target)
        for name, module, q in pairs:
            self.module_to_name[module] = name
            self._module_to_quantizer[module] = q
            self._name_to_quantizer[name] = q
            q.module_to_name[module] = name

    # ---- dispatch --------------------------------------------------------------------
    def child_for(self, module):
        """The candidate assigned to ``module`` (None before setup or for other modules)."""
        return self._module_to_quantizer.get(module)

    def quantize_layer(self, module, input=None, hessian=None, nsamples=None, **kw  # pylint: disable=redefined-builtin
                       ) -> Union[torch.Tensor, QuantizationResult]:
        child = self._module_to_quantizer.get(module)
        if child is None:
            raise RuntimeError("Module is not assigned to any child quantizer. Ensure setup() has been called.")
        return child.quantize_layer(module, input, hessian, **kw)

    def execute_post_processing(self):
        for q in self.quantizers:
            q.execute_post_processing()
        self.module_to_name = {}
        self._module_to_quantizer = {}

    def _all_children_gptq(self) -> bool:
        return bool(self._name_to_quantizer) and all(isinstance(q, GPTQ) for q in self._name_to_quantizer.values())

    def get_quant_config(self) -> dict:
        """mixed_gptq config: the default candidate plus a per-module bit map."""
        base = self.quantizers[0]
        cfg = base.get_quant_config()
        cfg["quant_method"] = "mixed_gptq"
        cfg["module_wbits"] = {n: q.wbits for n, q in self._name_to_quantizer.items()}
        return cfg

    def finalize_quant_config_for_save(self, quant_config, quantized_layer_names, num_hidden_layers=None):
        return self.quantizers[0].finalize_quant_config_for_save(
            quant_config, quantized_layer_names, num_hidden_layers=num_hidden_layers)

    def create_inference_layer(self, result, linear_module, **kwargs):
        return self.quantizers[0].create_inference_layer(result, linear_module, **kwargs)
