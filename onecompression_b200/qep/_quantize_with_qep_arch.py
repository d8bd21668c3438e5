"""Block-wise QEP driver (reference: onecomp/qep/_quantize_with_qep_arch.py).

Per decoder block, in the reference's order: layers that share one input form a
group; each group's Hessian H (from the block with the already quantized layers)
and cross term C (against the full-precision block) are accumulated over the
calibration set; every layer of the group is corrected, quantized, and replaced by
its dequantized weight before the next group is measured; finally both blocks'
outputs become the next block's inputs.

What differs from the reference is only where time goes:

* activations stay in HBM between blocks instead of travelling to the host and back;
* the full-precision block runs once per block: the inputs of all groups are
  captured in that pass (the reference re-runs it for every group);
* the quantized block's passes stop at the layer whose input is being measured;
* one inverse-Hessian factor per group serves the correction and the column loop of
  every layer in it (the reference factors per layer, three times);
* the cross term is not accumulated for a group none of whose layers is corrected;
* with a process group, tokens are sharded over ranks for H and C (one all-reduce per
  group) and weight rows are sharded over ranks for the correction and the column
  loop (one all-gather per layer).
"""

from __future__ import annotations

import copy
from collections import OrderedDict
from logging import getLogger
from typing import Optional

import torch
import torch.nn.functional as F
from torch import nn

from .. import kernels
from ..quantizer._quantizer import Quantizer
from ..quantizer.gptq._gptq import GPTQ
from ._qep_config import QEPConfig
from .blockwise import (
    StopForward, call_block, forward_input, get_blocks_and_inputs, move_to_device,
)

logger = getLogger(__name__)


@torch.no_grad()
def make_grouped_module(block, inps, kwargs, device):
    """Groups of Linear modules that receive the very same input tensor object in one
    forward of a single sample, split further by in_features (reference :47-115)."""
    seen = []

    def hook(module, inp, _out):
        seen.append((module, inp[0] if isinstance(inp, tuple) else inp))

    handles = [m.register_forward_hook(hook) for m in block.modules() if isinstance(m, nn.Linear)]
    try:
        call_block(block, inps[:1].to(device), kwargs)
    finally:
        for h in handles:
            h.remove()
    groups, index = [], {}
    for module, tensor in seen:
        key = id(tensor)
        if key not in index:
            index[key] = len(groups)
            groups.append([])
        groups[index[key]].append(module)
    del seen
    result = []
    for group in groups:
        by_dim = OrderedDict()
        for module in group:
            by_dim.setdefault(module.in_features, []).append(module)
        result.extend(by_dim.values())
    return result


def _stop_hook(sink):
    def pre_hook(_module, args):
        sink(args[0] if isinstance(args, tuple) else args)
        raise StopForward()

    return pre_hook


@torch.no_grad()
def compute_hessian_and_crossterm(block_q, block_f, module_q, module_f, inps_q, inps_f, kwargs,
                                  batch_size, device, dist=None):
    """(H, C, nsamples) for one layer, running both blocks chunk by chunk
    (reference :118-201).  Each forward stops at the measured layer."""
    acc = kernels.MomentAccumulator(module_q.in_features, device, cross=True)
    got = {}
    hq = module_q.register_forward_pre_hook(_stop_hook(lambda x: got.__setitem__("q", x)))
    hf = module_f.register_forward_pre_hook(_stop_hook(lambda x: got.__setitem__("f", x)))
    try:
        for first in range(0, inps_q.size(0), batch_size):
            for blk, inps in ((block_q, inps_q), (block_f, inps_f)):
                try:
                    call_block(blk, inps[first : first + batch_size].to(device), kwargs)
                except StopForward:
                    pass
            acc.add(got["q"], got["f"])
    finally:
        hq.remove()
        hf.remove()
    h, c, n = acc.finalize()
    if dist is not None:
        h, c, n = dist.reduce_moments(h, c, n)
    return h, c, n


@torch.no_grad()
def _compute_per_module_hessians(block, modules, inps, kwargs, batch_size, device, dist=None):
    """Independent Hessians of MoE expert layers from the tokens routed to each
    (reference :204-272).  A module that saw no token maps to None."""
    accs = {m: kernels.MomentAccumulator(m.in_features, device) for m in modules}
    got = {}

    def make(m):
        def hook(_mod, inp, _out):
            got[m] = inp[0] if isinstance(inp, tuple) else inp
        return hook

    handles = [m.register_forward_hook(make(m)) for m in modules]
    try:
        for first in range(0, inps.size(0), batch_size):
            call_block(block, inps[first : first + batch_size].to(device), kwargs)
            for m, x in got.items():
                if x.numel():
                    accs[m].add(x)
            got.clear()
    finally:
        for h in handles:
            h.remove()
    out = {}
    for m, acc in accs.items():
        h, _, n = acc.finalize()
        if dist is not None:
            h, _, n = dist.reduce_moments(h, None, n)
        out[m] = (h, n) if n > 0 else None
    return out


def _gptq_of(quantizer, module):
    """The GPTQ instance that quantizes ``module``: the quantizer itself, the candidate a
    mixed-precision quantizer assigned to the module, or None for other quantizers."""
    if isinstance(quantizer, GPTQ):
        return quantizer
    child_for = getattr(quantizer, "child_for", None)
    child = child_for(module) if child_for is not None else None
    return child if isinstance(child, GPTQ) else None


def _rtn_fallback_result(module, quantizer, name):
    """RTN-quantize a module that saw no calibration token, as a GPTQResult so that it goes
    through the same save path as its calibrated siblings (reference :290-320): unpacked
    integer codes, fp16 scales / zeros [G, out], no permutation."""
    from ..quantizer.gptq._gptq import GPTQResult

    wbits = GPTQ.resolve_bits(name, quantizer.wbits, quantizer.mlp_wbits, quantizer.module_wbits)
    groupsize = GPTQ.resolve_groupsize(name, quantizer.groupsize, quantizer.mlp_groupsize)
    weight = module.weight.data
    out = kernels.rtn_quantize(weight if weight.dtype in (torch.float16, torch.bfloat16) else weight.half(),
                               wbits, groupsize, quantizer.sym)
    scales = out["scales"].to(torch.float16).cpu()
    zeros = out["zeros"].to(torch.float16).cpu()
    if groupsize != -1:
        scales, zeros = scales.T, zeros.T
    result = GPTQResult(
        dequantized_weight=out["dequantized"].to(weight.dtype).cpu(), wbits=wbits, groupsize=groupsize,
        actorder=False, sym=quantizer.sym, qweight=out["codes"].cpu(), scales=scales, qzeros=zeros,
        perm=None,
    )
    # The block continues with compute_dequantized_weight() (fp16 scales), as the reference's
    # driver does (:599-603), not with RTN's own fp32-scale reconstruction.
    return result


_RMSNORM_BODY = (
    "input_dtype = hidden_states.dtype",
    "hidden_states = hidden_states.to(torch.float32)",
    "variance = hidden_states.pow(2).mean(-1, keepdim=True)",
    "hidden_states = hidden_states * torch.rsqrt(variance + self.variance_epsilon)",
    "return self.weight * hidden_states.to(input_dtype)",
)
_rmsnorm_classes: dict = {}


def _is_plain_rmsnorm(module) -> bool:
    """True for modules whose forward is, line for line, the Llama-style RMSNorm (fp32 statistics,
    downcast, then weight product) - the only formula the fused kernel reproduces."""
    cls = type(module)
    if cls not in _rmsnorm_classes:
        ok = False
        try:
            import inspect

            lines = [ln.strip() for ln in inspect.getsource(cls.forward).splitlines()]
            body = tuple(ln for ln in lines if ln and not ln.startswith(("def ", "#", '"""')))
            ok = body == _RMSNORM_BODY
        except (OSError, TypeError):
            ok = False
        _rmsnorm_classes[cls] = ok
    return (_rmsnorm_classes[cls] and hasattr(module, "variance_epsilon")
            and getattr(module, "weight", None) is not None and module.weight.dtype == torch.float16)


_ROPE_BODY = (
    "cos = cos.unsqueeze(unsqueeze_dim)",
    "sin = sin.unsqueeze(unsqueeze_dim)",
    "q_embed = (q * cos) + (rotate_half(q) * sin)",
    "k_embed = (k * cos) + (rotate_half(k) * sin)",
    "return q_embed, k_embed",
)
_ROTATE_HALF_BODY = (
    "x1 = x[..., : x.shape[-1] // 2]",
    "x2 = x[..., x.shape[-1] // 2 :]",
    "return torch.cat((-x2, x1), dim=-1)",
)
_GATED_MLP_BODY = (
    "down_proj = self.down_proj(self.act_fn(self.gate_proj(x)) * self.up_proj(x))",
    "return down_proj",
)
_source_checks: dict = {}
_declined_logged: set = set()


def _code_lines(fn):
    """Stripped source lines of ``fn`` without blank lines and comments ((), if unavailable)."""
    import inspect

    try:
        src = inspect.getsource(inspect.unwrap(fn))
    except (OSError, TypeError, ValueError):
        return ()
    return tuple(ln.strip() for ln in src.splitlines() if ln.strip() and not ln.strip().startswith("#"))


def _ends_with(fn, body) -> bool:
    key = (fn, body)
    if key not in _source_checks:
        lines = _code_lines(fn)
        _source_checks[key] = len(lines) > len(body) and lines[-len(body):] == body
    return _source_checks[key]


def _is_plain_gated_mlp(module) -> bool:
    """True for the gated MLP of Llama / Qwen blocks: down(act(gate(x)) * up(x)) with SiLU."""
    if not all(hasattr(module, a) for a in ("gate_proj", "up_proj", "down_proj", "act_fn")):
        return False
    act = module.act_fn
    silu = type(act) is nn.SiLU or (
        isinstance(act, nn.Module) and "forward" not in act.__dict__
        and _code_lines(type(act).forward)[-1:] == ("return nn.functional.silu(input)",))
    return silu and _ends_with(type(module).forward, _GATED_MLP_BODY)


def _plain_rope_namespace(module):
    """The python module that defines ``module``'s class, if its ``apply_rotary_pos_emb`` and
    ``rotate_half`` are, line for line, the Llama formulation; else None."""
    import sys

    ns = sys.modules.get(type(module).__module__)
    fn, rot = getattr(ns, "apply_rotary_pos_emb", None), getattr(ns, "rotate_half", None)
    if fn is None or rot is None or not callable(fn):
        return None
    head = [ln for ln in _code_lines(fn) if ln.startswith("def ")]
    if not head or head[0] != "def apply_rotary_pos_emb(q, k, cos, sin, unsqueeze_dim=1):":
        return None
    return ns if _ends_with(fn, _ROPE_BODY) and _ends_with(rot, _ROTATE_HALF_BODY) else None


class _FusedOps:
    """While active, elementwise chains of the given blocks run as single CUDA kernels with the
    rounding points of the unfused operators: plain RMSNorm modules (``norms``), and the rotary
    embedding and SwiGLU of Llama-style attention / MLP code (``elementwise``).  Anything whose
    source differs from the recognised formulation, and any input the kernels do not take, runs
    the model's own code."""

    def __init__(self, blocks, norms=True, elementwise=True):
        self.norm_mods, self.mlp_mods, self.rope_spaces = [], [], []
        for b in blocks:
            for m in b.modules():
                if "forward" in m.__dict__:
                    continue
                if norms and _is_plain_rmsnorm(m):
                    self.norm_mods.append(m)
                elif elementwise and _is_plain_gated_mlp(m):
                    self.mlp_mods.append(m)
                else:
                    self._note_declined(m, norms, elementwise)
                if elementwise and hasattr(m, "q_proj") and hasattr(m, "k_proj"):
                    ns = _plain_rope_namespace(m)
                    if ns is not None and all(ns is not x for x, _ in self.rope_spaces):
                        self.rope_spaces.append((ns, ns.apply_rotary_pos_emb))
                    elif ns is None:
                        self._say_once(("rope", type(m)), "rotary embedding of %s is not the recognised "
                                       "formulation: it runs the model's own operators", type(m).__name__)

    @staticmethod
    def _say_once(key, message, *args):
        """One log line per module class whose code is not recognised: the passes then run the model's
        own elementwise operators for it (same results, more kernels - e.g. after a transformers
        release that rewords a forward)."""
        if key not in _declined_logged:
            _declined_logged.add(key)
            logger.info("fused block operators: " + message, *args)

    def _note_declined(self, m, norms, elementwise):
        name = type(m).__name__.lower()
        if norms and "rmsnorm" in name and getattr(m, "weight", None) is not None:
            self._say_once(("norm", type(m)), "%s is not the recognised RMSNorm (fp32 statistics, downcast, "
                           "weight product; fp16 weight): it runs the model's own operators", type(m).__name__)
        elif elementwise and all(hasattr(m, a) for a in ("gate_proj", "up_proj", "down_proj")):
            self._say_once(("mlp", type(m)), "%s is not the recognised gated MLP (down(act(gate(x)) * up(x)) with "
                           "SiLU): it runs the model's own operators", type(m).__name__)

    def __enter__(self):
        for m in self.norm_mods:
            def fused_norm(x, _m=m):
                if x.is_cuda and x.dtype == torch.float16:
                    return kernels.rmsnorm_f16(x, _m.weight, _m.variance_epsilon)
                return type(_m).forward(_m, x)

            m.forward = fused_norm
        for m in self.mlp_mods:
            def fused_mlp(x, _m=m):
                gate, up = _m.gate_proj(x), _m.up_proj(x)
                if (gate.is_cuda and gate.dtype == torch.float16 and up.dtype == torch.float16
                        and gate.shape == up.shape and gate.is_contiguous() and up.is_contiguous()):
                    # not in place: a memoised gate_proj hands out views of its record
                    return _m.down_proj(kernels.swiglu_f16(gate, up))
                return _m.down_proj(_m.act_fn(gate) * up)

            m.forward = fused_mlp
        for ns, original in self.rope_spaces:
            def fused_rope(q, k, cos, sin, unsqueeze_dim=1, _orig=original, **kw):
                if (unsqueeze_dim == 1 and not kw and kernels.rope_supported(q, cos, sin)
                        and kernels.rope_supported(k, cos, sin)):
                    return kernels.rope_f16(q, cos, sin), kernels.rope_f16(k, cos, sin)
                return _orig(q, k, cos, sin, unsqueeze_dim, **kw)

            ns.apply_rotary_pos_emb = fused_rope
        return self

    def __exit__(self, *exc):
        for m in self.norm_mods + self.mlp_mods:
            m.__dict__.pop("forward", None)
        for ns, original in self.rope_spaces:
            ns.apply_rotary_pos_emb = original
        return False


class _ForwardMemo:
    """Keeps outputs of sub-modules of the quantized block that can no longer change, so that
    later passes over the same inputs skip them.

    The passes of one block all start from the same inputs and the block's layers are
    replaced in execution order.  A sub-module that contains no layer still waiting to be
    quantized, and that runs before the first such layer, therefore produces the same output
    in every later pass: its output is recorded once (per chunk of sequences, in HBM) and the
    module is then answered from the record.  Candidates are the block's children and their
    parameter-holding children (norms, projections, the attention module as a whole).
    """

    def __init__(self, block, pending, n_seq, device, reserve_bytes=8 << 30):
        self.pending = set(pending)          # target Linear modules not yet quantized
        self.n_seq = n_seq
        self.device = device
        self.reserve = reserve_bytes
        self.first = 0                       # first sequence of the chunk being forwarded
        self.cands = []
        for child in block.children():
            self.cands.append(child)
            for sub in child.children():
                if any(True for _ in sub.parameters()):
                    self.cands.append(sub)
        self.inside = {m: {x for x in m.modules() if isinstance(x, nn.Linear)} for m in self.cands}
        self.cache = {}                      # module -> stored output (tensor or tuple)
        self._recording = {}
        self._is_tuple = {}
        self._handles = []
        self._stubbed = []
        self._chunk = 0

    def mark_done(self, module):
        self.pending.discard(module)

    def _free_bytes(self):
        free, _ = torch.cuda.mem_get_info(self.device)
        return free + torch.cuda.memory_reserved(self.device) - torch.cuda.memory_allocated(self.device)

    def _store(self, module, out):
        rec = self._recording[module]
        if rec is False:
            return
        items = out if isinstance(out, tuple) else (out,)
        tensors = [t for t in items if isinstance(t, torch.Tensor)]
        if any(t.dim() < 2 or t.shape[0] != self._chunk for t in tensors) or not tensors:
            self._recording[module] = False      # not a per-sequence output: leave it alone
            return
        if rec is None:
            need = sum(self.n_seq * t[0].numel() * t.element_size() for t in tensors)
            if need + self.reserve > self._free_bytes():
                self._recording[module] = False
                return
            rec = [torch.empty((self.n_seq,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
                   if isinstance(t, torch.Tensor) else t for t in items]
            self._recording[module] = rec
            self._is_tuple[module] = isinstance(out, tuple)
        for buf, t in zip(rec, items):
            if isinstance(t, torch.Tensor):
                buf[self.first : self.first + t.shape[0]].copy_(t)

    def begin_pass(self, record=True):
        for m in self.cands:
            if m in self.cache:
                bufs, is_tuple = self.cache[m]

                def stub(*_a, _bufs=bufs, _tuple=is_tuple, **_k):
                    outs = [b[self.first : self.first + self._chunk] if isinstance(b, torch.Tensor) else b
                            for b in _bufs]
                    return tuple(outs) if _tuple else outs[0]

                self._stubbed.append((m, m.__dict__.get("forward")))
                m.forward = stub
            elif record and not (self.inside[m] & self.pending):
                self._recording[m] = None
                self._handles.append(m.register_forward_hook(
                    lambda mod, _inp, out: self._store(mod, out)))

    def set_chunk(self, first, size):
        self.first, self._chunk = first, size

    def end_pass(self, complete=True):
        for h in self._handles:
            h.remove()
        self._handles = []
        for m, previous in self._stubbed:
            if previous is None:
                del m.forward                # back to the class's forward
            else:
                m.forward = previous
        self._stubbed = []
        for m, rec in self._recording.items():
            if complete and rec not in (None, False):
                self.cache[m] = (rec, self._is_tuple.get(m, False))
        self._recording = {}
        # a cached parent answers for its children: drop their records
        for m in list(self.cache):
            for other in self.cands:
                if other is not m and other in self.cache and other in set(m.modules()):
                    del self.cache[other]

    def release(self):
        self.cache = {}


class BlockQuantizer:
    """Quantizes the layers of one decoder block with error propagation."""

    def __init__(self, quantizer: Quantizer, qep_config: QEPConfig, batch_size: int, device,
                 dist=None, cache_budget_bytes: Optional[int] = None, memoize: bool = True,
                 profile: bool = False, fuse_rmsnorm: bool = True, fuse_elementwise: bool = True,
                 stack_layers: bool = True, high_priority: bool = True):
        self.memoize = memoize
        # The block's own chain of kernels runs on a high-priority stream; the prefetched
        # full-precision pass of the next block (``prefetch``) runs on a normal-priority side
        # stream.  The block scheduler then gives SMs to the chain first, and the side stream's
        # kernels fill the SMs the latency-bound phases (factorisation, column loop) leave idle
        # instead of competing with the throughput-bound ones.
        self.high_priority = high_priority
        self._main = None
        # Llama-style RMSNorm modules of the block run as one kernel during the passes (same
        # rounding points as the module; the row sum is formed in another order)
        self.fuse_rmsnorm = fuse_rmsnorm
        self.fuse_elementwise = fuse_elementwise
        self.stack_layers = stack_layers
        self._stream_io = None
        # with profile=True every phase is bracketed by device synchronisation and its wall
        # time is added to self.timings (seconds per phase name); off by default
        self.profile = profile
        self.timings = {}
        self._side = None
        self._prefetched = None
        self.quantizer = quantizer
        self.cfg = qep_config
        self.batch_size = batch_size
        self.device = torch.device(device)
        self.dist = dist
        self.cache_budget_bytes = cache_budget_bytes

    def _tick(self, name, t0):
        if not self.profile:
            return t0
        import time

        torch.cuda.synchronize(self.device)
        now = time.perf_counter()
        if name is not None:
            self.timings[name] = self.timings.get(name, 0.0) + now - t0
        return now

    def _budget(self):
        if self.cache_budget_bytes is not None:
            return self.cache_budget_bytes
        # memory the process could still use: free on the device plus what torch's caching
        # allocator holds but has not handed out
        free, _total = torch.cuda.mem_get_info(self.device)
        free += torch.cuda.memory_reserved(self.device) - torch.cuda.memory_allocated(self.device)
        return int(free * 0.5)

    def _classify(self, block, groups):
        """(regular groups, expert modules) among the target layers of ``block``."""
        qz = self.quantizer
        regular, experts = [], []
        for group in groups:
            targets = [m for m in group if m in qz.module_to_name]
            if not targets:
                continue
            if any(".experts." in qz.module_to_name[m] for m in targets):
                experts.extend(targets)
            else:
                regular.append(group)
        # experts the single-sample grouping pass never routed to (reference :436-461)
        known = set(experts)
        for _n, m in block.named_modules():
            name = qz.module_to_name.get(m) if isinstance(m, nn.Linear) else None
            if name is not None and ".experts." in name and m not in known:
                experts.append(m)
                known.add(m)
        return regular, experts

    @torch.no_grad()
    def _full_precision_pass(self, block, inps_f, kwargs):
        """One pass of the still unmodified block over the full-precision inputs: its outputs
        (the next block's full-precision inputs) and the input of every group that will need a
        cross term.  Independent of everything the quantized stream does, so it may run ahead
        on another CUDA stream (see ``prefetch``)."""
        qz, dev, bs = self.quantizer, self.device, self.batch_size
        block_f = copy.deepcopy(block)
        names = {m: n for n, m in block.named_modules() if isinstance(m, nn.Linear)}
        mods_f = {n: m for n, m in block_f.named_modules() if isinstance(m, nn.Linear)}
        self._io("before_read_f", 0, 1)
        regular, _experts = self._classify(block, make_grouped_module(block, inps_f, kwargs, dev))
        heads, need_c = [], {}
        for group in regular:
            head = names[group[0]]
            heads.append(head)
            targets = [qz.module_to_name[m] for m in group if m in qz.module_to_name]
            need_c[head] = any(not self._excluded(n) for n in targets)
        n_seq, seq = inps_f.shape[0], inps_f.shape[1]
        cache_bytes = sum(n_seq * seq * mods_f[h].in_features * 2 for h in heads if need_c[h])
        use_cache = cache_bytes <= self._budget()
        caches, handles, cursor = {}, [], {"first": 0}
        if use_cache:
            for head in heads:
                if not need_c[head]:
                    continue
                caches[head] = torch.empty((n_seq, seq, mods_f[head].in_features), dtype=inps_f.dtype, device=dev)

                def make(head):
                    def pre_hook(_m, args):
                        x = args[0] if isinstance(args, tuple) else args
                        caches[head][cursor["first"] : cursor["first"] + x.shape[0]].copy_(x)
                    return pre_hook

                handles.append(mods_f[head].register_forward_pre_hook(make(head)))
        next_f = torch.empty_like(inps_f)
        try:
            with _FusedOps([block_f], self.fuse_rmsnorm, self.fuse_elementwise):
                for first in range(0, n_seq, bs):
                    cursor["first"] = first
                    self._io("before_read_f", first, min(bs, n_seq - first))
                    y = call_block(block_f, inps_f[first : first + bs].to(dev), kwargs)
                    next_f[first : first + bs].copy_(y)
                    self._io("after_write_f", first, min(bs, n_seq - first), next_f)
        finally:
            for h in handles:
                h.remove()
        return {"block_f": block_f, "mods_f": mods_f, "need_c": need_c, "caches": caches,
                "use_cache": use_cache, "next_f": next_f}

    @torch.no_grad()
    def prefetch(self, block, inps_f, kwargs):
        """Start the full-precision pass of ``block`` (the block that ``run`` will get next) on a
        side stream.  It only depends on ``inps_f`` and on the block's untouched weights, so it
        overlaps with the latency-bound factorisations and column loops of the current block."""
        if self._side is None:
            self._side = torch.cuda.Stream(self.device)
        main = torch.cuda.current_stream(self.device)
        ready = torch.cuda.Event()
        ready.record(main)
        self._side.wait_event(ready)
        inps_f.record_stream(self._side)
        with torch.cuda.stream(self._side):
            res = self._full_precision_pass(block, inps_f, kwargs)
            done = torch.cuda.Event()
            done.record(self._side)
        self._prefetched = (block, res, done)

    def _take_prefetched(self, block):
        if self._prefetched is None or self._prefetched[0] is not block:
            self._prefetched = None
            return None
        _blk, res, done = self._prefetched
        self._prefetched = None
        main = torch.cuda.current_stream(self.device)
        main.wait_event(done)
        for t in [res["next_f"], *res["caches"].values()]:
            t.record_stream(main)
        for p_ in res["block_f"].parameters():
            p_.data.record_stream(main)
        return res

    def _io(self, what, *args):
        """Chunk-level notifications for a caller that streams activations from / to the host."""
        fn = getattr(self._stream_io, what, None) if self._stream_io is not None else None
        if fn is not None:
            fn(*args)

    @torch.no_grad()
    def run(self, block_q, inps_q, inps_f, kwargs, on_layer_done=None, next_block=None, stream_io=None):
        """Returns (next inps_q, next inps_f).  ``block_q`` must be on the device; its
        target layers end up holding their dequantized weights.  With ``next_block`` (the block
        the following call will process, already on the device and unmodified) its
        full-precision pass is started on a side stream as soon as its inputs exist.
        The layers' results travel to the host in the background and are complete on return.
        ``stream_io`` lets a caller move the activations in and out while the block is processed:
        any of ``before_read_f(first, size)``, ``before_read_q(first, size)`` (called before sequences
        first..first+size of ``inps_f`` / ``inps_q`` are read for the first time: make the current
        stream wait for them there), ``after_write_f(first, size, next_f)`` and
        ``after_write_q(first, size, next_q)`` (called when those sequences of the outputs have been
        enqueued: start copying them out on another stream)."""
        self._stream_io = stream_io
        try:
            with kernels.deferred_host_copies():
                if not self.high_priority or self.profile:
                    return self._run_block(block_q, inps_q, inps_f, kwargs, on_layer_done, next_block)
                caller = torch.cuda.current_stream(self.device)
                if self._main is None:
                    self._main = torch.cuda.Stream(self.device, priority=-1)     # lower number: higher priority
                self._main.wait_stream(caller)
                with torch.cuda.stream(self._main):
                    next_q, next_f = self._run_block(block_q, inps_q, inps_f, kwargs, on_layer_done, next_block)
                caller.wait_stream(self._main)
                for t in (next_q, next_f):
                    t.record_stream(caller)
                return next_q, next_f
        finally:
            self._stream_io = None

    def _run_block(self, block_q, inps_q, inps_f, kwargs, on_layer_done=None, next_block=None):
        qz, dev, bs = self.quantizer, self.device, self.batch_size
        t0 = self._tick(None, 0.0)
        fp = self._take_prefetched(block_q)
        if fp is None:
            fp = self._full_precision_pass(block_q, inps_f, kwargs)
        block_f, mods_f, next_f = fp["block_f"], fp["mods_f"], fp["next_f"]
        use_cache = fp["use_cache"]
        if next_block is not None and not self.profile:
            self.prefetch(next_block, next_f, kwargs)
        with _FusedOps([block_q, block_f], self.fuse_rmsnorm, self.fuse_elementwise):
            return self._run_quantized(block_q, inps_q, inps_f, kwargs, on_layer_done, fp, t0)

    def _run_quantized(self, block_q, inps_q, inps_f, kwargs, on_layer_done, fp, t0):
        qz, dev, bs = self.quantizer, self.device, self.batch_size
        block_f, mods_f, next_f, use_cache = fp["block_f"], fp["mods_f"], fp["next_f"], fp["use_cache"]
        self._io("before_read_q", 0, 1)
        groups_q = make_grouped_module(block_q, inps_q, kwargs, dev)
        names_q = {m: n for n, m in block_q.named_modules() if isinstance(m, nn.Linear)}
        regular, experts = self._classify(block_q, groups_q)
        n_seq = inps_q.shape[0]
        need_c = [fp["need_c"][names_q[g[0]]] for g in regular]
        caches = [fp["caches"].get(names_q[g[0]]) for g in regular]
        t0 = self._tick("pass_full_precision", t0)
        memo = None
        if self.memoize and torch.device(inps_q.device).type == "cuda":
            pending = [m for g in regular for m in g if m in qz.module_to_name] + list(experts)
            memo = _ForwardMemo(block_q, pending, n_seq, dev)

        for gi, group in enumerate(regular):
            d = group[0].in_features
            acc = kernels.MomentAccumulator(d, dev, cross=need_c[gi])
            if memo is not None:
                memo.begin_pass(record=True)
            cur = {}
            hq = group[0].register_forward_pre_hook(_stop_hook(lambda x: cur.__setitem__("q", x)))
            hf = None
            if need_c[gi] and not use_cache:
                hf = mods_f[names_q[group[0]]].register_forward_pre_hook(
                    _stop_hook(lambda x: cur.__setitem__("f", x)))
            try:
                for first in range(0, n_seq, bs):
                    if memo is not None:
                        memo.set_chunk(first, min(bs, n_seq - first))
                    if gi == 0:
                        self._io("before_read_q", first, min(bs, n_seq - first))
                    try:
                        call_block(block_q, inps_q[first : first + bs].to(dev), kwargs)
                    except StopForward:
                        pass
                    xf = None
                    if need_c[gi]:
                        if use_cache:
                            xf = caches[gi][first : first + bs]
                        else:
                            try:
                                call_block(block_f, inps_f[first : first + bs].to(dev), kwargs)
                            except StopForward:
                                pass
                            xf = cur["f"]
                    acc.add(cur["q"], xf)
            finally:
                hq.remove()
                if hf is not None:
                    hf.remove()
                if memo is not None:
                    memo.end_pass(complete=True)
            caches[gi] = None
            h, c, n = acc.finalize()
            t0 = self._tick(f"pass_quantized+moments[{gi}]", t0)
            if self.dist is not None:
                # the factorisation needs H only: the reduction of C runs beside it
                h, c, n = self.dist.reduce_moments(h, c, n, fixed_split=True, defer_cross=not self.profile)
                t0 = self._tick("allreduce", t0)
            factors = {}
            plan = []            # [(modules sharing one call, factor, excluded)]
            for module in group:
                name = qz.module_to_name.get(module)
                if name is None:
                    continue
                child = _gptq_of(qz, module)
                factor = None
                if child is not None:
                    key = (child.percdamp, child.actorder)
                    if key not in factors:
                        factors[key] = kernels.factor_hessian(h, child.percdamp, child.actorder)
                        t0 = self._tick("factor", t0)
                    factor = factors[key]
                excluded = self._excluded(name)
                skey = None
                if child is not None and self.stack_layers and (self.dist is None or child.bitpack_on_quantize):
                    skey = child.stack_key(module)
                    if skey is not None:
                        skey = skey + (excluded,)
                for entry in plan:
                    if skey is not None and entry["key"] == skey:
                        entry["modules"].append(module)
                        break
                else:
                    plan.append({"key": skey, "modules": [module], "factor": factor, "excluded": excluded,
                                 "child": child})
            if self.dist is not None:
                self.dist.wait_cross()
            for entry in plan:
                mods, excluded = entry["modules"], entry["excluded"]
                if len(mods) > 1:
                    if self.dist is not None:
                        results = self.dist.quantize_rows_stacked(
                            entry["child"], mods, h, None if excluded else c, self.cfg, entry["factor"])
                        for module in mods:
                            entry["child"].results.pop(qz.module_to_name[module], None)
                    else:
                        results = entry["child"].quantize_stacked(
                            mods, h, entry["factor"], None if excluded else c, self.cfg.percdamp,
                            self.cfg.perccorr)
                    for module in mods:
                        name = qz.module_to_name[module]
                        qz.results[name] = results[module]
                        self._install_dequantized(module, name)
                else:
                    name = qz.module_to_name[mods[0]]
                    self._quantize_one(mods[0], name, h, None if excluded else c, n, entry["factor"])
                t0 = self._tick("correct+quantize", t0)
                for module in mods:
                    name = qz.module_to_name[module]
                    if memo is not None:
                        memo.mark_done(module)
                    if on_layer_done is not None:
                        on_layer_done(f"{name}, no weight correction" if excluded else name)

        if experts:
            per_module = _compute_per_module_hessians(block_q, experts, inps_q, kwargs, bs, dev, self.dist)
            shared = []
            for module in experts:
                name = qz.module_to_name[module]
                entry = per_module[module]
                if entry is None:
                    child = _gptq_of(qz, module)
                    if child is not None:
                        logger.warning(
                            "Expert layer %s received no tokens during calibration; falling back to "
                            "RTN so it stays quantized like its sibling experts", name)
                        qz.results[name] = _rtn_fallback_result(module, child, name)
                        self._install_dequantized(module, name)
                        if on_layer_done is not None:
                            on_layer_done(name)
                    else:
                        logger.warning("Expert layer %s received no tokens during calibration; skipping", name)
                        if on_layer_done is not None:
                            on_layer_done(f"{name}, skipped: no tokens")
                    continue
                child = _gptq_of(qz, module)
                if (child is not None and child.stack_key(module) is not None
                        and (self.dist is None or child.bitpack_on_quantize)):
                    shared.append((module, child, entry[0]))     # quantized together below
                    continue
                self._quantize_one(module, name, entry[0], None, entry[1], None)
                if on_layer_done is not None:
                    on_layer_done(name)
            # experts are independent small problems: several at a time on separate streams, and
            # whole layers per rank instead of row slabs when there are ranks
            by_child = {}
            for module, child, h_e in shared:
                by_child.setdefault(id(child), (child, []))[1].append((module, h_e))
            for child, items in by_child.values():
                if self.dist is not None:
                    done = self.dist.quantize_independent(child, items)
                else:
                    done = child.quantize_independent(items)
                for module, _h in items:
                    name = qz.module_to_name[module]
                    if child is not qz:
                        child.results.pop(name, None)
                    qz.results[name] = done[module]
                    self._install_dequantized(module, name)
                    if on_layer_done is not None:
                        on_layer_done(name)

        next_q = torch.empty_like(inps_q)
        if memo is not None and not experts:
            memo.begin_pass(record=False)
            try:
                for first in range(0, n_seq, bs):
                    memo.set_chunk(first, min(bs, n_seq - first))
                    y = call_block(block_q, inps_q[first : first + bs].to(dev), kwargs)
                    next_q[first : first + bs].copy_(y)
                    self._io("after_write_q", first, min(bs, n_seq - first), next_q)
            finally:
                memo.end_pass(complete=False)
                memo.release()
        else:
            if memo is not None:
                memo.release()
            self._io("before_read_q", 0, n_seq)
            forward_input(inps_q, block_q, kwargs, bs, dev, out=next_q)
            self._io("after_write_q", 0, n_seq, next_q)
        del block_f
        self._tick("pass_propagate", t0)
        return next_q, next_f

    def _excluded(self, name):
        return any(k in name for k in self.cfg.exclude_layer_keywords)

    def _quantize_one(self, module, name, h, c, n, factor):
        qz = self.quantizer
        extra = {"factor": factor} if factor is not None else {}
        child = _gptq_of(qz, module)
        if self.dist is not None and child is not None:
            self.dist.quantize_rows(child, module, h, c, self.cfg, factor)
            if child is not qz:
                qz.results[name] = child.results.pop(name)
        else:
            qz.quantize_with_qep(
                module, quant_input_activation=None, original_input_activation=None,
                percdamp=self.cfg.percdamp, perccorr=self.cfg.perccorr, hessian=h, delta_hatX=c,
                nsamples=n if qz.flag_nsamples else None, **extra,
            )
        self._install_dequantized(module, name)

    def _install_dequantized(self, module, name):
        result = self.quantizer.results.get(name)
        if result is None:
            return
        w_hat = result.__dict__.get("_device_dequantized")
        try:
            if w_hat is None:
                w_hat = result.compute_dequantized_weight().to(self.device)
            module.weight.data = w_hat.to(module.weight.dtype).reshape(module.weight.shape)
        except (ValueError, NotImplementedError):
            logger.error("Failed to compute dequantized weight for %s. Keeping original weights.", name)
        result.__dict__.pop("_device_dequantized", None)


@torch.no_grad()
def run_quantize_with_qep_arch(model_config, quantizer: Quantizer, qep_config: QEPConfig,
                               calibration_config=None, *, report_progress: bool = True,
                               model=None, model_inputs=None, batch_size: int = 16, dist=None,
                               activations_on_device: bool = True):
    """Quantize every target layer of a decoder-only model block by block with QEP
    (reference :323-627).

    ``model`` / ``model_inputs`` ({"input_ids": LongTensor [N, S], …}) can be given
    directly; otherwise ``model_config.load_model(device_map="cpu")`` supplies the model
    and ``calibration_config.model_inputs`` the calibration batch (tokenising a text
    corpus is not part of this package).  Results land in ``quantizer.results``.
    """
    if model is None:
        model = model_config.load_model(device_map="cpu")
    if model_inputs is None:
        model_inputs = getattr(calibration_config, "model_inputs", None)
        if model_inputs is None:
            raise ValueError("pass model_inputs (or a calibration_config that carries them)")
    device = torch.device(qep_config.device or "cuda")
    if device.type != "cuda":
        raise RuntimeError("run_quantize_with_qep_arch computes on a CUDA device only")

    quantizer.setup(model)
    store = device if activations_on_device else torch.device("cpu")
    # embeddings (and whatever precedes the first block) run where the model lives
    blocks, inps, kwargs = get_blocks_and_inputs(model, model_inputs, batch_size, store_device=store)
    inps_q, inps_f = inps, inps.clone()
    kwargs = move_to_device(kwargs, device)

    block_modules = {m for block in blocks for m in block.modules()}
    remaining = {n for m, n in quantizer.module_to_name.items() if m in block_modules}
    total = len(remaining)
    done = {"k": 0}

    def on_layer_done(label):
        remaining.discard(label.split(",")[0])
        done["k"] += 1
        if report_progress:
            logger.info("[progress] QEP %d/%d %s", done["k"], total, label)

    runner = BlockQuantizer(quantizer, qep_config, batch_size, device, dist=dist)
    for idx, block in enumerate(blocks):
        if not remaining:
            logger.info("All target layers quantized -- skipping remaining blocks.")
            break
        block_q = block.to(device)
        upcoming = None
        if idx + 1 < len(blocks) and remaining:
            upcoming = blocks[idx + 1].to(device)      # its full-precision pass runs ahead
        inps_q, inps_f = runner.run(block_q, inps_q, inps_f, kwargs, on_layer_done, next_block=upcoming)
        mse = F.mse_loss(inps_q.float(), inps_f.float()).item()
        logger.info("Block %d MSE: %.6e", idx + 1, mse)
        block_q.cpu()
    # every factorisation checks the status word of the fp32 tensor-core products issued before it;
    # this covers the products of the last layers
    with torch.cuda.device(device):
        torch.cuda.synchronize(device)
        kernels.check_gemm_status()
    quantizer.execute_post_processing()
