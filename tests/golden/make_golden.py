"""Generate the golden fixtures in this directory from the reference itself.

Run once, in a container that has the OneComp v1.4.0 source tree, as

    python tests/golden/make_golden.py /path/to/OneCompression

It imports the reference's own functions (with three third-party module roots
that are absent here - lm_eval, ortools, primefac - replaced by inert stubs;
none of them is touched by the path), runs them on small seeded inputs on CPU
and stores inputs and outputs as ``.npz``.  The tests never need the reference:
they read only the ``.npz`` files.
"""

from __future__ import annotations

import importlib.abc
import importlib.machinery
import os
import sys
import types

import numpy as np
import torch

_STUB_ROOTS = ("lm_eval", "ortools", "primefac")


class _Stub(types.ModuleType):
    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)
        return _Stub(self.__name__ + "." + name)

    def __call__(self, *a, **k):
        return _Stub(self.__name__ + "()")


class _Finder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, fullname, path, target=None):
        if fullname.split(".")[0] in _STUB_ROOTS:
            return importlib.machinery.ModuleSpec(fullname, self, is_package=True)
        return None

    def create_module(self, spec):
        m = _Stub(spec.name)
        m.__path__ = []
        return m

    def exec_module(self, module):
        pass


def _import_reference(root):
    sys.meta_path.insert(0, _Finder())
    sys.path.insert(0, root)


HERE = os.path.dirname(os.path.abspath(__file__))


def _np(t):
    if t is None:
        return np.zeros((0,), dtype=np.int64)
    if t.dtype == torch.float16:
        return t.numpy().view(np.uint16)  # stored as raw bits
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)  # raw bits as well
    return t.numpy()


def synth_layer(seed, out, d, ntok, outliers=4, dead=()):
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(out, d, generator=g) * 0.02).half()
    x = torch.randn(ntok, d, generator=g)
    idx = torch.randperm(d, generator=g)[:outliers]
    x[:, idx] *= 20
    for c in dead:
        x[:, c] = 0
    return w, x.half()


# (name, out, d, ntok, kwargs)
GPTQ_CASES = [
    ("b4_g128_asym", 32, 256, 1024, dict(wbits=4, groupsize=128, sym=False)),
    ("b3_g128_sym", 32, 256, 1024, dict(wbits=3, groupsize=128, sym=True)),
    ("b4_g32_asym_stale", 32, 256, 1024, dict(wbits=4, groupsize=32, sym=False)),
    ("b2_g64_asym", 32, 256, 1024, dict(wbits=2, groupsize=64, sym=False)),
    ("b8_perchannel_sym", 32, 256, 1024, dict(wbits=8, groupsize=-1, sym=True)),
    ("b4_perchannel_asym", 32, 256, 1024, dict(wbits=4, groupsize=-1, sym=False)),
    ("b4_g128_asym_actorder", 32, 256, 1024, dict(wbits=4, groupsize=128, sym=False, actorder=True)),
    ("b3_g128_sym_actorder", 32, 256, 1024, dict(wbits=3, groupsize=128, sym=True, actorder=True)),
    ("b4_g32_ragged_d160", 32, 160, 640, dict(wbits=4, groupsize=32, sym=False)),
    ("b4_g128_dead", 32, 256, 1024, dict(wbits=4, groupsize=128, sym=False, _dead=(3, 130))),
    ("b4_g128_block64", 32, 256, 1024, dict(wbits=4, groupsize=128, sym=True, blocksize=64)),
    ("b4_g128_asym_mse", 32, 256, 1024, dict(wbits=4, groupsize=128, sym=False, mse=True)),
    ("b3_perchannel_sym_mse", 32, 256, 1024, dict(wbits=3, groupsize=-1, sym=True, mse=True)),
]


def main(ref_root):
    _import_reference(ref_root)
    from onecomp.quantizer.gptq import _gptq as ref_gptq
    from onecomp.quantizer.gptq import gptq_layer as ref_layer
    from onecomp.qep import _quantize_with_qep_arch as ref_arch

    torch.set_num_threads(1)

    # ---- packing -----------------------------------------------------------
    pack = {}
    g = torch.Generator().manual_seed(11)
    for bits in (2, 3, 4, 8):
        codes = torch.randint(0, 2**bits, (64, 96), generator=g, dtype=torch.int32)
        zeros = torch.randint(0, 2**bits, (3, 64), generator=g, dtype=torch.int32)
        zeros[0, :4] = 0  # stored value becomes -1 and must be masked
        pack[f"codes{bits}"] = codes.numpy()
        pack[f"zeros{bits}"] = zeros.numpy()
        pack[f"qweight{bits}"] = ref_layer.pack_int_weights(codes, bits).numpy()
        pack[f"qzeros{bits}"] = ref_layer.pack_zeros(zeros - 1, bits).numpy()
        pack[f"unpacked{bits}"] = ref_layer.unpack_int_weights(
            ref_layer.pack_int_weights(codes, bits), bits, (64, 96)
        ).numpy()
    np.savez_compressed(os.path.join(HERE, "pack.npz"), **pack)

    # ---- find_params ---------------------------------------------------------
    fp = {}
    g = torch.Generator().manual_seed(12)
    x = torch.randn(24, 40, generator=g) * 0.05
    x[0] = 0  # all-zero row
    x[1] = x[1].abs()  # minimum clipped to 0
    x[2] = -x[2].abs()  # maximum clipped to 0
    x[3, 0] = 0.7  # outlier
    fp["x"] = x.numpy()
    for bits in (2, 3, 4, 8):
        for sym in (False, True):
            ex = ref_gptq.GPTQExcecutor()
            ex.configure(bits, perchannel=True, sym=sym, mse=False)
            ex.find_params(x.clone(), weight=True)
            fp[f"scale_b{bits}_s{int(sym)}"] = ex.scale.numpy()
            fp[f"zero_b{bits}_s{int(sym)}"] = ex.zero.numpy()
            q = ref_gptq.quantize(x, ex.scale, ex.zero, ex.maxq)
            fp[f"q_b{bits}_s{int(sym)}"] = q.numpy()
            fp[f"dq_b{bits}_s{int(sym)}"] = ref_gptq.dequantize(q, ex.scale, ex.zero, ex.maxq).numpy()
    ex = ref_gptq.GPTQExcecutor()
    ex.configure(4, perchannel=True, sym=False, mse=True, norm=2.4, grid=100)
    ex.find_params(x.clone(), weight=True)
    fp["scale_mse"] = ex.scale.numpy()
    fp["zero_mse"] = ex.zero.numpy()
    np.savez_compressed(os.path.join(HERE, "find_params.npz"), **fp)

    # ---- moments ---------------------------------------------------------------
    mom = {}
    g = torch.Generator().manual_seed(13)
    xq = (torch.randn(20, 16, 64, generator=g)).half()  # 20 seqs -> slices of 8,8,4
    xf = (xq.float() * (1 + 0.03 * torch.randn(20, 16, 64, generator=g))).half()
    lin = torch.nn.Linear(64, 8, bias=False).half()
    qz = ref_gptq.GPTQ(wbits=4, groupsize=-1)
    h, n = qz.calculate_hessian(lin, xq)
    mom.update(xq=_np(xq), xf=_np(xf), H=h.numpy(), n=np.int64(n))
    mom["C_generic"] = qz.calculate_delta_hatX(lin, xq, xf).numpy()

    class _Blk(torch.nn.Module):
        def __init__(self, lin):
            super().__init__()
            self.lin = lin

        def forward(self, x, **kw):
            return self.lin(x)

    bq, bf = _Blk(torch.nn.Linear(64, 8, bias=False).half()), _Blk(torch.nn.Linear(64, 8, bias=False).half())
    hh, cc, nn_ = ref_arch.compute_hessian_and_crossterm(
        bq, bf, bq.lin, bf.lin, xq, xf, {}, 6, torch.device("cpu")
    )
    mom.update(H_arch=hh.numpy(), C_arch=cc.numpy(), n_arch=np.int64(nn_), arch_chunk=np.int64(6))
    np.savez_compressed(os.path.join(HERE, "moments.npz"), **mom)

    # ---- run_gptq / quantize_layer / dequantize ----------------------------------
    for k, (name, out, d, ntok, kw) in enumerate(GPTQ_CASES):
        kw = dict(kw)
        dead = kw.pop("_dead", ())
        w, x = synth_layer(100 + k, out, d, ntok, dead=dead)
        lin = torch.nn.Linear(d, out, bias=False).half()
        lin.weight.data = w.clone()
        blocksize = kw.pop("blocksize", 128)
        qz = ref_gptq.GPTQ(blocksize=blocksize, **kw)
        qz.module_to_name = {lin: "layer"}
        h, n = qz.calculate_hessian(lin, x.unsqueeze(0))
        raw = ref_gptq.run_gptq(
            h.clone(), lin, blocksize=blocksize, percdamp=0.01, wbits=kw["wbits"],
            groupsize=kw["groupsize"], actorder=kw.get("actorder", False), mse=kw.get("mse", False),
            sym=kw["sym"],
        )
        u = ref_gptq._compute_inverse_hessian(_prep_h(h.clone(), raw["perm"]), 0.01)
        res = qz.quantize_layer(lin, None, hessian=h.clone())
        deq = res.compute_dequantized_weight()
        np.savez_compressed(
            os.path.join(HERE, f"gptq_{name}.npz"),
            W=_np(w), H=h.numpy(), n=np.int64(n), blocksize=np.int64(blocksize),
            wbits=np.int64(kw["wbits"]), groupsize=np.int64(kw["groupsize"]),
            sym=np.int64(kw["sym"]), actorder=np.int64(kw.get("actorder", False)),
            mse=np.int64(kw.get("mse", False)),
            codes=raw["qweight"].numpy(), scales=_np(raw["scales"]), qzeros=raw["qzeros"].numpy(),
            perm=_np(raw["perm"]), U=u.numpy(),
            qweight_packed=res.qweight.numpy(), qzeros_packed=res.qzeros.numpy(),
            dequantized=_np(deq),
        )

    # ---- QEP weight correction -----------------------------------------------------
    w, x = synth_layer(300, 32, 128, 1024)
    g = torch.Generator().manual_seed(301)
    xq = (x.float() * (1 + 0.05 * torch.randn(x.shape, generator=g))).half()
    lin = torch.nn.Linear(128, 32, bias=False).half()
    lin.weight.data = w.clone()
    qz = ref_gptq.GPTQ(wbits=4, groupsize=128, sym=False)
    qz.module_to_name = {lin: "layer"}
    h, n = qz.calculate_hessian(lin, xq.unsqueeze(0))
    c = qz.calculate_delta_hatX(lin, xq.unsqueeze(0), x.unsqueeze(0))
    qz.adjust_weight(lin, None, None, original_hessian=h, original_delta_hatX=c,
                     percdamp=0.01, perccorr=0.5)
    adjusted = lin.weight.data.clone()
    lin.weight.data = w.clone()
    qz.quantize_with_qep(lin, None, None, percdamp=0.01, perccorr=0.5,
                         hessian=h.clone(), delta_hatX=c.clone())
    res = qz.results["layer"]
    np.savez_compressed(
        os.path.join(HERE, "qep_adjust.npz"),
        W=_np(w), H=h.numpy(), C=c.numpy(), n=np.int64(n), adjusted=_np(adjusted),
        qweight_packed=res.qweight.numpy(), qzeros_packed=res.qzeros.numpy(),
        scales=_np(res.scales), dequantized=_np(res.compute_dequantized_weight()),
    )
    # ---- RTN fallback for experts without tokens -----------------------------------------
    from onecomp.quantizer.rtn.rtn_impl import run_rtn

    rtn = {}
    w, _ = synth_layer(400, 32, 128, 64)
    w[3] = 0
    w[4] = w[4].abs()
    lin = torch.nn.Linear(128, 32, bias=False).half()
    lin.weight.data = w.clone()
    rtn["W"] = _np(w)
    for bits, gs, sym in ((4, 32, False), (4, 32, True), (3, -1, False), (2, 64, True)):
        r = run_rtn(lin, wbits=bits, groupsize=gs, sym=sym)
        key = f"b{bits}_g{gs}_s{int(sym)}"
        rtn[f"codes_{key}"] = r["quantized_weight"].numpy()
        rtn[f"scale_{key}"] = _np(r["scale"])
        rtn[f"zero_{key}"] = _np(r["zero"])
        rtn[f"deq_{key}"] = _np(r["dequantized_weight"])
    np.savez_compressed(os.path.join(HERE, "rtn.npz"), **rtn)

    # ---- bf16 module: moments, correction, GPTQ, RTN on bfloat16 weights and activations ----------
    b = {}
    w, x = synth_layer(500, 32, 256, 1024)
    g = torch.Generator().manual_seed(501)
    w, x = w.bfloat16(), x.bfloat16()
    xq = (x.float() * (1 + 0.05 * torch.randn(x.shape, generator=g))).bfloat16()
    lin = torch.nn.Linear(256, 32, bias=False).bfloat16()
    lin.weight.data = w.clone()
    qz = ref_gptq.GPTQ(wbits=4, groupsize=64, sym=False)
    qz.module_to_name = {lin: "layer"}
    h, n = qz.calculate_hessian(lin, xq.unsqueeze(0))
    c = qz.calculate_delta_hatX(lin, xq.unsqueeze(0), x.unsqueeze(0))
    raw = ref_gptq.run_gptq(h.clone(), lin, blocksize=128, percdamp=0.01, wbits=4, groupsize=64,
                            actorder=False, mse=False, sym=False)
    b.update(W=_np(w), xq=_np(xq), xf=_np(x), H=h.numpy(), C=c.numpy(), n=np.int64(n),
             codes=raw["qweight"].numpy(), scales=_np(raw["scales"]), qzeros=raw["qzeros"].numpy())
    qz.adjust_weight(lin, None, None, original_hessian=h, original_delta_hatX=c, percdamp=0.01, perccorr=0.5)
    b["adjusted"] = _np(lin.weight.data.clone())
    lin.weight.data = w.clone()
    qz.quantize_with_qep(lin, None, None, percdamp=0.01, perccorr=0.5, hessian=h.clone(), delta_hatX=c.clone())
    res = qz.results["layer"]
    deq = res.compute_dequantized_weight()
    b.update(qep_qweight_packed=res.qweight.numpy(), qep_qzeros_packed=res.qzeros.numpy(),
             qep_scales=_np(res.scales), qep_dequantized=_np(deq),
             qep_installed=_np(deq.to(torch.bfloat16)))      # what the driver puts into the module
    lin.weight.data = w.clone()
    r = run_rtn(lin, wbits=4, groupsize=32, sym=False)
    b.update(rtn_codes=r["quantized_weight"].numpy(), rtn_scale=_np(r["scale"]), rtn_zero=_np(r["zero"]),
             rtn_deq=_np(r["dequantized_weight"]))
    b["rtn_deq_is_bf16"] = np.int64(r["dequantized_weight"].dtype == torch.bfloat16)
    np.savez_compressed(os.path.join(HERE, "bf16.npz"), **b)
    layer_state_fixture(ref_gptq, ref_layer)
    driver_fixtures(ref_gptq, ref_arch)
    print("golden fixtures written to", HERE)


def layer_state_fixture(ref_gptq, ref_layer):
    """What the save path writes per layer and into config.json: the buffers of the reference's
    GPTQLinear built from a result (onecomp/quantizer/gptq/gptq_layer.py:395-433, 576-628) for four of
    the GPTQ cases above, and the quantization_config of plain and mixed-precision quantizers
    (onecomp/quantizer/gptq/_gptq.py:480-566)."""
    import json

    out = {}
    wanted = ("b4_g128_asym", "b4_g128_asym_actorder", "b3_g128_sym", "b8_perchannel_sym")
    for k, (name, rows, d, ntok, kw) in enumerate(GPTQ_CASES):
        if name not in wanted:
            continue
        kw = dict(kw)
        kw.pop("_dead", None)
        w, x = synth_layer(100 + k, rows, d, ntok)
        lin = torch.nn.Linear(d, rows, bias=True).half()
        lin.weight.data = w.clone()
        g = torch.Generator().manual_seed(900 + k)
        lin.bias.data = (torch.randn(rows, generator=g) * 0.1).half()
        qz = ref_gptq.GPTQ(**kw)
        qz.module_to_name = {lin: "layer"}
        h, _n = qz.calculate_hessian(lin, x.unsqueeze(0))
        res = qz.quantize_layer(lin, None, hessian=h.clone())
        layer = ref_layer.GPTQLinear.from_quantization_result(res, bias=lin.bias.data, device="cpu",
                                                              pack_weights=True, use_gemlite=False)
        state = layer.state_dict()
        out[f"{name}/keys"] = np.array(list(state))
        for key, t in state.items():
            out[f"{name}/{key}"] = _np(t)
            out[f"{name}/{key}/dtype"] = np.array(str(t.dtype))
    names = [f"model.layers.{i}.{n}" for i in range(2) for n in
             ("self_attn.q_proj", "self_attn.o_proj", "mlp.gate_proj", "mlp.down_proj")] + ["lm_head"]
    configs = {
        "plain": dict(wbits=4, groupsize=128, sym=False, actorder=True),
        "mixed": dict(wbits=4, groupsize=128, mlp_wbits=3, mlp_groupsize=64,
                      module_wbits={"model.layers.1.self_attn.q_proj": 2}),
    }
    for tag, kw in configs.items():
        qz = ref_gptq.GPTQ(**kw)
        cfg = qz.get_quant_config()
        out[f"config/{tag}/kwargs"] = np.array(json.dumps(kw))
        out[f"config/{tag}/quant_config"] = np.array(json.dumps(cfg, sort_keys=True))
        final = qz.finalize_quant_config_for_save(dict(cfg), names, num_hidden_layers=2)
        out[f"config/{tag}/final"] = np.array(json.dumps(final, sort_keys=True))
    out["config/names"] = np.array(names)
    np.savez_compressed(os.path.join(HERE, "layer_state.npz"), **out)


class _FakeModelConfig:
    """What the reference's driver asks of a ModelConfig: the model and a tokenizer."""

    def __init__(self, model):
        self._model = model

    def load_model(self, device_map=None):  # pylint: disable=unused-argument
        return self._model

    def load_tokenizer(self):
        return None


def _run_reference_driver(ref_gptq, ref_arch, model, ids, quantizer_kw, tag, extra=None):
    """The reference's run_quantize_with_qep_arch (onecomp/qep/_quantize_with_qep_arch.py:323-627)
    on ``model`` with the token ids ``ids`` on CPU.  Records, in call order, what the driver hands
    to ``quantize_with_qep`` for every layer (the layer's weight at that moment, H, C or nothing)
    and every layer's result; layers that took the RTN fallback carry no quantization time."""
    from onecomp.qep._qep_config import QEPConfig

    original = ref_arch.prepare_calibration_dataset
    ref_arch.prepare_calibration_dataset = lambda **_kw: {"input_ids": ids}
    calls = []

    class Recording(ref_gptq.GPTQ):
        def quantize_with_qep(self, module, quant_input_activation, original_input_activation=None,
                              percdamp=0.01, perccorr=0.5, hessian=None, delta_hatX=None, nsamples=None):
            calls.append((self.module_to_name[module], module.weight.data.clone(), hessian.clone(),
                          None if delta_hatX is None else delta_hatX.clone()))
            return super().quantize_with_qep(module, quant_input_activation, original_input_activation,
                                             percdamp=percdamp, perccorr=perccorr, hessian=hessian,
                                             delta_hatX=delta_hatX, nsamples=nsamples)

    qz = Recording(**quantizer_kw)
    try:
        ref_arch.run_quantize_with_qep_arch(
            model_config=_FakeModelConfig(model), quantizer=qz,
            qep_config=QEPConfig(device="cpu", percdamp=0.01, perccorr=0.5),
            calibration_config=None, report_progress=False)
    finally:
        ref_arch.prepare_calibration_dataset = original
    out = {"ids": ids.numpy(), "order": np.array([c[0] for c in calls])}
    for k, v in (extra or {}).items():
        out[k] = v
    for name, p in model.state_dict().items():
        # the model after the run: target layers hold their dequantized weights
        out[f"final/{name}"] = _np(p.detach().cpu())
    for name, w, h, c in calls:
        # no layer's own weight has changed before its turn
        assert torch.equal(w, torch.from_numpy(extra[f"init/{name}.weight"].view(np.int16)).view(w.dtype))
        out[f"H/{name}"] = h.numpy()
        if c is not None:
            out[f"C/{name}"] = c.numpy()
    out["results"] = np.array(list(qz.results))
    for name, r in qz.results.items():
        out[f"qweight/{name}"] = r.qweight.numpy()
        out[f"qzeros/{name}"] = _np(r.qzeros)
        out[f"scales/{name}"] = _np(r.scales)
        out[f"packed/{name}"] = np.int64(bool(r.qweight_is_packed))
        out[f"rtn/{name}"] = np.int64(r.quantization_time is None)
        if r.perm is not None:
            out[f"perm/{name}"] = r.perm.numpy()
    np.savez_compressed(os.path.join(HERE, f"driver_{tag}.npz"), **out)


def _run_reference_generic_driver(ref_gptq, model, ids, quantizer_kw, tag, extra):
    """The reference's generic driver run_quantize_with_qep (onecomp/qep/_quantize_with_qep.py:35-133)
    on CPU: one forward per layer, every layer computes its own H (calculate_hessian) and C
    (calculate_delta_hatX) from captured activations.  Records both per layer, the order, and the
    results."""
    from onecomp.qep import _quantize_with_qep as ref_generic
    from onecomp.qep._qep_config import QEPConfig

    original = ref_generic.prepare_calibration_dataset
    ref_generic.prepare_calibration_dataset = lambda **_kw: {"input_ids": ids}
    order, hs, cs = [], {}, {}

    class Recording(ref_gptq.GPTQ):
        def calculate_hessian(self, module, input):  # pylint: disable=redefined-builtin
            h, n = super().calculate_hessian(module, input)
            name = self.module_to_name[module]
            if name not in hs:
                order.append(name)
                hs[name] = h.clone()
            return h, n

        def calculate_delta_hatX(self, module, quant_input_activation, original_input_activation):
            c = super().calculate_delta_hatX(module, quant_input_activation, original_input_activation)
            cs[self.module_to_name[module]] = c.clone()
            return c

    qz = Recording(**quantizer_kw)
    try:
        ref_generic.run_quantize_with_qep(
            model_config=_FakeModelConfig(model), quantizer=qz,
            qep_config=QEPConfig(general=True, device="cpu", percdamp=0.01, perccorr=0.5),
            calibration_config=None, report_progress=False)
    finally:
        ref_generic.prepare_calibration_dataset = original
    out = {"ids": ids.numpy(), "order": np.array(order), "results": np.array(list(qz.results))}
    out.update(extra)
    for name, p in model.state_dict().items():
        out[f"final/{name}"] = _np(p.detach().cpu())
    for name in order:
        out[f"H/{name}"] = hs[name].numpy()
        if name in cs:
            out[f"C/{name}"] = cs[name].numpy()
    for name, r in qz.results.items():
        out[f"qweight/{name}"] = r.qweight.numpy()
        out[f"qzeros/{name}"] = _np(r.qzeros)
        out[f"scales/{name}"] = _np(r.scales)
        out[f"packed/{name}"] = np.int64(bool(r.qweight_is_packed))
    np.savez_compressed(os.path.join(HERE, f"driver_{tag}.npz"), **out)


def driver_fixtures(ref_gptq, ref_arch):
    """Block-wise QEP driver of the reference on the seeded toy models of tests/toy_models.py."""
    sys.path.insert(0, os.path.dirname(HERE))
    import toy_models

    torch.set_num_threads(1)
    for tag, kw in (("llama_b4", dict(wbits=4, groupsize=32, sym=False)),
                    ("llama_b3_actorder", dict(wbits=3, groupsize=32, sym=True, actorder=True))):
        model = toy_models.tiny_llama(seed=0)
        init = {f"init/{k}": _np(v.detach().clone()) for k, v in model.state_dict().items()}
        _run_reference_driver(ref_gptq, ref_arch, model, toy_models.llama_ids(0), kw, tag, extra=init)
    model = toy_models.tiny_llama(seed=0)
    init = {f"init/{k}": _np(v.detach().clone()) for k, v in model.state_dict().items()}
    _run_reference_generic_driver(ref_gptq, model, toy_models.llama_ids(0), dict(wbits=4, groupsize=32, sym=False),
                                  "generic_llama_b4", init)
    model = toy_models.routed_moe(seed=0)
    init = {f"init/{k}": _np(v.detach().clone()) for k, v in model.state_dict().items()}
    _run_reference_driver(ref_gptq, ref_arch, model, toy_models.moe_ids(0),
                          dict(wbits=4, groupsize=16, sym=False, exclude_layer_keywords=["router"]),
                          "moe", extra=init)


def _prep_h(h, perm):
    dead = torch.diag(h) == 0
    h[dead, dead] = 1
    if perm is not None:
        h = h[perm][:, perm]
    return h


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path to the OneCompression source tree>")
    main(sys.argv[1])
