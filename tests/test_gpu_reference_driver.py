"""The block driver against the reference's own driver.

``tests/golden/driver_*.npz`` hold what the reference's ``run_quantize_with_qep_arch``
(onecomp/qep/_quantize_with_qep_arch.py:323-627) did on the seeded toy models of
``tests/toy_models.py`` on CPU: the order of the layers, which layers it corrected, the Hessian and
cross term it handed to each layer, every layer's result, which expert layers fell back to RTN, and
the model it left behind.  Here this package's driver runs on the same weights and token ids on the
GPU and is compared with that record at three levels:

1. decisions: layer order, corrected / uncorrected layers, RTN fallbacks, result flags;
2. kernels on the reference's inputs: every layer re-quantized from the reference's own (W, H, C)
   must reproduce the reference's codes and scales (north-star tolerances);
3. the driver end to end: its own H and C against the reference's, and its results.

Level 3 compares two different fp16 forward passes (CPU operators there, cuBLAS / CUDA operators
here).  They differ in rare last-bit roundings of activations, so H agrees to about 1e-5 while no
quantized layer lies upstream and drifts afterwards, once single differing codes of earlier layers
have changed the activations; the tolerances below say which bar is which.
"""

import numpy as np
import pytest
import torch

import toy_models
from conftest import bits16, f16, load_golden
from oracle import gptq_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

LLAMA_CASES = {
    "llama_b4": dict(wbits=4, groupsize=32, sym=False),
    "llama_b3_actorder": dict(wbits=3, groupsize=32, sym=True, actorder=True),
}
MOE_KW = dict(wbits=4, groupsize=16, sym=False, exclude_layer_keywords=["router"])


def _rel(a, b):
    a, b = torch.as_tensor(a).double(), torch.as_tensor(b).double()
    nb = b.norm().item()
    return ((a - b).norm().item() / nb) if nb > 0 else (a - b).norm().item()


def _load_model(z, build):
    model = build(seed=0)
    state = {k[len("init/"):]: v for k, v in z.items() if k.startswith("init/")}
    sd = model.state_dict()
    for k, v in state.items():
        assert sd[k].dtype == torch.float16
        sd[k].copy_(f16(v).reshape(sd[k].shape))
    return model


def _spy_class():
    from onecompression_b200 import GPTQ

    class Spy(GPTQ):
        """Records what the driver hands to every layer (per-layer calls: no stacking, no batching).
        With ``forced`` (name -> weight) the driver continues after each layer with that weight in
        place of the layer's own dequantized weight."""

        def quantize_with_qep(self, module, *a, **kw):
            name = self.module_to_name[module]
            self.calls.append((name, kw["hessian"].detach().cpu().clone(),
                               None if kw.get("delta_hatX") is None else kw["delta_hatX"].detach().cpu().clone()))
            out = super().quantize_with_qep(module, *a, **kw)
            forced = getattr(self, "forced", None)
            if forced is not None:
                self.own_dequantized[name] = self.results[name].__dict__["_device_dequantized"].cpu()
                self.results[name].__dict__["_device_dequantized"] = forced[name].to(module.weight.device)
            return out

    return Spy


def _run_driver(model, ids, quantizer):
    from onecompression_b200 import QEPConfig
    from onecompression_b200.qep._quantize_with_qep_arch import run_quantize_with_qep_arch

    run_quantize_with_qep_arch(None, quantizer, QEPConfig(device=DEV, percdamp=0.01, perccorr=0.5), None,
                               model=model, model_inputs={"input_ids": ids}, report_progress=False,
                               batch_size=16)
    return quantizer


def _ref_codes(z, name, bits):
    qw = z[f"qweight/{name}"]
    if int(z[f"packed/{name}"]):
        out = z[f"init/{name}.weight"].shape
        return orc.unpack_qweight(qw, bits, out)
    return qw


def _our_codes(res):
    if res.qweight_is_packed:
        return orc.unpack_qweight(res.qweight.numpy(), res.wbits, res.qweight_original_shape)
    return res.qweight.numpy()


def _layer_from_reference_inputs(z, name, kw):
    """One layer through this package's quantize_with_qep from the reference driver's (W, H, C)."""
    from onecompression_b200 import GPTQ

    w = f16(z[f"init/{name}.weight"])
    lin = torch.nn.Linear(w.shape[1], w.shape[0], bias=False).half()
    lin.weight.data = w.clone()
    lin = lin.to(DEV)
    q = GPTQ(**kw)
    q.module_to_name = {lin: name}
    h = torch.from_numpy(z[f"H/{name}"]).to(DEV)
    c = torch.from_numpy(z[f"C/{name}"]).to(DEV) if f"C/{name}" in z else None
    q.quantize_with_qep(lin, None, None, percdamp=0.01, perccorr=0.5, hessian=h, delta_hatX=c)
    return q.results[name]


def _scale_ulps(res, z, name):
    s = bits16(res.scales).astype(np.int64).reshape(-1)
    sref = z[f"scales/{name}"].astype(np.int64).reshape(-1)
    return np.abs(s - sref)


@pytest.mark.parametrize("tag", sorted(LLAMA_CASES))
def test_layers_from_the_reference_drivers_inputs(tag):
    """Level 2: the reference driver's own (W, H, C) per layer through the CUDA kernels."""
    z = load_golden(f"driver_{tag}.npz")
    kw = LLAMA_CASES[tag]
    same = total = 0
    skipped_perm = []
    for name in z["order"]:
        name = str(name)
        res = _layer_from_reference_inputs(z, name, kw)
        if kw.get("actorder"):
            if not np.array_equal(res.perm.numpy(), z[f"perm/{name}"]):
                skipped_perm.append(name)      # torch.argsort is not stable: ties may order differently
                continue
        eq = _our_codes(res) == _ref_codes(z, name, kw["wbits"])
        same += int(eq.sum())
        total += eq.size
        assert eq.mean() >= 0.99, f"{name}: {eq.mean():.5f} identical codes"
        assert (_scale_ulps(res, z, name) <= 1).mean() >= 0.99, name
    print(f"[{tag}] layers with another column order: {len(skipped_perm)} of {len(z['order'])} {skipped_perm}")
    assert len(skipped_perm) <= 2
    assert same / total >= 0.999, f"{same / total:.5f} identical codes over {total}"


@pytest.mark.parametrize("tag", sorted(LLAMA_CASES))
def test_block_driver_follows_reference_driver_layer_by_layer(tag):
    """Levels 1 and 3 on the two-layer Llama, layer by layer: after each layer the run continues with
    the weight the reference's driver installed for it (from the fixture), so every layer's H and C
    are measured behind the same quantized weights as in the reference and differ only by the
    rounding of the two fp16 forward passes."""
    z = load_golden(f"driver_{tag}.npz")
    kw = LLAMA_CASES[tag]
    ids = torch.from_numpy(z["ids"])
    spy = _spy_class()(**kw)
    spy.calls, spy.own_dequantized = [], {}
    spy.forced = {str(n): f16(z[f"final/{n}.weight"]).reshape(z[f"init/{n}.weight"].shape) for n in z["order"]}
    model = _load_model(z, toy_models.tiny_llama)
    _run_driver(model, ids, spy)

    assert [c[0] for c in spy.calls] == [str(n) for n in z["order"]]
    assert sorted(spy.results) == sorted(str(n) for n in z["results"])
    same, total, perm_differs = 0, 0, []
    for name, h, c in spy.calls:
        assert (c is None) == (f"C/{name}" not in z), name          # mlp.down_proj: no correction
        eh = _rel(h, z[f"H/{name}"])
        ec = None if c is None else _rel(c, z[f"C/{name}"])
        res = spy.results[name]
        if kw.get("actorder") and not np.array_equal(res.perm.numpy(), z[f"perm/{name}"]):
            perm_differs.append(name)
            frac = float("nan")
        else:
            eq = _our_codes(res) == _ref_codes(z, name, kw["wbits"])
            same += int(eq.sum())
            total += eq.size
            frac = eq.mean()
            assert frac >= 0.99, (name, frac)
        print(f"[{tag}] {name}: H rel {eh:.2e}, C rel {'-' if ec is None else f'{ec:.2e}'}, codes {frac:.5f}")
        # H: about the north-star bar for the attention layers of block 0; further down the last-bit
        # differences between the CPU's and the GPU's fp16 operators (softmax, SiLU, the residual
        # sums of a whole block) add up to a few 1e-5
        blk = int(name.split(".")[2])
        assert eh < (2e-5 if (".layers.0.self_attn." in name) else 1e-4 if blk == 0 else 5e-4), (name, eh)
        if ec is not None:
            if not np.any(z[f"C/{name}"]):
                assert ec == 0.0, name          # q, k, v of block 0: nothing quantized upstream
            else:
                # C is made of differences of activations a few percent apart: the same last-bit
                # differences weigh 1/0.03 times more than in H (and block 1 sees them through all
                # of block 0)
                assert ec < (1e-3 if blk == 0 else 5e-3), (name, ec)
    print(f"[{tag}] layers with another column order: {len(perm_differs)} {perm_differs}; "
          f"identical codes {same / max(1, total):.5f}")
    assert len(perm_differs) <= 2
    # 64-wide layers amplify: H within 1e-5 and C within 3e-4 still flip a few codes per thousand in
    # the corrected layers (from the reference's exact inputs the same kernels reach 99.9 %, see
    # test_layers_from_the_reference_drivers_inputs)
    assert same / total >= 0.995, same / total


@pytest.mark.parametrize("tag", sorted(LLAMA_CASES))
def test_block_driver_against_reference_driver_free_running(tag):
    """Levels 1 and 3 with nothing forced.  On a 64-wide model one differing code in o_proj (1 of
    4096, from a last-bit difference of the forward passes) moves the next layer's Hessian by
    about 3e-3, so position-by-position agreement decays layer by layer; what stays comparable is
    what the north star asks of a whole layer: its reconstruction error."""
    from onecompression_b200 import GPTQ

    z = load_golden(f"driver_{tag}.npz")
    kw = LLAMA_CASES[tag]
    ids = torch.from_numpy(z["ids"])
    spy = _spy_class()(**kw)
    spy.calls = []
    model = _load_model(z, toy_models.tiny_llama)
    _run_driver(model, ids, spy)

    assert [c[0] for c in spy.calls] == [str(n) for n in z["order"]]
    assert sorted(spy.results) == sorted(str(n) for n in z["results"])
    for name, h, c in spy.calls:
        assert (c is None) == (f"C/{name}" not in z), name
        if ".layers.0.self_attn." in name and not name.endswith("o_proj"):
            assert _rel(h, z[f"H/{name}"]) < 1e-5 and not c.any() and not np.any(z[f"C/{name}"])
            eq = _our_codes(spy.results[name]) == _ref_codes(z, name, kw["wbits"])
            if not kw.get("actorder") or np.array_equal(spy.results[name].perm.numpy(), z[f"perm/{name}"]):
                assert eq.mean() >= 0.999, (name, eq.mean())
    # reconstruction error per block, each side with its own Hessians
    for blk in (0, 1):
        e_got = e_ref = 0.0
        for name, h, _c in spy.calls:
            if int(name.split(".")[2]) != blk:
                continue
            w0 = f16(z[f"init/{name}.weight"])
            mod = dict(model.named_modules())[name]
            e_got += orc.reconstruction_error(w0, mod.weight.data.cpu(), h, 1)
            e_ref += orc.reconstruction_error(w0, f16(z[f"final/{name}.weight"]).reshape(w0.shape),
                                              torch.from_numpy(z[f"H/{name}"]), 1)
        print(f"[{tag}] block {blk}: reconstruction error {e_got:.6e} vs reference {e_ref:.6e} "
              f"({(e_got - e_ref) / e_ref:+.3%})")
        assert abs(e_got - e_ref) <= (0.005 if blk == 0 else 0.03) * e_ref, (blk, e_got, e_ref)

    # the production path (stacked layers, one factor per group) gives the very same results
    plain = GPTQ(**kw)
    _run_driver(_load_model(z, toy_models.tiny_llama), ids, plain)
    for name, r in spy.results.items():
        p = plain.results[name]
        assert torch.equal(p.qweight, r.qweight) and torch.equal(p.scales, r.scales) \
            and torch.equal(p.qzeros, r.qzeros), name


def test_expert_hessians_and_fallbacks_against_reference_driver():
    """The routed mixture: per-expert Hessians from routed tokens only (reference
    _compute_per_module_hessians, :204-272), experts missed by the one-sample grouping, experts
    without any token (RTN fallback), the uncorrected expert layers."""
    from onecompression_b200 import GPTQ

    z = load_golden("driver_moe.npz")
    ids = torch.from_numpy(z["ids"])
    spy = _spy_class()(**MOE_KW)
    spy.calls = []
    model = _load_model(z, toy_models.routed_moe)
    _run_driver(model, ids, spy)

    # decisions: same layers in the same order, experts uncorrected, the same fallbacks
    assert [c[0] for c in spy.calls] == [str(n) for n in z["order"]]
    assert sorted(spy.results) == sorted(str(n) for n in z["results"])
    for name, _h, c in spy.calls:
        assert (c is None) == (f"C/{name}" not in z), name
        assert (c is None) == (".experts." in name)
    for name in z["results"]:
        name = str(name)
        res = spy.results[name]
        is_rtn = bool(z[f"rtn/{name}"])
        assert (res.quantization_time is None) == is_rtn, name
        assert bool(res.qweight_is_packed) == bool(z[f"packed/{name}"]), name
        if is_rtn:
            # no Hessian involved: the fallback is the same arithmetic on the same weight
            assert np.array_equal(res.qweight.numpy(), z[f"qweight/{name}"]), name
            assert np.array_equal(bits16(res.scales), z[f"scales/{name}"]), name
            assert np.array_equal(bits16(res.qzeros), z[f"qzeros/{name}"]), name
            mod = dict(model.named_modules())[name]
            assert np.array_equal(bits16(mod.weight.data).reshape(-1), z[f"final/{name}.weight"].reshape(-1)), name
    same = total = 0
    for name, h, c in spy.calls:
        blk = int(name.split(".")[2])
        eh = _rel(h, z[f"H/{name}"])
        # same dead columns (channels an expert never sees)
        assert np.array_equal(np.diag(h.numpy()) == 0, np.diag(z[f"H/{name}"]) == 0), name
        res = spy.results[name]
        eq = _our_codes(res) == _ref_codes(z, name, MOE_KW["wbits"])
        same += int(eq.sum())
        total += eq.size
        print(f"[moe] {name}: H rel {eh:.2e}, codes {eq.mean():.5f}")
        if blk == 0 and (name.endswith(".pre") or name.endswith("gate_proj") or name.endswith("up_proj")):
            # routed inputs of block 0 sit behind one quantized layer (`pre`) only
            assert eh < (1e-5 if name.endswith(".pre") else 1e-3), (name, eh)
        assert eh < 5e-3, (name, eh)
    print(f"[moe] identical codes over all calibrated layers: {same / total:.5f}")
    assert same / total >= 0.99

    # level 2 for the experts: the reference's own per-expert H through the kernels
    same = total = 0
    for name in z["order"]:
        name = str(name)
        res = _layer_from_reference_inputs(z, name, {k: v for k, v in MOE_KW.items() if k != "exclude_layer_keywords"})
        eq = _our_codes(res) == _ref_codes(z, name, MOE_KW["wbits"])
        same += int(eq.sum())
        total += eq.size
        assert (_scale_ulps(res, z, name) <= 1).mean() >= 0.99, name
    assert same / total >= 0.999, f"{same / total:.5f}"

    # batched experts (the production path) give the same results as the per-layer calls
    plain = GPTQ(**MOE_KW)
    _run_driver(_load_model(z, toy_models.routed_moe), ids, plain)
    for name, r in spy.results.items():
        p = plain.results[name]
        assert torch.equal(p.qweight, r.qweight) and torch.equal(p.scales, r.scales) \
            and torch.equal(p.qzeros, r.qzeros), name


def test_generic_driver_follows_reference_generic_driver():
    """The architecture-independent driver (reference run_quantize_with_qep,
    onecomp/qep/_quantize_with_qep.py:35-133): one forward pass per layer, every layer forms its own
    H (slices of eight sequences) and C from captured activations through
    Quantizer.calculate_hessian / calculate_delta_hatX.  Same comparison as for the block-wise driver:
    after each layer the run continues with the weight the reference installed."""
    from onecompression_b200 import GPTQ, QEPConfig
    from onecompression_b200.qep import run_quantize_with_qep

    z = load_golden("driver_generic_llama_b4.npz")
    kw = LLAMA_CASES["llama_b4"]
    order, hs, cs = [], {}, {}

    class Spy(GPTQ):
        def calculate_hessian(self, module, input):  # pylint: disable=redefined-builtin
            h, n = super().calculate_hessian(module, input)
            name = self.module_to_name[module]
            if name not in hs:
                order.append(name)
                hs[name] = h.detach().cpu().clone()
            return h, n

        def calculate_delta_hatX(self, module, quant_input_activation, original_input_activation):
            c = super().calculate_delta_hatX(module, quant_input_activation, original_input_activation)
            cs[self.module_to_name[module]] = c.detach().cpu().clone()
            return c

        def quantize_with_qep(self, module, *a, **k):
            out = super().quantize_with_qep(module, *a, **k)
            name = self.module_to_name[module]
            forced = f16(z[f"final/{name}.weight"]).reshape(z[f"init/{name}.weight"].shape)
            self.results[name].__dict__["_device_dequantized"] = forced.to(module.weight.device)
            return out

    spy = Spy(**kw)
    model = _load_model(z, toy_models.tiny_llama).to(DEV)
    ids = torch.from_numpy(z["ids"]).to(DEV)
    run_quantize_with_qep(None, spy, QEPConfig(general=True, device=DEV, percdamp=0.01, perccorr=0.5), None,
                          model=model, model_inputs={"input_ids": ids}, report_progress=False, batch_size=16)
    assert order == [str(n) for n in z["order"]]
    assert sorted(spy.results) == sorted(str(n) for n in z["results"])
    same = total = 0
    for name in order:
        blk = int(name.split(".")[2])
        assert (name in cs) == (f"C/{name}" in z), name                 # mlp.down_proj: no correction
        eh = _rel(hs[name], z[f"H/{name}"])
        ec = _rel(cs[name], z[f"C/{name}"]) if name in cs else None
        eq = _our_codes(spy.results[name]) == _ref_codes(z, name, kw["wbits"])
        same += int(eq.sum())
        total += eq.size
        print(f"[generic] {name}: H rel {eh:.2e}, C rel {'-' if ec is None else f'{ec:.2e}'}, codes {eq.mean():.5f}")
        assert eh < (2e-5 if (".layers.0.self_attn." in name) else 1e-4 if blk == 0 else 5e-4), (name, eh)
        if ec is not None:
            if not np.any(z[f"C/{name}"]):
                assert ec == 0.0, name
            else:
                assert ec < (1e-3 if blk == 0 else 5e-3), (name, ec)
        assert eq.mean() >= 0.99, (name, eq.mean())
    print(f"[generic] identical codes {same / total:.5f}")
    assert same / total >= 0.995
    # the model holds the forced (= the reference's) weights now
    for name in order:
        mod = dict(model.named_modules())[name]
        assert np.array_equal(bits16(mod.weight.data).reshape(-1), z[f"final/{name}.weight"].reshape(-1))
