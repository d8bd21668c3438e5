"""What a saved model holds per layer, against the reference's own inference layer.

``tests/golden/layer_state.npz`` stores the state dict of the reference's
``GPTQLinear.from_quantization_result`` (onecomp/quantizer/gptq/gptq_layer.py:395-433, 576-628) for
four GPTQ cases and the ``quantization_config`` of a plain and a mixed-precision quantizer
(onecomp/quantizer/gptq/_gptq.py:480-566).  This package's layer, built from the same packed result,
must expose the same keys with the same shapes, dtypes and values, and its quantizers must write
the same configuration.  No kernel runs here (packed inputs stay packed)."""

import json

import numpy as np
import pytest
import torch

from conftest import f16, load_golden


def _tensor(arr, dtype):
    if dtype == "torch.float16":
        return f16(arr)
    return torch.from_numpy(np.ascontiguousarray(arr))


@pytest.mark.parametrize("case", ["b4_g128_asym", "b4_g128_asym_actorder", "b3_g128_sym", "b8_perchannel_sym"])
def test_inference_layer_state_matches_reference_layer(case):
    from onecompression_b200.quantizer.gptq._gptq import GPTQResult
    from onecompression_b200.quantizer.gptq.gptq_layer import GPTQLinear

    z = load_golden("layer_state.npz")
    g = load_golden(f"gptq_{case}.npz")
    keys = [str(k) for k in z[f"{case}/keys"]]
    want = {k: _tensor(z[f"{case}/{k}"], str(z[f"{case}/{k}/dtype"])) for k in keys}
    out_features, in_features = g["codes"].shape
    gs, bits, act = int(g["groupsize"]), int(g["wbits"]), bool(g["actorder"])
    scales = f16(g["scales"])
    result = GPTQResult(
        wbits=bits, groupsize=gs, actorder=act, sym=bool(g["sym"]),
        qweight=torch.from_numpy(g["qweight_packed"]), scales=scales, qzeros=torch.from_numpy(g["qzeros_packed"]),
        perm=torch.from_numpy(g["perm"]) if act else None, qweight_is_packed=True, qzeros_is_packed=True,
        qweight_original_shape=(out_features, in_features))
    layer = GPTQLinear.from_quantization_result(result, bias=want["bias"], device="cpu", pack_weights=True)
    state = layer.state_dict()
    assert sorted(state) == sorted(keys)
    for k in keys:
        assert state[k].dtype == want[k].dtype, (k, state[k].dtype, want[k].dtype)
        assert tuple(state[k].shape) == tuple(want[k].shape), (k, state[k].shape, want[k].shape)
        assert torch.equal(state[k], want[k]), k
    assert state["qweight"].shape == (in_features * bits // 32, out_features)
    assert state["g_idx"].dtype == torch.int32 and state["g_idx"].shape == (in_features,)


@pytest.mark.parametrize("tag", ["plain", "mixed"])
def test_quantization_config_matches_reference(tag):
    from onecompression_b200 import GPTQ

    z = load_golden("layer_state.npz")
    kw = json.loads(str(z[f"config/{tag}/kwargs"]))
    q = GPTQ(**kw)
    cfg = q.get_quant_config()
    assert cfg == json.loads(str(z[f"config/{tag}/quant_config"]))
    names = [str(n) for n in z["config/names"]]
    final = q.finalize_quant_config_for_save(dict(cfg), names, num_hidden_layers=2)
    assert final == json.loads(str(z[f"config/{tag}/final"]))
