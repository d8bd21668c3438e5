import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name):
    """Load a fixture; fp16 tensors are stored as raw uint16 bits."""
    z = np.load(os.path.join(GOLDEN, name))
    return {k: z[k] for k in z.files}


def f16(bits):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.float16).copy())


def bf16(bits):
    """bfloat16 tensor from its raw bits (fixtures store bf16 as uint16)."""
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16).copy()).view(torch.bfloat16)


def bits16(t):
    """Raw bits of an fp16 / bf16 tensor as a uint16 array."""
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def gptq_case_names():
    return sorted(
        f[len("gptq_") : -len(".npz")] for f in os.listdir(GOLDEN) if f.startswith("gptq_")
    )
