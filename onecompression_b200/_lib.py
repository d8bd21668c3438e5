"""ctypes binding of libonecomp_b200.so (the C ABI declared in include/onecomp_b200.h).

There is no CPU fallback: if the library is missing, every compute call raises.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_longlong, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libonecomp_b200.so")

# name -> (restype, argtypes); mirrors include/onecomp_b200.h one to one
_P, _I, _L, _F = c_void_p, c_int, c_longlong, c_float
SIGNATURES = {
    "oc_version": (_I, []),
    "oc_last_error": (c_char_p, []),
    "oc_launch_count": (_L, []),
    "oc_launch_count_reset": (_L, []),
    "oc_moment_accum": (_I, [_P, _P, _P, _L, _I, _L, _P, _P, _L, _F, _F, _I, _I, _I, _I, _P, _P]),
    "oc_moment_static_capacity": (_L, []),
    "oc_moment_accum_static": (_I, [_P, _P, _L, _I, _L, _P, _P, _L, _F, _F, _I, _I, _I, _P, _P]),
    "oc_mirror_upper": (_I, [_P, _L, _I, _P]),
    "oc_hinv_workspace_bytes": (_L, [_I]),
    "oc_hinv_factor": (_I, [_P, _L, _I, _F, _F, _I, _I, _P, _L, _P, _P, _P, _P, _P, _P, _L, _P]),
    "oc_gptq_workspace_bytes": (_L, [_I, _I, _I]),
    "oc_gptq_quantize": (_I, [_P, _L, _I, _I, _P, _L, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _P, _P,
                              _P, _P, _P, _L, _P, _P, _L, _I, _P, _L, _P]),
    "oc_hinv_factor_batched": (_I, [_I, _P, _I, _F, _I, _P, _P, _P, _P, _P, _P, _P, _L, _P]),
    "oc_gptq_quantize_batched": (_I, [_I, _P, _L, _I, _I, _P, _L, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I,
                                      _P, _P, _P, _P, _P, _P, _P, _I, _P, _L, _P]),
    "oc_rtn_quantize": (_I, [_P, _L, _I, _I, _I, _I, _I, _P, _P, _P, _P, _I, _P]),
    "oc_qep_workspace_bytes": (_L, [_I, _I]),
    "oc_qep_adjust": (_I, [_P, _L, _I, _I, _P, _L, _P, _L, _P, _P, _F, _I, _P, _L, _P]),
    "oc_rmsnorm_f16": (_I, [_P, _L, _P, _F, _L, _I, _P, _L, _P]),
    "oc_rope_f16": (_I, [_P, _P, _P, _P, _L, _I, _I, _I, _L, _L, _L, _L, _L, _L, _L, _L, _I, _P]),
    "oc_swiglu_f16": (_I, [_P, _P, _P, _L, _I, _P]),
    "oc_pack_qweight": (_I, [_P, _I, _I, _I, _P, _P]),
    "oc_unpack_qweight": (_I, [_P, _I, _I, _I, _P, _P]),
    "oc_pack_qzeros": (_I, [_P, _I, _I, _I, _I, _P, _P]),
    "oc_unpack_qzeros": (_I, [_P, _I, _I, _I, _I, _P, _P]),
    "oc_dequantize_packed": (_I, [_P, _P, _P, _P, _I, _I, _I, _P, _L, _P]),
    "oc_gemm_f32": (_I, [_P, _L, _P, _L, _P, _L, _I, _I, _I, _F, _F, _I, _I, _I, _P]),
    "oc_set_gemm_engine": (_I, [_I]),
    "oc_set_gemm_tile_shape": (_I, [_I]),
    "oc_gemm_tile_choice": (_I, [_I, _I, _I, _I, _I]),
    "oc_gemm_tc_status": (_I, []),
}

OC_ERR_UNSUPPORTED = -3

_lib = None


class KernelError(RuntimeError):
    """A C-ABI call returned a negative status."""

    def __init__(self, name, code, message):
        super().__init__(f"{name} failed ({code}): {message}")
        self.code = code


def load():
    """Load the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m onecompression_b200.build`. "
            "This package has no CPU or PyTorch fallback."
        )
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def call(name, *args):
    """Call an int-returning entry point and raise KernelError on failure."""
    lib = load()
    rc = getattr(lib, name)(*args)
    if rc != 0:
        raise KernelError(name, rc, lib.oc_last_error().decode())
    return rc


def ptr(t):
    """Device pointer of a tensor (or None)."""
    return None if t is None else t.data_ptr()


def stream_handle():
    import torch

    return torch.cuda.current_stream().cuda_stream
