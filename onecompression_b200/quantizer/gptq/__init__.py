from ._gptq import GPTQ, GPTQResult, run_gptq  # noqa: F401
from .gptq_layer import (  # noqa: F401
    GPTQLinear, PACKABLE_WBITS, is_packable_wbits, make_g_idx, normalize_scale_zero, pack_int_weights,
    pack_zeros, unpack_int_weights, unpack_zeros,
)
