"""B200-native GPTQ / QEP layer quantization behind OneComp's quantizer API.

All arithmetic runs in ``libonecomp_b200.so`` (hand-written sm_100a CUDA, loaded
through its C ABI with ctypes).  There is no CPU or PyTorch fallback.
"""

from . import kernels  # noqa: F401
from .qep import QEPConfig  # noqa: F401
from .quantizer import QuantizationResult, Quantizer  # noqa: F401
from .quantizer.gptq import GPTQ, GPTQResult, run_gptq  # noqa: F401
from .quantizer.autobit import AutoBitQuantizer  # noqa: F401

__version__ = "0.1.0"
