from ._qep_config import QEPConfig  # noqa: F401
from ._quantize_with_qep import capture_input_activations, run_quantize_with_qep  # noqa: F401
from ._quantize_with_qep_arch import run_quantize_with_qep_arch  # noqa: F401
