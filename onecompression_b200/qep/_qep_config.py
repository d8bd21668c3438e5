"""QEP options (reference: onecomp/qep/_qep_config.py:12-57)."""

from dataclasses import dataclass, field


@dataclass
class QEPConfig:
    """general: generic per-layer driver instead of the block-wise one (not built
    here: the block-wise driver is the default path); percdamp / perccorr: damping
    and strength of the weight correction; device: where to compute;
    exclude_layer_keywords: layers quantized without correction."""

    general: bool = False
    percdamp: float = 0.01
    perccorr: float = 0.5
    device: str = None
    exclude_layer_keywords: list[str] = field(default_factory=lambda: ["mlp.down_proj"])
