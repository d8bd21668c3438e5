from .save import build_quantization_config, load_quantized_layers, quantized_state_dict, save_quantized_model  # noqa: F401
from .unfuse_moe import RoutedExperts, fuse_moe_experts, unfuse_moe_experts  # noqa: F401
