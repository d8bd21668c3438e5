from .chunked_quantization import accumulate_moments, quantize_group, run_chunked_quantization  # noqa: F401
