from ._quantizer import QuantizationResult, Quantizer, ResultLoader  # noqa: F401
