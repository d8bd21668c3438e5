from ._autobit import AutoBitQuantizer, effective_bits_per_param, solve_assignment  # noqa: F401
