from ._autobit import (AutoBitQuantizer, collect_activation_stats, effective_bits_per_param,  # noqa: F401
                       solve_assignment)
