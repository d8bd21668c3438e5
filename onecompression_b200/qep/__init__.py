from ._qep_config import QEPConfig  # noqa: F401
