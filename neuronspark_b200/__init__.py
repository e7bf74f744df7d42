"""neuronspark_b200 — B200 (sm_100a) kernels for NeuronSpark's PLIF scan path.

Submodules mirror the reference's ``atomic_ops`` files for this path:
``parallel_scan``, ``fp16_codec``, ``lateral_inhibition``. ``install`` rebinds
the reference's own modules to these implementations.
"""
from ._lib import (NSBError, set_tuning, set_wait_limit_ns, set_time_split, last_time_split,  # noqa: F401
                   last_launch_info, set_scan_rotation, last_scan_rotation,
                   device_error_word, LIB_PATH)

__version__ = "0.1.0"
