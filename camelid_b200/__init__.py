"""camelid_b200 — B200 (sm_100a) decode engine behind Camelid's resident-GPU boundary.

The package is a thin ctypes layer over ``libcamelid_b200.so`` (built in-tree by
``python -m camelid_b200.build``).  There is no CPU path: importing loads the library and
every compute call needs a B200.
"""
from ._lib import CmldError, lib, lib_path, declared_symbols  # noqa: F401
from .engine import (  # noqa: F401
    Q8_0, Q4_K, Q6_K, F32, Q8_0_HOST36, ACT_Q8_0, ACT_Q8_K,
    DeviceBuffer, Weight, ResidentDecode, EngineConfig,
    act_row_bytes, device_count,
)
