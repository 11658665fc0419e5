"""B200-native BESS knowledge-graph-embedding training step.

``capi``        ctypes view of the C ABI (include/kge_b200.h)
``poplar_kge``  the reference's host interface (Settings, Batch, Predictions, Engine) on top of
                the compiled ``libpoplar_kge`` module
``build``       compiles both shared libraries for sm_100a, in tree

The directory name carries a hyphen, so it is imported through the loader module
``distributed_kge_poplar_b200`` at the repository root.
"""

from . import capi  # noqa: F401
from . import poplar_kge  # noqa: F401

__all__ = ["capi", "poplar_kge"]
