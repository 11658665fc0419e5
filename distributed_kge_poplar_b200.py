"""Import name for the package directory ``distributed-kge-poplar_b200/``.

A hyphen cannot appear in an ``import`` statement; importing this module loads the package
from that directory and registers it under ``distributed_kge_poplar_b200``.
"""

import importlib.util
import sys
from pathlib import Path

_dir = Path(__file__).resolve().parent / "distributed-kge-poplar_b200"
_spec = importlib.util.spec_from_file_location(
    __name__, _dir / "__init__.py", submodule_search_locations=[str(_dir)]
)
_module = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _module
_spec.loader.exec_module(_module)
