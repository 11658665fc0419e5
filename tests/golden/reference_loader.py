"""Import the reference's pure-Python files unchanged, for generating fixtures.

The reference's ``poplar_kge.py`` imports two Poplar SDK modules (``libpvti``,
``libpoplar_kge``) and its dataset module imports ``ogb.lsc``; none is
installed.  Empty stand-ins are placed in ``sys.modules`` so the files import
as they are; nothing of the SDK is emulated.  Only fixture generation and the
CPU tests that validate the oracle use this, and only where a checkout of the
reference is present: the directory named by ``REFERENCE_ROOT``, or a directory
``reference`` beside this repository.
"""

from __future__ import annotations

import os
import sys
import types
from pathlib import Path

REFERENCE_ROOT = Path(os.environ.get("REFERENCE_ROOT") or Path(__file__).resolve().parents[3] / "reference")


def available() -> bool:
    return (REFERENCE_ROOT / "tests/python/reference_model.py").exists()


def load():
    """Returns (poplar_kge, poplar_kge_dataset, reference_model) of the reference."""
    if not available():
        raise RuntimeError(f"no reference checkout at {REFERENCE_ROOT}")
    if "libpvti" not in sys.modules:
        pvti = types.ModuleType("libpvti")
        pvti.createTraceChannel = lambda name: name
        pvti.instrument_fn = lambda channel: (lambda fn: fn)
        sys.modules["libpvti"] = pvti
    if "ogb" not in sys.modules:
        ogb = types.ModuleType("ogb")
        ogb.lsc = types.ModuleType("ogb.lsc")
        sys.modules["ogb"], sys.modules["ogb.lsc"] = ogb, ogb.lsc
    saved = {k: sys.modules.pop(k, None) for k in ("libpoplar_kge", "poplar_kge")}
    engine_stub = types.ModuleType("libpoplar_kge")
    engine_stub.Engine = None
    engine_stub.__file__ = str(REFERENCE_ROOT / "build" / "libpoplar_kge.so")
    sys.modules["libpoplar_kge"] = engine_stub
    sys.path[:0] = [str(REFERENCE_ROOT / "src/python"), str(REFERENCE_ROOT / "tests/python")]
    try:
        import poplar_kge as ref_kge
        import poplar_kge_dataset as ref_data
        import reference_model as ref_model
    finally:
        del sys.path[:2]
        # leave no reference module under a name the product also uses
        for name in ("poplar_kge", "poplar_kge_dataset", "reference_model", "libpoplar_kge"):
            sys.modules.pop(name, None)
        for name, mod in saved.items():
            if mod is not None:
                sys.modules[name] = mod
    return ref_kge, ref_data, ref_model


def fix_adam_step(model) -> None:
    """torch >= 1.12 wants the Adam ``step`` entry as a tensor; the reference stores
    the int it read from the engine (tests/python/reference_model.py:54-66)."""
    import torch

    for entry in model.opt.state.values():
        entry["step"] = torch.tensor(float(entry["step"]))
