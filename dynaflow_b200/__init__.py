"""dynaflow_b200: B200-native execution backend behind DynaFlow's scheduling API.

The host-facing modules mirror the reference package ``dynaflow`` one to one
(``config``, ``interface``, ``manager``, ``matching``, ``utils``, ``executor``,
``runtime``); ``install_as_dynaflow()`` makes them importable under that name so
that host glue and policy files written against the reference load unchanged.
The compute path lives in ``ops`` (ctypes over ``libdynaflow_b200.so``).
"""
from __future__ import annotations

import importlib
import sys

__version__ = "0.1.0"

_MIRRORED = ("config", "interface", "manager", "matching", "utils", "executor", "executor.compiler",
             "executor.cudagraph", "runtime", "runtime.env", "runtime.engine")


def install_as_dynaflow(force: bool = False) -> None:
    """Registers this package and its mirrored submodules as ``dynaflow[.x]`` in
    ``sys.modules``. Refuses to shadow an already imported ``dynaflow`` unless ``force``."""
    existing = sys.modules.get("dynaflow")
    this = sys.modules[__name__]
    if existing is not None and existing is not this and not force:
        raise RuntimeError("a different 'dynaflow' package is already imported")
    sys.modules["dynaflow"] = this
    for name in _MIRRORED:
        sys.modules[f"dynaflow.{name}"] = importlib.import_module(f"{__name__}.{name}")
