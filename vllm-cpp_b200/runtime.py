"""The host runtime (C++: page pools, block tables, state slots, scheduler), built on first use."""
from __future__ import annotations

import importlib.util
import sys

from .csrc import build as _build

_mod = None


def runtime():
    global _mod
    if _mod is None:
        path = _build.build_runtime()
        spec = importlib.util.spec_from_file_location("_vcb_runtime", str(path))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        sys.modules.setdefault("_vcb_runtime", mod)
        _mod = mod
    return _mod
