"""Import shim for the compiled native module ``blitz_core`` living in ``blitz_scale_b200/_lib``."""
from __future__ import annotations

import importlib.machinery
import importlib.util
import sys
from pathlib import Path

_dir = Path(__file__).resolve().parent.parent / "_lib"


def _load():
    if "blitz_core" in sys.modules:
        return sys.modules["blitz_core"]
    cands = sorted(_dir.glob("blitz_core*.so"))
    if not cands:
        raise ImportError(f"native module blitz_core not built: run `python -m blitz_scale_b200.build` ({_dir})")
    loader = importlib.machinery.ExtensionFileLoader("blitz_core", str(cands[0]))
    spec = importlib.util.spec_from_loader("blitz_core", loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    sys.modules["blitz_core"] = mod
    return mod


_m = _load()
globals().update({k: getattr(_m, k) for k in dir(_m) if not k.startswith("__")})
