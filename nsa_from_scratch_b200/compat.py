"""Drop-in shim: after `install()`, the module names the reference's callers import
(`nsa.triton.compressed|selected|sliding|gating|forward|backward|fp8`, `nsa.cuda`) resolve to
this package, so the reference's model, benchmarks and tests run on these kernels unchanged.
`nsa.reference` (and everything else under `nsa`) still comes from the reference checkout
when it is importable; otherwise a minimal `nsa.reference` with NSAConfig is provided."""
from __future__ import annotations

import importlib
import sys
import types

_MAP = {
    "nsa.triton.compressed": "compressed", "nsa.triton.selected": "selected", "nsa.triton.sliding": "sliding",
    "nsa.triton.gating": "gating", "nsa.triton.forward": "forward", "nsa.triton.backward": "backward",
    "nsa.triton.fp8": "fp8", "nsa.cuda": "native",
}


def install() -> None:
    pkg = __name__.rsplit(".", 1)[0]
    try:
        importlib.import_module("nsa")
    except ImportError:
        nsa = types.ModuleType("nsa")
        nsa.__path__ = []
        sys.modules["nsa"] = nsa
        ref = types.ModuleType("nsa.reference")
        ref.NSAConfig = importlib.import_module(pkg + ".config").NSAConfig
        sys.modules["nsa.reference"] = ref
    if "nsa.triton" not in sys.modules:
        tri = types.ModuleType("nsa.triton")
        tri.__path__ = []
        sys.modules["nsa.triton"] = tri
    for name, ours in _MAP.items():
        mod = importlib.import_module(f"{pkg}.{ours}")
        sys.modules[name] = mod
        parent, _, leaf = name.rpartition(".")
        setattr(sys.modules[parent], leaf, mod)
