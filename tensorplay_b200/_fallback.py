"""Builder of the thin packages that are PyTorch's under another path: ``make(name, base, search, extra)`` returns a module
that shows ``base``'s namespace, looks further names up in the ``search`` modules (PyTorch keeps many of the names that
the reference lists at a package's top level in sub-modules), and carries ``extra`` definitions of its own. Sub-module
paths below it resolve to ``base``'s sub-modules as the same objects."""
from __future__ import annotations

import importlib
import sys
import types
from typing import Dict, Iterable, Optional


def make(name: str, base: str, search: Iterable[str] = (), extra: Optional[Dict[str, object]] = None, doc: str = "") -> types.ModuleType:
    base_mod = importlib.import_module(base)
    mod = types.ModuleType(name, doc or f"{base} under this framework's path.")
    mod.__path__ = list(getattr(base_mod, "__path__", []))  # (the front finder maps sub-modules to base's, never re-executes)
    mod.__dict__["__wrapped_base__"] = base_mod
    search = tuple(search)
    extra = dict(extra or {})

    def lookup(attr):
        if attr in extra:
            return extra[attr]
        try:
            return getattr(base_mod, attr)
        except AttributeError:
            pass
        for s in search:
            try:
                m = importlib.import_module(s)
            except ImportError:
                continue
            if hasattr(m, attr):
                return getattr(m, attr)
        try:
            return importlib.import_module(f"{base}.{attr}")
        except ImportError:
            raise AttributeError(f"module {name!r} has no attribute {attr!r}") from None
    mod.__getattr__ = lookup
    mod.__dir__ = lambda: sorted(set(dir(base_mod)) | set(extra))
    sys.modules[name] = mod
    return mod
