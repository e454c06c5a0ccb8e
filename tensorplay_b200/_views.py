"""Import views for the domain packs. The reference spreads a pack over many small modules
(``metrics/classification/accuracy.py``, ``lumen/_core/layer/grad_cam.py``, ``quantum/_gates.py`` ...); here a pack
is a few files by kind of state. ``install(package)`` keeps every module path of the reference importable: a
sub-module name without a file resolves to a view whose attributes are looked up in the pack's namespace (in the
pack's ``functional`` namespace for paths below ``functional``), so ``from tensorplay.metrics.classification.accuracy
import BinaryAccuracy`` finds the class that ``tensorplay.metrics.BinaryAccuracy`` names."""
from __future__ import annotations

import importlib
import importlib.util
import sys
import types


class _ViewLoader:
    def __init__(self, package: str, namespace: str):
        self.package, self.namespace = package, namespace

    def create_module(self, spec):
        pkg = importlib.import_module(self.namespace)
        target = pkg
        if ".functional" in spec.name[len(self.package):] and hasattr(pkg, "functional"):
            target = pkg.functional
        mod = types.ModuleType(spec.name, f"View of {target.__name__}.")
        mod.__path__ = []           # deeper names resolve the same way

        def lookup(attr, _t=target, _p=pkg, _n=spec.name):
            if attr.startswith("__"):
                raise AttributeError(attr)
            try:
                return getattr(_t, attr)
            except AttributeError:
                if _t is not _p:
                    try:
                        return getattr(_p, attr)
                    except AttributeError:
                        pass
                raise AttributeError(f"module {_n!r} has no attribute {attr!r} (looked up in {_t.__name__})") from None
        mod.__getattr__ = lookup
        return mod

    def exec_module(self, module):
        pass


class _ViewFinder:
    """``from pack.some.view import Name`` makes Python try ``pack.some.view.Name`` as a module when the view has no
    such attribute. So that a misspelt class still raises ImportError instead of coming back as an empty view, names
    that cannot be module names of the reference are refused: anything with an upper-case letter, and anything
    deeper below the pack than its module tree goes (one level more below ``functional``)."""

    def __init__(self, package: str, max_depth: int, namespace: str, names=None):
        self.package, self.max_depth, self.namespace = package, max_depth, namespace
        self.names = None if names is None else frozenset(names)

    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(self.package + "."):
            return None
        parts = fullname[len(self.package) + 1:].split(".")
        depth = len(parts) - (1 if parts[0] == "functional" else 0)
        if depth > self.max_depth or any(c.isupper() for c in parts[-1]):
            return None
        if self.names is not None and parts[0] not in self.names:
            return None
        return importlib.util.spec_from_loader(fullname, _ViewLoader(self.package, self.namespace))


def install(package: str, max_depth: int = 3, namespace: str = "", names=None) -> None:
    """Appended to ``sys.meta_path``: real files of the pack are found first (and PyTorch's module of the same path
    where the package falls back to PyTorch). ``max_depth``: levels of module names below the pack in the reference's
    tree; ``namespace``: the module whose attributes the views show (default: the package itself); ``names``: the only
    first-level module names that get a view (a package outside the domain packs lists them, so that a misspelt module
    name still raises ``ModuleNotFoundError``)."""
    if not [f for f in sys.meta_path if isinstance(f, _ViewFinder) and f.package == package]:
        sys.meta_path.append(_ViewFinder(package, max_depth, namespace or package, names))
