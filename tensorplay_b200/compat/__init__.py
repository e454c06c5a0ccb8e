"""Make ``import tensorplay`` (and every ``tensorplay.x.y``) resolve to this package, for code written
against the reference. Every aliased name maps to the *same* module object as its
``tensorplay_b200`` spelling, so process-wide state (symmetric arena, registries) exists once."""
import importlib
import importlib.util
import sys


class _AliasLoader:
    def __init__(self, real: str):
        self.real = real

    def create_module(self, spec):
        return importlib.import_module(self.real)

    def exec_module(self, module):
        pass


class _AliasFinder:
    def __init__(self, name: str):
        self.name = name

    def find_spec(self, fullname, path=None, target=None):
        if fullname != self.name and not fullname.startswith(self.name + "."):
            return None
        real = "tensorplay_b200" + fullname[len(self.name):]
        try:
            importlib.import_module(real)
        except ImportError:
            return None
        return importlib.util.spec_from_loader(fullname, _AliasLoader(real))


def install_alias(name: str = "tensorplay") -> None:
    import tensorplay_b200
    if not [f for f in sys.meta_path if isinstance(f, _AliasFinder) and f.name == name]:
        sys.meta_path.insert(0, _AliasFinder(name))     # before the path finder: no second copies
    sys.modules.setdefault(name, tensorplay_b200)
