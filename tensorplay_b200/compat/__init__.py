"""Make ``import tensorplay`` resolve to this package (for code written against the reference)."""
import importlib
import sys


def install_alias(name: str = "tensorplay") -> None:
    import tensorplay_b200
    sys.modules.setdefault(name, tensorplay_b200)
    for sub in ("nn", "nn.functional", "optim", "amp", "serialization", "distributed", "utils",
                "ops", "autograd", "cuda", "profiler"):
        try:
            mod = importlib.import_module(f"tensorplay_b200.{sub}")
        except Exception:
            continue
        sys.modules.setdefault(f"{name}.{sub}", mod)
