"""``autograd``: torch's engine (replaces the reference's tpx engine, tpx/src/Engine.cpp:229-879);
the fused kernels of this package plug in as ``autograd.Function`` nodes."""
from torch.autograd import *  # noqa: F401,F403
from torch.autograd import (Function, backward, enable_grad, forward_ad, functional, grad,  # noqa: F401
                            gradcheck, gradgradcheck, graph, inference_mode, no_grad, profiler,
                            set_grad_enabled)


def __getattr__(name):
    """Names not defined here resolve to PyTorch's autograd (functional jacobian / hessian / jvp / vjp, graph hooks, mode queries)."""
    import importlib
    for mod in ['torch.autograd', 'torch.autograd.functional', 'torch.autograd.graph', 'torch.autograd.grad_mode', 'torch']:
        try:
            return getattr(importlib.import_module(mod), name)
        except (ImportError, AttributeError):
            continue
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
