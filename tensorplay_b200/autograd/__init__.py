"""``autograd``: torch's engine (replaces the reference's tpx engine, tpx/src/Engine.cpp:229-879);
the fused kernels of this package plug in as ``autograd.Function`` nodes."""
from torch.autograd import *  # noqa: F401,F403
from torch.autograd import (Function, backward, enable_grad, forward_ad, functional, grad,  # noqa: F401
                            gradcheck, gradgradcheck, graph, inference_mode, no_grad, profiler,
                            set_grad_enabled)
