"""``optim``: the optimizer zoo. AdamW / Adam run the fused multi-tensor sm_100a kernel on CUDA
(fp32 master + moments, bf16 parameter emit in the same pass); the rest of the zoo is torch's;
``Muon`` is implemented here (the reference ships it in tensorplay/optim, P3)."""
from torch.optim import (ASGD, LBFGS, SGD, Adadelta, Adafactor, Adagrad, Adamax, NAdam, Optimizer,  # noqa: F401
                         RAdam, RMSprop, Rprop, SparseAdam, lr_scheduler, swa_utils)

from .adamw import Adam, AdamW
from .muon import Muon

__all__ = ["ASGD", "LBFGS", "SGD", "Adadelta", "Adafactor", "Adagrad", "Adamax", "NAdam", "Optimizer",
           "RAdam", "RMSprop", "Rprop", "SparseAdam", "lr_scheduler", "swa_utils", "Adam", "AdamW", "Muon"]
