"""``optim``: the optimizer zoo. AdamW / Adam, SGD, Adagrad, RMSprop and Adafactor run fused
sm_100a kernels on CUDA (fp32 state and master weights, bf16 parameter emit in the same pass); the
rest of the zoo is torch's; ``Muon`` is implemented here (the reference ships it in tensorplay/optim, P3)."""
from torch.optim import (ASGD, LBFGS, Adadelta, Adamax, NAdam, Optimizer,  # noqa: F401
                         RAdam, Rprop, SparseAdam, lr_scheduler, swa_utils)

from .adamw import Adam, AdamW
from .fused import SGD, Adafactor, Adagrad, RMSprop
from .muon import Muon

__all__ = ["ASGD", "LBFGS", "SGD", "Adadelta", "Adafactor", "Adagrad", "Adamax", "NAdam", "Optimizer",
           "RAdam", "RMSprop", "Rprop", "SparseAdam", "lr_scheduler", "swa_utils", "Adam", "AdamW", "Muon"]


import contextlib as _contextlib


@_contextlib.contextmanager
def swap_in_optimizer_params_and_state(optimizer, swapin_parameters, swapin_optim_state):
    """Temporarily run ``optimizer`` on replacement parameters and state (functional / stateless use:
    step on copies, evaluate hyper-parameter changes, meta-learning inner loops).

    ``swapin_parameters`` maps names to tensors in the order of the packed parameter indices;
    ``swapin_optim_state`` has the layout of ``optimizer.state_dict()`` (``state`` keyed by index,
    ``param_groups`` whose ``params`` are index lists). On exit the optimizer's own groups and state
    are back in place; whatever the steps inside wrote stays in the swapped-in tensors and dicts."""
    params = list(swapin_parameters.values())
    packed_state = swapin_optim_state.get("state", {})
    snapshots = [dict(g) for g in optimizer.param_groups]
    original_state = optimizer.state
    try:
        from collections import defaultdict
        new_state = defaultdict(dict)
        for live, packed in zip(optimizer.param_groups, swapin_optim_state["param_groups"]):
            live["params"] = [params[i] for i in packed["params"]]
            for k, v in packed.items():
                if k != "params":
                    live[k] = v
            for i in packed["params"]:
                if i in packed_state:
                    new_state[params[i]] = packed_state[i]
        optimizer.state = new_state
        yield optimizer
    finally:
        for g, snap in zip(optimizer.param_groups, snapshots):
            g.clear()
            g.update(snap)
        optimizer.state = original_state

from .. import _views as _views  # noqa: E402

_views.install(__name__, max_depth=1,
               names=("_stateless", "_utils", "adafactor"))
