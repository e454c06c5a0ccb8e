"""``nn.parallel``: ``DistributedDataParallel`` (own bucketed reducer, one process per GPU) and ``DataParallel`` (one
process over several devices, ``data_parallel.py``)."""
from .data_parallel import DataParallel, data_parallel, gather, scatter  # noqa: F401


def __getattr__(name):
    if name == "DistributedDataParallel":
        from ...distributed.ddp import DistributedDataParallel
        return DistributedDataParallel
    import torch.nn.parallel as _p
    return getattr(_p, name)
