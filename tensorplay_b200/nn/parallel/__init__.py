"""``nn.parallel``: DistributedDataParallel (own bucketed reducer) and DataParallel."""
from torch.nn.parallel import DataParallel  # noqa: F401


def __getattr__(name):
    if name == "DistributedDataParallel":
        from ...distributed.ddp import DistributedDataParallel
        return DistributedDataParallel
    raise AttributeError(name)
