"""Distributed checkpoint (DCP): every rank writes its own shards, rank 0 writes the metadata;
loading re-shards to whatever layout the destination ``state_dict`` describes (different world
size included). On-disk layout follows the reference's (tensorplay/distributed/checkpoint/
filesystem.py:56-80): one data file per rank ``__{rank}_0.distcp`` (a ``.mega`` container here)
plus ``.metadata``; ``async_save`` stages to host memory and writes in the background
(state_dict_saver.py:235-346, staging.py)."""
from typing import Protocol, Tuple, runtime_checkable


@runtime_checkable
class CheckpointableTensor(Protocol):
    """A tensor subclass that tells the checkpoint where its local pieces sit in the global tensor (duck-typed:
    anything with these four attributes is saved piece by piece and re-sharded on load)."""
    global_shape: Tuple[int, ...]
    global_offsets: Tuple[Tuple[int, ...], ...]
    local_offsets: Tuple[Tuple[int, ...], ...]
    local_sizes: Tuple[Tuple[int, ...], ...]


from .api import (MegaStorageReader, MegaStorageWriter, ShardedTensor, Stateful, async_save, engine_state_dict, load, load_engine_state_dict, save)
from .hf_storage import (HuggingFaceStorageReader, HuggingFaceStorageWriter, consolidate_to_hf, load_hf, save_hf)
from .planner import DefaultLoadPlanner, DefaultSavePlanner, ReadItem, SavePlan, WriteItem
from .state_dict import (StateDictOptions, get_model_state_dict, get_optimizer_state_dict, get_state_dict,
                         set_model_state_dict, set_optimizer_state_dict, set_state_dict)

__all__ = ["MegaStorageReader", "MegaStorageWriter", "ShardedTensor", "Stateful", "save", "async_save", "load",
           "engine_state_dict", "load_engine_state_dict", "DefaultSavePlanner", "DefaultLoadPlanner", "SavePlan",
           "WriteItem", "ReadItem", "HuggingFaceStorageWriter", "HuggingFaceStorageReader", "save_hf", "load_hf",
           "consolidate_to_hf", "StateDictOptions", "get_model_state_dict", "get_optimizer_state_dict",
           "get_state_dict", "set_model_state_dict", "set_optimizer_state_dict", "set_state_dict"]


def __getattr__(name):
    """Planner, storage, metadata and state-dict helper names that this package does not define resolve to PyTorch's distributed checkpoint (usable through ``save(..., storage_writer=...)`` / ``load(..., storage_reader=...)``)."""
    import importlib
    for mod in ['torch.distributed.checkpoint', 'torch.distributed.checkpoint.state_dict', 'torch.distributed.checkpoint.metadata', 'torch.distributed.checkpoint.planner', 'torch.distributed.checkpoint.optimizer', 'torch.distributed.checkpoint.state_dict_saver', 'torch.distributed.checkpoint.state_dict_loader', 'torch.distributed.checkpoint.filesystem']:
        try:
            return getattr(importlib.import_module(mod), name)
        except (ImportError, AttributeError):
            continue
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
