"""Pipeline parallelism: stages, micro-batching and the GPipe / 1F1B / interleaved-1F1B schedules
over point-to-point send/recv (NCCL on GPUs, gloo on CPU ranks), overlapped with compute by
batched non-blocking p2p. API after tensorplay/distributed/pipelining (``PipelineStage``
stage.py:1039-1558, schedules.py: ``ScheduleGPipe`` :658, ``Schedule1F1B`` :766-946,
``ScheduleInterleaved1F1B`` :1636; microbatch.py)."""
from .microbatch import merge_chunks, split_args_kwargs_into_chunks
from .schedules import (PipelineScheduleMulti, PipelineScheduleSingle, Schedule1F1B, ScheduleGPipe,
                        ScheduleInterleaved1F1B, ScheduleLoopedBFS)
from .stage import PipelineStage

__all__ = ["PipelineStage", "ScheduleGPipe", "Schedule1F1B", "ScheduleInterleaved1F1B", "ScheduleLoopedBFS",
           "PipelineScheduleSingle", "PipelineScheduleMulti", "split_args_kwargs_into_chunks", "merge_chunks"]


def __getattr__(name):
    """The tracing front-end (``pipeline``, ``Pipe``, ``SplitPoint``, ``pipe_split``, ``build_stage``) and the zero-bubble schedule classes resolve to PyTorch's; they work with PyTorch's stage objects, the schedules defined here with :class:`PipelineStage`."""
    import importlib
    for mod in ['torch.distributed.pipelining', 'torch.distributed.pipelining.schedules']:
        try:
            return getattr(importlib.import_module(mod), name)
        except (ImportError, AttributeError):
            continue
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
