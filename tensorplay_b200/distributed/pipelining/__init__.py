"""Pipeline parallelism: stages, micro-batching and schedules over point-to-point send/recv (NCCL
on GPUs, gloo on CPU ranks) with batched non-blocking p2p.

``schedules.py``: GPipe, 1F1B (one stage per rank) and the breadth-first looped schedule;
``runtime.py``: the action-table runtime with depth-first interleaved 1F1B, interleaved zero bubble
(split input / weight backward), the V-shaped zero-bubble placements and CSV-driven schedules.
API after tensorplay/distributed/pipelining (``PipelineStage`` stage.py:1039-1558, schedules.py:
``ScheduleGPipe`` :658, ``Schedule1F1B`` :766-946, ``_PipelineScheduleRuntime`` :1277,
``ScheduleInterleaved1F1B`` :1636, ``ScheduleInterleavedZeroBubble`` :1723, ``ScheduleZBVZeroBubble``
:1886, ``ScheduleDualPipeV`` :2057; ``_backward.py``; microbatch.py); ``frontend.py``: ``pipeline`` / ``Pipe`` /
``SplitPoint`` / ``pipe_split`` (_IR.py:447-756), cutting an fx trace of the model's containers."""
from .frontend import Pipe, SplitPoint, build_stage, pipe_split, pipeline
from .microbatch import merge_chunks, split_args_kwargs_into_chunks
from .runtime import (Action, PipelineScheduleRuntime, ScheduleDualPipeV, ScheduleFromCSV, ScheduleInterleaved1F1B,
                      ScheduleInterleavedZeroBubble, ScheduleZBVZeroBubble, greedy_zero_bubble_order,
                      interleaved_1f1b_order, loop_placement, simulate, v_placement)
from .schedules import PipelineScheduleMulti, PipelineScheduleSingle, Schedule1F1B, ScheduleGPipe, ScheduleLoopedBFS
from .stage import PipelineStage

_PipelineScheduleRuntime = PipelineScheduleRuntime

__all__ = ["PipelineStage", "ScheduleGPipe", "Schedule1F1B", "ScheduleInterleaved1F1B", "ScheduleLoopedBFS",
           "ScheduleInterleavedZeroBubble", "ScheduleZBVZeroBubble", "ScheduleDualPipeV", "ScheduleFromCSV",
           "PipelineScheduleRuntime", "PipelineScheduleSingle", "PipelineScheduleMulti", "Action", "simulate",
           "interleaved_1f1b_order", "greedy_zero_bubble_order", "loop_placement", "v_placement",
           "split_args_kwargs_into_chunks", "merge_chunks", "pipeline", "Pipe", "SplitPoint", "pipe_split",
           "build_stage"]


def __getattr__(name):
    """Names without a definition here resolve to PyTorch's pipelining package."""
    import importlib
    for mod in ['torch.distributed.pipelining', 'torch.distributed.pipelining.schedules']:
        try:
            return getattr(importlib.import_module(mod), name)
        except (ImportError, AttributeError):
            continue
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
