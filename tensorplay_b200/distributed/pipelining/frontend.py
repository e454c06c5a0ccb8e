"""Graph-splitting front end: ``pipeline(module, mb_args, split_spec=...)`` cuts a model into stage
modules and ``Pipe.build_stage`` wraps one of them in this package's :class:`PipelineStage`.

The reference exports the model and splits the exported graph (tensorplay/distributed/pipelining/
_IR.py:447-756: ``pipe_split`` :447, ``SplitPoint`` :484, ``Pipe`` :514, ``pipeline`` :700-756). Here the
model is traced with ``torch.fx`` at the granularity the split needs and no finer: only the containers
that lie on the path to a split point are traced, every other sub-module (each transformer block, the
embedding, the head) stays an opaque call, so blocks whose ``forward`` branches on tensor properties or
calls custom autograd functions never meet the tracer. Stage boundaries carry one tensor (what
:class:`PipelineStage` sends); a cut that would need several tensors to cross is refused with the names
of the values.
"""
from __future__ import annotations

from enum import Enum
from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.fx as fx
from torch import nn
from torch.fx.passes.split_module import split_module

from .stage import PipelineStage


class SplitPoint(Enum):
    BEGINNING = 1
    END = 2


_active_tracer: List[Optional[fx.Tracer]] = [None]


def pipe_split() -> None:
    """Marker: a call of ``pipe_split()`` in a traced ``forward`` starts the next stage there. Outside of
    :func:`pipeline` it does nothing."""
    tr = _active_tracer[0]
    if tr is not None:
        # a call without tensor arguments leaves no trace by itself: record the node explicitly
        tr.create_proxy("call_function", pipe_split, (), {})
    return None


class _CoarseTracer(fx.Tracer):
    """Traces only the ancestors of split points (and the root); everything else is a leaf."""

    def __init__(self, open_modules: set):
        super().__init__()
        self.open_modules = open_modules

    def is_leaf_module(self, m: nn.Module, qualname: str) -> bool:
        return qualname not in self.open_modules


def _ancestors(name: str) -> List[str]:
    parts = name.split(".")
    return [".".join(parts[:i]) for i in range(1, len(parts))]


class Pipe(nn.Module):
    """The split model: ``submod_0 .. submod_{n-1}`` chained. Calling it runs every stage locally."""

    def __init__(self, split_gm: fx.GraphModule, stages: List[nn.Module], examples: Optional[List[tuple]] = None):
        super().__init__()
        self.split_gm = split_gm
        self.stages = nn.ModuleList(stages)
        self.num_stages = len(stages)
        self._examples = examples  # per stage: (input example, output example) or None

    def forward(self, *args, **kwargs):
        return self.split_gm(*args, **kwargs)

    def get_stage_module(self, stage_index: int) -> nn.Module:
        if not 0 <= stage_index < self.num_stages:
            raise IndexError(f"stage {stage_index} of {self.num_stages}")
        return self.stages[stage_index]

    def info(self) -> Dict[str, object]:
        return {"num_stages": self.num_stages,
                "parameters_per_stage": [sum(p.numel() for p in s.parameters()) for s in self.stages]}

    def build_stage(self, stage_index: int, device=None, group=None) -> PipelineStage:
        """This package's runtime stage for ``stage_index`` (moved to ``device`` if given). When example
        micro-batch inputs were passed to :func:`pipeline`, the stage knows its activation shapes and the
        first step needs no shape hand-shake."""
        mod = self.get_stage_module(stage_index)
        if device is not None:
            mod = mod.to(device)
        if device is None:
            p = next(mod.parameters(), None)
            device = p.device if p is not None else torch.device("cpu")
        ex_in = ex_out = None
        if self._examples is not None:
            ex_in, ex_out = self._examples[stage_index]
            if stage_index == 0:
                ex_in = None   # the first stage receives its input from the caller, not from a peer
        return PipelineStage(mod, stage_index, self.num_stages, device=device, group=group,
                             input_args=ex_in, output_args=ex_out)


def build_stage(pipe: Pipe, stage_index: int, device=None, group=None) -> PipelineStage:
    return pipe.build_stage(stage_index, device=device, group=group)


def _assign_stages(gm: fx.GraphModule, split_spec: Dict[str, SplitPoint]) -> Dict[fx.Node, int]:
    part = 0
    out: Dict[fx.Node, int] = {}
    seen = set()
    for node in gm.graph.nodes:
        if node.op == "call_function" and node.target is pipe_split:
            part += 1
            out[node] = part
            continue
        bump_after = False
        if node.op == "call_module" and node.target in split_spec:
            seen.add(node.target)
            if split_spec[node.target] == SplitPoint.BEGINNING:
                part += 1
            else:
                bump_after = True
        out[node] = part
        if bump_after:
            part += 1
    missing = set(split_spec) - seen
    if missing:
        raise ValueError(f"pipeline: split points {sorted(missing)} are not called in the traced forward")
    return out


def _check_single_tensor_boundaries(split_gm: fx.GraphModule, n: int) -> None:
    """Stage i+1 must take exactly the output of stage i (one value), stage 0 the model inputs."""
    calls = [nd for nd in split_gm.graph.nodes if nd.op == "call_module"]
    if len(calls) != n:
        raise RuntimeError(f"pipeline: expected {n} stage calls in the split graph, found {len(calls)}")
    for i, nd in enumerate(calls):
        if i == 0:
            continue
        srcs = list(nd.all_input_nodes)
        prev = calls[i - 1]
        bad = [s for s in srcs if s is not prev and not (s.op == "call_function" and prev in s.all_input_nodes)]
        if len(srcs) != 1 or bad:
            names = [s.name for s in srcs]
            raise NotImplementedError(
                f"pipeline: stage {i} needs {names} from earlier stages; a stage boundary here carries one tensor "
                "(the previous stage's output). Move the split point, or fold the extra values into the stage.")


def pipeline(module: nn.Module, mb_args: Sequence = (), mb_kwargs: Optional[dict] = None,
             split_spec: Optional[Dict[str, SplitPoint]] = None,
             split_policy: Optional[Callable[[fx.GraphModule], fx.GraphModule]] = None) -> Pipe:
    """Split ``module`` into pipeline stages.

    ``split_spec`` maps sub-module names (``"layers.4"``) to :class:`SplitPoint`: ``BEGINNING`` starts a new
    stage before that sub-module's call, ``END`` after it. ``pipe_split()`` calls inside the traced part of
    the model cut as well. ``split_policy`` may rewrite the traced graph (insert ``pipe_split`` calls) before
    it is cut. ``mb_args`` / ``mb_kwargs`` are example inputs of ONE micro-batch: when given, the stages run
    once on them so that each stage records the shape of what it receives and sends.
    """
    split_spec = dict(split_spec or {})
    for name in split_spec:
        try:
            module.get_submodule(name)
        except AttributeError as e:
            raise ValueError(f"pipeline: no sub-module named {name!r}") from e
    open_modules = {""}
    for name in split_spec:
        open_modules.update(_ancestors(name))
    tracer = _CoarseTracer(open_modules)
    _active_tracer[0] = tracer
    try:
        graph = tracer.trace(module)
    finally:
        _active_tracer[0] = None
    gm = fx.GraphModule(module, graph)
    if split_policy is not None:
        gm = split_policy(gm)
    part_of = _assign_stages(gm, split_spec)
    n = max(part_of.values()) + 1 if part_of else 1
    # the markers themselves carry no computation
    for node in list(gm.graph.nodes):
        if node.op == "call_function" and node.target is pipe_split:
            part_of.pop(node, None)
            gm.graph.erase_node(node)
    gm.recompile()
    split_gm = split_module(gm, module, lambda node: part_of.get(node, 0), keep_original_order=True)
    stages = [getattr(split_gm, f"submod_{i}") for i in range(n) if hasattr(split_gm, f"submod_{i}")]
    if len(stages) != n:
        raise RuntimeError("pipeline: a stage came out empty (two split points with nothing between them)")
    _check_single_tensor_boundaries(split_gm, n)
    examples = None
    if len(mb_args) or mb_kwargs:
        examples = []
        with torch.no_grad():
            x = stages[0](*mb_args, **(mb_kwargs or {}))
            first_in = mb_args[0] if len(mb_args) else next(iter(mb_kwargs.values()))
            examples.append((first_in, x))
            for s in stages[1:]:
                y = s(x)
                examples.append((x, y))
                x = y
        for i, (a, b) in enumerate(examples):
            if not isinstance(b, torch.Tensor):
                raise NotImplementedError(f"pipeline: stage {i} returns {type(b).__name__}; stages pass one tensor")
    return Pipe(split_gm, stages, examples)
