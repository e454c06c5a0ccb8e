"""Selective activation checkpointing: keep the outputs of the expensive ops (GEMMs, attention)
of a checkpointed region and recompute only the cheap ones (norms, RoPE, SwiGLU, residual adds).

The checkpointing driver runs the region once under :func:`record` (no autograd graph): the
participating ops append their outputs to the record. In backward it runs the region again under
:func:`replay`: the same ops, in the same order, take their stored output instead of computing
it, while still building the autograd graph whose backward needs only their inputs.
Capability reference: selective policies of tensorplay/utils/checkpoint.py:210-547.
"""
from __future__ import annotations

import contextlib
import threading
from typing import List, Optional, Tuple

_tls = threading.local()


@contextlib.contextmanager
def record():
    """Collect the outputs stashed by participating ops; yields the list."""
    prev, rec = getattr(_tls, "rec", None), []
    _tls.rec = rec
    try:
        yield rec
    finally:
        _tls.rec = prev


@contextlib.contextmanager
def replay(saved: List[Tuple]):
    """Hand the recorded outputs back, in order, to the same sequence of ops."""
    prev = getattr(_tls, "rep", None)
    state = {"items": saved, "next": 0}
    _tls.rep = state
    try:
        yield
        if state["next"] != len(saved):
            raise RuntimeError(f"selective checkpoint replay consumed {state['next']} of {len(saved)} saved outputs: "
                               "the recomputation did not run the same ops as the forward pass")
    finally:
        _tls.rep = prev


def active() -> bool:
    return getattr(_tls, "rec", None) is not None or getattr(_tls, "rep", None) is not None


def stash(*tensors) -> None:
    rec = getattr(_tls, "rec", None)
    if rec is not None:
        rec.append(tensors)


def take() -> Optional[Tuple]:
    rep = getattr(_tls, "rep", None)
    if rep is None:
        return None
    if rep["next"] >= len(rep["items"]):
        raise RuntimeError("selective checkpoint replay ran more ops than the forward pass recorded")
    item = rep["items"][rep["next"]]
    rep["next"] += 1
    return item


@contextlib.contextmanager
def recompute():
    """Marks the forward that a checkpointing driver runs again in backward only to rebuild the autograd
    graph: the VALUE of the region's result is discarded (backward starts from the incoming gradient), so an
    op that produces that result as its last step may skip the step (see :func:`recomputing`)."""
    prev = getattr(_tls, "recompute", False)
    _tls.recompute = True
    try:
        yield
    finally:
        _tls.recompute = prev


def recomputing() -> bool:
    return bool(getattr(_tls, "recompute", False))
