"""Stateless spellings of the metrics: ``functional.mean_squared_error(preds, target)`` builds the
class of that name (``MeanSquaredError``), feeds it the one batch and returns its value. The ranking
and correlation functions written as functions in the first place are re-exported as they are.
Keyword arguments that ``update`` of the class accepts go to ``update``, the rest to the constructor."""
from __future__ import annotations

import inspect
import sys

from . import ranking as _ranking
from .ranking import *  # noqa: F401,F403

_SPECIAL = {"peak_signal_noise_ratio": "PeakSignalNoiseRatio", "bleu_score": "BLEUScore", "rouge_score": "ROUGEScore",
            "chrf_score": "CHRFScore", "sacre_bleu_score": "SacreBLEUScore", "bert_score": "BERTScore", "clip_score": "CLIPScore",
            "squad": "SQuAD", "retrieval_average_precision": "RetrievalMAP", "retrieval_reciprocal_rank": "RetrievalMRR",
            "retrieval_normalized_dcg": "RetrievalNormalizedDCG", "word_error_rate": "WordErrorRate",
            "char_error_rate": "CharErrorRate", "match_error_rate": "MatchErrorRate", "perplexity": "Perplexity", "word_information_lost": "WordInfoLost",
            "word_information_preserved": "WordInfoPreserved"}


def _class_for(name: str):
    pkg = sys.modules[__package__]
    if name in _SPECIAL and hasattr(pkg, _SPECIAL[name]):
        return getattr(pkg, _SPECIAL[name])
    key = name.replace("_", "").lower()
    for cand in dir(pkg):
        if cand.lower() == key and (inspect.isclass(getattr(pkg, cand)) or callable(getattr(pkg, cand))) and cand[0].isupper():
            return getattr(pkg, cand)
    return None


def _make(name: str, cls):
    def fn(*args, **kwargs):
        probe = cls if inspect.isclass(cls) else None
        upd = set()
        if probe is not None:
            upd = {p for p in inspect.signature(probe.update).parameters if p != "self"}
        to_update = {k: kwargs.pop(k) for k in list(kwargs) if k in upd}
        metric = cls(**kwargs)
        metric.update(*args, **to_update)
        return metric.compute()
    fn.__name__ = fn.__qualname__ = name
    fn.__doc__ = f"One-batch value of :class:`{getattr(cls, '__name__', name)}`."
    return fn


def __getattr__(name: str):
    if name.startswith("__"):
        raise AttributeError(name)
    pkg = sys.modules[__package__]
    if name in pkg.__dict__ and not name[0].isupper() and callable(pkg.__dict__[name]):
        return pkg.__dict__[name]                      # already a function (matrices, pit_permutate, ssim, ...)
    cls = _class_for(name)
    if cls is None:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    fn = _make(name, cls)
    globals()[name] = fn
    return fn


def __dir__():
    return sorted(set(globals()) | set(dir(_ranking)))


# the reference has a package at this path: deeper module names resolve to views of the pack
__path__: list = []
