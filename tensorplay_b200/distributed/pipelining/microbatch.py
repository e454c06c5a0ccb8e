"""Micro-batch splitting / merging along the batch dimension."""
from __future__ import annotations

from typing import Any, List, Sequence, Tuple

import torch


def _split(x: Any, n: int, dim: int = 0) -> List[Any]:
    if isinstance(x, torch.Tensor):
        if x.shape[dim] % n:
            raise ValueError(f"batch dimension {x.shape[dim]} is not divisible into {n} micro-batches")
        return list(torch.chunk(x, n, dim=dim))
    return [x] * n


def split_args_kwargs_into_chunks(args: Sequence[Any], kwargs: dict, chunks: int) -> Tuple[List[tuple], List[dict]]:
    a = [_split(v, chunks) for v in args]
    k = {key: _split(v, chunks) for key, v in (kwargs or {}).items()}
    return ([tuple(col[i] for col in a) for i in range(chunks)],
            [{key: col[i] for key, col in k.items()} for i in range(chunks)])


def merge_chunks(chunks: Sequence[Any], dim: int = 0) -> Any:
    if not chunks:
        return None
    if isinstance(chunks[0], torch.Tensor):
        if chunks[0].dim() == 0:
            return torch.stack(list(chunks))
        return torch.cat(list(chunks), dim=dim)
    if isinstance(chunks[0], (tuple, list)):
        return type(chunks[0])(merge_chunks([c[i] for c in chunks], dim) for i in range(len(chunks[0])))
    return list(chunks)
