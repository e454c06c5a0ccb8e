"""Tensor comparison helpers (tensorplay/utils/comparison.py)."""
import torch


def allclose(input, other, rtol: float = 1e-05, atol: float = 1e-08, equal_nan: bool = False) -> bool:
    """``|input - other| <= atol + rtol * |other|`` everywhere; ``other`` moves to ``input``'s device."""
    if input.device != other.device:
        other = other.to(input.device)
    return bool(torch.allclose(input, other.to(input.dtype), rtol=rtol, atol=atol, equal_nan=equal_nan))
