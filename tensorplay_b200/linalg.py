"""``linalg``: PyTorch's package plus the three functions the reference adds to it (tensorplay/linalg/__init__.py:
``vdot``, ``polar``, ``matrix_sqrth``)."""
import torch as _torch
from torch.linalg import *  # noqa: F401,F403


def vdot(x, y, *, out=None):
    """Conjugating dot product of two 1-D tensors."""
    return _torch.vdot(x, y, out=out)


def polar(A, side: str = "right"):
    """Polar decomposition from the SVD ``A = W S Vh``: ``A = U P`` (``side="right"``, ``P = V S Vh``) or ``A = P U``
    (``side="left"``, ``P = W S Wh``), ``U = W Vh`` with orthonormal columns (or rows), ``P`` Hermitian positive
    semi-definite."""
    if side not in ("right", "left"):
        raise ValueError("side must be 'right' or 'left'")
    W, S, Vh = _torch.linalg.svd(A, full_matrices=False)
    U = W @ Vh
    if side == "right":
        P = (Vh.mH * S.unsqueeze(-2)) @ Vh
    else:
        P = (W * S.unsqueeze(-2)) @ W.mH
    return U, P


def matrix_sqrth(A, UPLO: str = "L"):
    """Principal square root of a Hermitian positive semi-definite matrix through its eigendecomposition (eigenvalues
    that round-off made slightly negative count as zero)."""
    w, V = _torch.linalg.eigh(A, UPLO=UPLO)
    return (V * w.clamp_min(0).sqrt().unsqueeze(-2)) @ V.mH


def __getattr__(name):
    return getattr(_torch.linalg, name)
