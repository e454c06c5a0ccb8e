"""State construction and conversion helpers (the reference's ``tensorplay/quantum/_state.py``):
basis / product / random states, normalisation and inner products, density matrices, partial trace,
fidelity, Bloch-vector conversions."""
from __future__ import annotations

import math
from typing import Dict, Sequence, Union

import torch
from torch import Tensor

from .gates import _cdtype, n_qubits_of, pauli_matrix, zero_state


def zeros_state(n_qubits: int, batch: int = 1, dtype=torch.complex64, device=None) -> Tensor:
    return zero_state(n_qubits, batch, dtype, device)


def flatten(state: Tensor) -> Tensor:
    """``[batch, 2, ..., 2]`` -> ``[batch, 2^n]``."""
    return state.reshape(state.shape[0], -1)


def unflatten(vec: Tensor) -> Tensor:
    n = int(round(math.log2(vec.shape[-1])))
    return vec.reshape([vec.shape[0]] + [2] * n)


def basis_state(bits: Union[str, Sequence[int], int], n_qubits: int = None, batch: int = 1, dtype=torch.complex64,
                device=None) -> Tensor:
    """Computational basis state from a bit string (qubit 0 first), a bit list or an index."""
    if isinstance(bits, int):
        idx, n = bits, n_qubits
    else:
        b = [int(c) for c in bits]
        n = len(b)
        idx = int("".join(str(c) for c in b), 2)
    s = torch.zeros(batch, 2 ** n, dtype=_cdtype(dtype), device=device)
    s[:, idx] = 1
    return unflatten(s)


def state_from_bases(indices: Sequence[int], amplitudes: Sequence[complex], n_qubits: int, dtype=torch.complex64,
                     device=None) -> Tensor:
    s = torch.zeros(1, 2 ** n_qubits, dtype=_cdtype(dtype), device=device)
    for i, a in zip(indices, amplitudes):
        s[0, i] = a
    return unflatten(normalize(s))


def plus_state(n_qubits: int, batch: int = 1, dtype=torch.complex64, device=None) -> Tensor:
    s = torch.full((batch, 2 ** n_qubits), 2.0 ** (-n_qubits / 2), dtype=_cdtype(dtype), device=device)
    return unflatten(s)


def product_state(qubits: Sequence[Tensor]) -> Tensor:
    """Tensor product of single-qubit states ``[2]`` (qubit 0 first): ``[1, 2, ..., 2]``."""
    s = torch.ones(1, dtype=qubits[0].dtype, device=qubits[0].device)
    for q in qubits:
        s = torch.kron(s, q.reshape(2))
    return unflatten(s[None])


def random_state(n_qubits: int, batch: int = 1, dtype=torch.complex64, device=None, generator=None) -> Tensor:
    """Haar-random pure states (normalised complex Gaussians)."""
    re = torch.randn(batch, 2 ** n_qubits, 2, dtype=torch.float64, generator=generator)
    return unflatten(normalize(torch.view_as_complex(re)).to(_cdtype(dtype)).to(device))


def encode_state(x: Tensor, dtype=torch.complex64) -> Tensor:
    """Amplitude encoding of real rows ``[batch, 2^n]`` (zero-padded to a power of two, normalised)."""
    d = 1 << max(0, (x.shape[-1] - 1).bit_length())
    v = torch.zeros(x.shape[0], d, dtype=_cdtype(dtype), device=x.device)
    v[:, : x.shape[-1]] = x.to(v.dtype)
    return unflatten(normalize(v))


def norm(state: Tensor) -> Tensor:
    return flatten(state).norm(dim=-1)


def normalize(state: Tensor) -> Tensor:
    flat = state.reshape(state.shape[0], -1)
    return (flat / flat.norm(dim=-1, keepdim=True).clamp(min=1e-30)).reshape(state.shape)


def inner(a: Tensor, b: Tensor) -> Tensor:
    """``<a|b>`` per batch entry."""
    return (flatten(a).conj() * flatten(b)).sum(-1)


def global_phase(state: Tensor) -> Tensor:
    """Phase of the largest amplitude per batch entry (dividing it out fixes the gauge)."""
    flat = flatten(state)
    big = flat.gather(1, flat.abs().argmax(dim=1, keepdim=True))[:, 0]
    return torch.angle(big)


def to_density(state: Tensor) -> Tensor:
    v = flatten(state)
    return v[:, :, None] * v.conj()[:, None, :]


def density_mixture(states: Sequence[Tensor], probs: Sequence[float]) -> Tensor:
    return sum(p * to_density(s) for s, p in zip(states, probs))


def density_to_state(rho: Tensor) -> Tensor:
    """Dominant eigenvector of each density matrix (exact for pure states, up to a phase)."""
    vals, vecs = torch.linalg.eigh(rho)
    return unflatten(vecs[..., -1])


def partial_trace(rho: Tensor, keep: Sequence[int], n_qubits: int) -> Tensor:
    """Reduced density matrix of the qubits ``keep`` (in the given order)."""
    b = rho.shape[0]
    t = rho.reshape([b] + [2] * (2 * n_qubits))
    keep = list(keep)
    drop = [q for q in range(n_qubits) if q not in keep]
    for q in sorted(drop, reverse=True):                       # trace one qubit at a time
        n_now = (t.dim() - 1) // 2
        t = torch.diagonal(t, dim1=1 + q, dim2=1 + n_now + q).sum(-1)
    left = sorted(keep)
    perm = [left.index(q) for q in keep]
    k = len(keep)
    t = t.permute([0] + [1 + p for p in perm] + [1 + k + p for p in perm])
    return t.reshape(b, 2 ** k, 2 ** k)


def fidelity(a: Tensor, b: Tensor) -> Tensor:
    """``|<a|b>|^2`` for two pure states, ``<a|rho|a>`` for a pure state and a density matrix, and the
    Uhlmann fidelity for two density matrices."""
    a_is_rho = a.dim() == 3 and a.shape[-1] == a.shape[-2] and not _is_state(a)
    b_is_rho = b.dim() == 3 and b.shape[-1] == b.shape[-2] and not _is_state(b)
    if not a_is_rho and not b_is_rho:
        return inner(a, b).abs() ** 2
    if a_is_rho and not b_is_rho:
        a, b, a_is_rho, b_is_rho = b, a, False, True
    if not a_is_rho:
        v = flatten(a)
        return torch.einsum("bi,bij,bj->b", v.conj(), b, v).real
    vals, vecs = torch.linalg.eigh(a)
    sq = (vecs * vals.clamp(min=0).sqrt()[:, None, :]) @ vecs.conj().transpose(-1, -2)
    ev = torch.linalg.eigvalsh(sq @ b @ sq).clamp(min=0)
    return ev.sqrt().sum(-1) ** 2


def _is_state(t: Tensor) -> bool:
    # a [batch, 2, 2] tensor is ambiguous (two qubits as a state, or one-qubit density matrices):
    # it is a state exactly when its squared norm is 1 and its trace is not
    if t.dim() != 3 or t.shape[1:] != (2, 2):
        return t.dim() != 3
    tr = torch.diagonal(t, dim1=-2, dim2=-1).sum(-1)
    return not bool(torch.allclose(tr.real, torch.ones_like(tr.real), atol=1e-5) and torch.allclose(t, t.conj().transpose(-1, -2), atol=1e-5))


def sv2bloch(state: Tensor) -> Tensor:
    """Bloch vector ``[batch, 3]`` of single-qubit states ``[batch, 2]``."""
    return dens2bloch(to_density(state))


def dens2bloch(rho: Tensor) -> Tensor:
    return torch.stack([torch.einsum("bij,ji->b", rho, pauli_matrix(p, rho.dtype, rho.device)).real for p in "XYZ"], -1)


def bloch2dens(r: Tensor, dtype=torch.complex64) -> Tensor:
    eye = torch.eye(2, dtype=_cdtype(dtype), device=r.device)
    out = eye.expand(r.shape[0], 2, 2).clone()
    for i, p in enumerate("XYZ"):
        out = out + r[:, i, None, None].to(out.dtype) * pauli_matrix(p, dtype, r.device)
    return out / 2


def bloch2sv(r: Tensor, dtype=torch.complex64) -> Tensor:
    """Pure state ``[batch, 2]`` of a unit Bloch vector: ``cos(theta/2)|0> + e^{i phi} sin(theta/2)|1>``."""
    theta = torch.acos(r[:, 2].clamp(-1, 1))
    phi = torch.atan2(r[:, 1], r[:, 0])
    cd = _cdtype(dtype)
    return torch.stack((torch.cos(theta / 2).to(cd), torch.polar(torch.sin(theta / 2), phi).to(cd)), -1)


def state_from_counts(counts: Dict[str, int], dtype=torch.complex64) -> Tensor:
    """State with amplitudes ``sqrt(frequency)`` (phases are not observable in counts)."""
    n = len(next(iter(counts)))
    tot = sum(counts.values())
    s = torch.zeros(1, 2 ** n, dtype=_cdtype(dtype))
    for bits, c in counts.items():
        s[0, int(bits, 2)] = math.sqrt(c / tot)
    return unflatten(s)


def density_from_counts(counts: Dict[str, int], dtype=torch.complex64) -> Tensor:
    """Diagonal density matrix of the measured distribution."""
    n = len(next(iter(counts)))
    tot = sum(counts.values())
    d = torch.zeros(2 ** n, dtype=_cdtype(dtype))
    for bits, c in counts.items():
        d[int(bits, 2)] = c / tot
    return torch.diag(d)[None]


# the reference has a package at this path: deeper module names resolve to views of the pack
__path__: list = []
