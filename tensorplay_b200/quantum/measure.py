"""Reading a state: probabilities, expectation values, sampling, read-out error
(the reference's ``tensorplay/quantum/_measurement.py`` surface)."""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Union

import torch
from torch import Tensor

from .gates import apply_gate, h_matrix, n_qubits_of, pauli_matrix, sdg_matrix


def probs(state: Tensor) -> Tensor:
    """``[batch, 2^n]`` probabilities of the computational basis."""
    return (state.real ** 2 + state.imag ** 2).reshape(state.shape[0], -1)


def marginal_probs(state: Tensor, wires: Sequence[int]) -> Tensor:
    n = n_qubits_of(state)
    p = probs(state).reshape([state.shape[0]] + [2] * n)
    drop = [a + 1 for a in range(n) if a not in wires]
    if drop:
        p = p.sum(dim=drop)
    order = sorted(wires)
    perm = [0] + [order.index(w) + 1 for w in wires]
    return p.permute(perm).reshape(state.shape[0], -1)


def apply_pauli_word(state: Tensor, word: str, wires: Optional[Sequence[int]] = None) -> Tensor:
    wires = list(range(len(word))) if wires is None else list(wires)
    for ch, w in zip(word, wires):
        if ch.upper() != "I":
            state = apply_gate(state, pauli_matrix(ch, state.dtype, state.device), w)
    return state


def expectation(state: Tensor, observable: Union[str, Tensor], wires: Optional[Sequence[int]] = None) -> Tensor:
    """``<psi| O |psi>`` per batch entry; ``O`` is a Pauli word or a dense matrix on ``wires``."""
    if isinstance(observable, str):
        phi = apply_pauli_word(state, observable, wires)
    else:
        wires = list(range(n_qubits_of(state))) if wires is None else list(wires)
        phi = apply_gate(state, observable, wires)
    b = state.shape[0]
    return (state.conj().reshape(b, -1) * phi.reshape(b, -1)).sum(-1).real


def joint_expectation(state: Tensor, words: Sequence[str]) -> Tensor:
    return torch.stack([expectation(state, w) for w in words], -1)


def apply_measurement_basis(state: Tensor, word: str, wires: Optional[Sequence[int]] = None) -> Tensor:
    """Rotate so that measuring Z on every wire measures the Pauli word."""
    wires = list(range(len(word))) if wires is None else list(wires)
    for ch, w in zip(word.upper(), wires):
        if ch == "X":
            state = apply_gate(state, h_matrix(state.dtype, state.device), w)
        elif ch == "Y":
            state = apply_gate(state, sdg_matrix(state.dtype, state.device), w)
            state = apply_gate(state, h_matrix(state.dtype, state.device), w)
    return state


def sample_indices(state: Tensor, shots: int, generator=None) -> Tensor:
    """``[batch, shots]`` basis indices drawn from the state's distribution, on its device."""
    return torch.multinomial(probs(state).float(), shots, replacement=True, generator=generator)


def gen_bitstrings(n: int, device=None) -> Tensor:
    idx = torch.arange(2 ** n, device=device)
    return ((idx[:, None] >> torch.arange(n - 1, -1, -1, device=device)) & 1).to(torch.int64)


def measure(state: Tensor, shots: int = 1, generator=None) -> Tensor:
    """``[batch, shots, n]`` measured bits (qubit 0 first)."""
    n = n_qubits_of(state)
    idx = sample_indices(state, shots, generator)
    return (idx[..., None] >> torch.arange(n - 1, -1, -1, device=idx.device)) & 1


def counts_from_indices(idx: Tensor, n: int) -> List[Dict[str, int]]:
    out = []
    for row in idx.cpu().tolist():
        c: Dict[str, int] = {}
        for v in row:
            k = format(v, f"0{n}b")
            c[k] = c.get(k, 0) + 1
        out.append(c)
    return out


def expectation_from_counts(counts: Dict[str, int], word: Optional[str] = None) -> float:
    """Mean of the +-1 parity of the measured bits (restricted to the non-identity letters)."""
    tot = sum(counts.values())
    acc = 0
    for bits, c in counts.items():
        par = sum(int(b) for i, b in enumerate(bits) if word is None or word[i].upper() != "I")
        acc += c * (1 - 2 * (par & 1))
    return acc / max(1, tot)


def readout_error_matrix(p01: float, p10: float, dtype=torch.float32, device=None) -> Tensor:
    """Column-stochastic ``[[P(0|0), P(0|1)], [P(1|0), P(1|1)]]``."""
    return torch.tensor([[1 - p10, p01], [p10, 1 - p01]], dtype=dtype, device=device)


def apply_readout_error(p: Tensor, matrix: Tensor, n: int) -> Tensor:
    """Mix a ``[batch, 2^n]`` distribution with the same single-qubit confusion matrix on every qubit."""
    q = p.reshape([p.shape[0]] + [2] * n)
    for a in range(1, n + 1):
        q = torch.movedim(torch.tensordot(q, matrix.to(q.dtype), dims=([a], [1])), -1, a)
    return q.reshape(p.shape[0], -1)


def density_probs(rho: Tensor) -> Tensor:
    return torch.diagonal(rho, dim1=-2, dim2=-1).real


def expectation_from_density(rho: Tensor, observable: Tensor) -> Tensor:
    return torch.einsum("bij,ji->b", rho, observable.to(rho.dtype)).real


def commuting_groups(words: Sequence[str]) -> List[List[str]]:
    """Greedy grouping of Pauli words that commute qubit-wise (one measurement basis per group)."""
    def ok(a, b):
        return all(x == "I" or y == "I" or x == y for x, y in zip(a.upper(), b.upper()))
    groups: List[List[str]] = []
    for w in words:
        for g in groups:
            if all(ok(w, v) for v in g):
                g.append(w)
                break
        else:
            groups.append([w])
    return groups


# the reference has a package at this path: deeper module names resolve to views of the pack
__path__: list = []
