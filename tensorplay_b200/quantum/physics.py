"""Hamiltonians, time evolution, noise channels on density matrices and parameter-shift gradients
(the reference's ``_hamiltonian.py``, ``_dynamics.py``, ``_noise.py`` and ``_gradients.py``)."""
from __future__ import annotations

import math
from typing import Callable, List, Optional, Sequence, Tuple

import torch
from torch import Tensor

from . import gates as G
from .measure import expectation


class Hamiltonian:
    """Real linear combination of Pauli words, ``H = sum_k c_k P_k``."""

    def __init__(self, terms: Sequence[Tuple[float, str]]):
        self.terms = [(float(c), w.upper()) for c, w in terms]
        self.n_qubits = len(self.terms[0][1]) if self.terms else 0

    def matrix(self, dtype=torch.complex64, device=None) -> Tensor:
        return sum(c * G.pauli_string_matrix(w, dtype, device) for c, w in self.terms)

    def expectation(self, state: Tensor) -> Tensor:
        return sum(c * expectation(state, w) for c, w in self.terms)

    def evolve(self, state: Tensor, t: float, steps: int = 1, order: int = 1) -> Tensor:
        return trotter_evolve(state, self, t, steps, order)


def energy(state: Tensor, h: Hamiltonian) -> Tensor:
    return h.expectation(state)


def energy_from_density(rho: Tensor, h: Hamiltonian) -> Tensor:
    return torch.einsum("bij,ji->b", rho, h.matrix(rho.dtype, rho.device)).real


def trotter_evolve(state: Tensor, h: Hamiltonian, t: float, steps: int = 1, order: int = 1) -> Tensor:
    """``exp(-i H t)`` by a first- or second-order product formula; every factor is an exact Pauli
    rotation."""
    dt = t / steps
    wires = list(range(h.n_qubits))
    seq = h.terms if order == 1 else [(c / 2, w) for c, w in h.terms] + [(c / 2, w) for c, w in reversed(h.terms)]
    for _ in range(steps):
        for c, w in seq:
            if set(w) == {"I"}:
                state = G.apply_global_phase(state, -c * dt)
            else:
                state = G.apply_pauli_rotation(state, 2 * c * dt, w, wires)
    return state


def matrix_exp_evolve(state: Tensor, h: Hamiltonian, t: float) -> Tensor:
    u = torch.linalg.matrix_exp(-1j * t * h.matrix(torch.complex128, state.device)).to(state.dtype)
    return G.apply_gate(state, u, list(range(h.n_qubits)))


def sesolve(h: Hamiltonian, state: Tensor, times: Sequence[float]) -> List[Tensor]:
    """States of the Schroedinger equation at ``times`` (exact propagator per interval)."""
    out, prev = [], 0.0
    for t in times:
        state = matrix_exp_evolve(state, h, t - prev)
        out.append(state)
        prev = t
    return out


# ----------------------------------------------------------------------------- density matrices / noise
def density_matrix(state: Tensor) -> Tensor:
    v = state.reshape(state.shape[0], -1)
    return v[:, :, None] * v.conj()[:, None, :]


def apply_channel(rho: Tensor, kraus: Sequence[Tensor], wire: int, n: int) -> Tensor:
    """``sum_k K rho K^+`` with single-qubit Kraus operators acting on ``wire``."""
    from .circuit import expand_to_register
    out = torch.zeros_like(rho)
    for k in kraus:
        full = expand_to_register(k.to(rho.dtype).to(rho.device), [wire], n)
        out = out + full @ rho @ full.conj().transpose(-1, -2)
    return out


def bit_flip_kraus(p: float, dtype=torch.complex64):
    return [math.sqrt(1 - p) * G.i_matrix(dtype), math.sqrt(p) * G.x_matrix(dtype)]


def phase_flip_kraus(p: float, dtype=torch.complex64):
    return [math.sqrt(1 - p) * G.i_matrix(dtype), math.sqrt(p) * G.z_matrix(dtype)]


def depolarizing_kraus(p: float, dtype=torch.complex64):
    return [math.sqrt(1 - p) * G.i_matrix(dtype)] + [math.sqrt(p / 3) * G.pauli_matrix(c, dtype) for c in "XYZ"]


def pauli_kraus(px: float, py: float, pz: float, dtype=torch.complex64):
    return [math.sqrt(max(0.0, 1 - px - py - pz)) * G.i_matrix(dtype), math.sqrt(px) * G.x_matrix(dtype),
            math.sqrt(py) * G.y_matrix(dtype), math.sqrt(pz) * G.z_matrix(dtype)]


def amplitude_damping_kraus(gamma: float, dtype=torch.complex64):
    k0 = torch.tensor([[1, 0], [0, math.sqrt(1 - gamma)]], dtype=dtype)
    k1 = torch.tensor([[0, math.sqrt(gamma)], [0, 0]], dtype=dtype)
    return [k0, k1]


def apply_bit_flip(rho, p, wire, n): return apply_channel(rho, bit_flip_kraus(p, rho.dtype), wire, n)
def apply_phase_flip(rho, p, wire, n): return apply_channel(rho, phase_flip_kraus(p, rho.dtype), wire, n)
def apply_depolarizing(rho, p, wire, n): return apply_channel(rho, depolarizing_kraus(p, rho.dtype), wire, n)
def apply_amplitude_damping(rho, g, wire, n): return apply_channel(rho, amplitude_damping_kraus(g, rho.dtype), wire, n)


def dissipator(rho: Tensor, c: Tensor) -> Tensor:
    cd = c.conj().transpose(-1, -2)
    return c @ rho @ cd - 0.5 * (cd @ c @ rho + rho @ cd @ c)


def lindbladian(rho: Tensor, h: Tensor, collapse: Sequence[Tensor]) -> Tensor:
    out = -1j * (h @ rho - rho @ h)
    for c in collapse:
        out = out + dissipator(rho, c)
    return out


def mesolve(h: Tensor, rho: Tensor, times: Sequence[float], collapse: Sequence[Tensor] = (),
            substeps: int = 20) -> List[Tensor]:
    """Lindblad master equation by classical RK4 with ``substeps`` per output interval."""
    out, prev = [], 0.0
    for t in times:
        dt = (t - prev) / substeps
        for _ in range(substeps):
            k1 = lindbladian(rho, h, collapse)
            k2 = lindbladian(rho + 0.5 * dt * k1, h, collapse)
            k3 = lindbladian(rho + 0.5 * dt * k2, h, collapse)
            k4 = lindbladian(rho + dt * k3, h, collapse)
            rho = rho + dt / 6 * (k1 + 2 * k2 + 2 * k3 + k4)
        out.append(rho)
        prev = t
    return out


# ----------------------------------------------------------------------------- gradients
def param_shift(fn: Callable[[Tensor], Tensor], params: Tensor, shift: float = math.pi / 2) -> Tensor:
    """Gradient of a scalar expectation ``fn(params)`` whose parameters enter through gates
    ``exp(-i theta P / 2)``: ``(f(theta + s) - f(theta - s)) / (2 sin s)`` per parameter."""
    grads = torch.zeros_like(params)
    flat = params.detach().reshape(-1)
    for i in range(flat.numel()):
        plus, minus = flat.clone(), flat.clone()
        plus[i] += shift
        minus[i] -= shift
        with torch.no_grad():
            d = fn(plus.view_as(params)) - fn(minus.view_as(params))
        grads.view(-1)[i] = d.sum() / (2 * math.sin(shift))
    return grads


def apply_reset(rho: Tensor, wire: int, n: int) -> Tensor:
    """Reset channel: the qubit is put in |0> whatever its state (Kraus operators |0><0| and |0><1|)."""
    k0 = torch.tensor([[1, 0], [0, 0]], dtype=rho.dtype)
    k1 = torch.tensor([[0, 1], [0, 0]], dtype=rho.dtype)
    return apply_channel(rho, [k0, k1], wire, n)


class Lindbladian:
    """Generator of open-system dynamics ``d rho / dt = -i [H, rho] + sum_k D[c_k](rho)``."""

    def __init__(self, hamiltonian: Tensor, collapse: Sequence[Tensor] = ()):
        self.h, self.collapse = hamiltonian, list(collapse)

    def __call__(self, rho: Tensor) -> Tensor:
        return lindbladian(rho, self.h, self.collapse)

    def evolve(self, rho: Tensor, times: Sequence[float], substeps: int = 20) -> List[Tensor]:
        return mesolve(self.h, rho, times, self.collapse, substeps)

    def superoperator(self) -> Tensor:
        """Matrix of the generator on row-major vectorised density matrices."""
        d = self.h.shape[-1]
        eye = torch.eye(d, dtype=self.h.dtype)
        sup = -1j * (torch.kron(self.h, eye) - torch.kron(eye, self.h.transpose(-1, -2).contiguous()))
        for c in self.collapse:
            cdc = c.conj().transpose(-1, -2) @ c
            sup = sup + torch.kron(c, c.conj()) - 0.5 * (torch.kron(cdc, eye) + torch.kron(eye, cdc.transpose(-1, -2).contiguous()))
        return sup


def sample_energy(state: Tensor, h: Hamiltonian, shots: int = 1024, generator=None) -> Tensor:
    """Energy estimated from measurements: one basis rotation and ``shots`` samples per group of
    qubit-wise commuting terms, parities averaged per term."""
    from .measure import apply_measurement_basis, commuting_groups, sample_indices
    n = h.n_qubits
    coeff = {}
    for c, w in h.terms:
        coeff[w] = coeff.get(w, 0.0) + c
    total = torch.zeros(state.shape[0], dtype=torch.float64)
    words = [w for w in coeff if set(w) != {"I"}]
    total += sum(c for w, c in coeff.items() if set(w) == {"I"})
    for group in commuting_groups(words):
        basis = ["I"] * n
        for w in group:
            for i, ch in enumerate(w):
                if ch != "I":
                    basis[i] = ch
        idx = sample_indices(apply_measurement_basis(state, "".join(basis)), shots, generator)
        bits = (idx[..., None] >> torch.arange(n - 1, -1, -1)) & 1          # [batch, shots, n]
        for w in group:
            sel = torch.tensor([ch != "I" for ch in w])
            par = bits[..., sel].sum(-1) & 1
            total += coeff[w] * (1 - 2 * par).double().mean(-1)
    return total


# the reference has a package at this path: deeper module names resolve to views of the pack
__path__: list = []
