"""State-vector quantum simulation on the tensor primitives (the ``tensorplay.quantum`` pack).

States are ``[batch, 2, ..., 2]`` complex tensors with qubit 0 leading; density matrices are
``[batch, 2^n, 2^n]``. Gates stay differentiable in their angles; on a B200 one-qubit and
controlled one-qubit gates on complex64 states run in a streaming CUDA kernel when no gradient
is required.

    >>> from tensorplay_b200 import quantum as tq
    >>> bell = tq.Circuit(2); bell.h(0); bell.cx(0, 1)
    >>> tq.probs(bell())            # tensor([[0.5, 0.0, 0.0, 0.5]])
    >>> tq.expectation(bell(), "ZZ")   # tensor([1.])
"""
from .circuit import (GATE_TABLE, Circuit, efficient_su2, entanglement_pairs, expand_to_register, nlocal_circuit,
                      qft_circuit, real_amplitudes)
from .gates import *  # noqa: F401,F403
from .gates import apply_controlled, apply_gate, n_qubits_of, zero_state
from .measure import (apply_measurement_basis, apply_pauli_word, apply_readout_error, commuting_groups,
                      counts_from_indices, density_probs, expectation, expectation_from_counts,
                      expectation_from_density, gen_bitstrings, joint_expectation, marginal_probs, measure, probs,
                      readout_error_matrix, sample_indices)
from .physics import (Hamiltonian, Lindbladian, apply_reset, sample_energy, amplitude_damping_kraus, apply_amplitude_damping, apply_bit_flip, apply_channel,
                      apply_depolarizing, apply_phase_flip, bit_flip_kraus, density_matrix, depolarizing_kraus,
                      dissipator, energy, energy_from_density, lindbladian, matrix_exp_evolve, mesolve, param_shift,
                      pauli_kraus, phase_flip_kraus, sesolve, trotter_evolve)
from .states import (basis_state, bloch2dens, bloch2sv, dens2bloch, density_from_counts, density_mixture,  # noqa: E402
                     density_to_state, encode_state, fidelity, flatten, global_phase, inner, norm, normalize,
                     partial_trace, plus_state, product_state, random_state, state_from_bases, state_from_counts,
                     sv2bloch, to_density, unflatten, zeros_state)


def encode_w(wires) -> str:
    """Wire indices as a dictionary key: ``[1, 3, 2] -> "1.3.2"`` (tensorplay/quantum/_helpers.py:107)."""
    import operator
    if isinstance(wires, int):
        wires = [wires]
    return ".".join(str(operator.index(w)) for w in wires)


def decode_w(key) -> list:
    """Inverse of :func:`encode_w`: ``"1.3.2" -> [1, 3, 2]``."""
    if not key:
        raise ValueError("a wire key must not be empty")
    return [int(part) for part in str(key).split(".")]

from .. import _views as _views  # noqa: E402

_views.install(__name__, max_depth=1)
