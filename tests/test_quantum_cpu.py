"""Quantum pack on CPU: gates against dense linear algebra, circuits, measurement, dynamics, noise."""
import math

import torch

from tensorplay_b200 import quantum as tq


def test_bell_state_probs_and_expectations():
    c = tq.Circuit(2)
    c.h(0)
    c.cx(0, 1)
    s = c()
    torch.testing.assert_close(tq.probs(s), torch.tensor([[0.5, 0.0, 0.0, 0.5]]))
    torch.testing.assert_close(tq.expectation(s, "ZZ"), torch.tensor([1.0]))
    torch.testing.assert_close(tq.expectation(s, "XX"), torch.tensor([1.0]))
    torch.testing.assert_close(tq.expectation(s, "ZI"), torch.tensor([0.0]))
    bits = tq.measure(s, shots=64, generator=torch.Generator().manual_seed(0))
    assert bits.shape == (1, 64, 2) and bool((bits[..., 0] == bits[..., 1]).all())


def test_apply_gate_matches_dense_matrix_on_any_wires():
    g = torch.Generator().manual_seed(1)
    n = 4
    state = torch.randn(3, 2 ** n, dtype=torch.complex128)
    state = (state / state.norm(dim=1, keepdim=True)).reshape([3] + [2] * n)
    for wires in ([2], [3, 0], [1, 3, 2]):
        u = tq.random_unitary(len(wires), torch.complex128, generator=g)
        out = tq.apply_gate(state, u, wires)
        full = tq.expand_to_register(u, wires, n)
        ref = (state.reshape(3, -1) @ full.T).reshape(out.shape)
        torch.testing.assert_close(out, ref)
    # controlled gate = block matrix on (controls, target)
    out = tq.apply_crx(state, 0.7, 3, 1)
    ref = tq.apply_gate(state, tq.controlled_matrix(tq.rot_x_matrix(0.7, torch.complex128)), [3, 1])
    torch.testing.assert_close(out, ref)


def test_qft_circuit_equals_dft_matrix():
    n = 3
    m = tq.qft_circuit(n).matrix()
    torch.testing.assert_close(m, tq.qft_matrix(n), atol=1e-6, rtol=1e-6)


def test_parameter_gradients_autograd_equals_parameter_shift():
    ansatz = tq.real_amplitudes(3, reps=2)
    h = tq.Hamiltonian([(0.5, "ZZI"), (-0.3, "IXX"), (0.2, "YIY")])
    params = torch.randn(ansatz.n_params, generator=torch.Generator().manual_seed(2), dtype=torch.float64)
    ansatz.dtype = torch.complex128

    def f(p):
        return h.expectation(ansatz(p)).sum()
    p = params.clone().requires_grad_()
    f(p).backward()
    torch.testing.assert_close(p.grad, tq.param_shift(f, params), atol=1e-8, rtol=1e-6)
    # batched parameters: one state per row
    batch = torch.stack((params, params + 0.1))
    assert ansatz(batch).shape[0] == 2


def test_trotter_converges_to_exact_evolution_and_keeps_norm():
    h = tq.Hamiltonian([(1.0, "ZZ"), (0.7, "XI"), (0.4, "IX")])
    s0 = tq.apply_h(tq.zero_state(2, dtype=torch.complex128), 0)
    exact = tq.matrix_exp_evolve(s0, h, 0.8)
    e1 = (tq.trotter_evolve(s0, h, 0.8, steps=50, order=1) - exact).abs().max()
    e2 = (tq.trotter_evolve(s0, h, 0.8, steps=50, order=2) - exact).abs().max()
    assert e2 < e1 < 2e-2 and e2 < 2e-4
    torch.testing.assert_close(tq.probs(exact).sum(-1), torch.ones(1, dtype=torch.float64))
    # energy is conserved by the exact propagator
    torch.testing.assert_close(tq.energy(exact, h), tq.energy(s0, h))


def test_channels_preserve_trace_and_damp():
    s = tq.apply_x(tq.zero_state(2), 0)                 # |10>
    rho = tq.density_matrix(s)
    out = tq.apply_amplitude_damping(rho, 0.3, 0, 2)
    torch.testing.assert_close(torch.diagonal(out, dim1=-2, dim2=-1).real.sum(-1), torch.ones(1))
    torch.testing.assert_close(tq.density_probs(out), torch.tensor([[0.3, 0.0, 0.7, 0.0]]))
    dep = tq.apply_depolarizing(rho, 0.75, 0, 2)          # p = 3/4: qubit 0 fully mixed
    torch.testing.assert_close(tq.density_probs(dep), torch.tensor([[0.5, 0.0, 0.5, 0.0]]))
    z0 = tq.expand_to_register(tq.z_matrix(), [0], 2)
    torch.testing.assert_close(tq.expectation_from_density(dep, z0), torch.zeros(1), atol=1e-6, rtol=0)


def test_lindblad_decay_rate():
    # single qubit, H = 0, collapse sqrt(gamma) sigma_minus: excited population decays as exp(-gamma t)
    gamma = 0.5
    sm = torch.tensor([[0, 1], [0, 0]], dtype=torch.complex128) * math.sqrt(gamma)
    rho = torch.tensor([[[0, 0], [0, 1]]], dtype=torch.complex128)
    out = tq.mesolve(torch.zeros(2, 2, dtype=torch.complex128), rho, [1.0, 2.0], [sm])
    assert abs(out[0][0, 1, 1].real.item() - math.exp(-gamma)) < 1e-6
    assert abs(out[1][0, 1, 1].real.item() - math.exp(-2 * gamma)) < 1e-6


def test_readout_error_and_marginals():
    s = tq.apply_x(tq.zero_state(2), 1)                 # |01>
    p = tq.apply_readout_error(tq.probs(s), tq.readout_error_matrix(0.1, 0.2), 2)
    torch.testing.assert_close(p, torch.tensor([[0.8 * 0.1, 0.8 * 0.9, 0.2 * 0.1, 0.2 * 0.9]]))
    torch.testing.assert_close(tq.marginal_probs(s, [1]), torch.tensor([[0.0, 1.0]]))
    assert tq.commuting_groups(["ZZ", "ZI", "XX", "IX"]) == [["ZZ", "ZI"], ["XX", "IX"]]
    assert tq.expectation_from_counts({"00": 30, "11": 30, "01": 20}, "ZZ") == 0.5


def test_extra_gates_are_unitary_and_match_definitions():
    c = torch.complex128
    for m in (tq.sh_matrix(c), tq.sswap_matrix(c), tq.dcx_matrix(c), tq.ecr_matrix(c), tq.rccx_matrix(c), tq.rc3x_matrix(c),
              tq.single_excitation_matrix(0.7, c), tq.xx_plus_yy_matrix(0.7, 0.3, c), tq.xx_minus_yy_matrix(0.7, 0.3, c),
              tq.multirz_matrix(0.9, 3, c)):
        torch.testing.assert_close(m @ m.conj().transpose(-1, -2), torch.eye(m.shape[-1], dtype=c), atol=1e-10, rtol=0)
    torch.testing.assert_close(tq.sh_matrix(c) @ tq.sh_matrix(c), tq.h_matrix(c), atol=1e-10, rtol=0)
    torch.testing.assert_close(tq.sswap_matrix(c) @ tq.sswap_matrix(c), tq.swap_matrix(c), atol=1e-10, rtol=0)
    # generators: XX+YY and XX-YY rotations, multi-qubit Z rotation
    xx, yy = tq.pauli_string_matrix("XX", c), tq.pauli_string_matrix("YY", c)
    torch.testing.assert_close(tq.xx_plus_yy_matrix(0.7, 0.0, c), torch.linalg.matrix_exp(-1j * 0.7 / 4 * (xx + yy)), atol=1e-10, rtol=0)
    torch.testing.assert_close(tq.xx_minus_yy_matrix(0.7, 0.0, c), torch.linalg.matrix_exp(-1j * 0.7 / 4 * (xx - yy)), atol=1e-10, rtol=0)
    torch.testing.assert_close(tq.multirz_matrix(0.9, 3, c), tq.pauli_rotation_matrix(0.9, "ZZZ", c), atol=1e-10, rtol=0)
    # relative-phase Toffoli acts as CCX on the computational basis up to phases
    assert torch.equal(tq.rccx_matrix(c).abs(), tq.mcx_matrix(2, c).abs())
    assert torch.equal(tq.rc3x_matrix(c).abs(), tq.mcx_matrix(3, c).abs())
    s = tq.apply_dcx(tq.basis_state("10", dtype=c), 0, 1)          # CX(0,1): |11>, then CX(1,0): |01>
    torch.testing.assert_close(tq.probs(s), torch.tensor([[0.0, 1.0, 0.0, 0.0]], dtype=torch.float64))
    e = tq.apply_single_excitation(tq.basis_state("01", dtype=c), math.pi, 0, 1)
    torch.testing.assert_close(tq.probs(e), torch.tensor([[0.0, 0.0, 1.0, 0.0]], dtype=torch.float64), atol=1e-12, rtol=0)


def test_state_helpers():
    c = torch.complex128
    g = torch.Generator().manual_seed(0)
    s = tq.random_state(3, batch=4, dtype=c, generator=g)
    torch.testing.assert_close(tq.norm(s), torch.ones(4, dtype=torch.float64))
    assert tq.unflatten(tq.flatten(s)).shape == s.shape
    torch.testing.assert_close(tq.inner(s, s), torch.ones(4, dtype=c))
    torch.testing.assert_close(tq.fidelity(s, s), torch.ones(4, dtype=torch.float64))
    plus = tq.plus_state(2, dtype=c)
    torch.testing.assert_close(tq.probs(plus), torch.full((1, 4), 0.25, dtype=torch.float64))
    prod = tq.product_state([torch.tensor([1, 0], dtype=c), torch.tensor([0, 1], dtype=c)])
    torch.testing.assert_close(prod, tq.basis_state("01", dtype=c))
    assert torch.equal(tq.basis_state(5, 3, dtype=c), tq.basis_state("101", dtype=c))
    # partial trace of a Bell pair is maximally mixed; of a product state it is the factor
    bell = tq.Circuit(2, dtype=c)
    bell.h(0)
    bell.cx(0, 1)
    rho = tq.to_density(bell())
    torch.testing.assert_close(tq.partial_trace(rho, [0], 2), torch.eye(2, dtype=c)[None] / 2)
    three = tq.to_density(tq.apply_h(tq.basis_state("010", dtype=c), 2))
    red = tq.partial_trace(three, [2, 1], 3)                   # order (qubit 2, qubit 1) = |+>|1>
    want = tq.to_density(tq.product_state([torch.tensor([1, 1], dtype=c) / math.sqrt(2), torch.tensor([0, 1], dtype=c)]))
    torch.testing.assert_close(red, want)
    # mixed-state fidelity and eigen-recovery
    mix = tq.density_mixture([tq.basis_state("0", dtype=c), tq.basis_state("1", dtype=c)], [0.75, 0.25])
    assert abs(tq.fidelity(tq.basis_state("0", dtype=c), mix).item() - 0.75) < 1e-12
    assert abs(tq.fidelity(mix, mix).item() - 1.0) < 1e-9
    back = tq.density_to_state(rho)
    assert abs(tq.fidelity(back, bell()).item() - 1.0) < 1e-9
    # Bloch conversions round-trip
    r = torch.tensor([[0.0, 0.6, 0.8]], dtype=torch.float64)
    sv = tq.bloch2sv(r, c)
    torch.testing.assert_close(tq.sv2bloch(sv[:, None].reshape(1, 2)), r, atol=1e-12, rtol=0)
    torch.testing.assert_close(tq.dens2bloch(tq.bloch2dens(r, c)), r, atol=1e-12, rtol=0)
    enc = tq.encode_state(torch.tensor([[3.0, 4.0, 0.0]]))
    torch.testing.assert_close(tq.probs(enc), torch.tensor([[0.36, 0.64, 0.0, 0.0]]))
    counts = {"00": 30, "11": 10}
    torch.testing.assert_close(tq.probs(tq.state_from_counts(counts)), torch.tensor([[0.75, 0.0, 0.0, 0.25]]))
    torch.testing.assert_close(tq.density_probs(tq.density_from_counts(counts)), torch.tensor([[0.75, 0.0, 0.0, 0.25]]))


def test_reset_lindbladian_and_sampled_energy():
    c = torch.complex128
    rho = tq.to_density(tq.apply_h(tq.basis_state("01", dtype=c), 0))
    out = tq.apply_reset(rho, 0, 2)
    torch.testing.assert_close(tq.density_probs(out), torch.tensor([[0.0, 1.0, 0.0, 0.0]], dtype=torch.float64))
    gamma = 0.5
    sm = torch.tensor([[0, 1], [0, 0]], dtype=c) * math.sqrt(gamma)
    lind = tq.Lindbladian(torch.zeros(2, 2, dtype=c), [sm])
    r0 = torch.tensor([[[0, 0], [0, 1]]], dtype=c)
    assert abs(lind.evolve(r0, [1.0])[0][0, 1, 1].real.item() - math.exp(-gamma)) < 1e-6
    sup = lind.superoperator()
    torch.testing.assert_close((sup @ r0.reshape(4)).reshape(2, 2), lind(r0)[0], atol=1e-12, rtol=0)
    h = tq.Hamiltonian([(0.5, "ZZ"), (0.3, "XI"), (-0.2, "IX"), (0.1, "II")])
    state = tq.apply_ry(tq.apply_h(tq.zero_state(2), 0), 0.4, 1)
    est = tq.sample_energy(state, h, shots=20000, generator=torch.Generator().manual_seed(0))
    assert abs(est.item() - tq.energy(state, h).item()) < 0.02
