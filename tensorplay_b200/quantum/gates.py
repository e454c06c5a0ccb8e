"""Gate matrices and their application to state tensors.

A state is ``[batch, 2, 2, ...]``: one axis of size 2 per qubit after the batch axis, qubit 0
leading (the most significant bit of the amplitude index). Every gate goes through
:func:`apply_gate`; parametrised matrices are built from tensor operations, so a circuit stays
differentiable in its angles. (The layout and the ``apply_*`` / ``*_matrix`` naming follow the
reference's ``tensorplay/quantum/__init__.py:1-40`` and ``_gates.py``.)
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Union

import torch
from torch import Tensor

Angle = Union[float, Tensor]


def _cdtype(dtype) -> torch.dtype:
    if dtype in (torch.complex64, torch.complex128):
        return dtype
    return torch.complex128 if dtype == torch.float64 else torch.complex64


def _const(rows, dtype=torch.complex64, device=None) -> Tensor:
    return torch.tensor(rows, dtype=_cdtype(dtype), device=device)


def i_matrix(dtype=torch.complex64, device=None): return _const([[1, 0], [0, 1]], dtype, device)
def x_matrix(dtype=torch.complex64, device=None): return _const([[0, 1], [1, 0]], dtype, device)
def y_matrix(dtype=torch.complex64, device=None): return _const([[0, -1j], [1j, 0]], dtype, device)
def z_matrix(dtype=torch.complex64, device=None): return _const([[1, 0], [0, -1]], dtype, device)
def s_matrix(dtype=torch.complex64, device=None): return _const([[1, 0], [0, 1j]], dtype, device)
def sdg_matrix(dtype=torch.complex64, device=None): return _const([[1, 0], [0, -1j]], dtype, device)


def h_matrix(dtype=torch.complex64, device=None):
    r = 1 / math.sqrt(2)
    return _const([[r, r], [r, -r]], dtype, device)


def t_matrix(dtype=torch.complex64, device=None):
    return _const([[1, 0], [0, complex(math.cos(math.pi / 4), math.sin(math.pi / 4))]], dtype, device)


def tdg_matrix(dtype=torch.complex64, device=None):
    return dagger(t_matrix(dtype, device))


def sx_matrix(dtype=torch.complex64, device=None):
    return _const([[0.5 + 0.5j, 0.5 - 0.5j], [0.5 - 0.5j, 0.5 + 0.5j]], dtype, device)


def swap_matrix(dtype=torch.complex64, device=None):
    return _const([[1, 0, 0, 0], [0, 0, 1, 0], [0, 1, 0, 0], [0, 0, 0, 1]], dtype, device)


def iswap_matrix(dtype=torch.complex64, device=None):
    return _const([[1, 0, 0, 0], [0, 0, 1j, 0], [0, 1j, 0, 0], [0, 0, 0, 1]], dtype, device)


def pauli_matrix(name: str, dtype=torch.complex64, device=None) -> Tensor:
    return {"I": i_matrix, "X": x_matrix, "Y": y_matrix, "Z": z_matrix}[name.upper()](dtype, device)


def dagger(m: Tensor) -> Tensor:
    return m.conj().transpose(-1, -2)


def _angle(theta: Angle, dtype=torch.complex64, device=None) -> Tensor:
    real = torch.float64 if _cdtype(dtype) == torch.complex128 else torch.float32
    if not isinstance(theta, Tensor):
        return torch.tensor(float(theta), dtype=real, device=device)   # no detour through float32
    return theta.to(real)


def _stack2(a, b, c, d) -> Tensor:
    """``[[a, b], [c, d]]`` with broadcasting over a leading batch of angles."""
    return torch.stack((torch.stack((a, b), -1), torch.stack((c, d), -1)), -2)


def rot_x_matrix(theta: Angle, dtype=torch.complex64, device=None) -> Tensor:
    t = _angle(theta, dtype, device) / 2
    c, s = torch.cos(t).to(_cdtype(dtype)), torch.sin(t).to(_cdtype(dtype))
    return _stack2(c, -1j * s, -1j * s, c)


def rot_y_matrix(theta: Angle, dtype=torch.complex64, device=None) -> Tensor:
    t = _angle(theta, dtype, device) / 2
    c, s = torch.cos(t).to(_cdtype(dtype)), torch.sin(t).to(_cdtype(dtype))
    return _stack2(c, -s, s, c)


def rot_z_matrix(theta: Angle, dtype=torch.complex64, device=None) -> Tensor:
    t = _angle(theta, dtype, device) / 2
    e = torch.polar(torch.ones_like(t), t).to(_cdtype(dtype))
    z = torch.zeros_like(e)
    return _stack2(e.conj(), z, z, e)


def p_matrix(lam: Angle, dtype=torch.complex64, device=None) -> Tensor:
    t = _angle(lam, dtype, device)
    e = torch.polar(torch.ones_like(t), t).to(_cdtype(dtype))
    return _stack2(torch.ones_like(e), torch.zeros_like(e), torch.zeros_like(e), e)


phase_matrix = p_matrix


def u3_matrix(theta: Angle, phi: Angle, lam: Angle, dtype=torch.complex64, device=None) -> Tensor:
    t = _angle(theta, dtype, device) / 2
    phi, lam = _angle(phi, dtype, device), _angle(lam, dtype, device)
    cd = _cdtype(dtype)
    c, s = torch.cos(t).to(cd), torch.sin(t).to(cd)
    ep = torch.polar(torch.ones_like(phi), phi).to(cd)
    el = torch.polar(torch.ones_like(lam), lam).to(cd)
    return _stack2(c, -el * s, ep * s, ep * el * c)


def u2_matrix(phi: Angle, lam: Angle, dtype=torch.complex64, device=None) -> Tensor:
    return u3_matrix(math.pi / 2, phi, lam, dtype, device)


def rot_matrix(phi: Angle, theta: Angle, omega: Angle, dtype=torch.complex64, device=None) -> Tensor:
    """``RZ(omega) RY(theta) RZ(phi)``."""
    return rot_z_matrix(omega, dtype, device) @ rot_y_matrix(theta, dtype, device) @ rot_z_matrix(phi, dtype, device)


def globalphase_matrix(phi: Angle, dtype=torch.complex64, device=None) -> Tensor:
    t = _angle(phi, dtype, device)
    e = torch.polar(torch.ones_like(t), t).to(_cdtype(dtype))
    return _stack2(e, torch.zeros_like(e), torch.zeros_like(e), e)


def _kron(a: Tensor, b: Tensor) -> Tensor:
    return torch.kron(a, b)


def pauli_string_matrix(word: str, dtype=torch.complex64, device=None) -> Tensor:
    m = torch.ones(1, 1, dtype=_cdtype(dtype), device=device)
    for ch in word:
        m = _kron(m, pauli_matrix(ch, dtype, device))
    return m


def pauli_rotation_matrix(theta: Angle, word: str, dtype=torch.complex64, device=None) -> Tensor:
    """``exp(-i theta / 2 P)`` for a Pauli word ``P`` (``P @ P = I``)."""
    t = _angle(theta, dtype, device) / 2
    cd = _cdtype(dtype)
    p = pauli_string_matrix(word, dtype, device)
    eye = torch.eye(p.shape[0], dtype=cd, device=p.device)
    c, s = torch.cos(t).to(cd), torch.sin(t).to(cd)
    return c[..., None, None] * eye - 1j * s[..., None, None] * p


def rxx_matrix(theta, dtype=torch.complex64, device=None): return pauli_rotation_matrix(theta, "XX", dtype, device)
def ryy_matrix(theta, dtype=torch.complex64, device=None): return pauli_rotation_matrix(theta, "YY", dtype, device)
def rzz_matrix(theta, dtype=torch.complex64, device=None): return pauli_rotation_matrix(theta, "ZZ", dtype, device)
def rzx_matrix(theta, dtype=torch.complex64, device=None): return pauli_rotation_matrix(theta, "ZX", dtype, device)


def controlled_matrix(m: Tensor, n_controls: int = 1) -> Tensor:
    """Block matrix that applies ``m`` when all ``n_controls`` leading qubits are 1."""
    d = m.shape[-1]
    full = d * (2 ** n_controls)
    out = torch.eye(full, dtype=m.dtype, device=m.device).expand(*m.shape[:-2], full, full).clone()
    out[..., full - d:, full - d:] = m
    return out


def mcx_matrix(n_controls: int, dtype=torch.complex64, device=None) -> Tensor:
    return controlled_matrix(x_matrix(dtype, device), n_controls)


def qft_matrix(n: int, dtype=torch.complex64, device=None) -> Tensor:
    d = 2 ** n
    k = torch.arange(d, device=device, dtype=torch.float64)
    ang = 2 * math.pi * torch.outer(k, k) / d
    return (torch.polar(torch.ones_like(ang), ang) / math.sqrt(d)).to(_cdtype(dtype))


def random_unitary(n: int, dtype=torch.complex64, device=None, generator=None) -> Tensor:
    """Haar-distributed unitary on ``n`` qubits (QR of a complex Gaussian, phases fixed)."""
    d = 2 ** n
    a = torch.randn(d, d, dtype=torch.float64, generator=generator) + 1j * torch.randn(d, d, dtype=torch.float64, generator=generator)
    q, r = torch.linalg.qr(a)
    ph = torch.diagonal(r) / torch.diagonal(r).abs()
    return (q * ph).to(_cdtype(dtype)).to(device)


# ----------------------------------------------------------------------------- application
def zero_state(n_qubits: int, batch: int = 1, dtype=torch.complex64, device=None) -> Tensor:
    s = torch.zeros((batch,) + (2,) * n_qubits, dtype=_cdtype(dtype), device=device)
    s.view(batch, -1)[:, 0] = 1
    return s


def n_qubits_of(state: Tensor) -> int:
    return state.dim() - 1


def apply_gate(state: Tensor, matrix: Tensor, wires: Union[int, Sequence[int]]) -> Tensor:
    """Apply a ``2^k x 2^k`` unitary (optionally batched ``[batch, 2^k, 2^k]``) to ``wires``; the
    first wire is the most significant bit of the matrix index."""
    wires = [wires] if isinstance(wires, int) else list(wires)
    n, k = n_qubits_of(state), len(wires)
    if len(set(wires)) != k or any(w < 0 or w >= n for w in wires):
        raise ValueError(f"bad wires {wires} for {n} qubits")
    if matrix.shape[-1] != 2 ** k:
        raise ValueError("matrix size does not match the number of wires")
    matrix = matrix.to(state.dtype)
    if (k == 1 and matrix.dim() == 2 and state.is_cuda and state.dtype == torch.complex64
            and not (torch.is_grad_enabled() and (state.requires_grad or matrix.requires_grad))):
        from ._native import apply_1q_native
        out = apply_1q_native(state, matrix, wires[0], ())
        if out is not None:
            return out
    axes = [w + 1 for w in wires]
    rest = [a for a in range(1, n + 1) if a not in axes]
    perm = [0] + rest + axes
    s = state.permute(perm).reshape(state.shape[0], -1, 2 ** k)
    m = matrix if matrix.dim() == 3 else matrix.unsqueeze(0)
    s = torch.matmul(s, m.transpose(-1, -2))
    s = s.reshape([state.shape[0]] + [2] * n)
    inv = [0] * (n + 1)
    for i, p in enumerate(perm):
        inv[p] = i
    return s.permute(inv).contiguous()


def apply_controlled(state: Tensor, matrix: Tensor, controls: Sequence[int], targets: Union[int, Sequence[int]]) -> Tensor:
    targets = [targets] if isinstance(targets, int) else list(targets)
    controls = list(controls)
    if (len(targets) == 1 and matrix.dim() == 2 and state.is_cuda and state.dtype == torch.complex64
            and not (torch.is_grad_enabled() and (state.requires_grad or matrix.requires_grad))):
        from ._native import apply_1q_native
        out = apply_1q_native(state, matrix.to(state.dtype), targets[0], tuple(controls))
        if out is not None:
            return out
    return apply_gate(state, controlled_matrix(matrix.to(state.dtype), len(controls)), controls + targets)


def _fixed(name, mat_fn, k):
    def f(state: Tensor, *wires: int) -> Tensor:
        if len(wires) == 1 and not isinstance(wires[0], int):
            wires = tuple(wires[0])
        assert len(wires) == k, f"{name} acts on {k} wire(s)"
        return apply_gate(state, mat_fn(state.dtype, state.device), list(wires))
    f.__name__ = f"apply_{name}"
    f.__doc__ = f"Apply the {name.upper()} gate."
    return f


apply_i, apply_x, apply_y, apply_z = (_fixed(n, m, 1) for n, m in
                                      (("i", i_matrix), ("x", x_matrix), ("y", y_matrix), ("z", z_matrix)))
apply_h, apply_s, apply_sdg, apply_t, apply_tdg, apply_sx = (_fixed(n, m, 1) for n, m in (
    ("h", h_matrix), ("s", s_matrix), ("sdg", sdg_matrix), ("t", t_matrix), ("tdg", tdg_matrix), ("sx", sx_matrix)))
apply_swap, apply_iswap = _fixed("swap", swap_matrix, 2), _fixed("iswap", iswap_matrix, 2)


def _param(name, mat_fn, k, n_params=1):
    def f(state: Tensor, *args) -> Tensor:
        params, wires = args[:n_params], args[n_params:]
        if len(wires) == 1 and not isinstance(wires[0], int):
            wires = tuple(wires[0])
        assert len(wires) == k, f"{name} acts on {k} wire(s)"
        return apply_gate(state, mat_fn(*params, dtype=state.dtype, device=state.device), list(wires))
    f.__name__ = f"apply_{name}"
    f.__doc__ = f"Apply {name.upper()}(params..., wires...)."
    return f


apply_rx, apply_ry, apply_rz, apply_p = (_param(n, m, 1) for n, m in (
    ("rx", rot_x_matrix), ("ry", rot_y_matrix), ("rz", rot_z_matrix), ("p", p_matrix)))
apply_u3 = _param("u3", u3_matrix, 1, 3)
apply_u2 = _param("u2", u2_matrix, 1, 2)
apply_rot = _param("rot", rot_matrix, 1, 3)
apply_rxx, apply_ryy, apply_rzz, apply_rzx = (_param(n, m, 2) for n, m in (
    ("rxx", rxx_matrix), ("ryy", ryy_matrix), ("rzz", rzz_matrix), ("rzx", rzx_matrix)))


def apply_global_phase(state: Tensor, phi: Angle) -> Tensor:
    t = _angle(phi, state.dtype, state.device)
    return state * torch.polar(torch.ones_like(t), t).to(state.dtype)


def apply_pauli_rotation(state: Tensor, theta: Angle, word: str, wires: Sequence[int]) -> Tensor:
    return apply_gate(state, pauli_rotation_matrix(theta, word, state.dtype, state.device), list(wires))


def _ctrl(name, base, n_controls=1, n_params=0):
    def f(state: Tensor, *args) -> Tensor:
        params, wires = args[:n_params], args[n_params:]
        if len(wires) == 1 and not isinstance(wires[0], int):
            wires = tuple(wires[0])
        m = base(*params, dtype=state.dtype, device=state.device)
        return apply_controlled(state, m, list(wires[:n_controls]), list(wires[n_controls:]))
    f.__name__ = f"apply_{name}"
    return f


apply_cx = apply_cnot = _ctrl("cx", x_matrix)
apply_cy, apply_cz, apply_ch = _ctrl("cy", y_matrix), _ctrl("cz", z_matrix), _ctrl("ch", h_matrix)
apply_chadamard = apply_ch
apply_cs, apply_csdg, apply_csx = _ctrl("cs", s_matrix), _ctrl("csdg", sdg_matrix), _ctrl("csx", sx_matrix)
apply_crx, apply_cry, apply_crz, apply_cp = (_ctrl(n, m, 1, 1) for n, m in (
    ("crx", rot_x_matrix), ("cry", rot_y_matrix), ("crz", rot_z_matrix), ("cp", p_matrix)))
apply_ccx = apply_toffoli = _ctrl("ccx", x_matrix, 2)
apply_ccz = _ctrl("ccz", z_matrix, 2)
apply_cswap = _ctrl("cswap", swap_matrix, 1)


def apply_mcx(state: Tensor, controls: Sequence[int], target: int) -> Tensor:
    return apply_controlled(state, x_matrix(state.dtype, state.device), list(controls), target)


def apply_multirz(state: Tensor, theta: Angle, wires: Sequence[int]) -> Tensor:
    return apply_pauli_rotation(state, theta, "Z" * len(wires), wires)


# ----------------------------------------------------------------------------- further fixed and parametrised gates
def _matrix_power(m: Tensor, p: float) -> Tensor:
    """Principal ``p``-th power of a unitary through its eigen-decomposition."""
    vals, vecs = torch.linalg.eig(m.to(torch.complex128))
    return ((vecs * vals.pow(p)) @ torch.linalg.inv(vecs)).to(m.dtype)


def sh_matrix(dtype=torch.complex64, device=None): return _matrix_power(h_matrix(dtype, device), 0.5)
def sswap_matrix(dtype=torch.complex64, device=None): return _matrix_power(swap_matrix(dtype, device), 0.5)


def dcx_matrix(dtype=torch.complex64, device=None):
    """Double CNOT: ``CX(0, 1)`` followed by ``CX(1, 0)``."""
    cx01 = controlled_matrix(x_matrix(dtype, device))
    sw = swap_matrix(dtype, device)
    return (sw @ cx01 @ sw) @ cx01


def ecr_matrix(dtype=torch.complex64, device=None):
    r = 1 / math.sqrt(2)
    return _const([[0, 0, r, 1j * r], [0, 0, 1j * r, r], [r, -1j * r, 0, 0], [-1j * r, r, 0, 0]], dtype, device)


def rccx_matrix(dtype=torch.complex64, device=None):
    """Relative-phase Toffoli (Margolus): CCX up to phases ``-1`` on |101> and ``-i / i`` swaps on the last block."""
    m = torch.eye(8, dtype=_cdtype(dtype), device=device)
    m[5, 5] = -1
    m[6, 6], m[7, 7] = 0, 0
    m[6, 7], m[7, 6] = -1j, 1j
    return m


def rc3x_matrix(dtype=torch.complex64, device=None):
    """Relative-phase triple-controlled X."""
    m = torch.eye(16, dtype=_cdtype(dtype), device=device)
    m[12, 12], m[13, 13] = 1j, -1j
    m[14, 14], m[15, 15] = 0, 0
    m[14, 15], m[15, 14] = 1, -1
    return m


def single_excitation_matrix(theta: Angle, dtype=torch.complex64, device=None) -> Tensor:
    """Givens rotation in the {|01>, |10>} subspace by ``theta / 2``."""
    t = _angle(theta, dtype, device) / 2
    cd = _cdtype(dtype)
    c, s = torch.cos(t).to(cd), torch.sin(t).to(cd)
    one, z = torch.ones_like(c), torch.zeros_like(c)
    rows = [torch.stack(r, -1) for r in ((one, z, z, z), (z, c, -s, z), (z, s, c, z), (z, z, z, one))]
    return torch.stack(rows, -2)


def xx_plus_yy_matrix(theta: Angle, beta: Angle = 0.0, dtype=torch.complex64, device=None) -> Tensor:
    """``exp(-i theta/2 (XX + YY)/2)`` conjugated by ``RZ(beta)`` on qubit 0: acts on {|01>, |10>}."""
    t = _angle(theta, dtype, device) / 2
    b = _angle(beta, dtype, device)
    cd = _cdtype(dtype)
    c, s = torch.cos(t).to(cd), torch.sin(t).to(cd)
    em, ep = torch.polar(torch.ones_like(b), -b).to(cd), torch.polar(torch.ones_like(b), b).to(cd)
    one, z = torch.ones_like(c), torch.zeros_like(c)
    rows = [torch.stack(r, -1) for r in ((one, z, z, z), (z, c, -1j * s * em, z), (z, -1j * s * ep, c, z), (z, z, z, one))]
    return torch.stack(rows, -2)


def xx_minus_yy_matrix(theta: Angle, beta: Angle = 0.0, dtype=torch.complex64, device=None) -> Tensor:
    """``exp(-i theta/2 (XX - YY)/2)`` with phase ``beta``: acts on {|00>, |11>}."""
    t = _angle(theta, dtype, device) / 2
    b = _angle(beta, dtype, device)
    cd = _cdtype(dtype)
    c, s = torch.cos(t).to(cd), torch.sin(t).to(cd)
    em, ep = torch.polar(torch.ones_like(b), -b).to(cd), torch.polar(torch.ones_like(b), b).to(cd)
    one, z = torch.ones_like(c), torch.zeros_like(c)
    rows = [torch.stack(r, -1) for r in ((c, z, z, -1j * s * em), (z, one, z, z), (z, z, one, z), (-1j * s * ep, z, z, c))]
    return torch.stack(rows, -2)


def multirz_eigvals(theta: Angle, n: int, dtype=torch.complex64, device=None) -> Tensor:
    """Diagonal of ``exp(-i theta/2 Z^{(x) n})``: ``exp(-+ i theta/2)`` by the parity of the index."""
    t = _angle(theta, dtype, device) / 2
    idx = torch.arange(2 ** n, device=t.device)
    parity = torch.zeros_like(idx)
    for k in range(n):
        parity = parity ^ ((idx >> k) & 1)
    sign = (1 - 2 * parity).to(t.dtype)
    return torch.polar(torch.ones(2 ** n, dtype=t.dtype, device=t.device), -t[..., None] * sign).to(_cdtype(dtype))


def multirz_matrix(theta: Angle, n: int, dtype=torch.complex64, device=None) -> Tensor:
    return torch.diag_embed(multirz_eigvals(theta, n, dtype, device))


apply_shadamard, apply_sswap = _fixed("shadamard", sh_matrix, 1), _fixed("sswap", sswap_matrix, 2)
apply_dcx, apply_ecr = _fixed("dcx", dcx_matrix, 2), _fixed("ecr", ecr_matrix, 2)
apply_rccx, apply_rc3x = _fixed("rccx", rccx_matrix, 3), _fixed("rc3x", rc3x_matrix, 4)
apply_single_excitation = _param("single_excitation", single_excitation_matrix, 2)
apply_xx_plus_yy = _param("xx_plus_yy", xx_plus_yy_matrix, 2, 2)
apply_xx_minus_yy = _param("xx_minus_yy", xx_minus_yy_matrix, 2, 2)


# the reference has a package at this path: deeper module names resolve to views of the pack
__path__: list = []
