"""Circuit container and ansatz builders (the reference's ``tensorplay/quantum/_circuit.py``
surface: ``Circuit``, ``GATE_TABLE``, ``qft_circuit``, ``real_amplitudes``, ``efficient_su2``)."""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
from torch import Tensor, nn

from . import gates as G

# name -> (apply function, number of parameters, number of wires; 0 = variable)
GATE_TABLE: Dict[str, Tuple[Callable, int, int]] = {
    "i": (G.apply_i, 0, 1), "x": (G.apply_x, 0, 1), "y": (G.apply_y, 0, 1), "z": (G.apply_z, 0, 1),
    "h": (G.apply_h, 0, 1), "s": (G.apply_s, 0, 1), "sdg": (G.apply_sdg, 0, 1), "t": (G.apply_t, 0, 1),
    "tdg": (G.apply_tdg, 0, 1), "sx": (G.apply_sx, 0, 1),
    "rx": (G.apply_rx, 1, 1), "ry": (G.apply_ry, 1, 1), "rz": (G.apply_rz, 1, 1), "p": (G.apply_p, 1, 1),
    "u2": (G.apply_u2, 2, 1), "u3": (G.apply_u3, 3, 1), "rot": (G.apply_rot, 3, 1),
    "cx": (G.apply_cx, 0, 2), "cnot": (G.apply_cx, 0, 2), "cy": (G.apply_cy, 0, 2), "cz": (G.apply_cz, 0, 2),
    "ch": (G.apply_ch, 0, 2), "cs": (G.apply_cs, 0, 2), "csx": (G.apply_csx, 0, 2),
    "swap": (G.apply_swap, 0, 2), "iswap": (G.apply_iswap, 0, 2),
    "crx": (G.apply_crx, 1, 2), "cry": (G.apply_cry, 1, 2), "crz": (G.apply_crz, 1, 2), "cp": (G.apply_cp, 1, 2),
    "rxx": (G.apply_rxx, 1, 2), "ryy": (G.apply_ryy, 1, 2), "rzz": (G.apply_rzz, 1, 2), "rzx": (G.apply_rzx, 1, 2),
    "ccx": (G.apply_ccx, 0, 3), "toffoli": (G.apply_ccx, 0, 3), "ccz": (G.apply_ccz, 0, 3),
    "cswap": (G.apply_cswap, 0, 3),
}


class Circuit(nn.Module):
    """Ordered list of gates on ``n_qubits`` wires. Parameters are either fixed values given at
    build time or slots of the ``params`` tensor passed to the call (``circuit(params)``), which
    keeps the circuit differentiable and batched: ``params`` may be ``[n_params]`` or
    ``[batch, n_params]``."""

    def __init__(self, n_qubits: int, dtype=torch.complex64):
        super().__init__()
        self.n_qubits, self.dtype = n_qubits, dtype
        self.ops: List[tuple] = []   # (name, wires, [fixed values or ("slot", index)])
        self.n_params = 0

    def add(self, name: str, wires: Sequence[int], params: Sequence = ()) -> "Circuit":
        fn, n_p, n_w = GATE_TABLE[name]
        if n_w and len(wires) != n_w:
            raise ValueError(f"{name} acts on {n_w} wire(s)")
        vals = []
        params = list(params)
        for i in range(n_p):
            if i < len(params) and params[i] is not None:
                vals.append(params[i])
            else:
                vals.append(("slot", self.n_params))
                self.n_params += 1
        self.ops.append((name, tuple(wires), vals))
        return self

    def unitary(self, matrix: Tensor, wires: Sequence[int]) -> "Circuit":
        self.ops.append(("unitary", tuple(wires), [matrix]))
        return self

    def __getattr__(self, name):
        if name in GATE_TABLE:
            n_p, n_w = GATE_TABLE[name][1], GATE_TABLE[name][2]

            def method(*args):
                # wires first, then parameters: c.rx(0, theta), c.cx(0, 1), c.rx(0) leaves a free slot
                return self.add(name, args[:n_w], args[n_w:])
            return method
        return super().__getattr__(name)

    def forward(self, params: Optional[Tensor] = None, state: Optional[Tensor] = None) -> Tensor:
        batch = 1
        if params is not None and params.dim() == 2:
            batch = params.shape[0]
        if state is None:
            device = params.device if params is not None else None
            state = G.zero_state(self.n_qubits, batch, self.dtype, device)
        for name, wires, vals in self.ops:
            if name == "unitary":
                state = G.apply_gate(state, vals[0].to(state.device), list(wires))
                continue
            fn = GATE_TABLE[name][0]
            args = []
            for v in vals:
                if isinstance(v, tuple) and v and v[0] == "slot":
                    if params is None:
                        raise ValueError("this circuit has free parameters: call it with a params tensor")
                    args.append(params[..., v[1]])
                else:
                    args.append(v)
            state = fn(state, *args, *wires)
        return state

    def matrix(self, params: Optional[Tensor] = None) -> Tensor:
        """Dense unitary of the circuit (columns = images of the basis states)."""
        d = 2 ** self.n_qubits
        eye = torch.eye(d, dtype=self.dtype).reshape([d] + [2] * self.n_qubits)
        if params is not None:
            eye = eye.to(params.device)
        return self.forward(params, eye).reshape(d, d).transpose(0, 1)


def entanglement_pairs(n: int, kind: str = "linear") -> List[Tuple[int, int]]:
    if kind == "linear":
        return [(i, i + 1) for i in range(n - 1)]
    if kind == "circular":
        return [(i, (i + 1) % n) for i in range(n)] if n > 2 else [(0, 1)]
    if kind == "full":
        return [(i, j) for i in range(n) for j in range(i + 1, n)]
    raise ValueError(kind)


def nlocal_circuit(n: int, rotations: Sequence[str], entangler: str = "cx", reps: int = 1,
                   entanglement: str = "linear", final_rotation: bool = True) -> Circuit:
    c = Circuit(n)
    for rep in range(reps + (1 if final_rotation else 0)):
        for r in rotations:
            for q in range(n):
                c.add(r, (q,))
        if rep < reps:
            for a, b in entanglement_pairs(n, entanglement):
                c.add(entangler, (a, b))
    return c


def real_amplitudes(n: int, reps: int = 1, entanglement: str = "linear") -> Circuit:
    return nlocal_circuit(n, ["ry"], "cx", reps, entanglement)


def efficient_su2(n: int, reps: int = 1, entanglement: str = "linear") -> Circuit:
    return nlocal_circuit(n, ["ry", "rz"], "cx", reps, entanglement)


def qft_circuit(n: int, swaps: bool = True) -> Circuit:
    c = Circuit(n)
    for q in range(n):
        c.h(q)
        for k in range(q + 1, n):
            c.cp(k, q, math.pi / 2 ** (k - q))
    if swaps:
        for q in range(n // 2):
            c.swap(q, n - 1 - q)
    return c


def expand_to_register(matrix: Tensor, wires: Sequence[int], n: int) -> Tensor:
    """Dense ``2^n x 2^n`` matrix of a gate acting on ``wires`` of an ``n``-qubit register."""
    d = 2 ** n
    eye = torch.eye(d, dtype=matrix.dtype, device=matrix.device).reshape([d] + [2] * n)
    return G.apply_gate(eye, matrix, list(wires)).reshape(d, d).transpose(0, 1)


# the reference has a package at this path: deeper module names resolve to views of the pack
__path__: list = []
