"""Expert-parallel mixture-of-experts on peer-memory kernels.

``MoEWorkspace`` owns the symmetric buffers of one model (expert input / output buffers, the
histogram table, signal slots); ``expert_parallel_ffn`` is the autograd op

    y[t] = sum_k w[t,k] * down_e( swiglu( gate_up_e( x[t] ) ) ),   e = topk_idx[t,k]

with experts sharded over the ranks. Forward = route + dispatch (tokens land expert-sorted in
the owners' buffers) + three grouped tcgen05 GEMMs + combine (weighted pull). Backward mirrors
it: scaled dispatch of dy, grouped GEMM input/weight gradients, pull of dx, and the gate-weight
gradient from <dy[t], y_row>.
The public ``TokenSwitch`` API of the reference (tensorplay/distributed/_token_switch.py:43-132:
``create_routing / dispatch / combine``) is provided on top in
``tensorplay_b200.distributed._token_switch``.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import _ckpt

from .. import _native, ops
from ..ops._common import lib, status_word, stream_ptr
from .symm import NO_OFFSET, SymmArena

_SIGS = {
    "tpb_moe_route": [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p,
                      C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_size_t, C.c_int, C.c_uint32, C.c_double,
                      C.c_void_p, C.c_void_p],
    "tpb_symm_peer_ptrs": [C.c_size_t, C.c_void_p, C.c_int],
    "tpb_moe_dispatch": [C.c_void_p, C.c_longlong, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                         C.c_size_t, C.c_int, C.c_size_t, C.c_int, C.c_uint32, C.c_void_p, C.c_int,
                         C.c_void_p, C.c_void_p],
    "tpb_moe_combine": [C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p,
                        C.c_longlong, C.c_void_p, C.c_longlong, C.c_void_p, C.c_size_t, C.c_int, C.c_uint32,
                        C.c_int, C.c_double, C.c_void_p, C.c_void_p],
    "tpb_moe_signal": [C.c_size_t, C.c_int, C.c_uint32, C.c_void_p],
    "tpb_moe_rowdot": [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p],
}


def grouped_gemm(a: torch.Tensor, b: torch.Tensor, offs: torch.Tensor, *, mode: int = 0, b_mn: bool = False,
                 n: Optional[int] = None, k: Optional[int] = None, out: Optional[torch.Tensor] = None,
                 accumulate: bool = False, workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Ragged GEMM over expert segments (``offs`` int32 ``[G+1]`` on device, multiples of 128).

    mode 0: ``out[r] = a[r] @ b[e]^T`` (``b`` ``[G, N, K]``; with ``b_mn`` ``b`` is ``[G, K_red, N_out]``).
    mode 1: ``out[e] = a[rows_e]^T @ b[rows_e]`` -> ``[G, N, K]`` (``a`` ``[rows, N]``, ``b`` ``[rows, K]``).
    """
    G = offs.numel() - 1
    rows = a.shape[0]
    if mode == 0:
        if b_mn:
            kk, nn = b.shape[1], b.shape[2]
        else:
            nn, kk = b.shape[1], b.shape[2]
        if out is None:
            out = torch.empty(rows, nn, dtype=a.dtype, device=a.device)
    else:
        nn, kk = a.shape[1], b.shape[1]
        if out is None:
            out = torch.empty(G, nn, kk, dtype=a.dtype, device=a.device)
    if not (a.is_cuda and a.dtype == torch.bfloat16):
        o = offs.tolist()
        for e in range(G):
            r0, r1 = o[e], o[e + 1]
            if mode == 0:
                w = b[e].float() if b_mn else b[e].float().t()
                res = a[r0:r1].float() @ w
                out[r0:r1] = (out[r0:r1].float() + res if accumulate else res).to(out.dtype)
            else:
                res = a[r0:r1].float().t() @ b[r0:r1].float()
                out[e] = (out[e].float() + res if accumulate else res).to(out.dtype)
        return out
    L = lib()
    if workspace is None:
        workspace = torch.empty(L.tpb_grouped_workspace_ints(rows, G), dtype=torch.int32, device=a.device)
    code = L.tpb_grouped_gemm(a.data_ptr(), b.data_ptr(), out.data_ptr(), offs.data_ptr(), G, rows, nn, kk, mode,
                              int(b_mn), int(out.dtype == torch.float32), int(accumulate), workspace.data_ptr(),
                              status_word(a.device).data_ptr(), stream_ptr())
    _native.check(code, "tpb_grouped_gemm")
    if _native.flop_sinks:
        # the rows in use are a device-side quantity: count the rows of the buffer (an upper bound when the
        # buffer is sized for the worst case)
        _native.add_flops("tpb.grouped_gemm", 2 * rows * nn * kk)
    return out


def _swiglu_rows(gu: torch.Tensor, rows_dev: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` of the packed ``[cap, 2I]`` expert pre-activations, for the first
    ``rows_dev[0]`` rows only (a device scalar: the buffer is sized for the worst case)."""
    cap, two_i = gu.shape
    I = two_i // 2
    if not (gu.is_cuda and gu.dtype == torch.bfloat16 and I % 8 == 0):
        return ops.swiglu_packed(gu)
    out = torch.empty(cap, I, dtype=gu.dtype, device=gu.device)
    code = lib().tpb_swiglu_fwd_n(gu.data_ptr(), gu.data_ptr() + I * 2, out.data_ptr(), cap, I, two_i,
                                  rows_dev.data_ptr(), stream_ptr())
    _native.check(code, "tpb_swiglu_fwd_n")
    return out


def _swiglu_rows_bwd(dact: torch.Tensor, gu: torch.Tensor, rows_dev: torch.Tensor) -> torch.Tensor:
    cap, two_i = gu.shape
    I = two_i // 2
    if not (gu.is_cuda and gu.dtype == torch.bfloat16 and I % 8 == 0):
        g = gu.detach().float().requires_grad_()
        with torch.enable_grad():
            a = torch.nn.functional.silu(g[:, :I]) * g[:, I:]
        return torch.autograd.grad(a, g, dact.float())[0].to(gu.dtype)
    dgu = torch.empty_like(gu)
    code = lib().tpb_swiglu_bwd_n(dact.data_ptr(), gu.data_ptr(), gu.data_ptr() + I * 2, dgu.data_ptr(),
                                  dgu.data_ptr() + I * 2, cap, I, two_i, two_i, rows_dev.data_ptr(), stream_ptr())
    _native.check(code, "tpb_swiglu_bwd_n")
    return dgu


class MoEWorkspace:
    """Symmetric buffers for expert-parallel layers of one model (call collectively)."""

    def __init__(self, tokens: int, top_k: int, hidden: int, num_experts: int, group=None,
                 capacity_factor: float = 2.0, wait_s: float = 30.0, arena: Optional[SymmArena] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        assert num_experts % self.world == 0
        self.E, self.El, self.k, self.H, self.T = num_experts, num_experts // self.world, top_k, hidden, tokens
        avg = tokens * top_k
        self.cap = int((avg * capacity_factor + self.El * 128 + 127) // 128 * 128)
        self.wait_s = wait_s
        nbytes = 3 * self.cap * hidden * 2 + self.world * num_experts * 4 + (8 << 20)
        self.arena = arena or SymmArena._instance or SymmArena(nbytes + (64 << 20), group=group)
        a = self.arena
        raw = a.raw
        if not getattr(raw, "_moe_sigs", False):
            _native.register_sigs(raw, _SIGS)
            raw._moe_sigs = True
        self.raw = raw
        dev = a.device
        self.xbuf = a.alloc(self.cap * hidden, torch.bfloat16).view(self.cap, hidden)   # expert inputs
        self.ybuf = a.alloc(self.cap * hidden, torch.bfloat16).view(self.cap, hidden)   # expert outputs / dx rows
        self.dbuf = a.alloc(self.cap * hidden, torch.bfloat16).view(self.cap, hidden)   # dy rows (backward)
        self.rbuf = a.alloc(self.cap * 8, torch.bfloat16).view(self.cap, 8)             # per-row scalars (backward)
        self._ones8 = None
        # Which forward's rows xbuf / ybuf hold. A backward that finds its own forward's number here
        # (the forward ran immediately before it, as under per-layer activation recomputation) reuses
        # the dispatched inputs and the expert outputs instead of routing and computing them again.
        self.generation = 0
        self.counts = a.alloc(self.world * num_experts, torch.int32)
        self.counts_off = a.offset_of(self.counts)
        ptrs = (C.c_void_p * self.world)()
        _native.check(raw.tpb_symm_peer_ptrs(self.counts_off, ptrs, self.world), "tpb_symm_peer_ptrs")
        self.peer_tbl = torch.tensor([int(p) for p in ptrs], dtype=torch.int64, device=dev)
        self.slot_route = a.slots(self.world)
        self.slot_disp = a.slots(self.world)
        self.slot_done = a.slots(self.world)
        self.epoch = 0
        self.counter = torch.zeros(8, dtype=torch.int32, device=dev)
        self.status = status_word(dev)
        self.gws = torch.empty(lib().tpb_grouped_workspace_ints(self.cap, self.El), dtype=torch.int32, device=dev)

    # ---- primitives (each bumps the epoch it uses consistently on every rank)
    def route(self, topk_idx: torch.Tensor):
        self.epoch += 1
        n = topk_idx.numel()
        dev = topk_idx.device
        dst_rank = torch.empty(n, dtype=torch.int32, device=dev)
        dst_row = torch.empty(n, dtype=torch.int32, device=dev)
        offs2 = torch.empty(2 * self.El + 1, dtype=torch.int32, device=dev)  # offsets, then first padding rows
        offs = offs2[: self.El + 1]
        rows = torch.empty(1, dtype=torch.int32, device=dev)
        idx = topk_idx.reshape(-1).to(torch.int32).contiguous()
        code = self.raw.tpb_moe_route(idx.data_ptr(), n, self.E, self.peer_tbl.data_ptr(), self.counts_off,
                                      dst_rank.data_ptr(), dst_row.data_ptr(), offs2.data_ptr(), rows.data_ptr(),
                                      self.arena.offset_of(self.xbuf), self.H * 2, self.cap, self.arena.pad_off,
                                      self.slot_route, self.epoch, self.wait_s, self.status.data_ptr(), stream_ptr())
        _native.launch_count += 2
        _native.check(code, "tpb_moe_route")
        self.last_recv_rows = rows  # device scalar: padded rows this rank received (load statistic)
        return dst_rank, dst_row, offs

    def dispatch(self, x: torch.Tensor, dst_rank, dst_row, buf: torch.Tensor, scale=None) -> None:
        """Push rows of ``x [T, H]`` into ``buf`` on the owning ranks, then wait until every
        rank's rows have landed here."""
        self.epoch += 1
        code = self.raw.tpb_moe_dispatch(x.data_ptr(), x.stride(0), self.k, dst_row.numel(), dst_rank.data_ptr(),
                                         dst_row.data_ptr(), None if scale is None else scale.data_ptr(),
                                         self.arena.offset_of(buf), self.H, self.arena.pad_off, self.slot_disp,
                                         self.epoch, self.counter.data_ptr(), 0, self.status.data_ptr(), stream_ptr())
        _native.check(code, "tpb_moe_dispatch")
        code = self.raw.tpb_symm_wait_slots(self.arena.pad_off, self.slot_disp, self.epoch, self.wait_s,
                                            self.status.data_ptr(), stream_ptr())
        _native.launch_count += 2
        _native.check(code, "tpb_symm_wait_slots")

    def row_dots(self, a_rows: torch.Tensor, b_rows: torch.Tensor, rows_dev: torch.Tensor, dst_rank, dst_row,
                 tokens: int) -> torch.Tensor:
        """``out[t * k + j] = <a_rows[r], b_rows[r]>`` for the expert row ``r`` of assignment ``(t, j)``: the dot
        products are taken where the rows live and only the scalars cross NVLink (16 bytes per row instead of
        the row itself)."""
        code = self.raw.tpb_moe_rowdot(a_rows.data_ptr(), b_rows.data_ptr(), self.rbuf.data_ptr(), rows_dev.data_ptr(),
                                       self.cap, self.H, stream_ptr())
        _native.launch_count += 1
        _native.check(code, "tpb_moe_rowdot")
        if self._ones8 is None or self._ones8.shape[0] < tokens:
            self._ones8 = torch.zeros(tokens, 8, dtype=torch.bfloat16, device=a_rows.device)
            self._ones8[:, :2] = 1.0
        _, dots = self.combine(self.rbuf, dst_rank, dst_row, tokens=tokens, g=self._ones8, want_out=False, width=8)
        return dots

    def combine(self, buf: torch.Tensor, dst_rank, dst_row, w=None, tokens=None, g=None, want_out=True, width=None):
        """Signal that ``buf`` is complete on this rank, then pull: ``out[t] = sum_k w * buf_row``."""
        self.epoch += 1
        H = self.H if width is None else width
        tokens = tokens if tokens is not None else dst_row.numel() // self.k
        code = self.raw.tpb_moe_signal(self.arena.pad_off, self.slot_done, self.epoch, stream_ptr())
        _native.check(code, "tpb_moe_signal")
        out = torch.empty(tokens, H, dtype=torch.bfloat16, device=buf.device) if want_out else None
        dots = torch.empty(tokens * self.k, dtype=torch.float32, device=buf.device) if g is not None else None
        code = self.raw.tpb_moe_combine(self.arena.offset_of(buf), dst_rank.data_ptr(), dst_row.data_ptr(),
                                        None if w is None else w.data_ptr(), self.k, tokens, H,
                                        None if out is None else out.data_ptr(), H,
                                        None if g is None else g.data_ptr(), 0 if g is None else g.stride(0),
                                        None if dots is None else dots.data_ptr(), self.arena.pad_off,
                                        self.slot_done, self.epoch, 0, self.wait_s, self.status.data_ptr(),
                                        stream_ptr())
        _native.launch_count += 2
        _native.check(code, "tpb_moe_combine")
        return out, dots


class _EPFFNFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, topk_idx, topk_w, w_gate_up, w_down, ws: MoEWorkspace, result_is_region_output=False):
        T, H = x.shape
        dst_rank, dst_row, offs = ws.route(topk_idx)
        ws.dispatch(x, dst_rank, dst_row, ws.xbuf)
        rows_dev = offs[ws.El:]  # device scalar: rows of the expert buffers that are in use
        gu = grouped_gemm(ws.xbuf, w_gate_up, offs, workspace=ws.gws)                      # [cap, 2I]
        act = _swiglu_rows(gu, rows_dev)                                                    # [cap, I]
        grouped_gemm(act, w_down, offs, out=ws.ybuf, workspace=ws.gws)                      # [cap, H]
        wf = topk_w.reshape(-1).float().contiguous()
        if result_is_region_output and _ckpt.recomputing():
            # recomputation of a checkpointed block whose result this is: nobody reads the value (backward
            # starts from the incoming gradient), so the pull of the expert rows over NVLink is skipped
            y = x.new_empty(T, H)
        else:
            y, _ = ws.combine(ws.ybuf, dst_rank, dst_row, w=wf, tokens=T)
        ws.generation += 1
        ctx.gen = ws.generation
        ctx.ws = ws
        ctx.refs = (w_gate_up if hasattr(w_gate_up, "_tpb_grad_view") else None,
                    w_down if hasattr(w_down, "_tpb_grad_view") else None)
        if any(ctx.needs_input_grad):
            # a graph is being recorded: keep the routing and the expert activations for the backward
            ctx.save_for_backward(x, topk_idx, wf, w_gate_up, w_down, dst_rank, dst_row, offs, gu, act)
        else:
            ctx.save_for_backward(x, topk_idx, wf, w_gate_up, w_down)
        return y

    @staticmethod
    def backward(ctx, dy):
        saved = ctx.saved_tensors
        x, topk_idx, wf, w_gate_up, w_down = saved[:5]
        ws = ctx.ws
        T, H = x.shape
        dy = dy.contiguous()
        if len(saved) > 5 and ws.generation == ctx.gen:
            # no other forward used the workspace since: xbuf still holds this call's dispatched
            # rows and ybuf its expert outputs
            dst_rank, dst_row, offs, gu, act = saved[5:]
            xin = ws.xbuf
        else:
            # The buffers are shared between layers: route again (the row assignment only has to be
            # consistent within this backward) and recompute the expert activations.
            dst_rank, dst_row, offs = ws.route(topk_idx)
            ws.dispatch(x, dst_rank, dst_row, ws.xbuf)
            xin = ws.xbuf
            gu = grouped_gemm(xin, w_gate_up, offs, workspace=ws.gws)
            act = _swiglu_rows(gu, offs[ws.El:])
            grouped_gemm(act, w_down, offs, out=ws.ybuf, workspace=ws.gws)
        ws.generation += 1  # ybuf is overwritten below
        # dy rows, scaled by the gate weights, to the expert owners (padding rows of dbuf may hold
        # anything: they meet zero rows of xin / act in the weight gradients and their own output
        # rows are never pulled)
        ws.dispatch(dy, dst_rank, dst_row, ws.dbuf, scale=wf)
        dyr = ws.dbuf
        # gate-weight gradient <dy[t], y_row>: the owner of the row has w * dy[t] (just dispatched) and
        # y_row side by side, so it takes the dot product and only that scalar travels back; the token's
        # rank divides by w (top-k weights of a softmax are positive; a weight of exactly zero gets a
        # zero gradient)
        wdots = ws.row_dots(ws.dbuf, ws.ybuf, offs[ws.El:], dst_rank, dst_row, T)
        dots = torch.where(wf != 0, wdots / wf, torch.zeros_like(wdots))
        dact = grouped_gemm(dyr, w_down, offs, b_mn=True, workspace=ws.gws)                # [cap, I]
        dwd = _wgrad(dyr, act, offs, ctx.refs[1], ws)
        dgu = _swiglu_rows_bwd(dact, gu, offs[ws.El:])   # rows beyond the limit stay unwritten: no tile reads them
        dxr = grouped_gemm(dgu, w_gate_up, offs, b_mn=True, out=ws.ybuf, workspace=ws.gws)  # [cap, H]
        dwg = _wgrad(dgu, xin, offs, ctx.refs[0], ws)
        dx, _ = ws.combine(dxr, dst_rank, dst_row, tokens=T)
        return dx, None, dots.view(T, -1).to(dy.dtype), dwg, dwd, None, None


def _wgrad(dy_rows, x_rows, offs, ref, ws):
    if ref is not None and ref._tpb_grad_view is not None:
        grouped_gemm(dy_rows, x_rows, offs, mode=1, out=ref._tpb_grad_view,
                     accumulate=getattr(ref, "_tpb_grad_written", False), workspace=ws.gws)
        ref._tpb_grad_written = True
        return None
    return grouped_gemm(dy_rows, x_rows, offs, mode=1, workspace=ws.gws)


def expert_parallel_ffn(x: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor,
                        w_gate_up: torch.Tensor, w_down: torch.Tensor,
                        ws: Optional[MoEWorkspace] = None, num_experts: Optional[int] = None,
                        group=None, result_is_region_output: bool = False) -> torch.Tensor:
    """SwiGLU experts sharded over ranks. ``x [T, H]``, ``topk_idx/topk_w [T, k]`` (global expert
    ids), ``w_gate_up [E_local, 2I, H]``, ``w_down [E_local, H, I]`` (this rank's experts).
    ``result_is_region_output``: the caller only adds the result to the residual stream and returns it as
    the result of a checkpointed region; its recomputation then skips the final pull of the expert rows."""
    if ws is not None and x.is_cuda and x.dtype == torch.bfloat16:
        return _EPFFNFn.apply(x, topk_idx, topk_w, w_gate_up, w_down, ws, result_is_region_output)
    return expert_ffn_reference(x, topk_idx, topk_w, w_gate_up, w_down, group)


def expert_ffn_reference(x, topk_idx, topk_w, w_gate_up, w_down, group=None):
    """Plain PyTorch expert FFN. With several ranks every rank gathers all experts' weights
    (differentiably) and evaluates its own tokens densely - the oracle for the kernels."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world > 1:
        from torch.distributed.nn.functional import all_gather
        w_gate_up = torch.cat(all_gather(w_gate_up, group=group), dim=0)
        w_down = torch.cat(all_gather(w_down, group=group), dim=0)
    T, H = x.shape
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    E = w_gate_up.shape[0]
    I = w_down.shape[2]
    xf = x.float()
    for e in range(E):
        mask = topk_idx == e
        if not mask.any():
            continue
        tok, slot = mask.nonzero(as_tuple=True)
        h = xf[tok] @ w_gate_up[e].float().t()
        a = torch.nn.functional.silu(h[:, :I]) * h[:, I:]
        y = a @ w_down[e].float().t()
        out.index_add_(0, tok, y * topk_w[tok, slot].float().unsqueeze(-1))
    return out.to(x.dtype)


def topk_route(logits: torch.Tensor, k: int, renormalize: bool = True) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Softmax over experts, top-k, optional renormalisation; also returns the load-balance
    auxiliary loss ``E * sum_e f_e * P_e`` (fraction of assignments x mean router probability)."""
    probs = torch.softmax(logits.float(), dim=-1)
    w, idx = torch.topk(probs, k, dim=-1)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    E = logits.shape[-1]
    f = torch.zeros(E, dtype=torch.float32, device=logits.device)
    f.index_add_(0, idx.reshape(-1), torch.ones(idx.numel(), dtype=torch.float32, device=logits.device))
    f = f / idx.numel()
    aux = E * (f * probs.mean(dim=0)).sum()
    return idx, w, aux
