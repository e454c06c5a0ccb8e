"""Fused AdamW step over flat shards or tensor lists (sm_100a), plus grad-norm helpers.

Reference counterpart: ``_fused_adamw_`` multi-tensor apply,
p10/include/OptimizerMTA.cuh:560-748 and p10/src/backend/cuda/OptimizerKernels.cu.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import torch

from .. import _native
from ._common import lib, ptr, stream_ptr, use_native


def adamw_flat_(master: torch.Tensor, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor,
                grad: torch.Tensor, model: Optional[torch.Tensor], *, lr: float, beta1: float,
                beta2: float, eps: float, weight_decay: float, step: int, grad_scale: float = 1.0,
                maximize: bool = False, clip_coef: Optional[torch.Tensor] = None,
                found_inf: Optional[torch.Tensor] = None) -> None:
    """One AdamW step on a flat fp32 master/moment shard; writes the bf16/fp32 model copy."""
    n = master.numel()
    if use_native(master, grad):
        code = lib().tpb_adamw_flat(
            master.data_ptr(), exp_avg.data_ptr(), exp_avg_sq.data_ptr(), grad.data_ptr(),
            int(grad.dtype == torch.bfloat16), ptr(model),
            int(model is not None and model.dtype == torch.bfloat16), n, lr, beta1, beta2, eps,
            weight_decay, int(step), float(grad_scale), int(maximize), ptr(clip_coef),
            ptr(found_inf), stream_ptr())
        _native.check(code, "tpb_adamw_flat")
        return
    if found_inf is not None and float(found_inf) != 0.0:
        return
    g = grad.float() * grad_scale
    if clip_coef is not None:
        g = g * clip_coef.float()
    if maximize:
        g = -g
    master.mul_(1 - lr * weight_decay)
    exp_avg.mul_(beta1).add_(g, alpha=1 - beta1)
    exp_avg_sq.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    denom = exp_avg_sq.sqrt() / (bc2 ** 0.5) + eps
    master.addcdiv_(exp_avg, denom, value=-lr / bc1)
    if model is not None:
        model.copy_(master)


def _ptr_array(ts: Sequence[Optional[torch.Tensor]]):
    arr = (C.c_void_p * len(ts))()
    for i, t in enumerate(ts):
        arr[i] = None if t is None else t.data_ptr()
    return arr


def adamw_multi_(masters: List[torch.Tensor], exp_avgs: List[torch.Tensor],
                 exp_avg_sqs: List[torch.Tensor], grads: List[torch.Tensor],
                 models: Optional[List[torch.Tensor]], *, lr: float, beta1: float, beta2: float,
                 eps: float, weight_decay: float, step: int, grad_scale: float = 1.0,
                 maximize: bool = False, clip_coef: Optional[torch.Tensor] = None,
                 found_inf: Optional[torch.Tensor] = None) -> None:
    """Multi-tensor AdamW: all tensors of the list are updated by a handful of launches."""
    if not masters:
        return
    if use_native(masters[0], grads[0]):
        gb = grads[0].dtype == torch.bfloat16
        mb = models is not None and models[0].dtype == torch.bfloat16
        assert all((g.dtype == torch.bfloat16) == gb for g in grads)
        numel = (C.c_longlong * len(masters))(*[t.numel() for t in masters])
        code = lib().tpb_adamw_multi(
            len(masters), _ptr_array(masters), _ptr_array(exp_avgs), _ptr_array(exp_avg_sqs),
            _ptr_array(grads), _ptr_array(models) if models is not None else None, numel,
            int(gb), int(mb), lr, beta1, beta2, eps, weight_decay, int(step), float(grad_scale),
            int(maximize), ptr(clip_coef), ptr(found_inf), stream_ptr())
        _native.check(code, "tpb_adamw_multi")
        return
    for i in range(len(masters)):
        adamw_flat_(masters[i], exp_avgs[i], exp_avg_sqs[i], grads[i],
                    None if models is None else models[i], lr=lr, beta1=beta1, beta2=beta2, eps=eps,
                    weight_decay=weight_decay, step=step, grad_scale=grad_scale, maximize=maximize,
                    clip_coef=clip_coef, found_inf=found_inf)


def sumsq_(x: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """``out[0] += sum((x * scale)^2)`` without a host sync."""
    if use_native(x, out):
        code = lib().tpb_sumsq(x.data_ptr(), int(x.dtype == torch.bfloat16), x.numel(), scale,
                               out.data_ptr(), stream_ptr())
        _native.check(code, "tpb_sumsq")
    else:
        out[0] += (x.float() * scale).pow(2).sum()


def clip_coef_(sumsq: torch.Tensor, max_norm: float, coef: torch.Tensor,
               norm_out: Optional[torch.Tensor] = None) -> None:
    if use_native(sumsq, coef):
        code = lib().tpb_clip_coef(sumsq.data_ptr(), max_norm, coef.data_ptr(), ptr(norm_out),
                                   stream_ptr())
        _native.check(code, "tpb_clip_coef")
    else:
        nrm = sumsq.sqrt()
        if norm_out is not None:
            norm_out.copy_(nrm)
        coef.copy_(torch.clamp(max_norm / (nrm + 1e-6), max=1.0))


OPT_SGD, OPT_ADAGRAD, OPT_RMSPROP = 0, 1, 2
FLAG_NESTEROV, FLAG_MAXIMIZE, FLAG_CENTERED, FLAG_FIRST_STEP, FLAG_MOMENTUM = 1, 2, 4, 8, 16


def optim_multi_(algo: int, flags: int, params: List[torch.Tensor], s1: Optional[List[torch.Tensor]],
                 s2: Optional[List[torch.Tensor]], s3: Optional[List[torch.Tensor]], grads: List[torch.Tensor],
                 models: Optional[List[torch.Tensor]], *, lr: float, weight_decay: float = 0.0, a: float = 0.0,
                 b: float = 0.0, eps: float = 0.0, grad_scale: float = 1.0,
                 found_inf: Optional[torch.Tensor] = None) -> None:
    """One multi-tensor step of SGD / Adagrad / RMSprop on CUDA (``params``: fp32 weights or master
    copies; ``models``: the bf16 parameters to write alongside, or None). The meaning of ``a`` / ``b``
    and of the state lists follows ``tpb_optim_multi``."""
    if not params:
        return
    use_native(params[0], grads[0])
    gb = grads[0].dtype == torch.bfloat16
    assert all((g.dtype == torch.bfloat16) == gb for g in grads)
    numel = (C.c_longlong * len(params))(*[t.numel() for t in params])
    arr = lambda ts: _ptr_array(ts) if ts is not None else None  # noqa: E731
    code = lib().tpb_optim_multi(algo, flags, len(params), _ptr_array(params), arr(s1), arr(s2), arr(s3),
                                 _ptr_array(grads), arr(models), numel, int(gb), lr, weight_decay, a, b, eps,
                                 float(grad_scale), ptr(found_inf), stream_ptr())
    _native.check(code, "tpb_optim_multi")


def amp_unscale_(grads: List[torch.Tensor], inv_scale: torch.Tensor, found_inf: torch.Tensor) -> None:
    """``g *= inv_scale`` for every gradient (in place), ``found_inf[0] = 1`` if any holds inf / nan."""
    by_dtype = {}
    for g in grads:
        by_dtype.setdefault(g.dtype, []).append(g)
    for dt, gs in by_dtype.items():
        if gs[0].is_cuda and dt in (torch.float32, torch.bfloat16) and all(g.is_contiguous() for g in gs):
            use_native(gs[0])
            numel = (C.c_longlong * len(gs))(*[g.numel() for g in gs])
            code = lib().tpb_amp_unscale_multi(len(gs), _ptr_array(gs), numel, int(dt == torch.bfloat16),
                                               inv_scale.data_ptr(), found_inf.data_ptr(), stream_ptr())
            _native.check(code, "tpb_amp_unscale_multi")
        else:
            torch._amp_foreach_non_finite_check_and_unscale_(gs, found_inf, inv_scale)


def amp_update_scale_(scale: torch.Tensor, growth_tracker: torch.Tensor, found_inf: torch.Tensor,
                      growth_factor: float, backoff_factor: float, growth_interval: int) -> None:
    if scale.is_cuda:
        use_native(scale)
        code = lib().tpb_amp_update_scale(scale.data_ptr(), growth_tracker.data_ptr(), found_inf.data_ptr(),
                                          growth_factor, backoff_factor, int(growth_interval), stream_ptr())
        _native.check(code, "tpb_amp_update_scale")
    else:
        torch._amp_update_scale_(scale, growth_tracker, found_inf, growth_factor, backoff_factor, growth_interval)


def adafactor_step_(master: torch.Tensor, grad: torch.Tensor, model: Optional[torch.Tensor],
                    row_var: Optional[torch.Tensor], col_var: Optional[torch.Tensor], variance: Optional[torch.Tensor],
                    state: dict, *, lr: float, weight_decay: float, eps1: float, eps2: float, d: float, omb2: float,
                    rho: float, grad_scale: float = 1.0, found_inf: Optional[torch.Tensor] = None) -> None:
    """One fused Adafactor step of a vector or matrix on CUDA (fp32 weights and state; ``grad`` bf16 or fp32;
    ``model``: optional bf16 copy written in the same pass). ``state`` caches the scratch buffer."""
    if master.dim() > 1:
        R, C = master.shape
    else:
        R, C = 1, master.numel()
    L = lib()
    need = 4 + (R + C if R > 1 else 0)
    sc = state.get("_scratch")
    if sc is None or sc.numel() < need:
        sc = torch.empty(need, dtype=torch.float32, device=master.device)
        state["_scratch"] = sc
    code = L.tpb_adafactor_step(master.data_ptr(), grad.data_ptr(), int(grad.dtype == torch.bfloat16), ptr(model),
                                ptr(row_var), ptr(col_var), ptr(variance), sc.data_ptr(), R, C, float(lr),
                                float(weight_decay), float(eps1), float(eps2), float(d), float(omb2), float(rho),
                                float(grad_scale), ptr(found_inf), stream_ptr())
    _native.check(code, "tpb_adafactor_step")
