"""Cross-entropy on sm_100a row kernels.

Forward: one pass per row computes the online log-sum-exp and the loss. Backward: one pass
rewrites the logits buffer in place with ``(softmax - onehot) * g`` - the upstream gradient
and the mean-reduction factor are read from device memory, so nothing synchronises with the
host. Total traffic: logits read twice, written once.

Reference counterpart: composite log_softmax + nll_loss,
p10/src/backend/composite/LossNLL.cpp:97-265 and p10/src/backend/cuda/LossFillKernels.cu:354-470.
"""
from __future__ import annotations

import torch

from .. import _native
from ._common import lib, ptr, stream_ptr, use_native


class _CrossEntropyFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, target, ignore_index, reduction):
        V = logits.shape[-1]
        lg = logits.reshape(-1, V)
        if lg.stride(-1) != 1 or lg.stride(0) % 8:
            lg = lg.contiguous()
        tg = target.reshape(-1).to(torch.int64).contiguous()
        rows = lg.shape[0]
        loss = torch.empty(rows, dtype=torch.float32, device=lg.device)
        lse = torch.empty(rows, dtype=torch.float32, device=lg.device)
        code = lib().tpb_cross_entropy(lg.data_ptr(), tg.data_ptr(), loss.data_ptr(),
                                       lse.data_ptr(), None, rows, V, lg.stride(0),
                                       int(ignore_index), 1.0, stream_ptr())
        _native.check(code, "tpb_cross_entropy")
        inv_n = None
        if reduction == "mean":
            inv_n = (tg != ignore_index).sum().clamp_(min=1).float().reciprocal_().reshape(1)
        ctx.reduction = reduction
        ctx.ignore_index = ignore_index
        ctx.shape = logits.shape
        ctx.save_for_backward(lg, tg, lse, inv_n if inv_n is not None else torch.empty(0))
        if reduction == "mean":
            return loss.sum() * inv_n[0]
        if reduction == "sum":
            return loss.sum()
        return loss.view(target.shape)

    @staticmethod
    def backward(ctx, g):
        lg, tg, lse, inv_n = ctx.saved_tensors
        rows, V = lg.shape
        g = g.float().contiguous()
        g_scalar = g_rows = None
        if ctx.reduction == "none":
            g_rows = g.reshape(-1)
        else:
            g_scalar = g.reshape(1)
        # The logits buffer is dead after this point; its gradient is written over it.
        code = lib().tpb_cross_entropy_bwd(lg.data_ptr(), tg.data_ptr(), lse.data_ptr(),
                                           lg.data_ptr(), ptr(g_scalar),
                                           inv_n.data_ptr() if inv_n.numel() else None,
                                           ptr(g_rows), rows, V, lg.stride(0),
                                           int(ctx.ignore_index), stream_ptr())
        _native.check(code, "tpb_cross_entropy_bwd")
        return lg.view(ctx.shape), None, None, None


def cross_entropy(logits: torch.Tensor, target: torch.Tensor, ignore_index: int = -100,
                  reduction: str = "mean") -> torch.Tensor:
    """Cross-entropy over the last dim.

    On CUDA bf16 the backward pass overwrites the logits buffer with its gradient (the
    buffer is not needed again by autograd); do not reuse ``logits`` after ``backward``.
    """
    if logits.is_cuda and logits.dtype == torch.bfloat16 and use_native(logits):
        return _CrossEntropyFn.apply(logits, target, ignore_index, reduction)
    V = logits.shape[-1]
    out = torch.nn.functional.cross_entropy(logits.reshape(-1, V).float(), target.reshape(-1),
                                            ignore_index=ignore_index, reduction=reduction)
    return out if reduction != "none" else out.view(target.shape)
