"""Detection operators on this framework's kernels (``csrc/kernels/vision_ops.cu``), with a plain-PyTorch
formulation of each as the CPU path and the numerics oracle.

After tensorplay/vision/ops/boxes.py (``nms``, ``batched_nms``, ``box_area``, ``box_iou``) and
tensorplay/vision/ops/roi_align.py (``roi_align``, ``RoIAlign``). Operators without a kernel here
(``deform_conv2d``, ``ps_roi_align``, ``roi_pool`` ...) resolve to torchvision's.
"""
from __future__ import annotations

import math
from typing import List, Tuple, Union

import torch
from torch import Tensor, nn

from .. import _native
from ..ops._common import lib, ptr, stream_ptr, use_native


def box_area(boxes: Tensor) -> Tensor:
    return (boxes[..., 2] - boxes[..., 0]) * (boxes[..., 3] - boxes[..., 1])


def box_iou(boxes1: Tensor, boxes2: Tensor) -> Tensor:
    """Pairwise intersection over union of ``[N, 4]`` and ``[M, 4]`` boxes (x1, y1, x2, y2) -> ``[N, M]``."""
    lt = torch.max(boxes1[:, None, :2], boxes2[None, :, :2])
    rb = torch.min(boxes1[:, None, 2:], boxes2[None, :, 2:])
    wh = (rb - lt).clamp(min=0)
    inter = wh[..., 0] * wh[..., 1]
    union = box_area(boxes1)[:, None] + box_area(boxes2)[None, :] - inter
    return torch.where(union > 0, inter / union, torch.zeros_like(inter))


def nms_reference(boxes: Tensor, scores: Tensor, iou_threshold: float) -> Tensor:
    """Greedy suppression in plain PyTorch: indices of the kept boxes, by descending score."""
    order = torch.argsort(scores, descending=True, stable=True)
    iou = box_iou(boxes[order].float(), boxes[order].float())
    n = order.numel()
    removed = torch.zeros(n, dtype=torch.bool, device=boxes.device)
    keep = []
    for i in range(n):
        if removed[i]:
            continue
        keep.append(i)
        removed |= (iou[i] > iou_threshold) & (torch.arange(n, device=boxes.device) > i)
    return order[torch.tensor(keep, dtype=torch.long, device=boxes.device)] if keep else order[:0]


def nms(boxes: Tensor, scores: Tensor, iou_threshold: float) -> Tensor:
    """Indices of the boxes that survive greedy non-maximum suppression, sorted by descending score."""
    n = boxes.shape[0]
    if n == 0:
        return torch.empty(0, dtype=torch.long, device=boxes.device)
    if not (boxes.is_cuda and use_native(boxes)) or n > 32768:
        # the kernel's overlap bit matrix takes n * n / 8 bytes (134 MB at 32 768 boxes) and the plain formulation an
        # n x n float matrix: beyond that torchvision's operator, where it is installed
        if n > 4096:
            try:
                import torchvision.ops as _tvo
                return _tvo.nms(boxes.float(), scores.float(), iou_threshold)
            except ImportError:
                pass
        return nms_reference(boxes, scores, iou_threshold)
    b = boxes.detach().float().contiguous()
    order = torch.argsort(scores.detach(), descending=True, stable=True).contiguous()
    L = lib()
    words = (n + 63) // 64
    mask = torch.empty(n * words, dtype=torch.int64, device=boxes.device)
    keep = torch.empty(n, dtype=torch.uint8, device=boxes.device)
    n_keep = torch.empty(1, dtype=torch.int32, device=boxes.device)
    _native.check(L.tpb_nms(ptr(b), ptr(order), n, float(iou_threshold), ptr(mask), ptr(keep), ptr(n_keep),
                            stream_ptr()), "tpb_nms")
    return order[keep.bool()]


def batched_nms(boxes: Tensor, scores: Tensor, idxs: Tensor, iou_threshold: float) -> Tensor:
    """NMS within each category of ``idxs``: the categories are moved apart by more than the largest coordinate, so
    that boxes of different categories never overlap, and one suppression pass handles all of them."""
    if boxes.numel() == 0:
        return torch.empty(0, dtype=torch.long, device=boxes.device)
    span = boxes.max() - boxes.min() + 1
    shifted = boxes - boxes.min() + (idxs.to(boxes) * span)[:, None]
    return nms(shifted, scores, iou_threshold)


def _rois_tensor(boxes: Union[Tensor, List[Tensor]]) -> Tensor:
    if isinstance(boxes, (list, tuple)):
        parts = [torch.cat((torch.full((b.shape[0], 1), i, dtype=b.dtype, device=b.device), b), dim=1)
                 for i, b in enumerate(boxes)]
        return torch.cat(parts, dim=0)
    return boxes


def roi_align_reference(x: Tensor, rois: Tensor, output_size: Tuple[int, int], spatial_scale: float = 1.0,
                        sampling_ratio: int = -1, aligned: bool = False) -> Tensor:
    """RoIAlign written with tensor indexing (differentiable through ``x``): the oracle of the kernels."""
    ph, pw = output_size
    N, C, H, W = x.shape
    out = []
    xf = x.float()
    for roi in rois.float().tolist():
        bi = int(roi[0])
        off = 0.5 if aligned else 0.0
        sw, sh = roi[1] * spatial_scale - off, roi[2] * spatial_scale - off
        rw, rh = roi[3] * spatial_scale - off - sw, roi[4] * spatial_scale - off - sh
        if not aligned:
            rw, rh = max(rw, 1.0), max(rh, 1.0)
        bh, bw = rh / ph, rw / pw
        gh = sampling_ratio if sampling_ratio > 0 else int(math.ceil(rh / ph))
        gw = sampling_ratio if sampling_ratio > 0 else int(math.ceil(rw / pw))
        acc = xf.new_zeros(C, ph, pw)
        if gh > 0 and gw > 0:
            ys = sh + (torch.arange(ph, device=x.device)[:, None] * bh + (torch.arange(gh, device=x.device)[None, :] + 0.5) * bh / gh)
            xs = sw + (torch.arange(pw, device=x.device)[:, None] * bw + (torch.arange(gw, device=x.device)[None, :] + 0.5) * bw / gw)
            ys, xs = ys.reshape(-1).float(), xs.reshape(-1).float()            # [ph*gh], [pw*gw]
            vy = (ys >= -1) & (ys <= H)
            vx = (xs >= -1) & (xs <= W)
            yc, xc = ys.clamp(min=0), xs.clamp(min=0)
            y0 = yc.floor().long().clamp(max=H - 1)
            x0 = xc.floor().long().clamp(max=W - 1)
            y1, x1 = (y0 + 1).clamp(max=H - 1), (x0 + 1).clamp(max=W - 1)
            ly = torch.where(y0 >= H - 1, torch.zeros_like(yc), yc - y0)
            lx = torch.where(x0 >= W - 1, torch.zeros_like(xc), xc - x0)
            hy, hx = 1 - ly, 1 - lx
            plane = xf[bi]                                                     # [C, H, W]
            v = (plane[:, y0][:, :, x0] * (hy[:, None] * hx[None, :]) + plane[:, y0][:, :, x1] * (hy[:, None] * lx[None, :])
                 + plane[:, y1][:, :, x0] * (ly[:, None] * hx[None, :]) + plane[:, y1][:, :, x1] * (ly[:, None] * lx[None, :]))
            v = v * (vy[:, None] & vx[None, :])
            acc = v.view(C, ph, gh, pw, gw).sum(dim=(2, 4)) / (gh * gw)
        out.append(acc)
    res = torch.stack(out) if out else xf.new_zeros(0, C, ph, pw)
    return res.to(x.dtype)


class _RoIAlignFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, rois, ph, pw, spatial_scale, sampling_ratio, aligned):
        N, C, H, W = x.shape
        xc = x.contiguous()
        r = rois.detach().float().contiguous()
        K = r.shape[0]
        y = torch.empty((K, C, ph, pw), dtype=x.dtype, device=x.device)
        _native.check(lib().tpb_roi_align_fwd(ptr(xc), ptr(r), ptr(y), int(x.dtype == torch.bfloat16), N, C, H, W, K,
                                              ph, pw, float(spatial_scale), int(sampling_ratio), int(aligned),
                                              stream_ptr()), "tpb_roi_align_fwd")
        ctx.save_for_backward(r)
        ctx.cfg = (x.shape, x.dtype, ph, pw, spatial_scale, sampling_ratio, aligned)
        return y

    @staticmethod
    def backward(ctx, dy):
        (r,) = ctx.saved_tensors
        shape, dtype, ph, pw, spatial_scale, sampling_ratio, aligned = ctx.cfg
        N, C, H, W = shape
        dyc = dy.contiguous()
        dx = torch.zeros(shape, dtype=torch.float32, device=dy.device)
        _native.check(lib().tpb_roi_align_bwd(ptr(dyc), ptr(r), ptr(dx), int(dyc.dtype == torch.bfloat16), N, C, H, W,
                                              r.shape[0], ph, pw, float(spatial_scale), int(sampling_ratio),
                                              int(aligned), stream_ptr()), "tpb_roi_align_bwd")
        return dx.to(dtype), None, None, None, None, None, None


def roi_align(input: Tensor, boxes: Union[Tensor, List[Tensor]], output_size: Union[int, Tuple[int, int]],
              spatial_scale: float = 1.0, sampling_ratio: int = -1, aligned: bool = False) -> Tensor:
    """Region-of-interest align: ``input [N, C, H, W]``, ``boxes [K, 5]`` (batch index, x1, y1, x2, y2) or a list of
    ``[L_i, 4]`` per image -> ``[K, C, ph, pw]``."""
    rois = _rois_tensor(boxes)
    if isinstance(output_size, int):
        output_size = (output_size, output_size)
    ph, pw = int(output_size[0]), int(output_size[1])
    if input.is_cuda and input.dtype in (torch.float32, torch.bfloat16) and use_native(input):
        return _RoIAlignFn.apply(input, rois, ph, pw, spatial_scale, sampling_ratio, aligned)
    return roi_align_reference(input, rois, (ph, pw), spatial_scale, sampling_ratio, aligned)


class RoIAlign(nn.Module):
    def __init__(self, output_size, spatial_scale: float, sampling_ratio: int, aligned: bool = False):
        super().__init__()
        self.output_size, self.spatial_scale = output_size, spatial_scale
        self.sampling_ratio, self.aligned = sampling_ratio, aligned

    def forward(self, input: Tensor, rois: Union[Tensor, List[Tensor]]) -> Tensor:
        return roi_align(input, rois, self.output_size, self.spatial_scale, self.sampling_ratio, self.aligned)

    def extra_repr(self) -> str:
        return (f"output_size={self.output_size}, spatial_scale={self.spatial_scale}, "
                f"sampling_ratio={self.sampling_ratio}, aligned={self.aligned}")


def __getattr__(name):
    import importlib
    try:
        tvo = importlib.import_module("torchvision.ops")
    except ImportError as e:
        raise AttributeError(f"tensorplay_b200.vision.ops.{name}: no kernel here and torchvision is not installed") from e
    try:
        return getattr(tvo, name)
    except AttributeError:
        for sub in ("poolers", "boxes", "misc", "feature_pyramid_network"):
            m = importlib.import_module(f"torchvision.ops.{sub}")
            if hasattr(m, name):
                return getattr(m, name)
        raise
