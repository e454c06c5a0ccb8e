"""Detection operators: plain-PyTorch formulations on CPU, kernels against them on the GPU."""
import pytest
import torch

from tensorplay_b200.vision import ops as V


def _boxes(n, seed=0, span=60.0):
    g = torch.Generator().manual_seed(seed)
    b = torch.rand(n, 4, generator=g) * span
    b[:, 2:] = b[:, :2] + 1 + torch.rand(n, 2, generator=g) * 25
    return b, torch.rand(n, generator=g)


def test_box_iou_and_nms_reference():
    b = torch.tensor([[0., 0., 10., 10.], [1., 1., 11., 11.], [20., 20., 30., 30.], [0., 0., 10., 10.]])
    iou = V.box_iou(b, b)
    assert torch.allclose(iou.diag(), torch.ones(4)) and iou[0, 2] == 0 and abs(iou[0, 1] - 81 / 119) < 1e-6
    s = torch.tensor([0.9, 0.8, 0.7, 0.95])
    assert V.nms(b, s, 0.5).tolist() == [3, 2]            # 0 and 1 overlap the best box, 2 stands alone
    assert V.nms(b, s, 0.99).tolist() == [3, 1, 2]        # only the exact duplicate goes
    idx = torch.tensor([0, 1, 0, 1])
    assert sorted(V.batched_nms(b, s, idx, 0.5).tolist()) == [0, 2, 3]   # categories do not suppress each other
    assert V.nms(b[:0], s[:0], 0.5).numel() == 0


def test_roi_align_reference_properties():
    x = torch.arange(2 * 1 * 6 * 6, dtype=torch.float32).view(2, 1, 6, 6)
    # a box covering exactly one pixel centre region of a linear ramp returns the ramp's value there
    rois = torch.tensor([[1, 2.0, 3.0, 3.0, 4.0]])
    y = V.roi_align(x, rois, 1, 1.0, 2, aligned=True)
    assert abs(y.item() - (36 + 3.0 * 6 + 2.0)) < 1e-4     # centre (2.5, 3.5) - 0.5 -> pixel (x=2, y=3)
    per_image = V.roi_align(x, [torch.tensor([[0., 0., 4., 4.]]), torch.tensor([[2., 3., 3., 4.]])], 1, 1.0, 2, True)
    assert abs(per_image[1].item() - y.item()) < 1e-6
    assert V.RoIAlign((2, 3), 0.5, 2)(x, rois).shape == (1, 1, 2, 3)


@pytest.mark.gpu
@pytest.mark.parametrize("n", [1, 63, 64, 65, 1000, 5000])
def test_nms_kernel_matches_reference(n):
    b, s = _boxes(n, seed=n)
    for thr in (0.3, 0.7):
        got = V.nms(b.cuda(), s.cuda(), thr)
        assert torch.equal(got.cpu(), V.nms_reference(b, s, thr))
    idx = torch.randint(0, 4, (n,), generator=torch.Generator().manual_seed(1))
    assert torch.equal(V.batched_nms(b.cuda(), s.cuda(), idx.cuda(), 0.5).cpu(), V.batched_nms(b, s, idx, 0.5))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("aligned,sampling_ratio", [(False, 2), (True, 2), (True, -1), (False, -1)])
def test_roi_align_kernels_match_reference(dtype, aligned, sampling_ratio):
    torch.manual_seed(3)
    x = torch.randn(3, 5, 38, 50)
    rois = torch.tensor([[0, 1.5, 2.0, 45.0, 30.0], [2, 0.0, 0.0, 99.9, 75.9], [1, -6.0, -4.0, 10.0, 12.0],
                         [1, 80.0, 60.0, 120.0, 100.0], [0, 10.0, 10.0, 10.5, 10.5], [2, 33.3, 21.7, 71.2, 64.9]])
    xr = x.clone().requires_grad_(True)
    yr = V.roi_align_reference(xr, rois, (7, 5), 0.5, sampling_ratio, aligned)
    g = torch.randn_like(yr)
    (gr,) = torch.autograd.grad(yr, xr, g)
    xd = x.cuda().to(dtype).requires_grad_(True)
    y = V.roi_align(xd, rois.cuda(), (7, 5), 0.5, sampling_ratio, aligned)
    (gx,) = torch.autograd.grad(y, xd, g.cuda().to(dtype))
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    assert (y.float().cpu() - yr).abs().max() < tol * max(1.0, yr.abs().max().item())
    assert (gx.float().cpu() - gr).abs().max() < tol * max(1.0, gr.abs().max().item())


def test_batch_image_codecs_round_trip():
    from tensorplay_b200.vision import io as vio
    ims = [torch.randint(0, 255, (3, 32 + i, 40), dtype=torch.uint8) for i in range(5)]
    back = vio.decode_png_batch(vio.encode_png_batch(ims))
    assert all(torch.equal(a, b) for a, b in zip(ims, back))                       # PNG is lossless, order kept
    jp = vio.decode_jpeg_batch(vio.encode_jpeg_batch(ims, quality=95))
    assert [tuple(t.shape) for t in jp] == [tuple(t.shape) for t in ims]
