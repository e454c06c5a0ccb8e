"""``vision``: the detection operators with kernels of this framework (``vision.ops``: ``nms``, ``batched_nms``,
``box_iou``, ``box_area``, ``roi_align`` / ``RoIAlign``); models, transforms, datasets, io and the remaining operators
resolve to torchvision when it is installed (tensorplay/vision/**)."""
from . import ops  # noqa: F401


def __getattr__(name):
    import importlib
    try:
        tv = importlib.import_module("torchvision")
    except ImportError as e:
        raise AttributeError(f"tensorplay_b200.vision.{name}: torchvision is not installed") from e
    try:
        return getattr(tv, name)
    except AttributeError:
        return importlib.import_module(f"torchvision.{name}")

from .. import _views as _views  # noqa: E402

_views.install(__name__, max_depth=1)
