"""``vision``: the detection operators with kernels of this framework (``vision.ops``: ``nms``, ``batched_nms``,
``box_iou``, ``box_area``, ``roi_align`` / ``RoIAlign``); models, transforms, datasets, io and the remaining operators
resolve to torchvision when it is installed (tensorplay/vision/**)."""
from . import io, ops  # noqa: F401


def __getattr__(name):
    import importlib
    try:
        tv = importlib.import_module("torchvision")
    except ImportError as e:
        raise AttributeError(f"tensorplay_b200.vision.{name}: torchvision is not installed") from e
    try:
        return getattr(tv, name)
    except AttributeError:
        pass
    # helpers that the reference lists at the top of the pack: image grids and saving, tensor conversion
    for mod in ("torchvision.utils", "torchvision.transforms.functional", "torchvision.io"):
        m = importlib.import_module(mod)
        if hasattr(m, name):
            return getattr(m, name)
    aliases = {"from_image": ("torchvision.transforms.functional", "pil_to_tensor"),
               "from_file": ("torchvision.io", "read_image"),
               "set_backend": ("torchvision", "set_image_backend"), "get_backend": ("torchvision", "get_image_backend")}
    if name in aliases:
        mod, attr = aliases[name]
        return getattr(importlib.import_module(mod), attr)
    try:
        return importlib.import_module(f"torchvision.{name}")
    except ImportError:
        raise AttributeError(f"tensorplay_b200.vision has no attribute {name!r}") from None

from .. import _views as _views  # noqa: E402

_views.install(__name__, max_depth=1,
               names=("backend",))
