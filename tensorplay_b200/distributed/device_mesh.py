"""``DeviceMesh`` / ``init_device_mesh``: n-D named meshes with lazily created sub-groups
(torch's implementation; API as in tensorplay/distributed/device_mesh.py:89-681)."""
from torch.distributed.device_mesh import DeviceMesh, init_device_mesh  # noqa: F401

__all__ = ["DeviceMesh", "init_device_mesh"]
