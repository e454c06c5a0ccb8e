"""Import path of the ``.mega`` storage reader and writer (tensorplay/distributed/checkpoint/mega_storage.py); defined in
``api.py`` on top of the host runtime's container IO."""
from .api import MegaStorageReader, MegaStorageWriter  # noqa: F401
