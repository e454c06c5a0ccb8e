"""Error files of worker processes (tensorplay/distributed/elastic/multiprocessing/errors/__init__.py): the
definitions live in the package's ``__init__``; this module is their import path."""
from . import ERROR_FILE_ENV, ChildFailedError, ProcessFailure, _write_error_file, record  # noqa: F401
