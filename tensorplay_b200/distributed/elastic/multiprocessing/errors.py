"""Error files of worker processes (tensorplay/distributed/elastic/multiprocessing/errors/__init__.py): the
definitions live in the package's ``__init__``; this module is their import path."""
from . import ERROR_FILE_ENV, ChildFailedError, ProcessFailure, _write_error_file, record  # noqa: F401


import faulthandler as _faulthandler
import json as _json
import os as _os

from . import SignalException  # noqa: E402,F401


class ErrorHandler:
    """What ``record`` does, as an object (errors/error_handler.py in the reference): ``initialize`` turns on the
    fault handler (native crashes print the Python stacks), ``record_exception`` writes the error file,
    ``dump_error_file`` copies a child's root-cause file into this process's own error file."""

    def _error_file(self):
        return _os.environ.get(ERROR_FILE_ENV)

    def initialize(self) -> None:
        try:
            _faulthandler.enable(all_threads=True)
        except Exception:
            pass

    def record_exception(self, e: BaseException) -> None:
        path = self._error_file()
        if path:
            _write_error_file(path, e)

    def dump_error_file(self, rootcause_error_file: str, error_code: int = 0) -> None:
        with open(rootcause_error_file) as f:
            data = _json.load(f)
        if error_code and isinstance(data.get("message"), dict):
            data["message"]["errorCode"] = error_code
        mine = self._error_file()
        if mine:
            with open(mine, "w") as f:
                _json.dump(data, f)


_handler = ErrorHandler()


def get_error_handler() -> ErrorHandler:
    return _handler
