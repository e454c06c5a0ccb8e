"""Live debug endpoint of a rank: an HTTP server on 127.0.0.1 that returns the Python stacks of
every thread, the flight-recorder ring of collectives and the device status word
(tensorplay/distributed/debug/__init__.py). Started explicitly or with ``TP_DEBUG_SERVER_PORT``."""
from __future__ import annotations

import faulthandler
import io
import json
import os
import sys
import tempfile
import threading
import traceback
from http.server import BaseHTTPRequestHandler, HTTPServer
from typing import Optional

_server: Optional[HTTPServer] = None


def dump_stacks() -> str:
    """Python stack of every thread of this process."""
    out = io.StringIO()
    frames = sys._current_frames()
    for t in threading.enumerate():
        out.write(f"--- thread {t.name} ({t.ident})\n")
        fr = frames.get(t.ident)
        if fr is not None:
            out.write("".join(traceback.format_stack(fr)))
    return out.getvalue()


def dump_native_stacks() -> str:
    """faulthandler's view (also shows threads blocked inside native calls)."""
    with tempfile.TemporaryFile(mode="w+") as f:
        faulthandler.dump_traceback(file=f, all_threads=True)
        f.seek(0)
        return f.read()


class DebugHandler:
    """One endpoint of the debug server: ``path`` prefix, content type and ``handle() -> str``."""

    path = "/"
    content_type = "text/plain"

    def handle(self, request_path: str) -> str:
        raise NotImplementedError


class StacksHandler(DebugHandler):
    path = "/stacks"

    def handle(self, request_path: str) -> str:
        return dump_stacks()


class NativeStacksHandler(DebugHandler):
    path = "/native"

    def handle(self, request_path: str) -> str:
        return dump_native_stacks()


class FlightRecorderHandler(DebugHandler):
    path, content_type = "/flight", "application/json"

    def handle(self, request_path: str) -> str:
        from .. import flight_recorder
        return json.dumps({"rank": os.environ.get("RANK"), "entries": flight_recorder.entries()})


class StoreDumpHandler(DebugHandler):
    """Keys of a store registered with :func:`register_store` (values are not dumped)."""

    path, content_type = "/store", "application/json"
    store = None

    def handle(self, request_path: str) -> str:
        st = type(self).store
        if st is None:
            return json.dumps({"error": "no store registered"})
        n = st.num_keys() if hasattr(st, "num_keys") else None
        return json.dumps({"num_keys": n, "type": type(st).__name__})


class IndexHandler(DebugHandler):
    path, content_type = "/", "application/json"

    def handle(self, request_path: str) -> str:
        return json.dumps({"pid": os.getpid(), "rank": os.environ.get("RANK"), "endpoints": list_handlers()})


_handlers = {}


def register_handler(handler: DebugHandler) -> None:
    """Add (or replace) the endpoint at ``handler.path``."""
    _handlers[handler.path] = handler


def list_handlers():
    return sorted(p for p in _handlers if p != "/")


def default_handlers():
    return [StacksHandler(), NativeStacksHandler(), FlightRecorderHandler(), StoreDumpHandler(), IndexHandler()]


def register_store(store) -> None:
    StoreDumpHandler.store = store


for _h in default_handlers():
    register_handler(_h)


class _Handler(BaseHTTPRequestHandler):
    def log_message(self, *a):  # silence
        pass

    def do_GET(self):  # noqa: N802
        best = max((p for p in _handlers if p != "/" and self.path.startswith(p)), key=len, default="/")
        h = _handlers[best]
        try:
            body, ctype, code = h.handle(self.path), h.content_type, 200
        except Exception as e:  # a handler must not take the server down
            body, ctype, code = json.dumps({"error": repr(e)}), "application/json", 500
        data = body.encode()
        self.send_response(code)
        self.send_header("Content-Type", ctype)
        self.send_header("Content-Length", str(len(data)))
        self.end_headers()
        self.wfile.write(data)


def start_debug_server(port: int = 0) -> int:
    """Start (once) the endpoint on 127.0.0.1; returns the bound port."""
    global _server
    if _server is None:
        _server = HTTPServer(("127.0.0.1", port), _Handler)
        threading.Thread(target=_server.serve_forever, name="tp-debug-server", daemon=True).start()
    return _server.server_address[1]


def stop_debug_server() -> None:
    global _server
    if _server is not None:
        _server.shutdown()
        _server.server_close()
        _server = None


if os.environ.get("TP_DEBUG_SERVER_PORT"):
    start_debug_server(int(os.environ["TP_DEBUG_SERVER_PORT"]))
