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


class _Handler(BaseHTTPRequestHandler):
    def log_message(self, *a):  # silence
        pass

    def do_GET(self):  # noqa: N802
        if self.path.startswith("/stacks"):
            body, ctype = dump_stacks(), "text/plain"
        elif self.path.startswith("/native"):
            body, ctype = dump_native_stacks(), "text/plain"
        elif self.path.startswith("/flight"):
            from .. import flight_recorder
            body, ctype = json.dumps(flight_recorder.dump()), "application/json"
        else:
            body, ctype = json.dumps({"pid": os.getpid(), "rank": os.environ.get("RANK"),
                                      "endpoints": ["/stacks", "/native", "/flight"]}), "application/json"
        data = body.encode()
        self.send_response(200)
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
