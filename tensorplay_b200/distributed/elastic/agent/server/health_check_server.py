"""Liveness endpoint of an elastic agent: ``GET /`` (or ``/healthz``) answers 200 while the agent's
monitor loop keeps reporting progress and 503 once the last report is older than ``timeout`` seconds,
so that an orchestrator can restart an agent whose loop is wedged
(tensorplay/distributed/elastic/agent/server/health_check_server.py)."""
from __future__ import annotations

import json
import threading
import time
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Callable


class HealthCheckServer:
    def __init__(self, alive_callback: Callable[[], float], port: int, timeout: float, host: str = "127.0.0.1"):
        """``alive_callback()`` returns the time (``time.time()``) of the agent's last sign of life."""
        self._alive, self._timeout = alive_callback, timeout
        outer = self

        class Handler(BaseHTTPRequestHandler):
            def do_GET(self):  # noqa: N802
                age = time.time() - outer._alive()
                ok = age <= outer._timeout
                body = json.dumps({"healthy": ok, "seconds_since_last_report": round(age, 3)}).encode()
                self.send_response(200 if ok else 503)
                self.send_header("Content-Type", "application/json")
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)

            def log_message(self, *a):
                pass

        self._httpd = ThreadingHTTPServer((host, port), Handler)
        self.port = self._httpd.server_address[1]
        self._thread = threading.Thread(target=self._httpd.serve_forever, daemon=True)

    def start(self) -> None:
        self._thread.start()

    def stop(self) -> None:
        self._httpd.shutdown()
        self._httpd.server_close()


def create_healthcheck_server(alive_callback: Callable[[], float], port: int, timeout: float) -> HealthCheckServer:
    return HealthCheckServer(alive_callback, port, timeout)
