"""Tiny HTTP endpoint that dumps the stacks of all Python threads of this process.

Parity target in the reference: ``StatusHTTPServer`` (axlearn/common/status_server.py): started
by the trainer launcher so that a stuck job can be inspected with ``curl host:port``.
"""

from __future__ import annotations

import http.server
import threading
from typing import Optional

from axlearn_b200.common.utils import thread_stack_traces


class _Handler(http.server.BaseHTTPRequestHandler):
    def do_GET(self):  # pylint: disable=invalid-name
        body = "\n\n".join("\n".join(t) for t in thread_stack_traces()).encode()
        self.send_response(200)
        self.send_header("Content-Type", "text/plain; charset=utf-8")
        self.send_header("Content-Length", str(len(body)))
        self.end_headers()
        self.wfile.write(body)

    def log_message(self, *args):  # Quiet.
        del args


class StatusHTTPServer:
    def __init__(self, port: int, host: str = "127.0.0.1"):
        self._addr = (host, port)
        self._server: Optional[http.server.ThreadingHTTPServer] = None
        self._thread: Optional[threading.Thread] = None

    @property
    def port(self) -> int:
        return self._server.server_address[1] if self._server is not None else self._addr[1]

    def start(self) -> None:
        self._server = http.server.ThreadingHTTPServer(self._addr, _Handler)
        self._thread = threading.Thread(target=self._server.serve_forever, name="status-server", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        if self._server is not None:
            self._server.shutdown()
            self._server.server_close()
            self._server = None
