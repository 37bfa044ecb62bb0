"""A line writer that appends to a (possibly remote, mounted) file from a background thread
(reference: axlearn/cloud/common/writer.py:30-147): callers ``write()`` without ever waiting for
the file system; lines are flushed every ``flush_seconds`` and on exit.  Used to tee job output
to the shared output directory."""

from __future__ import annotations

import os
import queue
import sys
import threading
from typing import Optional


class BaseWriter:
    def write(self, data: str):
        raise NotImplementedError(type(self))


class FileWriter(BaseWriter):
    def __init__(self, *, output_path: str, flush_seconds: float = 1.0):
        self._output_path = output_path
        self._flush_seconds = flush_seconds
        self._queue: "queue.Queue[str]" = queue.Queue()
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._file = None
        self.flush_count = 0

    def __enter__(self):
        self._stop.clear()
        self._thread = threading.Thread(target=self._flush_loop, name="writer-flush", daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *args) -> Optional[bool]:
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
            self._thread = None
        self._drain()
        if self._file is not None:
            self._file.close()
            self._file = None
        return None

    def _drain(self):
        chunks = []
        while True:
            try:
                chunks.append(self._queue.get_nowait())
            except queue.Empty:
                break
        if not chunks:
            return
        if self._file is None:
            os.makedirs(os.path.dirname(os.path.abspath(self._output_path)), exist_ok=True)
            self._file = open(self._output_path, "a", encoding="utf-8")  # pylint: disable=consider-using-with
        self._file.write("".join(chunks))
        self._file.flush()
        self.flush_count += 1

    def _flush_loop(self):
        while not self._stop.wait(self._flush_seconds):
            self._drain()

    def write(self, data: str):
        if self._thread is None:
            raise ValueError("write() outside of the writer's context")
        self._queue.put(data)


def main(argv=None):
    """``python -m axlearn_b200.cloud.common.writer OUTPUT_PATH``: copies stdin to stdout and to
    the file (what the bastion pipes a job's output through)."""
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) != 1:
        raise SystemExit("usage: writer OUTPUT_PATH")
    with FileWriter(output_path=argv[0]) as w:
        for line in sys.stdin:
            sys.stdout.write(line)
            sys.stdout.flush()
            w.write(line)


if __name__ == "__main__":
    main()
