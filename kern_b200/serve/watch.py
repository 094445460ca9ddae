"""Fail-fast: a thread peeks on every peer control connection; a closed peer ends this process, so a rank
that died takes its group down at once instead of leaving the others inside a collective.
Reference counterpart: crates/kern-serve/src/watch.rs:22-39."""
from __future__ import annotations

import logging
import os
import select
import socket
import threading

log = logging.getLogger("kern.serve")


class Watch:
    def __init__(self, on_lost=None, interval: float = 0.2):
        self._socks: dict[socket.socket, str] = {}
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self.on_lost = on_lost or self._exit
        self.interval = interval
        self._thread = threading.Thread(target=self._run, name="kern-watch", daemon=True)
        self._thread.start()

    @staticmethod
    def _exit(who: str) -> None:
        log.error("peer lost who=%s", who)
        os._exit(1)

    def add(self, sock: socket.socket, who: str) -> None:
        with self._lock:
            self._socks[sock] = who

    def remove(self, sock: socket.socket) -> None:
        with self._lock:
            self._socks.pop(sock, None)

    def stop(self) -> None:
        self._stop.set()

    def _run(self) -> None:
        while not self._stop.wait(self.interval):
            with self._lock:
                socks = dict(self._socks)
            if not socks:
                continue
            try:
                ready, _, _ = select.select(list(socks), [], [], 0)
            except (OSError, ValueError):
                ready = list(socks)
            for s in ready:
                try:
                    closed = s.recv(1, socket.MSG_PEEK | socket.MSG_DONTWAIT) == b""
                except (BlockingIOError, InterruptedError):
                    closed = False
                except OSError:
                    closed = True
                if closed:
                    self.remove(s)
                    self.on_lost(socks[s])
