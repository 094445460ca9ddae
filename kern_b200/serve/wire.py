"""Control-plane framing between serving processes: little-endian u32 length + JSON body over TCP with
TCP_NODELAY; ``recv`` returns None on a clean close. bytes values travel as hex under ``{"hex": ...}``.
Reference counterpart: crates/kern-serve/src/pp/mod.rs:166-181."""
from __future__ import annotations

import json
import socket
import struct

MAX_FRAME = 1 << 30


def _enc(o):
    if isinstance(o, (bytes, bytearray)):
        return {"hex": bytes(o).hex()}
    if hasattr(o, "tolist"):
        return o.tolist()
    raise TypeError(f"cannot send {type(o).__name__}")


def _dec(d):
    if len(d) == 1 and "hex" in d and isinstance(d["hex"], str):
        return bytes.fromhex(d["hex"])
    return d


def send(sock: socket.socket, obj) -> None:
    body = json.dumps(obj, default=_enc, separators=(",", ":")).encode()
    sock.sendall(struct.pack("<I", len(body)) + body)


def _exact(sock: socket.socket, n: int) -> bytes | None:
    buf = bytearray()
    while len(buf) < n:
        chunk = sock.recv(n - len(buf))
        if not chunk:
            if buf:
                raise ConnectionError("peer closed in the middle of a frame")
            return None
        buf += chunk
    return bytes(buf)


def recv(sock: socket.socket):
    head = _exact(sock, 4)
    if head is None:
        return None
    (n,) = struct.unpack("<I", head)
    if n > MAX_FRAME:
        raise ConnectionError(f"frame of {n} bytes exceeds the limit")
    body = _exact(sock, n) if n else b""
    if body is None:
        raise ConnectionError("peer closed in the middle of a frame")
    return json.loads(body, object_hook=_dec)


def listen(host: str = "127.0.0.1", port: int = 0) -> socket.socket:
    s = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
    s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
    s.bind((host, port))
    s.listen(64)
    return s


def connect(addr: tuple[str, int], timeout: float = 60.0, retry_s: float = 0.05) -> socket.socket:
    import time

    deadline = time.monotonic() + timeout
    while True:
        try:
            s = socket.create_connection(addr, timeout=timeout)
            s.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
            s.settimeout(None)
            return s
        except OSError:
            if time.monotonic() > deadline:
                raise
            time.sleep(retry_s)


def accept(lsock: socket.socket) -> socket.socket:
    s, _ = lsock.accept()
    s.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
    return s
