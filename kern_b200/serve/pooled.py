"""A pooled KV tier behind the local prefix cache: whole pages, content-addressed, shared by every engine that can
reach the store. A page's key is a hash chain over the tokens up to and including it (and a salt naming the model and
page geometry), so equal keys mean equal prefixes. An admitted prompt first takes what the local prefix cache has, then
probes the tier for the pages that follow and fetches the longest present run into its fresh lease; a finished request
puts its full pages. Stores: `MemoryTier` (in-process, bounded) and `SsdTier` (one unlinked arena file used as a ring of
fixed-size chunks, positional reads and writes, never trusts a stored size).
Reference counterpart: crates/kern-pool/src/pooled.rs (keys, Probe, objects), crates/kern-serve/src/pool/mod.rs:46-150,
pool/ssd.rs:61-220 (arena ring), scheduler.rs:625-755 (probe / fetch / put around admission).
"""
from __future__ import annotations

import hashlib
import os
import struct
import tempfile
import threading
from collections import OrderedDict


def page_keys(tokens: list[int], unit: int, salt: bytes = b"") -> list[bytes]:
    """One 32-byte key per full page of `tokens`: key_i = sha256(key_{i-1} || page i's tokens)."""
    keys, prev = [], hashlib.sha256(b"kern-pooled-v1" + salt).digest()
    for p in range(len(tokens) // unit):
        h = hashlib.sha256(prev)
        h.update(struct.pack(f"<{unit}q", *tokens[p * unit:(p + 1) * unit]))
        prev = h.digest()
        keys.append(prev)
    return keys


class MemoryTier:
    def __init__(self, capacity_pages: int = 1 << 16):
        self.cap = capacity_pages
        self.store: OrderedDict[bytes, bytes] = OrderedDict()
        self.lock = threading.Lock()

    def probe(self, keys: list[bytes]) -> int:
        """How many leading keys are present (a run: the first miss ends it)."""
        with self.lock:
            n = 0
            for k in keys:
                if k not in self.store:
                    break
                n += 1
            return n

    def put(self, key: bytes, data: bytes) -> None:
        with self.lock:
            self.store[key] = bytes(data)
            self.store.move_to_end(key)
            while len(self.store) > self.cap:
                self.store.popitem(last=False)

    def get(self, key: bytes) -> bytes | None:
        with self.lock:
            d = self.store.get(key)
            if d is not None:
                self.store.move_to_end(key)
            return d


class SsdTier:
    """A ring of `chunks` fixed-size chunks in one arena file. The newest write overwrites the oldest chunk; the index
    (key -> chunk, generation) lives in memory, and every chunk starts with a header (magic, key, length, checksum)
    that a read verifies before trusting anything."""

    MAGIC = b"KRNCHNK1"
    HEADER = 8 + 32 + 8 + 32

    def __init__(self, directory: str, chunk_bytes: int, chunks: int):
        self.chunk = self.HEADER + chunk_bytes
        self.payload = chunk_bytes
        self.chunks = chunks
        fd, path = tempfile.mkstemp(prefix="kern-arena-", dir=directory)
        os.unlink(path)                      # the arena disappears with the process
        os.ftruncate(fd, self.chunk * chunks)
        self.fd = fd
        self.index: dict[bytes, int] = {}
        self.owner: list[bytes | None] = [None] * chunks
        self.head = 0
        self.lock = threading.Lock()
        self.reads = self.writes = self.corrupt = 0

    def probe(self, keys: list[bytes]) -> int:
        with self.lock:
            n = 0
            for k in keys:
                if k not in self.index:
                    break
                n += 1
            return n

    def put(self, key: bytes, data: bytes) -> None:
        if len(data) != self.payload:
            raise ValueError(f"a chunk holds {self.payload} bytes, not {len(data)}")
        with self.lock:
            if key in self.index:
                return
            at = self.head
            self.head = (self.head + 1) % self.chunks
            old = self.owner[at]
            if old is not None:
                self.index.pop(old, None)
            self.owner[at] = key
            self.index[key] = at
        head = self.MAGIC + key + struct.pack("<Q", len(data)) + hashlib.sha256(data).digest()
        os.pwrite(self.fd, head + data, at * self.chunk)
        self.writes += 1

    def get(self, key: bytes) -> bytes | None:
        with self.lock:
            at = self.index.get(key)
        if at is None:
            return None
        raw = os.pread(self.fd, self.chunk, at * self.chunk)
        self.reads += 1
        magic, k, (n,), digest = raw[:8], raw[8:40], struct.unpack("<Q", raw[40:48]), raw[48:80]
        data = raw[self.HEADER:self.HEADER + self.payload]
        if magic != self.MAGIC or k != key or n != self.payload or hashlib.sha256(data).digest() != digest:
            self.corrupt += 1               # overwritten since the lookup, or damaged: a miss, never wrong bytes
            with self.lock:
                if self.index.get(key) == at:
                    self.index.pop(key, None)
            return None
        return data

    def close(self) -> None:
        os.close(self.fd)


class PagedStates:
    """Reads and writes whole pages of every paged state of a runtime (one page = that page of every layer)."""

    def __init__(self, rt):
        self.rt = rt
        self.unit = rt.page_unit
        self.states = [(n, s["bytes_per_token"] * self.unit) for n, s in rt.doc["states"].items() if s.get("bytes_per_token")]
        self.stateful = any(s.get("bytes_per_seq") for s in rt.doc["states"].values())
        self.page_bytes = sum(b for _, b in self.states)

    def _flat(self, name):
        t = self.rt.tensor(name)
        return t.view(-1) if t.dtype.itemsize == 1 else t.view(-1).view(__import__("torch").uint8)

    def read(self, page: int) -> bytes:
        parts = []
        for name, n in self.states:
            parts.append(self._flat(name)[page * n:(page + 1) * n].cpu().numpy().tobytes())
        return b"".join(parts)

    def write(self, page: int, data: bytes) -> None:
        import numpy as np
        import torch

        at = 0
        for name, n in self.states:
            src = torch.from_numpy(np.frombuffer(data, np.uint8, n, at).copy())
            flat = self._flat(name)
            flat[page * n:(page + 1) * n] = src.to(flat.device)
            at += n


class PooledCache:
    """What the scheduler calls: `fetch` into a fresh lease after admission, `put` when a request finishes."""

    def __init__(self, rt, tier, salt: bytes = b""):
        self.pages = PagedStates(rt)
        self.tier = tier
        self.unit = self.pages.unit
        self.salt = salt + rt.doc.get("model", "").encode() + struct.pack("<II", self.unit, self.pages.page_bytes)
        self.enabled = not self.pages.stateful and bool(self.pages.states)
        self.fetched_pages = self.put_pages = self.probes = 0

    def fetch(self, prompt: list[int], have: int, lease_pages: list[int], at_most: int) -> int:
        """Pages of `prompt` beyond the first `have` tokens that the tier holds are copied into the lease's pages;
        returns the new count of tokens present (a multiple of the page size, never past `at_most`)."""
        if not self.enabled or have % self.unit:
            return have
        keys = page_keys(prompt[: at_most // self.unit * self.unit], self.unit, self.salt)
        first = have // self.unit
        if first >= len(keys):
            return have
        self.probes += 1
        # the chain makes key i depend on every earlier page, so a run may start anywhere
        n = self.tier.probe(keys[first:])
        got = 0
        for i in range(first, first + n):
            data = self.tier.get(keys[i])
            if data is None:
                break
            self.pages.write(lease_pages[i], data)
            got += 1
        self.fetched_pages += got
        return have + got * self.unit

    def put(self, tokens: list[int], page_ids: list[int], skip_pages: int = 0) -> int:
        if not self.enabled:
            return 0
        keys = page_keys(tokens, self.unit, self.salt)
        n = 0
        for i, k in enumerate(keys):
            if i < skip_pages or i >= len(page_ids):
                continue
            if self.tier.probe([k]):
                continue
            self.tier.put(k, self.pages.read(page_ids[i]))
            n += 1
        self.put_pages += n
        return n
