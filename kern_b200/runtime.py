"""``kern_b200.Runtime``: the Python face of the native executor.

Mirrors the reference's Python binding (crates/kern-py/src/lib.rs:47-245): construct from a manifest,
a kernels directory and a checkpoint; ``run`` / ``issue`` programs by name with a var assignment;
``region(name)`` views of runtime memory as torch tensors; ``offer`` / ``connect`` for rank groups;
``bind_host`` / ``enqueue_after`` for engines that own the states (vLLM / SGLang style hosts).
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

import os

from . import _native
from .models.common import KERNELS_DIR

os.environ.setdefault("KERN_B200_KERNELS", str(KERNELS_DIR))     # where a foreign package's `extern:` built-ins are found

_NP = {"bf16": np.uint16, "f16": np.float16, "f32": np.float32, "fp8e4m3": np.uint8, "fp8e8m0": np.uint8, "i8": np.int8,
       "i32": np.int32, "u32": np.uint32, "i64": np.int64, "u64": np.uint64, "u8": np.uint8}
_TORCH = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32, "i8": torch.int8, "i32": torch.int32,
          "i64": torch.int64, "u8": torch.uint8, "fp8e4m3": torch.uint8, "fp8e8m0": torch.uint8, "u32": torch.int32,
          "u64": torch.int64}


class _CudaView:
    """Minimal ``__cuda_array_interface__`` carrier so torch can view runtime memory without a copy."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 3,
                                         "strides": None}


def manifest_text(manifest) -> str:
    if isinstance(manifest, dict):
        return json.dumps(manifest)
    if isinstance(manifest, Path) or (isinstance(manifest, str) and not manifest.lstrip().startswith("{")):
        return Path(manifest).read_text()
    return manifest


def verify(manifest, strict_multicast: bool = False):
    """-> (native manifest | None, [diagnostics])."""
    return _native.verify(manifest_text(manifest), strict_multicast)


class Runtime:
    def __init__(self, manifest, kernels: str | Path | None = None, weights=None, gpu: int = 0,
                 topology: dict[str, tuple[int, int]] | None = None, tokens: int = 0, slots: int = 0,
                 memory_fraction: float = 0.9, stream: int | None = None, guard_bands: bool = False):
        if not _native.cuda_available():
            raise RuntimeError("kern_b200.Runtime needs a CUDA device; use kern_b200.cpu.CpuRuntime on a machine without one")
        text = manifest_text(manifest)
        self.gpu = gpu
        with torch.cuda.device(gpu):
            torch.zeros(1, device="cuda")   # the primary context the runtime shares with torch
            self._stream = torch.cuda.Stream(device=gpu) if stream is None else None
            raw = self._stream.cuda_stream if stream is None else stream
            self._rt = _native.Runtime(text, str(kernels or KERNELS_DIR), gpu, dict(topology or {}), tokens, slots,
                                       memory_fraction, raw, guard_bands)
        self.doc = json.loads(self._rt.manifest_json())
        pj = self._rt.protocol_json()
        self.protocol = json.loads(pj) if pj else None
        self.stream = raw
        if weights is not None:
            self.load_weights(weights)

    # ---- load ----
    def load_weights(self, weights) -> None:
        if isinstance(weights, (str, Path)):
            p = Path(weights)
            paths = sorted(str(x) for x in p.glob("*.safetensors")) if p.is_dir() else [str(p)]
        else:
            paths = [str(x) for x in weights]
        if not paths:
            raise FileNotFoundError(f"no safetensors files under {weights}")
        self._rt.load_weights(paths)

    def load_tensors(self, provider, skip=None) -> None:
        """Bind the weights from tensors already on the device: ``provider(name)`` returns the checkpoint
        tensor of that name (device-to-device copies by segment, the same `bind` rules as a file load).
        ``skip(name)``: a buffer bound only to such tensors is left for the caller to fill."""
        ranks = lambda g: self._rt.rank(g)
        pick = lambda t: t if isinstance(t, str) else t["tensors"][ranks(t["group"])]
        rng = lambda r, whole: (0, whole) if r is None else (tuple(r) if isinstance(r, list) else tuple(r["ranges"][ranks(r["group"])]))
        last = [None, None]          # consecutive segments of one tensor (row ranges) fetch it once

        def fetch(n):
            if last[0] != n:
                last[0], last[1] = n, provider(n)
            return last[1]

        for name, b in self.doc["buffers"].items():
            if b["kind"] not in ("weight", "source") or b.get("placement") == "host":
                continue
            if skip is not None and all(skip(pick(seg["tensor"])) for seg in b["bind"]):
                continue
            dst = self.tensor(name).view(-1)
            at = 0
            for seg in b["bind"]:
                t = fetch(pick(seg["tensor"]))
                t2 = t.reshape(t.shape[0], -1) if t.dim() > 1 else t.reshape(-1, 1)
                if "interleave" in seg:
                    u = provider(pick(seg["interleave"]["with"])).reshape(t2.shape)
                    n = seg["interleave"]["rows"]
                    part = torch.stack([t2.view(-1, n, t2.shape[1]), u.view(-1, n, t2.shape[1])], 1).reshape(-1)
                    del u
                else:
                    r, c = rng(seg.get("rows"), t2.shape[0]), rng(seg.get("cols"), t2.shape[1])
                    part = t2[r[0]:r[1], c[0]:c[1]].reshape(-1)
                if at + part.numel() > dst.numel():
                    raise ValueError(f"buffer `{name}`: bound tensors hold more than the buffer")
                dst[at:at + part.numel()] = part.to(dst.dtype)
                at += part.numel()
                del t, t2, part
            if at != dst.numel():
                raise ValueError(f"buffer `{name}`: bound tensors hold {at} elements, the buffer {dst.numel()}")
        torch.cuda.synchronize(self.gpu)

    def once(self) -> None:
        """Run every `once` program (after every peer is connected)."""
        self._rt.run_once_programs()

    # ---- memory ----
    def region(self, name: str) -> tuple[int, int]:
        return self._rt.region(name)

    def tensor(self, name: str) -> torch.Tensor:
        """Zero-copy torch view of a buffer (declared dtype and var-max shape) or a state (bytes)."""
        ptr, nbytes = self._rt.region(name)
        b = self.doc["buffers"].get(name)
        if b is None:
            return torch.as_tensor(_CudaView(ptr, (nbytes,), "|u1"), device=f"cuda:{self.gpu}")
        shape = [d if isinstance(d, int) else self.doc["vars"][d]["max"] for d in b["shape"]]
        dt = b["dtype"]
        es = np.dtype(_NP[dt]).itemsize
        raw = torch.as_tensor(_CudaView(ptr, (nbytes,), "|u1"), device=f"cuda:{self.gpu}")
        return raw.view(_TORCH[dt]).view(shape) if nbytes == es * int(np.prod(shape)) else raw

    def write(self, name: str, data, offset: int = 0) -> None:
        """Host -> device on the runtime's stream. ``data``: pinned torch tensor (no staging copy), any
        torch CPU tensor, numpy array or bytes."""
        if isinstance(data, torch.Tensor):
            assert data.device.type == "cpu" and data.is_contiguous()
            self._rt.write_input_ptr(name, data.data_ptr(), data.numel() * data.element_size(), offset)
        else:
            self._rt.write_input(name, np.ascontiguousarray(data) if not isinstance(data, (bytes, bytearray)) else data, offset)

    def read(self, name: str, count: int | None = None, offset: int = 0, out: torch.Tensor | None = None):
        """Device -> host of an output (or any buffer); synchronises the runtime's stream."""
        b = self.doc["buffers"][name]
        dt = b["dtype"]
        es = np.dtype(_NP[dt]).itemsize
        if out is not None:
            self._rt.read_output_ptr(name, out.data_ptr(), out.numel() * out.element_size(), offset)
            return out
        total = self._rt.region(name)[1] // es
        n = total if count is None else count
        raw = self._rt.read_output(name, n * es, offset)
        return np.frombuffer(raw, dtype=_NP[dt]).copy()

    # ---- execution ----
    def issue(self, program: str, vars: dict[str, int], eager: bool = False) -> int:
        rec = getattr(self, "_recorder", None)
        if rec is None:
            return self._rt.issue(program, vars, eager)
        import time

        t0 = time.perf_counter()
        n = self._rt.issue(program, vars, eager)
        p = self.protocol or {}
        rows = vars.get((p.get("rows") or {}).get("var"), 0)
        groups = vars.get((p.get("groups") or {}).get("var"), 0)
        ctx = vars.get((p.get("context") or {}).get("var"), 0) if p.get("context") else 0
        graph = bool(self.doc["programs"][program].get("graph")) and not eager
        rec.step(program, groups, rows, ctx, graph, 0.0, (time.perf_counter() - t0) * 1e6, n)
        return n

    def issue_range(self, program: str, vars: dict[str, int], lo: int, hi: int) -> int:
        """Calls [lo, hi) of `program`, eagerly and in order (what activation probes step a program with)."""
        return self._rt.issue_range(program, vars, lo, hi)

    def record(self, directory, rank: int = 0):
        """Start recording every issued step into Parquet traces under `directory` (see `kern_b200.trace`); returns the
        recorder (`rotate()` writes what is buffered, `record(None)` stops)."""
        if directory is None:
            rec, self._recorder = getattr(self, "_recorder", None), None
            if rec is not None:
                rec.rotate()
            return None
        from .trace import Recorder

        self._recorder = Recorder(directory, rank)
        return self._recorder

    def issue_timed(self, program: str, vars: dict[str, int]):
        """One eager run with an event between calls: [(label, op, ms, launches)] in call order."""
        return self._rt.issue_timed(program, vars)

    def run(self, program: str, vars: dict[str, int]) -> int:
        return self._rt.run(program, vars)

    def enqueue_after(self, program: str, vars: dict[str, int], stream: int) -> int:
        return self._rt.enqueue_after(program, vars, stream)

    def synchronize(self) -> None:
        self._rt.synchronize()

    # ---- stream-ordered signals between the device and the host (or another stream, stage or process) ----
    def _signals(self):
        from .ops.launcher import Kernels

        return Kernels.get(torch.device(f"cuda:{self.gpu}"))

    def mark(self) -> "Mark":
        """Enqueue a mark: once everything issued so far on the runtime's stream has run, the device writes the mark's
        sequence number into a pinned host word; `Mark.wait()` is the host's side (a deadline, no stream
        synchronisation). Reference: crates/kern-runtime/src/exec.rs:67-97."""
        import struct

        from .ops.launcher import ptr

        m = getattr(self, "_mark_word", None)
        if m is None:
            m = self._mark_word = torch.zeros(1, dtype=torch.int64, pin_memory=True)
            self._mark_seq = 0
        self._mark_seq += 1
        self._signals().launch("signals", "kern_mark", (1,), (32,), [ptr(m), struct.pack("<Q", self._mark_seq)], stream=self.stream)
        return Mark(m, self._mark_seq)

    def gate(self) -> "Gate":
        """A counter in pinned host memory that the host (or a peer's copy) advances and `hold` waits on."""
        return Gate(torch.zeros(1, dtype=torch.int64, pin_memory=True))

    def hold(self, gate: "Gate", want: int, timeout_s: float = 60.0, code: int = 901) -> None:
        """Enqueue a wait on the runtime's stream: what is issued after it runs once `gate` has been opened `want` times.
        The wait is bounded: after `timeout_s` it sets the error word to `code` and lets the stream go on
        (the host sees the error at its next `check_error`). Reference: exec.rs:103-113, 135-164."""
        import struct

        from .ops.launcher import i32, i64, ptr

        err = self._rt.region(self._error_name())[0] if self._error_name() else 0
        self._signals().launch("signals", "kern_hold", (1,), (32,),
                               [ptr(gate.word), struct.pack("<Q", want), i64(int(timeout_s * 1e9)), struct.pack("<Q", err), i32(code)],
                               stream=self.stream)

    def _error_name(self):
        for f in (self.protocol or {}).get("fills", []):
            if f["fill"] == "error":
                return f["name"]
        return "error" if "error" in self.doc["buffers"] else None

    def fetch(self, name: str, count: int | None = None) -> "Fetch":
        """Start reading an output into a pinned buffer of the runtime's pool, behind what is issued so far; the result
        is taken with `Fetch.get()`, which waits on a mark, not on the stream (later work may already be queued).
        Reference: exec.rs:257-277."""
        b = self.doc["buffers"][name]
        src = self.tensor(name).view(-1)
        n = src.numel() if count is None else count
        pool = self.__dict__.setdefault("_fetch_pool", {})
        free = pool.setdefault((name, n), [])
        dst = free.pop() if free else torch.empty(n, dtype=src.dtype, pin_memory=True)
        with torch.cuda.stream(torch.cuda.ExternalStream(self.stream, device=f"cuda:{self.gpu}")):
            dst.copy_(src[:n], non_blocking=True)
        return Fetch(dst, self.mark(), free, b["dtype"])

    def check_error(self) -> None:
        for f in (self.protocol or {}).get("fills", []):
            if f["fill"] == "error":
                code = int(self.read(f["name"], 1)[0])
                if code:
                    raise RuntimeError(f"device error word `{f['name']}` = {code}")
        if self._rt.checked:          # a checked kernel build: accesses it refused since the last call
            caught = list(self._rt.checked_failures())
            if caught:
                raise RuntimeError("checked kernels skipped accesses: " + "; ".join(caught))

    # ---- pool support ----
    def zero_slot(self, slot: int) -> None:
        self._rt.zero_slot(slot)

    def run_copies(self, copies: dict) -> None:
        """Execute a pool copy plan (half pages are copied whole: the tail rows are dead to the holder)."""
        if copies["pages"]:
            self._rt.copy_pages(list(copies["pages"]))
        if copies["slot"] is not None:
            self._rt.copy_slot(*copies["slot"])

    # ---- groups ----
    # ---- another process's pool (prefill tier -> decode tier) ----
    def export_states(self) -> dict[str, bytes]:
        """A handle per state of this runtime's pools, for a process that will push pages and slots into them."""
        return {name: self._rt.export_region(name) for name in self.doc["states"]}

    def map_pool(self, handles: dict[str, bytes]) -> dict[str, int]:
        """Map another process's exported states; the result goes to `push`."""
        return {name: self._rt.import_region(h) for name, h in handles.items()}

    def push(self, mapped: dict[str, int], plan: dict) -> None:
        """Run a push plan (`serve.pd.moves`): whole pages of every paged state, the slot of every per-sequence one,
        from this runtime's pools into the mapped ones, on this runtime's stream (one device copy per unit)."""
        for name, s in self.doc["states"].items():
            if s.get("bytes_per_token"):
                for a, b in plan["pages"]:
                    self._rt.push_unit(name, mapped[name], a, b)
            elif s.get("bytes_per_seq") and plan.get("slot") is not None:
                self._rt.push_unit(name, mapped[name], plan["slot"][0], plan["slot"][1])

    def state_bytes(self) -> dict[str, int]:
        """Bytes of every state's pool as allocated here (what a peer that maps them checks its copies against)."""
        return {name: int(self._rt.region(name)[1]) for name in self.doc["states"]}

    def push_state_unit(self, state: str, dst_ptr: int, src_unit: int, dst_unit: int) -> None:
        """One page or slot of `state` into the same-shaped mapped pool at `dst_ptr`."""
        self._rt.push_unit(state, dst_ptr, src_unit, dst_unit)

    def push_rows(self, state: str, dst_ptr: int, dst_bytes: int, runs, row_bytes: int) -> int:
        """The dealt rows of a paged state (runs of `kern_pool.deal`: source rows a group width apart, destination rows
        contiguous) into a mapped pool, as strided copies of at most 64 KiB. Reference: crates/kern-runtime/src/push.rs:400-434."""
        copies = _native.dealt_copies([tuple(r) for r in runs], row_bytes)
        self._rt.push_copies(state, 0, dst_ptr, dst_bytes, copies)
        return len(copies)

    def push_slot_part(self, state: str, dst_ptr: int, dst_bytes: int, from_slot: int, into_slot: int, segments, of: int,
                       part: int) -> int:
        """Member `part`'s columns of slot `from_slot` of a per-sequence state into slot `into_slot` of a mapped pool whose
        slots are 1/`of` the size (a decode group that shards the state by heads). `segments`: what a line of the slot
        holds, (rows, width bytes) each. Reference: crates/kern-runtime/src/push.rs:365-398."""
        mine = int(self.doc["states"][state]["bytes_per_seq"])
        line = _native.split_line(list(segments), of)
        if mine % line or mine % of:
            raise ValueError(f"state `{state}`: a slot of {mine} bytes is not whole lines of {line} bytes over {of} members")
        theirs = mine // of
        copies = _native.split_copies(list(segments), of, mine // line, part)
        self._rt.push_copies(state, from_slot * mine, dst_ptr + into_slot * theirs, dst_bytes - into_slot * theirs, copies)
        return len(copies)

    def export_buffers(self, names) -> dict[str, bytes]:
        """Handles of buffers another process will write (a pipeline stage's landing buffers)."""
        return {n: self._rt.export_region(n) for n in names}

    def push_bytes(self, name: str, dst_ptr: int, nbytes: int) -> None:
        """The first `nbytes` of buffer `name` into mapped memory of another process, on this runtime's stream."""
        self._rt.push_bytes(name, dst_ptr, nbytes)

    def check_guards(self) -> list[str]:
        """With `guard_bands=True` (test mode): the allocations whose canary bands were written over since load —
        "name (before)" / "name (after)" — the sign of a kernel that wrote outside its buffer without faulting."""
        return list(self._rt.check_guards())

    def rank(self, group: str) -> int:
        return self._rt.rank(group)

    def offer(self) -> dict[str, bytes]:
        return dict(self._rt.export_handles())

    def connect(self, group: str, members: list[dict[str, bytes]]) -> None:
        self._rt.connect(group, members)

    # ---- hosted ----
    @property
    def awaits_host(self) -> bool:
        return self._rt.awaits_host

    def bind_host(self, regions: dict[str, tuple[int, str, list[int], list[int]]]) -> None:
        self._rt.bind_host(regions)

    # ---- facts ----
    page_unit = property(lambda self: self._rt.page_unit)
    pages = property(lambda self: self._rt.pages)
    slots = property(lambda self: self._rt.slots)
    launches_total = property(lambda self: self._rt.launches_total)
    graphs = property(lambda self: self._rt.graphs)

    def banner(self) -> str:
        return self._rt.banner()


class Mark:
    """A point of the runtime's stream the host can wait for without synchronising the stream."""

    def __init__(self, word: torch.Tensor, seq: int):
        self.word, self.seq = word, seq

    def done(self) -> bool:
        return int(self.word[0]) >= self.seq

    def wait(self, timeout_s: float = 60.0) -> None:
        import time

        deadline = time.monotonic() + timeout_s
        while not self.done():
            if time.monotonic() > deadline:
                raise TimeoutError(f"mark {self.seq} did not land within {timeout_s:.0f} s (the device reached {int(self.word[0])})")
            time.sleep(0.00005)


class Gate:
    def __init__(self, word: torch.Tensor):
        self.word = word

    def open(self, n: int = 1) -> None:
        """Advance the count the device-side `hold` polls (a plain host store to pinned memory)."""
        self.word[0] += n

    @property
    def count(self) -> int:
        return int(self.word[0])


class Fetch:
    def __init__(self, buf: torch.Tensor, mark: Mark, free: list, dtype: str):
        self.buf, self.mark, self._free, self.dtype = buf, mark, free, dtype

    def get(self, timeout_s: float = 60.0) -> np.ndarray:
        self.mark.wait(timeout_s)
        out = self.buf.numpy().copy() if self.dtype != "bf16" else self.buf.view(torch.int16).numpy().copy()
        self._free.append(self.buf)
        return out
