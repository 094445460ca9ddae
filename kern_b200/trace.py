"""Step and kernel traces as Parquet, NVML counters, and the hooks that feed them.

Files: ``<dir>/date=YYYY-MM-DD/rank=<q>/HHMMSS.{steps,kernels,counters}.parquet`` (zstd). A file holds what was
recorded since the last rotate; ``rotate()`` closes the open batch (a quarter-hour timer or ``POST /kern/trace/rotate``).

  steps     seq, t_ns, program, groups, rows, context, graph, device_us, host_us, launches
  kernels   seq, call, label, op, start_us, end_us, launches          (per labelled call of a timed step)
  counters  t_ns, sm_mhz, mem_mhz, gpu_util, mem_util, power_w        (read-only NVML samples)

Timing is by CUDA events on the runtime's stream (device time) — a software-timestamp path that needs no profiler
attached. ``kern workload`` turns steps.parquet into a weighted bench workload.
Reference counterpart: crates/kern-trace/src/lib.rs:154-204 (schemas), :286-390 (Recorder),
crates/kern-runtime/src/trace.rs:226-283 (folding launches into steps), crates/kern-runtime/src/counters.rs:93-214.
"""
from __future__ import annotations

import threading
import time
from datetime import datetime, timezone
from pathlib import Path

STEP_FIELDS = ("seq", "t_ns", "program", "groups", "rows", "context", "graph", "device_us", "host_us", "launches")
KERNEL_FIELDS = ("seq", "call", "label", "op", "start_us", "end_us", "launches")
# sm_active / tensor_active / dram_bw: per mille of peak over the sampling interval, from the driver's performance
# monitoring samples (NVML GPM: SM utilisation, any-tensor-pipe utilisation, DRAM bandwidth utilisation); -1 where the
# device or the driver does not offer them
COUNTER_FIELDS = ("t_ns", "sm_mhz", "mem_mhz", "gpu_util", "mem_util", "power_w", "sm_active_pm", "tensor_active_pm", "dram_bw_pm")


def shape_of(groups: int, rows: int) -> str:
    """The shape class a step is counted under: decode (one row per sequence), round (a few), prefill (many)."""
    per = rows / max(1, groups)
    return "decode" if per <= 1 else ("round" if per <= 16 else "prefill")


def comm_ops(doc: dict) -> set[str]:
    """The ops of a manifest that count as communication on the kernels board: a launch that is one of the
    `extern:nccl_*` built-ins, or a call that is handed a `peer` buffer (the table of a buffer's copies on the other
    ranks). Reference: crates/kern-serve/src/kernels.rs:141-150."""
    peers = {n for n, b in doc.get("buffers", {}).items() if b.get("kind") == "peer"}
    out = {name for name, op in doc.get("ops", {}).items()
           if any(str(l.get("entry", "")).startswith("extern:nccl") for l in op.get("impl", {}).get("launches", []))}
    for prog in doc.get("programs", {}).values():
        for c in prog.get("calls", []):
            if any(a.get("buf") in peers for a in c.get("args", []) if isinstance(a, dict)):
                out.add(c["op"])
    return out


class Recorder:
    def __init__(self, directory: str | Path, rank: int = 0, clock=time.time_ns, comm: set[str] | None = None):
        """`comm`: the ops whose time is communication (`comm_ops(doc)`); sampled steps split their device time by it."""
        self.dir, self.rank, self.clock = Path(directory), rank, clock
        self._lock = threading.Lock()
        self._rows = {"steps": [], "kernels": [], "counters": []}
        self.seq = 0
        self.dropped = 0
        self.written: list[Path] = []
        self.comm = set(comm or ())
        # the kernels board's running totals (never reset by a rotate)
        self.steps_by: dict[tuple[str, str], int] = {}             # (program, shape) -> steps
        self.device_seconds = {"compute": 0.0, "comm": 0.0}
        self.comm_share = 0.0                                       # of the sampled steps' device time
        self._sampled = [0.0, 0.0]                                  # [comm ms, all ms] over the sampled steps
        self.started = time.monotonic()

    # ---- feeding ----
    def step(self, program: str, groups: int, rows: int, context: int, graph: bool, device_us: float, host_us: float,
             launches: int, calls=None) -> int:
        """One runtime call. `calls`: [(label, op, ms, launches)] of a timed (eager, per-call events) step."""
        with self._lock:
            self.seq += 1
            seq = self.seq
            self._rows["steps"].append((seq, self.clock(), program, groups, rows, context, bool(graph), float(device_us),
                                        float(host_us), int(launches)))
            key = (program, shape_of(groups, rows))
            self.steps_by[key] = self.steps_by.get(key, 0) + 1
            at = 0.0
            for i, (label, op, ms, n) in enumerate(calls or []):
                self._rows["kernels"].append((seq, i, label or "", op, at, at + ms * 1e3, int(n)))
                at += ms * 1e3
                self._sampled[1] += ms
                if op in self.comm:
                    self._sampled[0] += ms
            # a step's device time goes to compute and comm by the share the sampled steps have shown so far
            self.comm_share = self._sampled[0] / self._sampled[1] if self._sampled[1] > 0 else 0.0
            sec = float(device_us or host_us) / 1e6
            self.device_seconds["comm"] += sec * self.comm_share
            self.device_seconds["compute"] += sec * (1.0 - self.comm_share)
        return seq

    def counters(self, sm_mhz: int, mem_mhz: int, gpu_util: int, mem_util: int, power_w: float, sm_active_pm: int = -1,
                 tensor_active_pm: int = -1, dram_bw_pm: int = -1) -> None:
        with self._lock:
            self._rows["counters"].append((self.clock(), sm_mhz, mem_mhz, gpu_util, mem_util, power_w, int(sm_active_pm),
                                           int(tensor_active_pm), int(dram_bw_pm)))

    # ---- files ----
    def _path(self, kind: str, now: datetime) -> Path:
        d = self.dir / f"date={now:%Y-%m-%d}" / f"rank={self.rank}"
        d.mkdir(parents=True, exist_ok=True)
        return d / f"{now:%H%M%S}.{kind}.parquet"

    def rotate(self) -> list[Path]:
        """Write what is buffered and start afresh; returns the files written."""
        import pyarrow as pa
        import pyarrow.parquet as pq

        with self._lock:
            rows, self._rows = self._rows, {"steps": [], "kernels": [], "counters": []}
        now = datetime.now(timezone.utc)
        out = []
        for kind, fields in (("steps", STEP_FIELDS), ("kernels", KERNEL_FIELDS), ("counters", COUNTER_FIELDS)):
            if not rows[kind]:
                continue
            cols = list(zip(*rows[kind]))
            table = pa.table({f: list(c) for f, c in zip(fields, cols)})
            path = self._path(kind, now)
            n = 0
            while path.exists():          # two rotates inside one second
                n += 1
                path = path.with_name(f"{now:%H%M%S}-{n}.{kind}.parquet")
            pq.write_table(table, path, compression="zstd", compression_level=3, use_dictionary=["program", "label", "op"]
                           if kind != "counters" else False)
            out.append(path)
        self.written += out
        return out

    close = rotate


class Counters(threading.Thread):
    """Samples NVML (read only) into a recorder every `period` seconds: clocks, utilisation, power, and — where the
    device offers performance-monitoring samples (GPM) — the share of the interval the SMs, the tensor pipes and the DRAM
    interface were busy, computed by the driver from two consecutive samples. Nothing is set: streaming mode, clocks and
    every other setting stay as found. Reference counterpart: crates/kern-runtime/src/counters.rs:25-31,93-214 (SM MHz,
    SM / tensor active per mille, DRAM traffic every --trace-pm-us)."""

    def __init__(self, recorder: Recorder, gpu: int = 0, period: float = 0.2, nvml=None):
        super().__init__(name="kern-counters", daemon=True)
        self.rec, self.gpu, self.period = recorder, gpu, max(0.00005, period)
        self._halt = threading.Event()
        self.nvml = nvml
        self.gpm = False           # whether the last run found performance-monitoring samples

    def _gpm_open(self, nv, h):
        """Two sample buffers when the device supports GPM, else None."""
        try:
            if not nv.nvmlGpmQueryDeviceSupport(h).isSupportedDevice:
                return None
            a, b = nv.nvmlGpmSampleAlloc(), nv.nvmlGpmSampleAlloc()
            nv.nvmlGpmSampleGet(h, a)
            return [a, b]
        except Exception:
            return None

    def _gpm_read(self, nv, h, pair) -> tuple[int, int, int]:
        """Metrics between the previous sample and a new one (the buffers swap roles)."""
        nv.nvmlGpmSampleGet(h, pair[1])
        get = nv.c_nvmlGpmMetricsGet_t()
        get.version = nv.NVML_GPM_METRICS_GET_VERSION
        ids = (nv.NVML_GPM_METRIC_SM_UTIL, nv.NVML_GPM_METRIC_ANY_TENSOR_UTIL, nv.NVML_GPM_METRIC_DRAM_BW_UTIL)
        get.numMetrics = len(ids)
        get.sample1, get.sample2 = pair[0], pair[1]
        for i, m in enumerate(ids):
            get.metrics[i].metricId = m
        nv.nvmlGpmMetricsGet(get)
        pair[0], pair[1] = pair[1], pair[0]
        return tuple(int(round(10.0 * get.metrics[i].value)) for i in range(len(ids)))      # percent -> per mille

    def run(self) -> None:
        nv = self.nvml
        if nv is None:
            import pynvml as nv
        nv.nvmlInit()
        h = nv.nvmlDeviceGetHandleByIndex(self.gpu)
        pair = self._gpm_open(nv, h)
        self.gpm = pair is not None
        while not self._halt.wait(self.period):
            try:
                u = nv.nvmlDeviceGetUtilizationRates(h)
                pm = (-1, -1, -1)
                if pair is not None:
                    try:
                        pm = self._gpm_read(nv, h, pair)
                    except Exception:
                        pair, self.gpm = None, False          # not offered after all (permissions, MIG): go on without
                self.rec.counters(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM), nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_MEM),
                                  u.gpu, u.memory, nv.nvmlDeviceGetPowerUsage(h) / 1000.0, *pm)
            except Exception:
                self.rec.dropped += 1
        if pair is not None:
            for smp in pair:
                try:
                    nv.nvmlGpmSampleFree(smp)
                except Exception:
                    pass

    def stop(self) -> None:
        self._halt.set()


class TracedEngine:
    """Wraps an engine: every step is recorded (device time by CUDA events on the runtime's stream when there is a
    GPU, host time always); every `sample_every`-th step runs eagerly with per-call events so kernels.parquet gets
    the cost by call."""

    def __init__(self, engine, recorder: Recorder, sample_every: int = 0):
        self.eng, self.rec, self.sample_every = engine, recorder, sample_every
        self._n = 0

    def __getattr__(self, name):
        return getattr(self.eng, name)

    def step(self, batch, **kw):
        self._n += 1
        timed = bool(self.sample_every) and self._n % self.sample_every == 0 and hasattr(self.eng.rt, "issue_timed")
        groups = len(batch) + kw.get("pad", 0)
        rows = sum(len(t) for _, t in batch) + kw.get("pad", 0) * (len(batch[0][1]) if batch else 0)
        context = max((s.length + len(t) for s, t in batch), default=0)
        ev = None
        try:
            import torch
            if torch.cuda.is_available() and hasattr(self.eng.rt, "stream"):
                st = torch.cuda.ExternalStream(self.eng.rt.stream)
                ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True), st)
                ev[0].record(st)
        except Exception:
            ev = None
        t0 = time.perf_counter()
        out = self.eng.step(batch, timed=timed, **kw) if timed else self.eng.step(batch, **kw)
        host_us = (time.perf_counter() - t0) * 1e6
        device_us = 0.0
        if ev is not None:
            ev[1].record(ev[2])
            ev[1].synchronize()
            device_us = ev[0].elapsed_time(ev[1]) * 1e3
        fw = self.eng.forward_for(groups, [len(t) for _, t in batch] + [len(batch[0][1])] * kw.get("pad", 0), kw.get("round", False))
        self.rec.step(fw["name"], groups, rows, context, bool(fw.get("graph")) and not timed, device_us, host_us,
                      getattr(self.eng, "last_launches", 0), getattr(self.eng, "last_times", None) if timed else None)
        return out


def prometheus_lines(recorder: Recorder, kv: str = "paged") -> list[str]:
    """The kernels board of one rank from its recorder: device seconds by class (comm = the share of the sampled steps'
    time spent in `recorder.comm` ops; idle = wall clock not covered by a step), steps by program and shape, dropped
    records. Reference: crates/kern-serve/src/kernels.rs:188-222."""
    wall = time.monotonic() - recorder.started
    busy = recorder.device_seconds["compute"] + recorder.device_seconds["comm"]
    lines = ["# TYPE kern_device_seconds_total counter",
             f'kern_device_seconds_total{{class="compute"}} {recorder.device_seconds["compute"]:.6f}',
             f'kern_device_seconds_total{{class="comm"}} {recorder.device_seconds["comm"]:.6f}',
             f'kern_device_seconds_total{{class="idle"}} {max(0.0, wall - busy):.6f}',
             "# TYPE kern_step_compute_seconds_total counter", f"kern_step_compute_seconds_total {busy:.6f}",
             "# TYPE kern_steps_total counter"]
    for (program, shape), n in sorted(recorder.steps_by.items()):
        lines.append(f'kern_steps_total{{program="{program}",shape="{shape}",kv="{kv}"}} {n}')
    lines += ["# TYPE kern_trace_dropped_records_total counter", f"kern_trace_dropped_records_total {recorder.dropped}"]
    return lines


class Rotator(threading.Thread):
    """Closes the recorder's files at every boundary of `every_s` seconds of the wall clock (a quarter hour: the files of
    one directory line up across ranks), looking every `period` seconds, and whenever more than `max_rows` rows are
    buffered. Reference: crates/kern-serve/src/kernels.rs:294-343 (the 200 ms collector), kern-trace/src/lib.rs:154-204."""

    def __init__(self, recorder: Recorder, every_s: float = 900.0, period: float = 0.2, max_rows: int = 1_000_000, clock=time.time):
        super().__init__(name="kern-trace-rotate", daemon=True)
        self.rec, self.every_s, self.period, self.max_rows, self.clock = recorder, every_s, period, max_rows, clock
        self._halt = threading.Event()
        self.rotations = 0

    def due(self, last_slot: int) -> tuple[bool, int]:
        slot = int(self.clock() // self.every_s)
        rows = sum(len(v) for v in self.rec._rows.values())
        return (slot != last_slot and rows > 0) or rows > self.max_rows, slot

    def run(self) -> None:
        last = int(self.clock() // self.every_s)
        while not self._halt.wait(self.period):
            go, slot = self.due(last)
            if go:
                self.rec.rotate()
                self.rotations += 1
            last = slot

    def stop(self) -> None:
        self._halt.set()


# ---- kernel activity through CUPTI --------------------------------------------------------------------------------------
def launch_plan(doc: dict, program: str, vars: dict[str, int]) -> list[dict]:
    """The kernel launches one issue of `program` makes, in order, with the call they belong to: every launch of every
    call's op whose `when` range admits the var's value. [{call, label, op, entry}] — what `fold` lines kernel records
    up against. Reference counterpart: crates/kern-runtime/src/trace.rs:171-230 (launch tags)."""
    out = []
    for ci, c in enumerate(doc["programs"][program]["calls"]):
        for l in doc["ops"][c["op"]]["impl"]["launches"]:
            w = l.get("when")
            if w is not None:
                v = vars.get(w["var"])
                if v is None or v < w.get("min", 1) or v > w.get("max", 1 << 62):
                    continue
            out.append({"call": ci, "label": c.get("label", ""), "op": c["op"], "entry": l["entry"]})
    return out


def fold(records: list[dict], issues: list[tuple[str, list[dict]]]) -> list[dict]:
    """Attribute kernel activity records to (step, call): `issues` are the program issues in the order they were made,
    each a (step tag, `launch_plan`), and `records` the kernels the device ran (any order; sorted here by start). A
    plan's launches take the next records in order; a record whose kernel name does not contain the planned entry
    (externs carry library names and are not checked) ends the folding with an error rather than mis-attributing the
    rest. Returns one row per launch: step, call, label, op, entry, start_ns, end_ns, us.
    Reference counterpart: crates/kern-runtime/src/trace.rs:232-283 (fold into steps)."""
    recs = sorted(records, key=lambda r: r["start_ns"])
    rows, at = [], 0
    for step, plan in issues:
        for l in plan:
            if at >= len(recs):
                raise ValueError(f"step {step}: the trace ends {len(plan)} launches short (at `{l['entry']}` of call `{l['label']}`)")
            r = recs[at]
            if not l["entry"].startswith("extern:") and l["entry"] not in r["name"]:
                raise ValueError(f"step {step}: launch {at} is `{r['name']}`, the plan expected `{l['entry']}` (call `{l['label']}`)")
            rows.append({"step": step, **l, "start_ns": r["start_ns"], "end_ns": r["end_ns"], "us": (r["end_ns"] - r["start_ns"]) / 1e3})
            at += 1
    return rows


def by_call(rows: list[dict]) -> dict[str, dict]:
    """Folded launches summed by op: {op: {launches, total_us, calls}} longest first (one step or many)."""
    out: dict[str, dict] = {}
    seen = set()
    for r in rows:
        d = out.setdefault(r["op"], {"launches": 0, "total_us": 0.0, "calls": 0})
        d["launches"] += 1
        d["total_us"] += r["us"]
        if (r["step"], r["call"]) not in seen:
            seen.add((r["step"], r["call"]))
            d["calls"] += 1
    return dict(sorted(out.items(), key=lambda kv: -kv[1]["total_us"]))


class KernelTrace:
    """Every kernel this process launches while the trace is on, with its device start and end (CUPTI activity records,
    `csrc/runtime/cupti_trace.hpp`): no events around launches, graph replays included.

        with KernelTrace() as kt:
            engine.step(...)
            torch.cuda.synchronize()
        for name, stats in kt.by_kernel().items(): ...

    Reference counterpart: crates/kern-runtime/src/trace.rs:171-283 (launch tags and folding into steps)."""

    FIELDS = ("name", "start_ns", "end_ns", "stream", "grid", "block", "registers", "shared_bytes")

    def __init__(self):
        from . import _native

        self._n = _native
        ok, why = _native.cupti_available()
        if not ok:
            raise RuntimeError(f"kernel tracing is unavailable: {why}")
        self.records: list[dict] = []

    def __enter__(self):
        self._n.cupti_start()
        return self

    def collect(self) -> list[dict]:
        """Records since the last collect (synchronise the streams first); also appended to `self.records`."""
        new = [dict(zip(self.FIELDS, r)) for r in self._n.cupti_collect()]
        self.records += new
        return new

    def __exit__(self, *exc):
        self.records += [dict(zip(self.FIELDS, r)) for r in self._n.cupti_stop()]
        return False

    def by_kernel(self) -> dict[str, dict]:
        """name -> {launches, total_us, mean_us, max_us}, longest total first."""
        out: dict[str, dict] = {}
        for r in self.records:
            d = out.setdefault(r["name"], {"launches": 0, "total_us": 0.0, "max_us": 0.0})
            us = (r["end_ns"] - r["start_ns"]) / 1e3
            d["launches"] += 1
            d["total_us"] += us
            d["max_us"] = max(d["max_us"], us)
        for d in out.values():
            d["mean_us"] = d["total_us"] / d["launches"]
        return dict(sorted(out.items(), key=lambda kv: -kv[1]["total_us"]))

    def write(self, path) -> None:
        """The raw records as Parquet (zstd): name, start_ns, end_ns, stream, grid/block extents, registers, shared_bytes."""
        import pyarrow as pa
        import pyarrow.parquet as pq

        cols = {"name": [r["name"] for r in self.records], "start_ns": [r["start_ns"] for r in self.records],
                "end_ns": [r["end_ns"] for r in self.records], "stream": [r["stream"] for r in self.records],
                "registers": [r["registers"] for r in self.records], "shared_bytes": [r["shared_bytes"] for r in self.records]}
        for i, ax in enumerate("xyz"):
            cols["grid_" + ax] = [r["grid"][i] for r in self.records]
            cols["block_" + ax] = [r["block"][i] for r in self.records]
        pq.write_table(pa.table(cols), str(path), compression="zstd")
