"""Trace recorder: Parquet layout and schemas, rotate, the step -> workload loop, counters through a fake NVML."""
import time

import pyarrow.parquet as pq

from kern_b200 import trace
from kern_b200.cpu import CpuRuntime
from kern_b200.engine import Engine
from kern_b200.models import toy_int


def test_steps_and_kernels_files(tmp_path):
    rec = trace.Recorder(tmp_path, rank=3)
    eng = trace.TracedEngine(Engine(CpuRuntime(toy_int.build_manifest(False), tokens=16 * 20)), rec)
    s = eng.open(64)
    t = eng.step([(s, list(range(1, 20)))])[0][0]
    for _ in range(5):
        t = eng.step([(s, [t])])[0][0]
    rec.step("prefill", 1, 8, 8, False, 12.0, 20.0, 3, calls=[("l0.qkv", "qkv_proj", 0.004, 1), ("l0.attn", "attn", 0.008, 2)])
    files = rec.rotate()
    kinds = sorted(p.name.split(".")[1] for p in files)
    assert kinds == ["kernels", "steps"]
    assert all(p.parent.name == "rank=3" and p.parent.parent.name.startswith("date=") for p in files)
    steps = pq.ParquetFile(next(p for p in files if ".steps." in p.name)).read().to_pydict()
    assert list(steps) == list(trace.STEP_FIELDS)
    assert steps["program"][:2] == ["prefill", "decode"] and steps["rows"][0] == 19 and steps["groups"][1] == 1
    assert steps["context"][:3] == [19, 20, 21] and steps["seq"] == list(range(1, 8))
    kern = pq.ParquetFile(next(p for p in files if ".kernels." in p.name)).read().to_pydict()
    assert kern["label"] == ["l0.qkv", "l0.attn"] and kern["start_us"][1] == kern["end_us"][0] == 4.0
    assert rec.rotate() == []                     # nothing buffered: no empty files


def test_workload_from_steps(tmp_path):
    from kern_b200.cli import main

    rec = trace.Recorder(tmp_path)
    for _ in range(30):
        rec.step("decode", 16, 16, 900, True, 5000.0, 5100.0, 1)
    for _ in range(3):
        rec.step("prefill", 1, 2048, 2048, False, 90000.0, 90500.0, 400)
    steps = next(p for p in rec.rotate() if ".steps." in p.name)
    out = tmp_path / "w.toml"
    assert main(["workload", str(steps), "--out", str(out)]) == 0
    text = out.read_text()
    assert "groups = 16" in text and "chunk = 2048" in text and "context = 1024" in text
    assert trace.shape_of(16, 16) == "decode" and trace.shape_of(8, 56) == "round" and trace.shape_of(1, 2048) == "prefill"


class FakeNvml:
    NVML_CLOCK_SM, NVML_CLOCK_MEM = 1, 2

    class _U:
        gpu, memory = 77, 31

    def nvmlInit(self): pass
    def nvmlDeviceGetHandleByIndex(self, i): return i
    def nvmlDeviceGetUtilizationRates(self, h): return self._U()
    def nvmlDeviceGetClockInfo(self, h, which): return 1965 if which == 1 else 3996
    def nvmlDeviceGetPowerUsage(self, h): return 612000


def test_counters_sampler_reads_only(tmp_path):
    rec = trace.Recorder(tmp_path)
    c = trace.Counters(rec, period=0.01, nvml=FakeNvml())
    c.start()
    time.sleep(0.15)
    c.stop()
    c.join(2)
    f = next(p for p in rec.rotate() if ".counters." in p.name)
    t = pq.ParquetFile(f).read().to_pydict()
    assert len(t["t_ns"]) >= 3 and set(t["sm_mhz"]) == {1965} and t["power_w"][0] == 612.0


class FakeNvmlGpm(FakeNvml):
    """NVML with performance-monitoring samples: a sample is a counter reading; the metrics call turns two of them into
    percentages. Records every call so the test can see that nothing was set."""
    NVML_GPM_METRICS_GET_VERSION, NVML_GPM_METRIC_SM_UTIL, NVML_GPM_METRIC_ANY_TENSOR_UTIL, NVML_GPM_METRIC_DRAM_BW_UTIL = 1, 2, 5, 10

    class _Metric:
        metricId, value = 0, 0.0

    class c_nvmlGpmMetricsGet_t:
        def __init__(self):
            self.version = self.numMetrics = 0
            self.sample1 = self.sample2 = None
            self.metrics = [FakeNvmlGpm._Metric() for _ in range(16)]

    def __init__(self, supported=True):
        self.calls, self.n, self.supported = [], 0, supported

    def nvmlGpmQueryDeviceSupport(self, h):
        self.calls.append("query")
        return type("S", (), {"isSupportedDevice": int(self.supported)})()

    def nvmlGpmSampleAlloc(self):
        self.calls.append("alloc")
        return {"at": None}

    def nvmlGpmSampleGet(self, h, smp):
        self.n += 1
        smp["at"] = self.n
        self.calls.append("sample")

    def nvmlGpmMetricsGet(self, get):
        assert get.sample2["at"] == get.sample1["at"] + 1          # consecutive samples, older first
        for i, v in zip(range(get.numMetrics), (93.5, 61.25, 40.0)):
            assert get.metrics[i].metricId in (2, 5, 10)
            get.metrics[i].value = v
        self.calls.append("metrics")

    def nvmlGpmSampleFree(self, smp):
        self.calls.append("free")


def test_counters_sampler_reads_performance_monitoring_samples(tmp_path):
    """SM / tensor / DRAM busy shares per interval from the driver's samples, written per mille beside the clocks; a device
    without them gives -1 in those columns. The sampler only reads: no call that sets anything is made."""
    nv = FakeNvmlGpm()
    rec = trace.Recorder(tmp_path)
    c = trace.Counters(rec, period=0.01, nvml=nv)
    c.start()
    time.sleep(0.15)
    c.stop()
    c.join(2)
    assert c.gpm and set(nv.calls) == {"query", "alloc", "sample", "metrics", "free"} and nv.calls.count("free") == 2
    t = pq.ParquetFile(next(p for p in rec.rotate() if ".counters." in p.name)).read().to_pydict()
    assert len(t["t_ns"]) >= 3 and set(t["sm_active_pm"]) == {935} and set(t["tensor_active_pm"]) == {612} and set(t["dram_bw_pm"]) == {400}
    rec2 = trace.Recorder(tmp_path / "b")
    c2 = trace.Counters(rec2, period=0.01, nvml=FakeNvmlGpm(supported=False))
    c2.start()
    time.sleep(0.08)
    c2.stop()
    c2.join(2)
    t2 = pq.ParquetFile(next(p for p in rec2.rotate() if ".counters." in p.name)).read().to_pydict()
    assert not c2.gpm and set(t2["sm_active_pm"]) == {-1} and set(t2["sm_mhz"]) == {1965}


def test_kernel_records_fold_into_steps_and_calls():
    """Kernel activity records attributed to (step, call) by the launch plan of each issue: `when` ranges pick the
    launch an issue really makes, a name that does not match the plan stops the folding."""
    import pytest

    from kern_b200 import trace
    from kern_b200.models import dense

    doc = dense.build_manifest(dense.TOY)
    plan1 = trace.launch_plan(doc, "decode", {"seqs": 1, "tokens": 1})
    plan4 = trace.launch_plan(doc, "decode", {"seqs": 4, "tokens": 4})
    assert len(plan1) == len(plan4) > 10
    # one row: the weight-streaming kernel; four rows: a tensor-core tile (the op's `when` ranges)
    e1 = {l["label"]: l["entry"] for l in plan1}
    e4 = {l["label"]: l["entry"] for l in plan4}
    assert e1["l0.qkv"].startswith("kern_gemv_bf16") and e4["l0.qkv"].startswith("kern_gem") and e1["l0.qkv"] != e4["l0.qkv"]
    t, records = 1000, []
    for plan in (plan1, plan4):
        for l in plan:
            records.append({"name": f"void {l['entry']}<...>(...)", "start_ns": t, "end_ns": t + 2000})
            t += 2500
    rows = trace.fold(list(reversed(records)), [("s0", plan1), ("s1", plan4)])
    assert len(rows) == len(plan1) + len(plan4) and rows[0]["step"] == "s0" and rows[-1]["step"] == "s1"
    assert all(r["us"] == 2.0 for r in rows)
    ops = trace.by_call(rows)
    assert ops["attn_decode"]["calls"] == 2 * dense.TOY.layers
    with pytest.raises(ValueError, match="expected"):
        trace.fold(records, [("s0", plan4), ("s1", plan1)])        # the plans in the wrong order: names disagree
    with pytest.raises(ValueError, match="short"):
        trace.fold(records[:5], [("s0", plan1)])


def test_server_trace_flags_record_steps_calls_and_counters(tmp_path):
    """`kern server --trace-dir D --trace-sample 2 --trace-pm-us 10000`: the engine the scheduler drives is the traced
    one, sampled steps carry their cost by call, the sampler thread writes counters, and a rotate closes the files."""
    from types import SimpleNamespace

    from kern_b200 import cli
    from kern_b200.cpu import CpuRuntime
    from kern_b200.engine import Engine
    from kern_b200.models import dense
    from kern_b200.serve.scheduler import Request, Scheduler

    cfg = dense.TOY
    rt = CpuRuntime(dense.build_manifest(cfg), weights=dense.random_weights(cfg, seed=0, std=0.05), tokens=cfg.page_size * 16)
    rt.once()
    args = SimpleNamespace(trace_dir=str(tmp_path), trace_sample=2, trace_pm_us=10000, cpu=True, gpu=0)
    eng, rec, sampler = cli.trace_setup(args, Engine(rt), nvml=FakeNvmlGpm())
    assert rec is not None and sampler is not None
    sched = Scheduler(eng, chunk=16, max_seqs=2)
    for i in range(3):
        sched.submit(Request(id=str(i), prompt=list(range(2, 20 + i)), max_tokens=4))
    sched.run_until_idle()
    time.sleep(0.05)
    sampler.stop()
    sampler.join(2)
    rec.rotator.stop()
    kinds = {p.name.split(".")[1]: p for p in rec.rotate()}
    assert {"steps", "counters"} <= set(kinds)
    steps = pq.ParquetFile(kinds["steps"]).read().to_pydict()
    assert len(steps["seq"]) >= sched.stats.steps          # a scheduler step is one engine call, or several when it splits
    assert {"prefill", "decode"} <= set(steps["program"])
    assert set(pq.ParquetFile(kinds["counters"]).read().to_pydict()["tensor_active_pm"]) == {612}
    # without the flag nothing is wrapped
    plain = cli.trace_setup(SimpleNamespace(trace_dir=None), "engine")
    assert plain == ("engine", None, None)


def test_kernels_board_from_the_recorder_and_the_rotator(tmp_path):
    """The board of a traced rank: steps by program and shape, device seconds split into compute and comm by the share
    the sampled steps' calls show (comm = ops that run a collective built-in or take a peer table), idle = the rest of
    the wall clock; the rotator closes files at a boundary of its period and when too many rows are buffered."""
    from kern_b200.models import dense, dense_tp

    doc = dense_tp.build_manifest_tp(__import__("dataclasses").replace(dense.TOY, tp=2))
    comm = trace.comm_ops(doc)
    # the fused all-reduce + norm, and the two GEMMs whose epilogue pushes rows into the peers' staging buffers
    assert comm == {"allreduce_norm", "o_proj", "down_proj"}
    assert trace.comm_ops(dense.build_manifest(dense.TOY)) == set()
    rec = trace.Recorder(tmp_path, comm={"allreduce"})
    rec.step("decode", 8, 8, 100, True, 1000.0, 1100.0, 10)                       # nothing sampled yet: all compute
    rec.step("prefill", 1, 64, 64, False, 3000.0, 3100.0, 40, calls=[("a", "gemm", 2.0, 1), ("b", "allreduce", 1.0, 1)])
    rec.step("decode", 8, 8, 101, True, 3000.0, 3100.0, 10)
    lines = trace.prometheus_lines(rec)
    assert 'kern_steps_total{program="decode",shape="decode",kv="paged"} 2' in lines
    assert 'kern_steps_total{program="prefill",shape="prefill",kv="paged"} 1' in lines
    val = lambda cls: float(next(l for l in lines if f'class="{cls}"' in l).split()[-1])
    assert abs(val("comm") - 0.002) < 1e-9 and abs(val("compute") - 0.005) < 1e-9 and val("idle") >= 0.0
    # the rotator: a boundary of the period with rows buffered, or too many rows
    now = [1000.0]
    rot = trace.Rotator(rec, every_s=900.0, max_rows=5, clock=lambda: now[0])
    assert rot.due(int(1000 // 900)) == (False, 1)
    now[0] = 1801.0
    assert rot.due(1) == (True, 2)
    rec.rotate()
    assert rot.due(1) == (False, 2)                                               # nothing buffered: no empty files
    for _ in range(6):
        rec.step("decode", 1, 1, 5, True, 10.0, 11.0, 1)
    assert rot.due(2) == (True, 2)
