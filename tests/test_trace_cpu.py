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
