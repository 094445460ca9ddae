"""The kernel registry: family documents regenerated from the tree, the offline check, measured picks with their reports."""
import json

import pytest

from kern_b200 import _build, kernel_registry as R


@pytest.fixture()
def index(tmp_path, monkeypatch):
    monkeypatch.setattr(R, "INDEX", tmp_path / "kernel_index")
    monkeypatch.setattr(R, "PICKS", tmp_path / "kernel_index" / "picks.toml")
    monkeypatch.setenv("KERN_B200_CACHE", str(tmp_path / "cache"))
    _build.ensure_built()
    return tmp_path / "kernel_index"


def test_entries_come_from_the_sources_macros_included():
    gemv = R.entries_of(_build.KSRC / "gemv_bf16.cu")
    assert {"kern_gemv_bf16_tn_m1", "kern_gemv_bf16_tn_swiglu_m8"} <= set(gemv) and len(gemv) == 16      # token-pasted names
    moe = R.entries_of(_build.KSRC / "moe.cu")
    assert "kern_ep_fc2_bf16_combine_n256" in moe and "kern_moe_plan_ep" in moe
    assert not any(e.startswith("kern_gemm_bf16_tn") for e in moe)          # the included GEMM source's own entries are switched off
    assert "kern_attn_ragged_paged_d128" in R.entries_of(_build.KSRC / "attn_paged.cu")          # nested launch-bounds expression


def test_documents_check_clean_and_findings_name_what_is_wrong(index):
    paths = R.write_all()
    assert len(paths) == len(R.families()) and R.check() == []
    doc = R.load("moe")
    assert doc["family"]["source"] == "csrc/kernels/sm100/moe.cu" and doc["variant"][0]["name"] == "normal"
    sha = doc["variant"][0]["sha256"]
    idx = json.loads((_build.KOUT / "index.json").read_text())
    assert idx["moe"]["sha256"] == sha                                      # the identity a manifest's module pins
    # a tampered document
    p = index / "moe.toml"
    p.write_text(p.read_text().replace(sha, "0" * 64))
    errs = R.check()
    assert any("moe.toml" in e and "regenerates" in e for e in errs) and any("does not hash" in e for e in errs)
    p.unlink()
    assert any("moe.toml is missing" in e for e in R.check())


def test_a_pick_needs_a_variant_an_entry_and_a_report(index, tmp_path):
    R.write_all()
    report = tmp_path / "bench.json"
    with pytest.raises(ValueError, match="never recorded without"):
        R.pick("moe", "ep_fc2", "rows>192", "normal", report, entry="kern_ep_fc2_bf16_combine_n256")
    report.write_text(json.dumps({"p50_ms": {"n128": 1.0, "n256": 0.76}}))
    with pytest.raises(ValueError, match="no variant"):
        R.pick("moe", "ep_fc2", "rows>192", "tuned", report)
    with pytest.raises(ValueError, match="no entry"):
        R.pick("moe", "ep_fc2", "rows>192", "normal", report, entry="kern_nothing")
    rec = R.pick("moe", "ep_fc2", "rows>192", "normal", report, entry="kern_ep_fc2_bf16_combine_n256", measured="today here")
    assert R.picked("moe", "ep_fc2", "rows>192")["entry"] == "kern_ep_fc2_bf16_combine_n256"
    assert R.blob_path(rec["report"]).exists() and R.report_path(rec["report"]).exists()
    assert R.load("moe")["pick"][0]["report"] == rec["report"] and R.check() == []
    # a second measurement of the same (op, shape) replaces the first; the store keeps both reports
    report.write_text(json.dumps({"p50_ms": {"n128": 0.7, "n256": 0.76}}))
    R.pick("moe", "ep_fc2", "rows>192", "normal", report, entry="kern_ep_fc2_bf16_combine_n128")
    assert len(R.load_picks()) == 1 and R.picked("moe", "ep_fc2", "rows>192")["entry"].endswith("n128")
    R.report_path(R.picked("moe", "ep_fc2", "rows>192")["report"]).unlink()
    R.blob_path(R.picked("moe", "ep_fc2", "rows>192")["report"]).unlink()
    assert any("neither beside the index nor in the store" in e for e in R.check()) and R.check(require_reports=False) == []
