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


def test_import_a_foreign_cubin_with_entries_from_a_capture_and_land_it(index, tmp_path, monkeypatch):
    monkeypatch.setattr(R, "IMPORTED", index / "imported")
    foreign = tmp_path / "their_fmha.cubin"
    foreign.write_bytes(b"\x7fELF" + bytes(range(200)))
    import hashlib

    sha = hashlib.sha256(foreign.read_bytes()).hexdigest()
    cap = tmp_path / "launches.jsonl"
    launch = lambda sym, mod: {"kind": "launch", "t_ns": 1, "symbol": sym, "module": mod, "grid": [1, 1, 1], "block": [32, 1, 1], "smem": 0, "params": []}
    cap.write_text("\n".join(json.dumps(r) for r in [launch("fmha_fwd_d128", sha), launch("fmha_fwd_d64", sha), launch("other", "f" * 64)]) + "\n")
    with pytest.raises(ValueError, match="own sources"):
        R.import_cubin(foreign, "moe", entries=["x"])
    with pytest.raises(ValueError, match="no launch out of a module"):
        R.import_cubin(_build.KOUT / "moe.cubin", "their-fmha", capture_file=cap)
    doc = R.import_cubin(foreign, "their-fmha", capture_file=cap, origin="https://example.org/fmha@abc123")
    assert doc["variant"][0]["entries"] == ["fmha_fwd_d128", "fmha_fwd_d64"] and doc["variant"][0]["sha256"] == sha
    assert R.import_cubin(foreign, "their-fmha", entries=["ignored"])["variant"] == doc["variant"]      # the same bytes: nothing new
    assert R.module_decl("their-fmha") == {"source": "their_fmha.cubin", "sha256": sha}
    R.write_all()
    assert R.check() == []
    (index / "imported" / "their-fmha.toml").write_text((index / "imported" / "their-fmha.toml").read_text().replace('entries = ["fmha_fwd_d128", "fmha_fwd_d64"]', "entries = []"))
    assert any("lists no entry" in e for e in R.check())
    # landing: the foreign module from the store, one of the package's own from its build, one nowhere
    own = json.loads((_build.KOUT / "index.json").read_text())["norm_embed"]
    manifest = {"modules": {"fmha": R.module_decl("their-fmha"), "norm": {"source": own["source"], "sha256": own["sha256"]},
                            "ghost": {"source": "ghost.cubin", "sha256": "1" * 64}}}
    landed, missing = R.land(manifest, tmp_path / "pkg")
    assert sorted(landed) == [f"fmha-{sha[:12]}.cubin", f"norm-{own['sha256'][:12]}.cubin"] and len(missing) == 1 and "ghost" in missing[0]
    assert (tmp_path / "pkg" / landed[0]).read_bytes() in (foreign.read_bytes(), (_build.KOUT / own["source"]).read_bytes())
    assert R.land(manifest, tmp_path / "pkg")[0] == []                       # already there by content


def test_kernels_import_and_land_commands(index, tmp_path, monkeypatch, capsys):
    from kern_b200 import cli

    monkeypatch.setattr(R, "IMPORTED", index / "imported")
    foreign = tmp_path / "k.cubin"
    foreign.write_bytes(b"\x7fELFxyz")
    assert cli.main(["kernels", "import", str(foreign), "their-k", "--entry", "a", "--entry", "b"]) == 0
    assert "2 entries" in capsys.readouterr().out
    m = tmp_path / "m.json"
    m.write_text(json.dumps({"modules": {"k": R.module_decl("their-k")}}))
    assert cli.main(["kernels", "land", str(m), str(tmp_path / "out")]) == 0
    assert "1 landed, 0 missing" in capsys.readouterr().out
