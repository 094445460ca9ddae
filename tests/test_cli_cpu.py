"""`kern` subcommands on the CPU executor: verify (prints the protocol), cut, run, test (A/B verdicts), bench."""
import dataclasses
import json

import pytest

from kern_b200 import cli
from kern_b200.models import common, dense


@pytest.fixture(scope="module")
def pkg(tmp_path_factory):
    d = tmp_path_factory.mktemp("pkg")
    cfg = dense.TOY
    (d / "manifest.json").write_text(json.dumps(dense.build_manifest(cfg)))
    common.write_safetensors(d / "model.safetensors", dense.random_weights(cfg, seed=0, std=0.05))
    return d, cfg


def test_verify_prints_protocol_and_rejects(pkg, capsys, tmp_path):
    d, _ = pkg
    assert cli.main(["verify", str(d / "manifest.json")]) == 0
    out = capsys.readouterr().out
    assert "forward decode: up to 4 groups x 1 rows, emits next_token, graph" in out and "fill token" in out and "once load" in out
    bad = json.loads((d / "manifest.json").read_text())
    bad["vars"]["tokens"]["max"] = 0
    (tmp_path / "bad.json").write_text(json.dumps(bad))
    assert cli.main(["verify", str(tmp_path / "bad.json")]) == 1
    assert "max must be >= 1" in capsys.readouterr().out


def test_run_and_cut(pkg, capsys, tmp_path):
    d, cfg = pkg
    assert cli.main(["run", "--cpu", "--manifest", str(d / "manifest.json"), "--weights", str(d), "--prompt-ids", "5,6,7,8", "--steps", "4"]) == 0
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert len(line["tokens"]) == 4
    # per-layer KV states: a cut between the layers leaves each stage its own
    n_layer0 = next(i for i, c in enumerate(json.loads((d / "manifest.json").read_text())["programs"]["decode"]["calls"]) if c.get("label") == "l1.ln1")
    rc = cli.main(["cut", str(d / "manifest.json"), "--at", str(n_layer0), "--out", str(tmp_path / "stages")])
    out = capsys.readouterr().out
    # the toy's prefill and decode programs differ in length before the cut point, so this cut may be refused;
    # either way the command must answer, never crash
    assert rc in (0, 1) and ("stage 0" in out or "cannot cut" in out)


def test_ab_test_verdicts(pkg, capsys, tmp_path):
    d, cfg = pkg
    a = d / "manifest.json"
    assert cli.main(["test", str(a), str(a), "--cpu", "--weights", str(d), "--prompts", "2", "--decode-steps", "3"]) == 0
    assert "PASS: bit-identical" in capsys.readouterr().out
    # B: another launch geometry for the norm (an implementation change with identical values)
    doc = json.loads(a.read_text())
    doc["ops"]["norm"]["impl"]["launches"][0]["block"] = [128, 1, 1]
    (tmp_path / "b.json").write_text(json.dumps(doc))
    assert cli.main(["test", str(a), str(tmp_path / "b.json"), "--cpu", "--weights", str(d), "--prompts", "2", "--decode-steps", "3"]) == 0
    out = capsys.readouterr().out
    assert "diff op norm: impl" in out and "PASS" in out
    # every changed span was replayed on B from A's images of the same step, and wrote the same bytes
    replays = [l for l in out.splitlines() if l.startswith("replay program")]
    assert replays and all("bit-identical" in l for l in replays)
    # B: a different epsilon in the final norm changes the function -> not bit-identical; tiny eps stays within KL
    doc2 = json.loads(a.read_text())
    for l in doc2["ops"]["norm_last"]["impl"]["launches"]:
        l["args"][7] = {"f32": 0.5}
    (tmp_path / "c.json").write_text(json.dumps(doc2))
    rc = cli.main(["test", str(a), str(tmp_path / "c.json"), "--cpu", "--weights", str(d), "--prompts", "2", "--decode-steps", "3"])
    out = capsys.readouterr().out
    assert "diff op norm_last: impl" in out and rc in (1, 2) or "logit evidence" in out
    # the replay pins the difference to the span that holds the changed op, from identical inputs
    replays = [l for l in out.splitlines() if l.startswith("replay program")]
    assert replays and all("differs: " in l for l in replays)


def test_bench_and_kernels(pkg, capsys):
    d, _ = pkg
    assert cli.main(["bench", "--cpu", "--manifest", str(d / "manifest.json"), "--weights", str(d), "--capacity", "1024"]) == 0
    pts = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines()]
    assert len(pts) == 2 and all(p["p50_ms"] > 0 and p["min_ms"] <= p["p50_ms"] <= p["max_ms"] for p in pts)
    # the raw samples are kept; on the host executor the clock is the host's and nothing is flushed
    assert all(len(p["samples_ms"]) >= 3 and p["clock"] == "host" and not p["l2_flushed"] and p["host_p50_ms"] > 0 for p in pts)
    assert cli.main(["kernels"]) == 0
    assert "gemm_bf16.cubin" in capsys.readouterr().out


def test_bench_candidate_splices_and_picks(tmp_path, capsys):
    """`kern bench --candidate`: an op implementation from another manifest is spliced in, held to the same answers, priced."""
    import json

    from kern_b200.cli import main
    from kern_b200.models import common, dense

    cfg = dense.TOY
    doc = dense.build_manifest(cfg)
    mpath, wpath = tmp_path / "m.json", tmp_path / "w.safetensors"
    mpath.write_text(json.dumps(doc))
    common.write_safetensors(wpath, dense.random_weights(cfg, seed=1, std=0.08))
    # the candidate: the same norm op (another implementation would go here), interface unchanged
    cand = {"modules": {"norm_embed": doc["modules"]["norm_embed"]}, "ops": {"norm": doc["ops"]["norm"]}}
    cpath = tmp_path / "cand.json"
    cpath.write_text(json.dumps(cand))
    out = tmp_path / "picks.json"
    assert main(["bench", "--cpu", "--manifest", str(mpath), "--weights", str(wpath), "--candidate", str(cpath), "--out", str(out)]) == 0
    got = json.loads(out.read_text())
    assert got["held"] == "PASS" and len(got["picks"]) == 2 and all(p["pick"] in ("base", "candidate", "either") for p in got["picks"])
    bad = dict(cand, ops={"norm": {**doc["ops"]["norm"], "params": doc["ops"]["norm"]["params"][:2]}})
    cpath.write_text(json.dumps(bad))
    assert main(["bench", "--cpu", "--manifest", str(mpath), "--weights", str(wpath), "--candidate", str(cpath)]) == 1


def test_pick_fewest_ranges_within_noise():
    from kern_b200.testing.pick import Point, gaps, pick

    pts = [Point(1, {"gemv": 1.0, "tile": 3.0}), Point(4, {"gemv": 1.2, "tile": 2.9}), Point(8, {"gemv": 2.5, "tile": 2.6}, noise=0.2),
           Point(16, {"gemv": 9.0, "tile": 2.7}), Point(256, {"gemv": 99.0, "tile": 3.0})]
    got = pick(pts)
    assert got == [("gemv", 1, 8), ("tile", 9, 256)]            # the tie at 8 (within noise) extends the first range
    assert gaps(got, 512) == [(257, 512)] and gaps(got, 256) == []
    assert pick([Point(5, {"a": 1.0, "b": 1.05}, noise=0.1), Point(9, {"a": 2.0, "b": 1.0})]) == [("b", 1, 9)]


def test_native_kern_binary_verifies_and_cuts(tmp_path):
    """The C++ `kern` binary (manifest library + main, no Python or CUDA behind it): verify with the protocol, a
    diagnostic for a broken manifest, and cut into stage files."""
    import json
    import subprocess
    from kern_b200 import _build
    from kern_b200.models import dense

    exe = _build.build_cli()
    doc = dense.build_manifest(dense.TINY)
    good = tmp_path / "m.json"
    good.write_text(json.dumps(doc))
    p = subprocess.run([str(exe), "verify", str(good), "--protocol", "--greedy"], capture_output=True, text=True, timeout=60)
    assert p.returncode == 0 and p.stdout.startswith("ok:") and '"page_tables"' in p.stdout, p.stdout[:500]
    bad = dict(doc, surprise=1)
    (tmp_path / "bad.json").write_text(json.dumps(bad))
    p = subprocess.run([str(exe), "verify", str(tmp_path / "bad.json")], capture_output=True, text=True, timeout=60)
    assert p.returncode == 1 and "surprise" in p.stdout
    calls = len(doc["programs"]["prefill"]["calls"])
    (tmp_path / "st").mkdir()
    p = subprocess.run([str(exe), "cut", str(good), "--at", str(calls // 2), "--out", str(tmp_path / "st")],
                       capture_output=True, text=True, timeout=60)
    assert p.returncode == 0, p.stdout
    from kern_b200.runtime import verify
    for i in range(2):
        m, diags = verify(json.loads((tmp_path / "st" / f"stage{i}.json").read_text()))
        assert m is not None, diags[:3]


def test_run_with_activation_probes(tmp_path, capsys):
    """`kern run --probe-dir`: the program runs call range by call range and the asked-for calls' outputs land as
    tensors; the generated tokens are the ones an unprobed run gives."""
    import json
    import torch
    from kern_b200 import cli

    base = ["run", "--model", "toy", "--cpu", "--prompt-ids", "1,2,3,4,5", "--steps", "3"]
    assert cli.main(base) == 0
    plain = json.loads(capsys.readouterr().out.strip().splitlines()[-1])["tokens"]
    d = tmp_path / "probes"
    assert cli.main(base + ["--probe-dir", str(d), "--probe-labels", "l0.ln1,head"]) == 0
    probed = json.loads(capsys.readouterr().out.strip().splitlines()[-1])["tokens"]
    assert probed == plain
    index = json.loads((d / "index.json").read_text())
    labels = {e["label"] for e in index}
    assert "l0.ln1" in labels and any(l.endswith("head") for l in labels), labels
    first = next(e for e in index if e["label"] == "l0.ln1")
    t = torch.load(d / first["file"])
    assert list(t.shape) == first["shape"] and t.shape[0] == 5 and bool(torch.isfinite(t.float()).all())


def test_bench_samples_start_from_the_same_recurrent_state(capsys, tmp_path):
    """A model with a per-sequence state: every sample of a sweep point runs from the pre-image (the state is kept in a
    spare slot and put back), so the slot's bytes after the bench equal those after the context alone plus one call."""
    import numpy as np

    from kern_b200.cli import bench_points
    from kern_b200.cpu import CpuRuntime
    from kern_b200.models import hybrid

    cfg = hybrid.TOY_HYBRID
    w = hybrid.random_weights(cfg, seed=1, std=0.05)
    make = lambda: CpuRuntime(hybrid.build_manifest(cfg), weights=w, tokens=cfg.page_size * 16, slots=6)
    wl = {"seed": 3, "samples": 3, "sweep": [{"groups": 1, "rows": 1, "context": 9}]}
    rt = make()
    rt.once()
    seen = []
    real = rt.run_copies
    rt.run_copies = lambda c: (seen.append(c["slot"]), real(c))[1]
    rep = bench_points(rt, wl, quiet=True)
    assert len(rep["points"][0]["samples_ms"]) == 3
    # one copy out to the spare slot, then one back before each of the 4 + 3 calls
    assert len(seen) == 1 + 7 and seen[0] == tuple(reversed(seen[1])) and len(set(seen[1:])) == 1
