"""The pure C++ libraries under AddressSanitizer and UndefinedBehaviorSanitizer: the native `kern` binary (parser,
verifier, protocol projection, cut, serialiser) is rebuilt with both and run over real manifests and over malformed
input; any report fails the test. The GPU-side tool of this kind is closed where these tests run, so the host-side
libraries get the coverage that can be had. Reference counterpart: the reference's CI runs its crates' tests under
Miri / sanitizers for the same libraries (.github/workflows)."""
import json
import os
import shutil
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "csrc")


@pytest.fixture(scope="module")
def kern_asan(tmp_path_factory):
    cxx = shutil.which("g++")
    if cxx is None:
        pytest.skip("no g++")
    out = tmp_path_factory.mktemp("asan") / "kern_asan"
    srcs = [os.path.join(CSRC, "cli", "kern_main.cpp")] + sorted(
        os.path.join(CSRC, "manifest", f) for f in os.listdir(os.path.join(CSRC, "manifest")) if f.endswith(".cpp"))
    p = subprocess.run([cxx, "-O1", "-g", "-std=c++17", "-fsanitize=address,undefined", "-fno-sanitize-recover=undefined",
                        "-fno-omit-frame-pointer", "-I", CSRC, "-o", str(out), *srcs], capture_output=True, text=True, timeout=600)
    if p.returncode != 0:
        pytest.skip("the sanitizer runtimes are not installed: " + p.stderr[-300:])
    return str(out)


def run(exe, *args):
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1")
    return subprocess.run([exe, *args], capture_output=True, text=True, timeout=120, env=env)


def clean(p):
    return "Sanitizer" not in p.stderr and "runtime error" not in p.stderr


def test_verify_cut_and_print_are_clean_under_sanitizers(kern_asan, tmp_path):
    from kern_b200.models import dense, hybrid, moe, spec
    from kern_b200.serve import pp

    docs = {"dense": dense.build_manifest(dense.TINY), "hybrid": hybrid.build_manifest(hybrid.TINY_HYBRID),
            "moe": moe.build_manifest(moe.TINY_MOE), "spec": spec.build_manifest(dense.TINY)}
    for name, doc in docs.items():
        path = tmp_path / f"{name}.json"
        path.write_text(json.dumps(doc))
        p = run(kern_asan, "verify", str(path), "--protocol")
        assert p.returncode == 0 and clean(p), (name, p.stdout[-500:], p.stderr[-2000:])
        p = run(kern_asan, "print", str(path))
        assert p.returncode == 0 and clean(p), (name, p.stderr[-2000:])
    at = pp.layer_cuts(docs["dense"], 2)
    (tmp_path / "stages").mkdir()
    p = run(kern_asan, "cut", str(tmp_path / "dense.json"), "--at", ",".join(map(str, at)), "--out", str(tmp_path / "stages"))
    assert p.returncode == 0 and clean(p), p.stderr[-2000:]


def test_malformed_input_is_refused_cleanly_under_sanitizers(kern_asan, tmp_path):
    from kern_b200.models import dense

    text = json.dumps(dense.build_manifest(dense.TOY))
    cases = {"truncated": text[: len(text) // 2], "empty": "", "not_json": "{]", "wrong_types": text.replace('"max": 64', '"max": "x"', 1),
             "deep": "[" * 5000, "nul": text[:100] + "\\u0000" + text[100:]}
    doc = json.loads(text)
    doc["programs"]["decode"]["calls"][0]["args"] = [{"buf": "nope"}] * 40
    cases["bad_call"] = json.dumps(doc)
    doc = json.loads(text)
    next(iter(doc["buffers"].values()))["shape"] = [2 ** 62, 2 ** 62]
    cases["overflow"] = json.dumps(doc)
    for name, body in cases.items():
        path = tmp_path / f"{name}.json"
        path.write_text(body)
        p = run(kern_asan, "verify", str(path))
        assert p.returncode in (0, 1, 2) and clean(p), (name, p.returncode, p.stderr[-2000:])
