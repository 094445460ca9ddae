"""Kernel capture: the injection library's recorder (fed the calls it would see, without a driver), the lifter (its
skeleton must be a manifest op the verifier accepts) and the miner (passes, pointer classes, expressions) on a synthetic
serving run."""
import ctypes
import json
import os
import struct
import subprocess
import sys

import pytest

from kern_b200 import capture as K
from kern_b200.runtime import verify


class LaunchArgs(ctypes.Structure):
    _fields_ = [("f", ctypes.c_void_p)] + [(n, ctypes.c_uint) for n in ("gx", "gy", "gz", "bx", "by", "bz", "smem")] + \
               [("stream", ctypes.c_void_p), ("params", ctypes.POINTER(ctypes.c_void_p)), ("extra", ctypes.c_void_p)]


class AllocArgs(ctypes.Structure):
    _fields_ = [("dptr", ctypes.POINTER(ctypes.c_uint64)), ("bytes", ctypes.c_size_t)]


class MapArgs(ctypes.Structure):
    _fields_ = [("map", ctypes.c_void_p), ("dtype", ctypes.c_int), ("rank", ctypes.c_uint32), ("address", ctypes.c_void_p),
                ("dims", ctypes.POINTER(ctypes.c_uint64)), ("strides", ctypes.POINTER(ctypes.c_uint64)),
                ("box", ctypes.POINTER(ctypes.c_uint32)), ("elem", ctypes.POINTER(ctypes.c_uint32)),
                ("interleave", ctypes.c_int), ("swizzle", ctypes.c_int), ("l2", ctypes.c_int), ("oob", ctypes.c_int)]


RECORDER = r"""
import ctypes, os, struct, sys
sys.path.insert(0, os.getcwd())
from tests.test_capture_cpu import LaunchArgs, AllocArgs, MapArgs
lib = ctypes.CDLL(sys.argv[1])
assert lib.kern_capture_open() == 1
feed = lib.kern_capture_feed
feed.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_char_p]

def alloc(ptr, n):
    box = ctypes.c_uint64(ptr)
    a = AllocArgs(ctypes.pointer(box), n)
    feed(b"cuMemAlloc_v2", 1, ctypes.addressof(a), 0, None)

alloc(0x7f0000000000, 1 << 20)          # activations
alloc(0x7f0010000000, 1 << 24)          # weights
# a descriptor over the weights: 2-D bf16 [rows 512][k 256], box 64 x 128, 128-byte swizzle, 256-byte promotion
desc = (ctypes.c_ubyte * 128)(*[(7 * i + 3) % 251 for i in range(128)])
dims = (ctypes.c_uint64 * 2)(256, 512); strides = (ctypes.c_uint64 * 1)(512)
box = (ctypes.c_uint32 * 2)(64, 128); elem = (ctypes.c_uint32 * 2)(1, 1)
m = MapArgs(ctypes.addressof(desc), 9, 2, 0x7f0010000000 + 4096, dims, strides, box, elem, 0, 3, 3, 0)
feed(b"cuTensorMapEncodeTiled", 1, ctypes.addressof(m), 0, None)
# the launch: (descriptor, pointer into the activations, i32 rows, f32 eps, a 24-byte struct {ptr, i32, 0, u8...})
p0 = (ctypes.c_ubyte * 128)(*desc)
p1 = ctypes.c_uint64(0x7f0000000000 + 0x600)
p2 = ctypes.c_int(37)
p3 = ctypes.c_float(1e-6)
p4 = (ctypes.c_ubyte * 24)(*struct.pack("<QiiB7x", 0x7f0010000000 + 4096, 512, 0, 5))
ptrs = (ctypes.c_void_p * 5)(*[ctypes.addressof(x) for x in (p0, p1, p2, p3, p4)])
offs = (ctypes.c_size_t * 5)(0, 128, 136, 140, 144); sizes = (ctypes.c_size_t * 5)(128, 8, 4, 4, 24)
lib.kern_capture_layout(offs, sizes, 5)
la = LaunchArgs(0x1234, 148, 1, 1, 192, 1, 1, 99328, None, ptrs, None)
feed(b"cuLaunchKernel_ptsz", 0, ctypes.addressof(la), 0, b"kern_gemm_bf16_tn_n128")
# a failed allocation and a free are handled: nothing for the first, a record for the second
box2 = ctypes.c_uint64(0x7f0020000000); bad = AllocArgs(ctypes.pointer(box2), 64)
feed(b"cuMemAlloc_v2", 1, ctypes.addressof(bad), 2, None)
free = ctypes.c_uint64(0x7f0000000000)
feed(b"cuMemFree_v2", 0, ctypes.addressof(free), 0, None)
"""


@pytest.fixture(scope="module")
def recorded(tmp_path_factory):
    out = tmp_path_factory.mktemp("cap")
    env = dict(os.environ, KERN_CAPTURE_DIR=str(out))
    r = subprocess.run([sys.executable, "-c", RECORDER, str(K.library())], env=env, capture_output=True, text=True,
                       cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert r.returncode == 0, r.stderr
    files = list(out.glob("pid*/launches.jsonl"))
    assert len(files) == 1
    return K.Capture(K.load(files[0]))


def test_recorder_writes_what_the_calls_carried(recorded):
    kinds = [r["kind"] for r in recorded.records]
    assert kinds == ["alloc", "alloc", "tensormap", "launch", "free"]
    t = recorded.maps[0]
    assert (t["dtype"], t["rank"], t["dims"], t["strides"], t["box"], t["swizzle"]) == (9, 2, [256, 512], [512], [64, 128], 3)
    l = recorded.launches[0]
    assert l["symbol"] == "kern_gemm_bf16_tn_n128" and l["grid"] == [148, 1, 1] and l["block"] == [192, 1, 1] and l["smem"] == 99328
    assert [p["size"] for p in l["params"]] == [128, 8, 4, 4, 24]
    assert l["params"][0]["tensormaps"] == [{"at": 0, "id": 0}] and "pointers" not in l["params"][0]
    assert l["params"][1]["pointers"] == [{"at": 0, "base": "0x7f0000000000", "offset": 0x600, "bytes": 1 << 20}]
    assert l["params"][4]["pointers"][0]["offset"] == 4096


def test_lifted_skeleton_is_a_manifest_op(recorded):
    out = K.lift(recorded.launches[0], recorded, names={0x7f0010000000: "weights"})
    launch = out["op"]["impl"]["launches"][0]
    assert launch["params"] == ["bytes<128>", "inout buffer<u8>", "i32", "f32", "bytes<24>"]
    tm = launch["args"][0]["pack"]["fields"][0]["tensormap"]
    assert tm["dtype"] == "bf16" and tm["swizzle"] == 128 and tm["l2_promotion"] == 256 and tm["dims"] == [256, 512]
    assert launch["args"][2] == {"i32": 37} and abs(launch["args"][3]["f32"] - 1e-6) < 1e-12
    fields = launch["args"][4]["pack"]["fields"]
    assert fields == [{"at": 0, "param": tm["param"]}, {"at": 8, "i32": 512}, {"at": 16, "i32": 5}]
    assert out["pointers"] == {"0": "@weights+0x1000", "1": "@A+0x600"}
    assert any("4096 bytes into its allocation" in n for n in out["notes"])
    # the skeleton, with its module pinned, is an op the verifier takes
    launch["module"] = "m"
    doc = {"schema_version": 7, "model": "lifted", "vars": {"tokens": {"max": 64}}, "states": {},
           "buffers": {"w": {"dtype": "u8", "shape": [1 << 20], "kind": "inout"},
                       "x": {"dtype": "u8", "shape": ["tokens", 64], "kind": "inout"}},
           "modules": {"m": {"source": "m.cubin", "sha256": "0" * 64}},
           "ops": {"lifted": out["op"]},
           "programs": {"step": {"calls": [{"op": "lifted", "label": "l", "args": [{"buf": "w"}, {"buf": "x"}]}]}}}
    m, diags = verify(doc)
    assert m is not None, diags


def test_variants_group_by_shape(recorded):
    a = recorded.launches[0]
    b = json.loads(json.dumps(a))
    b["params"][1]["hex"] = struct.pack("<Q", 0x7f0000000000 + 0x9000).hex()     # another pointer: the same shape
    b["params"][1]["pointers"][0]["offset"] = 0x9000
    c = json.loads(json.dumps(a))
    c["params"][2]["hex"] = struct.pack("<i", 64).hex()                           # another row count: another shape
    got = K.variants([a, b, c])
    assert [n for _, n in got] == [2, 1]


def _launch(t_ns, symbol, grid, scalars, pointers):
    params = []
    for i, v in enumerate(scalars):
        params.append({"index": i, "offset": 4 * i, "size": 4, "hex": struct.pack("<i", v).hex()})
    for j, (base, off) in enumerate(pointers):
        i = len(scalars) + j
        params.append({"index": i, "offset": 64 + 8 * j, "size": 8, "hex": struct.pack("<Q", base + off).hex(),
                       "pointers": [{"at": 0, "base": hex(base), "offset": off, "bytes": 1 << 30}]})
    return {"kind": "launch", "t_ns": t_ns, "symbol": symbol, "module": None, "grid": grid, "block": [128, 1, 1], "smem": 0, "params": params}


def synthetic_run(token_counts, layers=4):
    """embed, then per layer (norm, gemm, attn), then head; weights per layer, a KV state shared by all layers'
    attention, activations from an arena whose offsets move from pass to pass."""
    W, S, A = 0x7f1000000000, 0x7f2000000000, 0x7f3000000000
    recs, t = [], 0
    for n, tok in enumerate(token_counts):
        t += 50_000_000                                     # requests are 50 ms apart
        arena = 0x1000 * (n % 3)
        recs.append(_launch(t, "embed", [tok, 1, 1], [tok], [(W, 0), (A, arena)]))
        for l in range(layers):
            t += 20_000
            recs.append(_launch(t, "norm", [tok, 1, 1], [tok, 4096], [(A, arena), (W, 0x100000 * l + 0x10), (A, arena + 0x40000)]))
            recs.append(_launch(t + 5_000, "gemm", [-(-tok // 128) * 8, 1, 1], [tok, 4096, 1024], [(A, arena + 0x40000), (W, 0x100000 * l + 0x4000)]))
            recs.append(_launch(t + 10_000, "attn", [-(-3 * tok // 64), 8, 1], [tok, l], [(S, 0), (A, arena)]))
        recs.append(_launch(t + 30_000, "head", [1, 1, 1], [tok], [(W, 0xF00000)]))
    return recs


def test_mine_finds_passes_classes_and_expressions():
    cap = K.Capture(synthetic_run([5, 64, 300, 1000, 77]))
    facts = K.mine(cap, min_launches=8, burst_gap=4)
    assert facts["passes"] == 5 and facts["classes"] == 1 and facts["launches_per_pass"] == 14
    assert facts["tokens"] == [5, 64, 300, 1000, 77] and facts["tokens_from"] != "given"
    e = facts["expressions"]
    assert K.expr_text(e["norm#0 grid.x"][0]) == "t"
    assert K.expr_text(e["gemm#2 grid.x"][0]) == "8*ceil(t/128)"
    assert K.expr_text(e["attn#1 grid.x"][0]) == "ceil(3*t/64)"
    assert "attn#1 p1+0" not in e                              # the layer index does not vary between passes
    p = facts["pointers"]
    assert p["norm p3+0"]["class"].startswith("weight") and p["gemm p4+0"]["class"].startswith("weight")
    assert p["attn p2+0"]["class"].startswith("state")
    assert p["norm p2+0"]["class"] == "workspace" and p["gemm p3+0"]["class"] == "workspace"
    assert p["head p1+0"]["class"].startswith("fixed (one call site")
    assert "core kernel" in K.report(facts) and not facts["unexplained"]


def test_mine_with_windows_holding_several_passes_and_given_tokens():
    recs = synthetic_run([16, 48])
    for r in recs:                                           # one window: passes 1 ms apart
        r["t_ns"] = r["t_ns"] // 100
    cap = K.Capture(recs)
    facts = K.mine(cap, gap_ms=5.0, tokens=[16, 48], min_launches=8, burst_gap=4)
    assert facts["windows"] == 1 and facts["passes"] == 2 and facts["tokens_from"] == "given"
    assert K.mine(cap, tokens=[1, 2, 3], min_launches=8, burst_gap=4)["error"].startswith("--tokens names 3")


def test_fit_reports_what_the_samples_cannot_tell_apart():
    assert [K.expr_text(e) for e in K.fit([(100, 1), (128, 1)])] == ["1"]
    both = [K.expr_text(e) for e in K.fit([(100, 1), (200, 2)])]
    assert "ceil(t/128)" in both and "ceil(t/256)" not in both and len(both) > 1     # 100, 200 fit several divisors
    assert K.fit([(3, 7), (5, 9)]) == []


def test_command_line(recorded, tmp_path, capsys):
    path = tmp_path / "launches.jsonl"
    path.write_text("\n".join(json.dumps(r) for r in recorded.records) + "\n{\"kind\":\"lau")   # a cut last line is tolerated
    assert K.main(["lift", str(path), "--symbol", "gemm_bf16", "--all"]) == 0
    out = json.loads(capsys.readouterr().out)
    assert out["launches_of_this_shape"] == 1 and out["op"]["impl"]["launches"][0]["entry"] == "kern_gemm_bf16_tn_n128"
    assert K.main(["lift", str(path), "--symbol", "nothing"]) == 1


def test_a_capture_taken_on_a_b200_lifts_into_ops_the_verifier_takes():
    """The fixture is the head of what the library wrote beside a tiny dense model's prefill on a B200 (modules,
    allocations, descriptors, the first 14 launches of the package's own kernels)."""
    path = os.path.join(os.path.dirname(__file__), "data", "capture_b200_tiny_dense.jsonl")
    cap = K.Capture(K.load(path))
    assert len(cap.launches) == 14 and len(cap.modules) == 7 and all(m["format"] == "elf" for m in cap.modules)
    pinned = {m["sha256"] for m in cap.modules}
    gemm = cap.of_symbol("kern_gemm_bf16_tn_n64")[0]
    out = K.lift(gemm, cap)
    launch = out["op"]["impl"]["launches"][0]
    assert launch["module"] in pinned and launch["block"] == [192, 1, 1] and launch["grid"] == [148, 1, 1]
    assert launch["params"][:2] == ["bytes<128>", "bytes<128>"]
    a, b = (launch["args"][i]["pack"]["fields"][0]["tensormap"] for i in (0, 1))
    assert a["dtype"] == b["dtype"] == "bf16" and a["swizzle"] == b["swizzle"] == 128 and a["box"][0] == b["box"][0] == 64
    for rec in cap.launches:                                  # every launch of the run lifts into a valid op
        out = K.lift(rec, cap)
        launch = out["op"]["impl"]["launches"][0]
        assert launch["module"] in pinned, rec["symbol"]
        launch["module"] = "m"
        n = len(out["op"]["params"])
        doc = {"schema_version": 7, "model": "lifted", "vars": {}, "states": {},
               "buffers": {f"b{i}": {"dtype": "u8", "shape": [1 << 20], "kind": "inout"} for i in range(n)},
               "modules": {"m": {"source": "m.cubin", "sha256": "0" * 64}}, "ops": {"lifted": out["op"]},
               "programs": {"step": {"calls": [{"op": "lifted", "label": "l", "args": [{"buf": f"b{i}"} for i in range(n)]}]}}}
        m, diags = verify(doc)
        assert m is not None, (rec["symbol"], diags)
