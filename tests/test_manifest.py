"""Manifest v7: typed parse, every verifier rule group, protocol projection, lanes, cut, candidates.

Each negative case edits one thing in a small valid manifest and names the diagnostic it must produce
(the verifier reports all problems at once, so a case checks `any(...)`).
Model for the shape of this suite: crates/kern-manifest/tests/{verify,protocol,lanes,cut,candidate}.rs.
"""
import copy
import glob
import json
import os

import pytest

from kern_b200 import _native as N

SHA = "ab" * 32
REF = os.environ.get("KERN_REFERENCE_DIR", "")      # the upstream tree, when one is mounted (fixture tests skip otherwise)


def base():
    return {
        "schema_version": 7,
        "model": "unit",
        "vars": {"tokens": {"max": 64, "axis": "rows"}, "seqs": {"max": 8, "axis": "groups"}},
        "states": {"kv": {"bytes_per_token": 64}},
        "buffers": {
            "ids": {"dtype": "i64", "shape": ["tokens"], "kind": "input", "fill": "token"},
            "slots": {"dtype": "i64", "shape": ["tokens"], "kind": "input", "fill": "slot", "domain": {"index_into": "kv"}},
            "table": {"dtype": "i32", "shape": ["seqs", 4], "kind": "input", "domain": {"index_into": "kv", "stride": 16}},
            "emb": {"dtype": "bf16", "shape": [256, 32], "kind": "weight", "bind": [{"tensor": "embed.weight"}]},
            "x": {"dtype": "bf16", "shape": ["tokens", 32], "kind": "workspace"},
            "y": {"dtype": "bf16", "shape": ["tokens", 32], "kind": "workspace"},
            "next": {"dtype": "i64", "shape": ["seqs"], "kind": "output", "fill": "tokens"},
        },
        "modules": {"k": {"source": "k.cubin", "sha256": SHA}},
        "ops": {
            "embed": {
                "params": ["in buffer<i64>", "in buffer<bf16>", "out buffer<bf16>", "i32"],
                "impl": {"launches": [{"module": "k", "entry": "embed", "block": [128, 1, 1], "grid": ["tokens", 1, 1]}]},
            },
            "attn": {
                "params": ["in buffer<bf16>", "in buffer<i64>", "in buffer<i32>", "inout state", "out buffer<bf16>"],
                "impl": {
                    "scratch": {"tmp": {"dtype": "f32", "shape": ["tokens", 8]}},
                    "launches": [
                        {"module": "k", "entry": "a1", "block": [64, 1, 1], "grid": [{"ceil_div": ["tokens", 4]}, 1, 1],
                         "params": ["in buffer<bf16>", "in buffer<i64>", "inout state", "out buffer<f32>"],
                         "args": [{"param": 0}, {"param": 1}, {"param": 3}, {"scratch": "tmp"}]},
                        {"module": "k", "entry": "a2", "block": [64, 1, 1], "grid": ["seqs", 1, 1],
                         "params": ["in buffer<f32>", "in buffer<i32>", "out buffer<bf16>"],
                         "args": [{"scratch": "tmp"}, {"param": 2}, {"param": 4}]},
                    ],
                },
            },
            "head": {
                "params": ["in buffer<bf16>", "out buffer<i64>"],
                "impl": {"launches": [{"module": "k", "entry": "head", "block": [32, 1, 1], "grid": ["seqs", 1, 1]}]},
            },
        },
        "programs": {
            "prefill": {"batch": {"groups": 1, "rows": "tokens"}, "calls": [
                {"op": "embed", "args": [{"buf": "ids"}, {"buf": "emb"}, {"buf": "x"}, {"var": "tokens"}]},
                {"op": "attn", "label": "layer.0", "args": [{"buf": "x"}, {"buf": "slots"}, {"buf": "table"}, {"state": "kv"}, {"buf": "y"}]},
                {"op": "head", "args": [{"buf": "y"}, {"buf": "next"}]},
            ]},
            "decode": {"batch": {"groups": 8, "rows": 1}, "graph": True, "calls": [
                {"op": "embed", "args": [{"buf": "ids"}, {"buf": "emb"}, {"buf": "x"}, {"var": "tokens"}]},
                {"op": "attn", "args": [{"buf": "x"}, {"buf": "slots"}, {"buf": "table"}, {"state": "kv"}, {"buf": "y"}]},
                {"op": "head", "args": [{"buf": "y"}, {"buf": "next"}]},
            ]},
        },
    }


def verify(doc, **kw):
    m, errs = N.verify(json.dumps(doc), **kw)
    return m, errs


def expect(doc, needle):
    m, errs = verify(doc)
    assert m is None, "expected a rejection"
    assert any(needle in e for e in errs), f"no diagnostic contains {needle!r}: {errs}"


def test_base_verifies_and_roundtrips():
    m, errs = verify(base())
    assert m is not None, errs
    again, errs2 = N.verify(m.to_json())
    assert again is not None, errs2
    assert json.loads(again.to_json()) == json.loads(m.to_json())


def edit(path, value=None, delete=False):
    d = base()
    cur = d
    for k in path[:-1]:
        cur = cur[k]
    if delete:
        del cur[path[-1]]
    else:
        cur[path[-1]] = value
    return d


CASES = [
    (edit(["schema_version"], 6), "unsupported schema_version"),
    (edit(["vars", "tokens", "max"], 0), "max must be >= 1"),
    (edit(["vars", "extra"], {"max": 4, "axis": "rows"}), "all count the `rows` axis"),
    (edit(["vars", "spare"], {"max": 4}), "var `spare` is never used"),
    (edit(["surprise"], 1), "unknown field `surprise`"),
    (edit(["buffers", "x", "colour"], "red"), "unknown field `colour`"),
    (edit(["states", "kv"], {}), "one of bytes_per_token / bytes / bytes_per_seq / host must be set"),
    (edit(["states", "kv"], {"bytes_per_token": 4, "bytes": 4}), "are exclusive"),
    (edit(["states", "idle"], {"bytes": 16}), "state `idle` is never used"),
    (edit(["buffers", "x", "shape"], ["nope", 32]), "unknown var `nope`"),
    (edit(["buffers", "ids", "dtype"], "f32"), "fill `token` needs an i32 or i64 buffer"),
    (edit(["buffers", "next", "fill"], "token"), "written into an input but the buffer is output"),
    (edit(["buffers", "x", "fill"], "token"), "a fill sits on an input or output"),
    (edit(["buffers", "slots", "domain"], {"index_into": "kv", "min": 0}), "mutually exclusive"),
    (edit(["buffers", "slots", "domain"], {"index_into": "ghost"}), "unknown buffer/state `ghost`"),
    (edit(["buffers", "slots", "domain"], {}), "empty (declare bounds"),
    (edit(["buffers", "slots", "domain"], {"min": 5, "max": 1}), "min 5"),
    (edit(["buffers", "emb", "bind"], []), "binds at least one checkpoint tensor"),
    (edit(["buffers", "x", "bind"], [{"tensor": "t"}]), "names checkpoint tensors for a weight or a source"),
    (edit(["buffers", "emb", "bind"], [{"tensor": "t", "rows": [4, 4]}]), "rows [4, 4) is empty"),
    (edit(["buffers", "x", "of"], "y"), "`of` only applies to peer buffers"),
    (edit(["buffers", "unused"], {"dtype": "f32", "shape": [4], "kind": "workspace"}), "buffer `unused` is never used"),
    (edit(["modules", "k", "sha256"], "xyz"), "is not 64 hex chars"),
    (edit(["modules", "k", "source"], "ftp://x/y"), "only https:// and hf: sources"),
    (edit(["modules", "spare"], {"source": "s.cubin", "sha256": SHA}), "module `spare` is never launched"),
    (edit(["ops", "embed", "impl", "launches", 0, "module"], "ghost"), "unknown module `ghost`"),
    (edit(["ops", "embed", "impl", "launches", 0, "block"], [2048, 1, 1]), "exceeds 1024 threads"),
    (edit(["ops", "embed", "impl", "launches", 0, "block"], [1, 1, 128]), "block.z 128 > 64"),
    (edit(["ops", "embed", "impl", "launches", 0, "grid"], [{"mul": ["tokens", 100000000]}, 1, 1]), "exceeds CUDA limit"),
    (edit(["ops", "embed", "impl", "launches", 0, "grid"], [0, 1, 1]), "evaluates to 0 at var upper bounds"),
    (edit(["ops", "embed", "impl", "launches", 0, "shared_mem"], 300000), "exceeds opt-in limit"),
    (edit(["ops", "embed", "impl", "launches", 0, "cluster"], [4, 8, 1]), "more than 16 blocks"),
    (edit(["ops", "embed", "impl", "launches", 0, "cluster"], [2, 1, 1]), "is not a multiple of cluster.x"),
    (edit(["ops", "embed", "impl", "launches", 0, "when"], {"var": "seqs", "min": 5, "max": 2}), "is empty"),
    (edit(["ops", "embed", "impl", "launches", 0, "entry"], "extern:foo"), "an extern entry has no module"),
    (edit(["ops", "embed", "impl", "launches"], []), "implementation has no launches"),
    (edit(["ops", "embed", "impl", "launches", 0, "args"], [{"param": 0}]), "takes 4 params, got 1 args"),
    (edit(["ops", "embed", "impl", "launches", 0, "params"],
          ["inout buffer<i64>", "in buffer<bf16>", "out buffer<bf16>", "i32"]), "writes through interface `in` param #0"),
    (edit(["ops", "embed", "params"], ["in buffer<i64>", "in buffer<bf16>", "out buffer<bf16>", "bytes<8>"]), "byte aggregate"),
    (edit(["ops", "attn", "impl", "launches", 0, "args"], [{"param": 0}, {"param": 1}, {"param": 3}, {"param": 4}]),
     "does not match launch param"),
    (edit(["ops", "attn", "impl", "scratch", "more"], {"dtype": "f32", "shape": [4]}), "scratch `more` is never used"),
    (edit(["ops", "head", "impl", "launches", 0, "params"], ["in buffer<bf16>", "in buffer<i64>"]), "read before any launch wrote it"),
    (edit(["ops", "spare"], {"params": ["i32"], "impl": {"launches": [{"module": "k", "entry": "e", "block": [1, 1, 1], "grid": [1, 1, 1]}]}}),
     "op `spare` is never called"),
    (edit(["programs", "decode", "calls", 0, "op"], "ghost"), "unknown op `ghost`"),
    (edit(["programs", "decode", "calls", 0, "args"], [{"buf": "ids"}]), "takes 4 params, got 1 args"),
    (edit(["programs", "decode", "calls", 0, "args", 1], {"buf": "x"}), "is read before ever being written"),
    (edit(["programs", "decode", "calls", 0, "args", 2], {"buf": "emb"}), "op writes to read-only weight buffer"),
    (edit(["programs", "decode", "calls", 0, "args", 0], {"buf": "table"}), "has dtype i32 but param expects i64"),
    (edit(["programs", "decode", "calls", 0, "args", 2], {"buf": "x", "offset": 3}), "is not 2-aligned"),
    (edit(["programs", "decode", "calls", 0, "args", 2], {"buf": "x", "offset": 1 << 20}), "is outside buffer `x`"),
    (edit(["programs", "decode", "calls", 0, "args", 3], {"f32": 1.0}), "does not match param `i32`"),
    (edit(["programs", "decode", "calls", 0, "args", 3], {"expr": {"mul": ["tokens", 1 << 40]}}), "exceeding i32 range"),
    (edit(["programs", "decode", "calls", 1, "args", 3], {"state": "ghost"}), "unknown state `ghost`"),
    (edit(["programs", "decode", "once"], True), "are exclusive"),
    (edit(["programs", "decode", "batch"], delete=True), "`graph` (captured per call shape) needs a `batch`"),
    (edit(["programs", "decode", "batch", "groups"], 0), "batch.groups must be >= 1"),
    (edit(["programs", "decode", "batch", "rows"], "ghost"), "batch.rows names unknown var `ghost`"),
    (edit(["programs", "decode", "calls", 0, "lane"], 2), "lanes are numbered densely"),
    (edit(["chat"], {"tool_parser": "Bad-Name"}), "lowercase letters, digits and underscores"),
    (edit(["cut"], {"id": "", "stage": 3, "stages": 2}), "a cut has an id"),
]


@pytest.mark.parametrize("doc,needle", CASES, ids=[c[1][:40] for c in CASES])
def test_rejections(doc, needle):
    expect(doc, needle)


def test_every_error_is_reported_at_once():
    d = base()
    d["vars"]["tokens"]["max"] = 0
    d["modules"]["k"]["sha256"] = "zz"
    d["programs"]["decode"]["calls"][0]["op"] = "ghost"
    _, errs = verify(d)
    assert len(errs) >= 3


def test_duplicate_key_and_constants():
    text = json.dumps(base())
    dup = text.replace('"model": "unit"', '"model": "unit", "model": "again"')
    m, errs = N.verify(dup)
    assert m is None and "duplicate key" in errs[0]
    d = base()
    d["constants"] = {"HID": 32, "PAGE": 16}
    d["buffers"]["x"]["shape"] = ["tokens", "HID"]
    d["buffers"]["table"]["domain"]["stride"] = "PAGE"
    m, errs = verify(d)
    assert m is not None, errs
    out = json.loads(m.to_json())
    assert out["buffers"]["x"]["shape"] == ["tokens", 32] and out["buffers"]["table"]["domain"]["stride"] == 16
    d["constants"]["tokens"] = 4
    _, errs = verify(d)
    assert any("conflicts with a var" in e for e in errs)


def topo():
    d = base()
    d["topology"] = {"groups": {"tp": 2}}
    d["buffers"]["x"]["export"] = True
    d["buffers"]["xp"] = {"dtype": "u64", "shape": [2], "kind": "peer", "of": "x", "group": "tp"}
    d["ops"]["ar"] = {"params": ["inout buffer<bf16>", "in buffer<u64>", "i32"],
                      "impl": {"launches": [{"module": "k", "entry": "ar", "block": [32, 1, 1], "grid": [1, 1, 1]}]}}
    d["programs"]["decode"]["calls"].insert(1, {"op": "ar", "args": [{"buf": "x"}, {"buf": "xp"}, {"rank": "tp"}]})
    return d


def test_topology_peer_and_multicast_declaration():
    m, errs = verify(topo())
    assert m is not None, errs
    # strict mode: a module of a multi-rank manifest must declare that it is multicast-free
    m, errs = verify(topo(), strict_multicast=True)
    assert m is None and any("must declare `multicast: false`" in e for e in errs)
    d = topo()
    d["modules"]["k"]["multicast"] = False
    m, errs = verify(d, strict_multicast=True)
    assert m is not None, errs
    d["modules"]["k"]["multicast"] = True
    _, errs = verify(d)
    assert any("the only declarable value is false" in e for e in errs)


@pytest.mark.parametrize("mut,needle", [
    (lambda d: d["buffers"]["xp"].update(dtype="i64"), "dtype must be u64"),
    (lambda d: d["buffers"]["xp"].update(shape=[3]), "has shape [2], one address per member"),
    (lambda d: d["buffers"]["xp"].update(of="y"), "is not exported"),
    (lambda d: d["buffers"]["xp"].update(of="xp"), "cannot be `of` itself"),
    (lambda d: d["buffers"]["xp"].update(group="ep"), "unknown topology group `ep`"),
    (lambda d: d["topology"]["groups"].update(ep=4), "topology group `ep` is never used"),
    (lambda d: d["ops"]["ar"]["impl"]["launches"].append({"entry": "extern:nccl_allreduce_bf16", "params": ["inout buffer<bf16>"], "args": [{"param": 0}]}),
     "runtime built-ins never receive peer memory"),
    (lambda d: d["states"]["kv"].update(shard={"by": "heads", "group": "tp", "segments": [[1, 64]]}), "splits a per-sequence state"),
    (lambda d: d["programs"]["decode"]["calls"][1].update(lane=1, after=[0]), "cross-rank work stays on lane 0"),
])
def test_multi_rank_rules(mut, needle):
    d = topo()
    mut(d)
    expect(d, needle)


def test_pack_and_tensormap_rules():
    d = base()
    d["ops"]["embed"]["impl"]["launches"][0].update(
        params=["in buffer<i64>", "bytes<192>", "i32"],
        args=[{"param": 0},
              {"pack": {"size": 192, "fields": [
                  {"at": 0, "tensormap": {"param": 1, "dtype": "bf16", "dims": [32, 256], "strides": [64], "box": [32, 64], "swizzle": 64}},
                  {"at": 128, "param": 2}, {"at": 136, "var": "tokens"}]}},
              {"param": 3}])
    m, errs = verify(d)
    assert m is not None, errs

    def with_tm(**kw):
        dd = copy.deepcopy(d)
        dd["ops"]["embed"]["impl"]["launches"][0]["args"][1]["pack"]["fields"][0]["tensormap"].update(kw)
        return dd

    expect(with_tm(strides=[60]), "not a positive multiple of 16")
    expect(with_tm(box=[32, 512]), "must be 1..=256")
    expect(with_tm(box=[64, 64]), "more than the 64 byte swizzle span")
    expect(with_tm(dims=[32, 4096]), "addresses")            # footprint beyond the bound buffer
    expect(with_tm(param=3), "which is not a buffer or state")
    dd = copy.deepcopy(d)
    dd["ops"]["embed"]["impl"]["launches"][0]["args"][1]["pack"]["fields"][1]["at"] = 100
    expect(dd, "overlaps")
    dd = copy.deepcopy(d)
    dd["ops"]["embed"]["impl"]["launches"][0]["args"][1]["pack"]["fields"][0]["at"] = 32
    expect(dd, "not 64-byte aligned")
    dd = copy.deepcopy(d)
    dd["ops"]["embed"]["impl"]["launches"][0]["args"][1]["pack"]["size"] = 128
    expect(dd, "bound to a `bytes<192>` param")


def test_protocol_projection():
    m, _ = verify(base())
    p = json.loads(m.protocol())
    assert p["rows"] == {"var": "tokens", "max": 64} and p["groups"] == {"var": "seqs", "max": 8}
    fills = {f["fill"]: f for f in p["fills"]}
    assert fills["token"]["axis"] == "rows" and fills["tokens"]["axis"] == "groups" and fills["slot"]["dtype"] == "i64"
    assert p["page_tables"] == [{"name": "table", "width": 4, "state": "kv", "stride": 16}]
    fw = {f["name"]: f for f in p["forwards"]}
    assert fw["decode"]["rows"] == 1 and fw["decode"]["groups"] == 8 and fw["decode"]["graph"] and fw["decode"]["emits"] == "next"
    assert fw["prefill"]["rows"] == "var"

    def perr(mut, needle):
        d = base()
        mut(d)
        mm, errs = verify(d)
        assert mm is not None, errs
        with pytest.raises(ValueError, match=needle):
            mm.protocol()

    perr(lambda d: d["vars"]["tokens"].pop("axis"), "no var has `axis: rows`")
    perr(lambda d: d["programs"]["decode"]["batch"].update(groups=80), "exceed")
    perr(lambda d: d["buffers"]["table"].update(dtype="i64") or d["ops"]["attn"]["params"].__setitem__(2, "in buffer<i64>")
         or d["ops"]["attn"]["impl"]["launches"][1]["params"].__setitem__(1, "in buffer<i64>"),
         "hands out i32 page and line indices")
    perr(lambda d: d["buffers"].update(temp={"dtype": "f32", "shape": ["seqs"], "kind": "input", "fill": "temperature"})
         or d["ops"]["head"]["params"].append("in buffer<f32>") or [c["args"].append({"buf": "temp"}) for p in d["programs"].values() for c in p["calls"] if c["op"] == "head"],
         "come together, all or none")


def test_lanes_happens_before():
    def laned(calls_edit):
        d = base()
        d["buffers"]["z"] = {"dtype": "bf16", "shape": ["tokens", 32], "kind": "workspace"}
        d["ops"]["copy"] = {"params": ["in buffer<bf16>", "out buffer<bf16>"],
                            "impl": {"launches": [{"module": "k", "entry": "cp", "block": [32, 1, 1], "grid": ["tokens", 1, 1]}]}}
        calls = d["programs"]["decode"]["calls"]
        # embed(x) ; [lane1: copy x->z] || attn x->y ; head(y) joins ; copy z -> y? keep simple
        calls.insert(1, {"op": "copy", "args": [{"buf": "x"}, {"buf": "z"}], "lane": 1, "after": [0]})
        calls.append({"op": "copy", "args": [{"buf": "z"}, {"buf": "x"}], "after": [1]})
        calls_edit(calls)
        return d

    m, errs = verify(laned(lambda c: None))
    assert m is not None, errs
    expect(laned(lambda c: c[-1].pop("after")), "is never joined")
    expect(laned(lambda c: c[1].pop("after")), "a side lane's first call names the lanes it runs `after`")
    expect(laned(lambda c: c[1]["args"].__setitem__(1, {"buf": "y"})), "neither runs after the other")
    expect(laned(lambda c: c[1].update(after=[1])), "names its own lane")


def test_cut_into_stages():
    d = base()
    # two layers with one state each, so each stage keeps its own
    d["states"]["kv2"] = {"bytes_per_token": 64}
    for p in d["programs"].values():
        p["calls"].insert(2, {"op": "attn", "label": "layer.1", "args": [{"buf": "y"}, {"buf": "slots"}, {"buf": "table"}, {"state": "kv2"}, {"buf": "x"}]})
        p["calls"][3]["args"][0] = {"buf": "x"}
    m, errs = verify(d)
    assert m is not None, errs
    stages = m.cut([2])
    assert len(stages) == 2
    s0, s1 = (json.loads(s.to_json()) for s in stages)
    assert s0["cut"]["stage"] == 0 and s1["cut"]["stages"] == 2 and s0["cut"]["id"] == s1["cut"]["id"]
    assert s0["buffers"]["y"]["kind"] == "output" and s1["buffers"]["y"]["kind"] == "input" and s1["buffers"]["y"]["export"]
    assert set(s0["states"]) == {"kv"} and set(s1["states"]) == {"kv2"}
    assert s1["buffers"]["table"]["domain"]["index_into"] == "kv2"      # re-pointed at the kept state
    assert "ids" not in s1["buffers"] and "next" not in s0["buffers"]
    with pytest.raises(ValueError, match="cannot be cut before call"):
        m.cut([9])
    with pytest.raises(ValueError, match="belongs to one stage"):
        base_m, _ = verify(base_two_calls_same_state())
        base_m.cut([2])


def base_two_calls_same_state():
    d = base()
    for p in d["programs"].values():
        p["calls"].insert(2, {"op": "attn", "args": [{"buf": "y"}, {"buf": "slots"}, {"buf": "table"}, {"state": "kv"}, {"buf": "x"}]})
        p["calls"][3]["args"][0] = {"buf": "x"}
    return d


def test_candidate_splice():
    m, _ = verify(base())
    cand = {"modules": {"k": {"source": "other.cubin", "sha256": "cd" * 32}},
            "ops": {"head": {"params": ["in buffer<bf16>", "out buffer<i64>"],
                             "impl": {"launches": [{"module": "k", "entry": "head_v2", "block": [64, 1, 1], "grid": ["seqs", 1, 1]}]}}}}
    out = json.loads(m.splice(json.dumps(cand)).to_json())
    assert out["ops"]["head"]["impl"]["launches"][0]["entry"] == "head_v2"
    renamed = out["ops"]["head"]["impl"]["launches"][0]["module"]
    assert renamed == "k@cdcdcdcd" and out["modules"][renamed]["source"] == "other.cubin" and "k" in out["modules"]
    cand["ops"]["head"]["params"] = ["in buffer<bf16>", "out buffer<i32>"]
    with pytest.raises(ValueError, match="are not the manifest's"):
        m.splice(json.dumps(cand))


def test_values_codecs():
    assert N.decode_values("bf16", N.encode_values("bf16", [1.0, -2.5, 0.1]))[:2] == [1.0, -2.5]
    assert N.decode_values("fp8e4m3", N.encode_values("fp8e4m3", [448.0, 1000.0, -0.5])) == [448.0, 448.0, -0.5]
    assert N.decode_values("fp8e8m0", N.encode_values("fp8e8m0", [1.0, 8.0, 0.25])) == [1.0, 8.0, 0.25]
    assert N.decode_values("f16", N.encode_values("f16", [0.5, 65504.0, 6e-8]))[:2] == [0.5, 65504.0]
    a, b = N.encode_values("f32", [1.0]), N.encode_values("f32", [1.0000001])
    assert N.ulp_distance("f32", a, b) == 1 and N.ulp_distance("f32", a, a) == 0
    z = N.ulp_distance("bf16", N.encode_values("bf16", [0.0]), N.encode_values("bf16", [-0.0]))
    assert z == 0


def test_registry_refs():
    assert N.registry_url("hf:org/repo/a/b.cubin@v1") == "https://huggingface.co/org/repo/resolve/v1/a/b.cubin"
    assert N.registry_url("hf:org/repo/x.cubin") == "https://huggingface.co/org/repo/resolve/main/x.cubin"
    assert N.registry_url("local.cubin") is None
    with pytest.raises(ValueError):
        N.registry_url("hf:org/repo")


@pytest.mark.skipif(not os.path.isdir(REF), reason="reference fixtures are not mounted")
def test_reference_fixtures_verify_in_milliseconds():
    files = [REF + "/examples/minimal.json"] + sorted(glob.glob(REF + "/crates/kern-manifest/tests/fixtures/**/*.json", recursive=True))
    assert len(files) >= 6
    for f in files:
        text = open(f).read()
        m, errs = N.verify(text)
        assert m is not None, (f, errs[:3])
        if f.endswith("k3/head.json"):
            assert N.verify_seconds(text, 3) < 0.05     # 570 kB, thousands of calls
            assert json.loads(m.protocol(sampled=False))["forwards"]
