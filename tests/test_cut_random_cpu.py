"""A cut changes a stage's signature, never its arithmetic. 400 random straight-line manifests (opaque ops over a few
workspaces, an input, an output and one state per layer) are cut at every position the library accepts; run
symbolically — an op's output is a hash of its name and of what it read — the stages, each fed what the stage before
holds under the names it takes in, must compute exactly what the whole manifest computes, and every state must live
in exactly one stage. Model for this test: crates/kern-manifest/tests/cut.rs (same idea, own generator and machine)."""
import json
import random

from kern_b200 import _native as N

SHA = "ab" * 32
OPS = {
    "f1": ["in buffer<bf16>", "out buffer<bf16>"],
    "f2": ["in buffer<bf16>", "in buffer<bf16>", "out buffer<bf16>"],
    "g": ["inout buffer<bf16>"],
    "sw": ["in buffer<bf16>", "inout state"],
    "sr": ["in state", "in buffer<bf16>", "out buffer<bf16>"],
}


def random_manifest(rng: random.Random) -> dict:
    ws = ["w0", "w1", "w2", "w3"]
    layers = rng.randint(2, 5)
    readable = ["x"]
    calls = []

    def pick():
        return rng.choice(readable)

    first = rng.choice(ws)
    calls.append({"op": "f1", "args": [{"buf": "x"}, {"buf": first}]})
    readable.append(first)
    for layer in range(layers):
        for _ in range(rng.randint(1, 4)):
            kind = rng.choice(["f1", "f2", "g", "sw", "sr"])
            out = rng.choice(ws)
            st = {"state": f"s{layer}"}
            if kind == "f1":
                c = {"op": "f1", "args": [{"buf": pick()}, {"buf": out}]}
            elif kind == "f2":
                c = {"op": "f2", "args": [{"buf": pick()}, {"buf": pick()}, {"buf": out}]}
            elif kind == "g":
                c = {"op": "g", "args": [{"buf": rng.choice(readable[1:])}]}
            elif kind == "sw":
                c = {"op": "sw", "args": [{"buf": pick()}, st]}
            else:
                c = {"op": "sr", "args": [st, {"buf": pick()}, {"buf": out}]}
            if kind in ("f1", "f2", "sr") and out not in readable:
                readable.append(out)
            c["label"] = f"l{layer}.c{len(calls)}"
            calls.append(c)
    calls.append({"op": "f1", "label": "head", "args": [{"buf": pick()}, {"buf": "y"}]})
    used_states = {a["state"] for c in calls for a in c["args"] if "state" in a}
    used_ws = {a["buf"] for c in calls for a in c["args"] if "buf" in a} & set(ws)
    bufs = {"x": {"dtype": "bf16", "shape": ["tokens", 8], "kind": "input"},
            "y": {"dtype": "bf16", "shape": ["tokens", 8], "kind": "output"}}
    for w in used_ws:
        bufs[w] = {"dtype": "bf16", "shape": ["tokens", 8], "kind": "workspace"}
    ops = {name: {"params": params, "impl": {"launches": [{"module": "k", "entry": name, "block": [32, 1, 1], "grid": ["tokens", 1, 1]}]}}
           for name, params in OPS.items() if any(c["op"] == name for c in calls)}
    return {"schema_version": 7, "model": "random", "vars": {"tokens": {"max": 16, "axis": "rows"}},
            "states": {s: {"bytes": 256} for s in used_states}, "buffers": bufs,
            "modules": {"k": {"source": "k.cubin", "sha256": SHA}}, "ops": ops, "programs": {"step": {"batch": {"groups": 1, "rows": "tokens"}, "calls": calls}}}


def h(*parts) -> int:
    x = 0xCBF29CE484222325
    for p in parts:
        for b in repr(p).encode():
            x = ((x ^ b) * 0x100000001B3) & ((1 << 64) - 1)
    return x


def run(doc: dict, mem: dict) -> None:
    """Symbolic execution of `step`: every value is a hash of how it was computed."""
    for c in doc["programs"]["step"]["calls"]:
        params = doc["ops"][c["op"]]["params"]
        key = lambda a: ("state", a["state"], a.get("offset", 0)) if "state" in a else ("buf", a["buf"])
        reads = [mem.get(key(a), h("unwritten", key(a))) for a, p in zip(c["args"], params) if p.startswith(("in ", "inout "))]
        for a, p in zip(c["args"], params):
            if p.startswith(("out ", "inout ")):
                mem[key(a)] = h(c["op"], reads, key(a)[0])


def test_every_accepted_cut_of_400_random_manifests_computes_the_whole():
    rng = random.Random(20)
    cuts_checked = refused = 0
    for i in range(400):
        doc = random_manifest(rng)
        m, errs = N.verify(json.dumps(doc), False)
        assert m is not None, (i, errs[:3])
        whole = {("buf", "x"): h("x")}
        run(doc, whole)
        ncalls = len(doc["programs"]["step"]["calls"])
        for at in range(1, ncalls):
            try:
                stages = [json.loads(s.to_json()) for s in m.cut([at])]
            except ValueError:
                refused += 1          # a state would belong to two stages, or the cut falls inside a lane
                continue
            cuts_checked += 1
            assert len(stages) == 2
            owners = [set(s["states"]) for s in stages]
            assert not (owners[0] & owners[1]) and owners[0] | owners[1] == set(doc["states"]), (i, at)
            mem = {("buf", "x"): h("x")}
            prev = None
            for s in stages:
                local = {k: v for k, v in mem.items() if k[0] == "state" and k[1] in s["states"]}
                for name, b in s["buffers"].items():
                    if b["kind"] == "input" or (b["kind"] == "inout" and b.get("export")):
                        src = ("buf", name)
                        assert src in mem, (i, at, name, "a stage takes in what nobody before it wrote")
                        local[src] = mem[src]
                run(s, local)
                # what the stage leaves: its outputs (and its states)
                for name, b in s["buffers"].items():
                    if b["kind"] in ("output", "inout"):
                        mem[("buf", name)] = local[("buf", name)]
                mem.update({k: v for k, v in local.items() if k[0] == "state"})
                prev = s
            assert mem[("buf", "y")] == whole[("buf", "y")], (i, at)
            for k, v in whole.items():
                if k[0] == "state":
                    assert mem[k] == v, (i, at, k)
    assert cuts_checked > 1500 and refused > 100, (cuts_checked, refused)
