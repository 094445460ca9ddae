"""JSON Schema of the manifest wire format (schema_version 7) and a small validator for it.

`python -m kern_b200 schema` prints the schema; `--check` compares it with the committed golden
`schema/manifest-v7.schema.json` (the continuous-integration gate: a change of the wire format must show up as a diff
of that file). The schema states the *shape* the C++ parser accepts (`csrc/manifest/parse.cpp`): field names, types,
enumerations, the one-of forms of args; what needs the whole document (names that must exist, launch geometry limits,
the race check) stays with the verifier. Numbers may everywhere be given as the name of a `constants` entry, so integer
positions also accept a string.
Reference: crates/kern-manifest/src/constants.rs:40-71 (schema generation), schema/manifest-v7.schema.json.
"""
from __future__ import annotations

import json
from pathlib import Path

GOLDEN = Path(__file__).resolve().parent.parent / "schema" / "manifest-v7.schema.json"

DTYPES = ["bf16", "f16", "f32", "fp8e4m3", "fp8e8m0", "i8", "i32", "u32", "i64", "u64", "u8"]
BUFFER_KINDS = ["input", "output", "inout", "weight", "source", "workspace", "carry", "peer"]


def _obj(props: dict, required: list[str] = (), extra=False) -> dict:
    return {"type": "object", "properties": props, "required": list(required), "additionalProperties": extra}


def _map(value: dict) -> dict:
    return {"type": "object", "additionalProperties": value}


def schema() -> dict:
    ref = lambda n: {"$ref": f"#/$defs/{n}"}
    uint = {"description": "an unsigned integer, or the name of a constant", "anyOf": [{"type": "integer", "minimum": 0}, {"type": "string"}]}
    sint = {"anyOf": [{"type": "integer"}, {"type": "string"}]}
    num = {"anyOf": [{"type": "number"}, {"type": "string"}]}
    string = {"type": "string"}
    boolean = {"type": "boolean"}
    uints = {"type": "array", "items": uint}
    defs = {
        "uint": uint,
        "dtype": {"type": "string", "enum": DTYPES},
        "dim": {"description": "an extent: a constant or the name of a var", "anyOf": [{"type": "integer", "minimum": 0}, string]},
        "expr": {
            "description": "an integer, a var name, or one of ceil_div / mul / add / clamp over sub-expressions",
            "anyOf": [
                {"type": "integer", "minimum": 0}, string,
                _obj({"ceil_div": {"type": "array", "prefixItems": [ref("expr"), uint], "minItems": 2, "maxItems": 2}}, ["ceil_div"]),
                _obj({"mul": {"type": "array", "prefixItems": [ref("expr"), uint], "minItems": 2, "maxItems": 2}}, ["mul"]),
                _obj({"add": {"type": "array", "items": ref("expr"), "minItems": 2, "maxItems": 2}}, ["add"]),
                _obj({"clamp": {"type": "array", "prefixItems": [ref("expr"), uint, uint], "minItems": 3, "maxItems": 3}}, ["clamp"]),
            ]},
        "param_type": {"type": "string", "description": "`in|out|inout buffer<dtype>`, `in|inout state`, a scalar dtype, or `bytes<n>`"},
        "var": _obj({"max": uint, "axis": {"type": "string", "enum": ["rows", "groups", "ranks"]}}, ["max"]),
        "host_tensor": _obj({"dtype": ref("dtype"), "shape": uints, "strides": uints}, ["dtype", "shape", "strides"]),
        "shard": _obj({"by": {"type": "string", "enum": ["position", "heads"]}, "group": string,
                       "segments": {"type": "array", "items": {"type": "array", "items": uint, "minItems": 2, "maxItems": 2}}},
                      ["by", "group"]),
        "state": _obj({"bytes_per_token": uint, "bytes": uint, "bytes_per_seq": uint, "host": ref("host_tensor"), "shard": ref("shard")}),
        "tensor_source": {"anyOf": [string, _obj({"group": string, "tensors": {"type": "array", "items": string}}, ["group", "tensors"])]},
        "ranges": {"anyOf": [{"type": "array", "items": uint, "minItems": 2, "maxItems": 2},
                             _obj({"group": string, "ranges": {"type": "array", "items": {"type": "array", "items": uint, "minItems": 2, "maxItems": 2}}},
                                  ["group", "ranges"])]},
        "segment": _obj({"tensor": ref("tensor_source"), "rows": ref("ranges"), "cols": ref("ranges"),
                         "interleave": _obj({"with": ref("tensor_source"), "rows": uint}, ["with", "rows"])}, ["tensor"]),
        "bound": {"anyOf": [{"type": "number"}, string]},
        "domain": _obj({"min": ref("bound"), "max": ref("bound"), "index_into": string, "stride": uint, "monotone": boolean}),
        "buffer": _obj({"dtype": ref("dtype"), "shape": {"type": "array", "items": ref("dim")}, "kind": {"type": "string", "enum": BUFFER_KINDS},
                        "placement": {"type": "string", "enum": ["device", "host"]}, "fill": string, "domain": ref("domain"),
                        "export": boolean, "of": string, "group": string, "bind": {"type": "array", "items": ref("segment")}},
                       ["dtype", "shape", "kind"]),
        "module": _obj({"source": string, "sha256": string, "multicast": {"const": False}}, ["source", "sha256"]),
        "tensormap": _obj({"param": uint, "dtype": string, "dims": uints, "strides": uints, "box": uints, "swizzle": uint,
                           "l2_promotion": uint, "oob_nan": boolean, "wrap": boolean}, ["param", "dtype", "dims", "box"]),
        "pack_field": _obj({"at": uint, "width": uint, "param": uint, "scratch": string, "var": string, "expr": ref("expr"),
                            "rank": string, "tensormap": ref("tensormap"), "i32": sint, "i64": sint, "f32": num, "u8": uint}, ["at"]),
        "pack": _obj({"size": uint, "fields": {"type": "array", "items": ref("pack_field")}}, ["size", "fields"]),
        "launch_arg": {
            "description": "exactly one of param | scratch | i32 | i64 | f32 | u8 | rank | pack",
            "oneOf": [_obj({k: v}, [k]) for k, v in (("param", uint), ("scratch", string), ("i32", sint), ("i64", sint), ("f32", num),
                                                    ("u8", uint), ("rank", string), ("pack", ref("pack")))]},
        "when": _obj({"var": string, "min": uint, "max": uint}, ["var"]),
        "algo": _obj({k: (sint if k in ("id", "split_k") else uint) for k in
                      ("id", "tile", "stages", "split_k", "reduction", "swizzle", "custom", "inner_shape", "cluster_shape")},
                     ["id", "tile", "stages", "split_k", "reduction", "swizzle", "custom", "inner_shape", "cluster_shape"]),
        "launch": _obj({"module": string, "entry": string, "params": {"type": "array", "items": ref("param_type")}, "when": ref("when"),
                        "args": {"type": "array", "items": ref("launch_arg")}, "algo": ref("algo"),
                        "block": {"type": "array", "items": uint, "minItems": 3, "maxItems": 3},
                        "grid": {"type": "array", "items": ref("expr"), "minItems": 3, "maxItems": 3},
                        "shared_mem": ref("expr"), "cluster": {"type": "array", "items": uint, "minItems": 3, "maxItems": 3},
                        "pdl": boolean}, ["entry"]),
        "scratch": _obj({"dtype": ref("dtype"), "shape": {"type": "array", "items": ref("dim")}}, ["dtype", "shape"]),
        "op": _obj({"params": {"type": "array", "items": ref("param_type")},
                    "impl": _obj({"scratch": _map(ref("scratch")), "launches": {"type": "array", "items": ref("launch")}}, ["launches"])},
                   ["params", "impl"]),
        "arg": {
            "description": "exactly one of buf | state (each with an optional byte offset) | var | expr | rank | a literal",
            "oneOf": [_obj({"buf": string, "offset": uint}, ["buf"]), _obj({"state": string, "offset": uint}, ["state"]),
                      _obj({"var": string}, ["var"]), _obj({"expr": ref("expr")}, ["expr"]), _obj({"rank": string}, ["rank"]),
                      _obj({"i32": sint}, ["i32"]), _obj({"i64": sint}, ["i64"]), _obj({"f32": num}, ["f32"]), _obj({"u8": uint}, ["u8"])]},
        "call": _obj({"label": string, "op": string, "args": {"type": "array", "items": ref("arg")}, "lane": uint, "after": uints},
                     ["op", "args"]),
        "batch": _obj({"groups": uint, "rows": ref("dim"), "context": string}, ["groups", "rows"]),
        "program": _obj({"batch": ref("batch"), "once": boolean, "derive": boolean, "graph": boolean,
                         "calls": {"type": "array", "items": ref("call")}}, ["calls"]),
    }
    return {
        "$schema": "https://json-schema.org/draft/2020-12/schema",
        "title": "kern manifest, schema_version 7",
        **_obj({
            "schema_version": {"const": 7}, "model": string, "constants": _map({"type": "number"}),
            "chat": _obj({"tool_parser": string}), "vars": _map(ref("var")),
            "topology": _obj({"groups": _map(uint)}, ["groups"]),
            "cut": _obj({"id": string, "stage": uint, "stages": uint}, ["id", "stage", "stages"]),
            "states": _map(ref("state")), "buffers": _map(ref("buffer")), "modules": _map(ref("module")),
            "ops": _map(ref("op")), "programs": _map(ref("program")),
        }, ["schema_version", "model", "vars", "states", "buffers", "modules", "ops", "programs"]),
        "$defs": defs,
    }


def text() -> str:
    return json.dumps(schema(), indent=1, sort_keys=False) + "\n"


# ---- a validator for the subset of JSON Schema used above ---------------------------------------------------------------
def validate(doc, sch: dict | None = None) -> list[str]:
    """Every violation as `path: message` (an empty list: the document has the shape of a manifest)."""
    root = sch or schema()
    errs: list[str] = []

    def typed(v, t: str) -> bool:
        if t == "object": return isinstance(v, dict)
        if t == "array": return isinstance(v, list)
        if t == "string": return isinstance(v, str)
        if t == "boolean": return isinstance(v, bool)
        if t == "integer": return isinstance(v, int) and not isinstance(v, bool)
        if t == "number": return isinstance(v, (int, float)) and not isinstance(v, bool)
        return True

    def check(v, s: dict, path: str, out: list[str]) -> None:
        if "$ref" in s:
            return check(v, root["$defs"][s["$ref"].rsplit("/", 1)[1]], path, out)
        if "const" in s and v != s["const"]:
            out.append(f"{path}: expected {s['const']!r}")
        if "type" in s and not typed(v, s["type"]):
            out.append(f"{path}: expected {s['type']}")
            return
        if "enum" in s and v not in s["enum"]:
            out.append(f"{path}: `{v}` is not one of {', '.join(s['enum'])}")
        if "minimum" in s and isinstance(v, (int, float)) and v < s["minimum"]:
            out.append(f"{path}: below {s['minimum']}")
        for key in ("anyOf", "oneOf"):
            if key in s:
                fits = 0
                for alt in s[key]:
                    sub: list[str] = []
                    check(v, alt, path, sub)
                    fits += not sub
                if fits == 0 or (key == "oneOf" and fits != 1):
                    out.append(f"{path}: {s.get('description') or ('matches %d of the allowed forms' % fits)}")
        if isinstance(v, dict) and ("properties" in s or "additionalProperties" in s):
            props = s.get("properties", {})
            for r in s.get("required", []):
                if r not in v:
                    out.append(f"{path}: missing field `{r}`")
            extra = s.get("additionalProperties", True)
            for k, x in v.items():
                if k in props:
                    check(x, props[k], f"{path}/{k}", out)
                elif extra is False:
                    out.append(f"{path}: unknown field `{k}`")
                elif isinstance(extra, dict):
                    check(x, extra, f"{path}/{k}", out)
        if isinstance(v, list):
            if "minItems" in s and len(v) < s["minItems"] or "maxItems" in s and len(v) > s["maxItems"]:
                out.append(f"{path}: expected {s.get('minItems', 0)}..{s.get('maxItems', 'any')} items")
            pre = s.get("prefixItems", [])
            for i, x in enumerate(v):
                if i < len(pre):
                    check(x, pre[i], f"{path}/{i}", out)
                elif "items" in s:
                    check(x, s["items"], f"{path}/{i}", out)

    check(doc, root, "", errs)
    return errs


def check_golden() -> bool:
    return GOLDEN.exists() and GOLDEN.read_text() == text()


def write_golden() -> Path:
    GOLDEN.parent.mkdir(exist_ok=True)
    GOLDEN.write_text(text())
    return GOLDEN
