"""The JSON Schema of the manifest wire format: the committed golden is what the generator writes, every built-in
manifest (and the C++ parser's own fixtures) has that shape, and shape errors are named with their path."""
import copy
import json

from kern_b200 import schema


def test_golden_is_up_to_date():
    assert schema.check_golden(), "run `python -m kern_b200 schema --write` and commit schema/manifest-v7.schema.json"
    doc = json.loads(schema.GOLDEN.read_text())
    assert doc["properties"]["schema_version"] == {"const": 7} and "launch_arg" in doc["$defs"]


def test_every_builtin_manifest_has_the_shape():
    from kern_b200.models import dense_tp, moe_ep, registry, spec

    sch = schema.schema()
    for name, (cfg, build, *_rest) in registry.families().items():
        if name in ("dense-8b", "hybrid-27b", "moe-30b-a3b"):
            continue      # the small configs of each family cover the same generators
        assert schema.validate(build(cfg), sch) == [], name
    from kern_b200.models import dense
    import dataclasses
    assert schema.validate(dense_tp.build_manifest_tp(dataclasses.replace(dense.TINY, tp=2)), sch) == []
    from kern_b200.parallel.coll_check import manifest as coll
    from kern_b200.testing.extern_gemm import manifest as ext
    assert schema.validate(coll(2, 64), sch) == [] and schema.validate(ext(64, 96, 128), sch) == []


def test_shape_errors_carry_their_path():
    from kern_b200.models import dense

    good = dense.build_manifest(dense.TINY)
    sch = schema.schema()
    bad = copy.deepcopy(good)
    bad["vars"]["tokens"]["axis"] = "cols"
    name = next(iter(bad["buffers"]))
    bad["buffers"][name]["surprise"] = 1
    bad["programs"]["decode"]["calls"][0]["args"][0] = {"buf": "x", "var": "tokens"}
    errs = schema.validate(bad, sch)
    assert any(e.startswith("/vars/tokens/axis") for e in errs)
    assert any(e.startswith(f"/buffers/{name}") and "surprise" in e for e in errs)
    assert any(e.startswith("/programs/decode/calls/0/args/0") for e in errs)
    assert len(errs) == 3, errs


def test_cli_check_and_validate(tmp_path, capsys):
    from kern_b200 import cli
    from kern_b200.models import dense

    assert cli.main(["schema", "--check"]) == 0
    p = tmp_path / "m.json"
    p.write_text(json.dumps(dense.build_manifest(dense.TINY)))
    assert cli.main(["schema", "--validate", str(p)]) == 0
    p.write_text(json.dumps({"schema_version": 6}))
    assert cli.main(["schema", "--validate", str(p)]) == 1
    assert "schema_version" in capsys.readouterr().out
