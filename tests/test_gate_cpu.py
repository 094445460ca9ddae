"""The serving gate (`kern gate`) on the host-memory executor: every scenario passes for a paged-KV decoder and for the
exact integer model with a per-sequence state slot (whose repeat hit needs the turn-boundary snapshot)."""
import pytest

from kern_b200 import cli


@pytest.mark.parametrize("model", ["toy", "toy-int-stateful", "tiny-latent"])
def test_gate_passes(model, capsys):
    assert cli.main(["gate", "--model", model, "--cpu"]) == 0
    out = capsys.readouterr().out
    assert "10 of 10 scenarios pass" in out and "FAIL" not in out


def test_gate_names_a_failure(capsys):
    """A pool too small for the scenarios' prompts: the scenario that cannot run is reported, not raised."""
    assert cli.main(["gate", "--model", "toy", "--cpu", "--capacity", "32", "--only", "conc1_equals_run"]) == 1
    assert "FAIL conc1_equals_run" in capsys.readouterr().out


def test_gate_spec_acceptance_on_a_package_with_rounds():
    """A target with a one-layer draft: round-by-round serving gives the tokens of one row per step, alone and in a
    burst, and proposals are being made (the acceptance rate itself is the draft's business)."""
    import dataclasses

    from kern_b200.cpu import CpuRuntime
    from kern_b200.engine import Engine
    from kern_b200.models import dense, spec
    from kern_b200.testing.gate import Gate

    T = dataclasses.replace(dense.TOY, max_tokens=64, max_seqs=4)
    w = spec.random_weights(T, None, seed=7, std=0.08)
    doc = spec.build_manifest(T, None, k=3)

    def make(tokens):
        rt = CpuRuntime(doc, weights=w, tokens=tokens)
        rt.once()
        return Engine(rt)

    g = Gate(make, T.vocab, T.page_size, T.page_size * 30, out_tokens=4)
    r = g.spec_acceptance()
    assert r.ok and "acceptance" in r.detail, r.line()
    assert g.kept_nothing().ok
