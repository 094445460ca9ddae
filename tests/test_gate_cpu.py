"""The serving gate (`kern gate`) on the host-memory executor: every scenario passes for a paged-KV decoder and for the
exact integer model with a per-sequence state slot (whose repeat hit needs the turn-boundary snapshot)."""
import pytest

from kern_b200 import cli


@pytest.mark.parametrize("model", ["toy", "toy-int-stateful", "tiny-latent"])
def test_gate_passes(model, capsys):
    assert cli.main(["gate", "--model", model, "--cpu"]) == 0
    out = capsys.readouterr().out
    assert "7 of 7 scenarios pass" in out and "FAIL" not in out


def test_gate_names_a_failure(capsys):
    """A pool too small for the scenarios' prompts: the scenario that cannot run is reported, not raised."""
    assert cli.main(["gate", "--model", "toy", "--cpu", "--capacity", "32", "--only", "conc1_equals_run"]) == 1
    assert "FAIL conc1_equals_run" in capsys.readouterr().out
