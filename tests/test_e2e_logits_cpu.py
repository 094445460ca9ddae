"""e2e-logits: record on one engine, judge the same model (passes) and a perturbed one (fails)."""
import numpy as np

from kern_b200.cpu import CpuRuntime
from kern_b200.models import dense
from kern_b200.testing import e2e
from kern_b200.testing.abtest import EngineSide


def side(weights):
    rt = CpuRuntime(dense.build_manifest(dense.TOY), weights=weights, tokens=16 * 24)
    rt.once()
    return EngineSide(rt)


def test_record_save_load_judge(tmp_path):
    cfg = dense.TOY
    w = dense.random_weights(cfg, seed=5, std=0.08)
    qs = e2e.plan(seed=1, count=3, vocab=cfg.vocab, lengths=(5, 30), max_tokens=6)
    assert [q.id for q in qs] == ["q0", "q1", "q2"] and e2e.plan(1, 3, cfg.vocab, (5, 30), 6)[1].prompt == qs[1].prompt
    rec = e2e.record(side(w), qs, source="toy@cpu")
    path = tmp_path / "rec.parquet"
    rec.save(path)
    back = e2e.Recording.load(path)
    assert back.source == "toy@cpu" and [r["output"] for r in back.rows] == [r["output"] for r in rec.rows]
    # the noise is what the engine's own batch shapes move a distribution by: tiny on the host executor, never negative
    assert all(len(r["top_ids"]) == 6 and len(r["top_ids"][0]) == e2e.TOP and 0.0 <= r["noise"] < 1e-3 for r in back.rows)
    assert e2e.record(side(w), qs[:2], source="solo", batch=1).rows[0]["noise"] == 0.0      # alone twice: the same bits
    text, code = e2e.summary(e2e.judge(back, side(w)))
    assert code == 0 and "PASS: 3/3" in text
    # the verdict over all positions: mean KL against the recording's own noise + 3 standard errors, with the means by
    # decode step and context depth
    assert 0.0 <= back.noise_mean < 1e-4
    text, code = e2e.summary(e2e.judge(back, side(w)), noise_mean=back.noise_mean)
    last = text.splitlines()[-1]
    assert code == 0 and last.startswith("PASS      mean KL") and "over 18 scored positions" in last
    assert "mean KL by decode step" in text and "mean KL by context depth" in text
    w2 = dict(w)
    w2["lm_head.weight"] = (w["lm_head.weight"].float() + 0.2 * (np.random.default_rng(0).standard_normal(w["lm_head.weight"].shape)).astype(np.float32)).to(w["lm_head.weight"].dtype)
    text, code = e2e.summary(e2e.judge(back, side(w2)), noise_mean=back.noise_mean)
    assert code == 1 and text.splitlines()[-1].startswith("FAIL      mean KL")


def test_kl_top_is_zero_on_itself_and_positive_off():
    row = np.random.default_rng(0).standard_normal(300).astype(np.float32)
    ids, lp = e2e.top_of(row)
    assert ids[0] == int(row.argmax()) and abs(e2e.kl_top(ids, lp, row)) < 1e-9
    assert e2e.kl_top(ids, lp, row[::-1].copy()) > 0.1


def test_batched_forced_run_gives_the_rows_of_the_solo_run():
    """The decode steps of several questions as one call (and in halves) visit the same positions: the rows agree with
    the solo run's up to the rounding a batch shape brings."""
    cfg = dense.TOY
    w = dense.random_weights(cfg, seed=5, std=0.08)
    s = side(w)
    prompts = [list(range(3, 3 + n)) for n in (5, 19, 11)]
    outs, rows, _ = s.free_run(prompts, 5, 8)
    per = [rows[i * 5:(i + 1) * 5] for i in range(3)]
    for b in (3, 2):
        got = s.batched_forced_run(prompts, outs, 8, b)
        assert [len(g) for g in got] == [5, 5, 5]
        for a, g in zip(per, got):
            assert max(float(np.abs(x - y).max()) for x, y in zip(a, g)) < 1e-2
            assert [int(x.argmax()) for x in a] == [int(y.argmax()) for y in g]
