"""Pipeline parallelism on CPU: a decoder cut into stages, each stage its own runtime, activations crossing the cuts;
the pipeline must emit exactly what the uncut engine emits, under the same scheduler."""
import pytest
import torch

from kern_b200.cpu import CpuRuntime
from kern_b200.engine import Engine
from kern_b200.models import dense, hybrid, latent
from kern_b200.serve import pp
from kern_b200.serve.scheduler import Request, Scheduler


def make(cfg, build, weights, n_stages, slots=0):
    doc = build(cfg)
    at = pp.layer_cuts(doc, n_stages)
    stages_doc = pp.cut(doc, at)
    assert [d["cut"]["stage"] for d in stages_doc] == list(range(n_stages))
    stages = [CpuRuntime(d, weights=weights, tokens=cfg.page_size * 24, slots=slots) for d in stages_doc]
    for rt in stages:
        rt.once()
    whole = CpuRuntime(doc, weights=weights, tokens=cfg.page_size * 24, slots=slots)
    whole.once()
    return pp.PipelineEngine(stages, whole.protocol), Engine(whole), stages_doc


@pytest.mark.parametrize("n_stages", [2])
def test_dense_pipeline_equals_uncut(n_stages):
    cfg = dense.TOY
    w = dense.random_weights(cfg, seed=2, std=0.08)
    pipe, single, docs = make(cfg, dense.build_manifest, w, n_stages)
    # states never travel: each layer's KV lives on exactly one stage
    owned = [set(d["states"]) for d in docs]
    assert set.union(*owned) == {f"kv.l{i}" for i in range(cfg.layers)} and not set.intersection(*owned)
    torch.manual_seed(0)
    prompts = [torch.randint(1, cfg.vocab, (n,)).tolist() for n in (13, 30, 4)]
    outs = []
    for eng in (single, pipe):
        sch = Scheduler(eng, chunk=16, max_seqs=3)
        reqs = [Request(id=str(i), prompt=p, max_tokens=5) for i, p in enumerate(prompts)]
        for r in reqs:
            sch.submit(r)
        sch.run_until_idle(500)
        assert sch.idle()
        outs.append([r.out for r in reqs])
    assert outs[0] == outs[1]
    assert pipe.moved_bytes > 0


def test_hybrid_pipeline_four_stages_with_state_slots():
    cfg = hybrid.TOY_HYBRID
    w = hybrid.random_weights(cfg, seed=4, std=0.08)
    pipe, single, docs = make(cfg, hybrid.build_manifest, w, 4, slots=5)
    assert sorted(s for d in docs for s in d["states"]) == sorted(["gdn.l0", "gdn.l1", "gdn.l2", "kv.l3"])
    torch.manual_seed(1)
    prompt = torch.randint(1, cfg.vocab, (22,)).tolist()
    res = []
    for eng in (single, pipe):
        s = eng.open(40)
        t = eng.step([(s, prompt[:10])])
        t = eng.step([(s, prompt[10:])])[0]
        out = [t[0]]
        for _ in range(4):
            out.append(eng.step([(s, [out[-1]])])[0][0])
        res.append(out)
    assert res[0] == res[1]


def test_latent_moe_pipeline_two_stages():
    """KDA + latent attention + routed experts cut in two: the row plan of the latent layers (`row_seq`, `row_len`)
    is made on the stage of the first latent layer and crosses the cut with the activations."""
    cfg = latent.TINY_LATENT
    w = latent.folded(cfg, latent.random_weights(cfg, seed=4, std=0.05))
    pipe, single, docs = make(cfg, latent.build_manifest, w, 2, slots=5)
    assert sorted(s for d in docs for s in d["states"]) == sorted(["kda.l0", "kv.l1", "kda.l2", "kv.l3"])
    torch.manual_seed(1)
    prompt = torch.randint(1, cfg.vocab, (22,)).tolist()
    res = []
    for eng in (single, pipe):
        s = eng.open(40)
        t = eng.step([(s, prompt[:10])])
        t = eng.step([(s, prompt[10:])])[0]
        out = [t[0]]
        for _ in range(4):
            out.append(eng.step([(s, [out[-1]])])[0][0])
        res.append(out)
    assert res[0] == res[1]


def test_layer_cuts_reject_more_stages_than_layers():
    with pytest.raises(ValueError):
        pp.layer_cuts(dense.build_manifest(dense.TOY), 3)
