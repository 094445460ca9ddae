"""Pipeline stages as GPU runtimes of one process: activations cross the cut by a device-to-device copy. With one
GPU both stages share the device; with more, stage s runs on GPU s."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_two_stage_pipeline_matches_uncut_on_gpu(cuda):
    from kern_b200.engine import Engine
    from kern_b200.models import dense
    from kern_b200.runtime import Runtime
    from kern_b200.serve import pp

    cfg = dense.TINY
    weights = dense.random_weights(cfg, seed=0, std=0.05)
    doc = dense.build_manifest(cfg)
    stage_docs = pp.cut(doc, pp.layer_cuts(doc, 2))
    ngpu = torch.cuda.device_count()
    stages = []
    for s, d in enumerate(stage_docs):
        rt = Runtime(d, gpu=s % ngpu, tokens=cfg.page_size * 64)
        rt.load_tensors(lambda name, g=s % ngpu: weights[name].to(f"cuda:{g}"))
        rt.once()
        stages.append(rt)
    whole = Runtime(doc, tokens=cfg.page_size * 64)
    whole.load_tensors(lambda name: weights[name].cuda())
    whole.once()
    pipe, single = pp.PipelineEngine(stages, whole.protocol, transfer=pp.device_transfer), Engine(whole)
    torch.manual_seed(0)
    prompts = [torch.randint(1, cfg.vocab, (n,)).tolist() for n in (70, 9)]
    res = []
    for eng in (single, pipe):
        seqs = [eng.open(120) for _ in prompts]
        toks = [t[0] for t in eng.step(list(zip(seqs, prompts)))]
        out = [list(toks)]
        for _ in range(4):
            toks = [t[0] for t in eng.step([(s, [t]) for s, t in zip(seqs, toks)])]
            out.append(list(toks))
        res.append(out)
        for s in seqs:
            eng.close(s)
    for rt in stages + [whole]:
        rt.check_error()
    assert res[0] == res[1]
