"""The MoE decoder's manifest through the CPU executor against the fp32 oracle."""
import pytest
import torch

from kern_b200.cpu import CpuRuntime
from kern_b200.engine import Engine
from kern_b200.models import moe
from kern_b200.runtime import verify


def test_manifest_verifies_at_full_size():
    for cfg in (moe.TOY_MOE, moe.MOE_30B):
        m, d = verify(moe.build_manifest(cfg))
        assert m is not None, d[:5]


def test_prefill_and_decode_match_oracle():
    cfg = moe.TOY_MOE
    w = moe.random_weights(cfg, seed=2, std=0.08)
    rt = CpuRuntime(moe.build_manifest(cfg), weights=w, tokens=16 * 24)
    rt.once()
    eng, oracle = Engine(rt), moe.MoeOracle(cfg, w)
    torch.manual_seed(0)
    prompts = [torch.randint(1, cfg.vocab, (n,)).tolist() for n in (17, 5)]
    seqs = [eng.open(40) for _ in prompts]
    caches = [oracle.new_cache() for _ in prompts]
    first = eng.step(list(zip(seqs, prompts)))
    logits = rt.tensor("logits")[:2].float()
    worst = max(float((logits[i] - oracle.forward(p, c)[-1]).abs().max()) for i, (p, c) in enumerate(zip(prompts, caches)))
    toks = [f[0] for f in first]
    for _ in range(4):
        refs = [oracle.forward([t], c)[-1] for t, c in zip(toks, caches)]
        nxt = eng.step([(s, [t]) for s, t in zip(seqs, toks)])
        logits = rt.tensor("logits")[:2].float()
        worst = max([worst] + [float((logits[i] - refs[i]).abs().max()) for i in range(2)])
        toks = [n[0] for n in nxt]
    assert worst < 0.15, worst


def test_block_scaled_experts_manifest_on_the_cpu_executor():
    """`mx_experts`: MXFP4 expert weights and MXFP8 expert activations. The manifest verifies, binds the packed checkpoint
    (`mx_checkpoint`), and on the host-memory executor the decoder's logits stay close to the bf16-expert oracle's (the
    quantisation is the only difference)."""
    import dataclasses

    import torch

    from kern_b200.cpu import CpuRuntime
    from kern_b200.engine import Engine
    from kern_b200.models import moe
    from kern_b200.runtime import verify

    cfg = dataclasses.replace(moe.TINY_MOE, name="tiny-moe-mx", mx_experts=True, moe_intermediate=128, layers=1, experts=8, top_k=2)
    doc = moe.build_manifest(cfg)
    m, diags = verify(doc)
    assert m is not None, diags[:5]
    w = moe.random_weights(cfg, seed=3, std=0.05)
    rt = CpuRuntime(doc, weights=moe.mx_checkpoint(cfg, w), tokens=cfg.page_size * 16)
    rt.once()
    eng = Engine(rt)
    oracle = moe.MoeOracle(cfg, w)
    torch.manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (21,)).tolist()
    seq = eng.open(40)
    eng.step([(seq, prompt)])
    logits = rt.tensor("logits")[:1].float()
    ref = oracle.forward(prompt, oracle.new_cache())[-1]
    err = float((logits[0] - ref).abs().max())
    assert err < 0.35 * float(ref.abs().max()) + 0.05, (err, float(ref.abs().max()))
    assert int(logits[0].argmax()) == int(ref.argmax()) or err < 0.1


@pytest.mark.parametrize("world", [1, 2, 8])
def test_fused_expert_parallel_manifests_verify(world):
    """The fused dispatch / combine layer and the decoder over sharded tokens are valid manifests at every group size:
    five launches per routed layer, none of them a barrier kernel or a library collective."""
    import dataclasses
    import json

    from kern_b200 import _native
    from kern_b200.models import moe, moe_ep
    from kern_b200.parallel import ep_check

    doc = ep_check.manifest_fused(world, 64, 1024, 512, 16, 4)
    m, errs = _native.verify(json.dumps(doc))
    assert m is not None, errs
    entries = [l["entry"] for c in doc["programs"]["step"]["calls"] for l in doc["ops"][c["op"]]["impl"]["launches"]]
    assert entries == ["kern_ep_publish", "kern_moe_plan_ep", "kern_ep_fc1_bf16_swiglu_n128", "kern_ep_fc2_bf16_combine_n128",
                       "kern_ep_finalize"]
    # from 193 rows of a rank on, the routed GEMMs switch to 256-wide tiles: one launch of each runs, whatever the count
    wide = ep_check.manifest_fused(world, 1024, 1024, 512, 16, 4)
    m, errs = _native.verify(json.dumps(wide))
    assert m is not None, errs
    for op, small, big in (("ep_fc1", "kern_ep_fc1_bf16_swiglu_n128", "kern_ep_fc1_bf16_swiglu_n256"),
                           ("ep_fc2", "kern_ep_fc2_bf16_combine_n128", "kern_ep_fc2_bf16_combine_n256")):
        ls = wide["ops"][op]["impl"]["launches"]
        assert [l["entry"] for l in ls] == [small, big]
        assert ls[0]["when"] == {"var": "rows", "max": 192} and ls[1]["when"] == {"var": "rows", "min": 193}
    # block-scaled form: one more launch (this rank's rows quantised once), the routed pair out of the MX module
    mx = ep_check.manifest_fused(world, 1024, 1024, 512, 16, 4, mx=True)
    m, errs = _native.verify(json.dumps(mx))
    assert m is not None, errs
    entries = [l["entry"] for c in mx["programs"]["step"]["calls"] for l in mx["ops"][c["op"]]["impl"]["launches"]]
    assert entries == ["kern_quant_mxfp8_rows", "kern_ep_publish", "kern_moe_plan_ep", "kern_ep_fc1_mxfp8_mxfp4_swiglu_mxfp8_n128",
                       "kern_ep_fc1_mxfp8_mxfp4_swiglu_mxfp8_n256", "kern_ep_fc2_mxfp8_mxfp4_combine_n128",
                       "kern_ep_fc2_mxfp8_mxfp4_combine_n256", "kern_ep_finalize"]
    assert mx["buffers"]["ep.q8"]["export"] and mx["buffers"]["ep.sf8"]["shape"] == [1024, 1024 // 32]
    cfg = dataclasses.replace(moe.TINY_MOE, experts=16, top_k=4)
    doc = moe_ep.build_manifest_ep_sharded(cfg, world)
    m, errs = _native.verify(json.dumps(doc))
    assert m is not None, errs
    used = {c["op"] for p in doc["programs"].values() for c in p["calls"]}
    assert {"ep_publish", "ep_plan", "ep_fc1", "ep_fc2", "ep_finalize"} <= used
    assert not any(l["entry"].startswith("extern:nccl") or l["entry"] == "kern_peer_barrier"
                   for o in used for l in doc["ops"][o]["impl"]["launches"])
    # every rank binds its own range of experts
    w1 = doc["buffers"]["w.l0.w1"]
    assert w1["shape"][0] == 16 // world and len(w1["bind"][0]["tensor"]["tensors"]) == world
