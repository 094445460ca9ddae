"""End to end on a GPU: manifest -> native runtime -> engine, against the PyTorch fp32 oracle."""
import json

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tiny(cuda, tmp_path_factory):
    from kern_b200.models import common, dense
    from kern_b200.runtime import Runtime, verify

    cfg = dense.TINY
    weights = dense.random_weights(cfg, seed=0, std=0.05)
    path = tmp_path_factory.mktemp("ckpt") / "model.safetensors"
    common.write_safetensors(path, weights)
    doc = dense.build_manifest(cfg)
    m, errs = verify(doc)
    assert m is not None, errs[:5]
    rt = Runtime(doc, weights=path, tokens=cfg.page_size * 64)
    rt.once()
    return cfg, weights, rt


def test_logits_match_oracle_prefill_and_decode(tiny):
    from kern_b200.engine import Engine
    from kern_b200.models.dense import DenseOracle

    cfg, weights, rt = tiny
    eng = Engine(rt)
    oracle = DenseOracle(cfg, weights, device="cuda")
    torch.manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (37,)).tolist()
    seq = eng.open(64)
    cache = oracle.new_cache()
    got = eng.step([(seq, prompt)])
    ref = oracle.forward(prompt, cache)[-1]
    logits = rt.tensor("logits")[0].float()
    assert torch.allclose(logits, ref, atol=0.08, rtol=0.05), float((logits - ref).abs().max())
    tok = got[0][0]
    for _ in range(6):
        ref = oracle.forward([tok], cache)[-1]
        got = eng.step([(seq, [tok])])
        logits = rt.tensor("logits")[0].float()
        assert torch.allclose(logits, ref, atol=0.08, rtol=0.05), float((logits - ref).abs().max())
        tok = got[0][0]
    rt.check_error()
    eng.close(seq)


def test_batched_generation_matches_single_and_graph_replays(tiny):
    from kern_b200.engine import Engine
    from kern_b200.models.dense import DenseOracle

    cfg, weights, rt = tiny
    eng = Engine(rt)
    oracle = DenseOracle(cfg, weights, device="cuda")
    rng = np.random.default_rng(1)
    prompts = [rng.integers(0, cfg.vocab, n).tolist() for n in (5, 16, 17, 40)]
    seqs = [eng.open(80) for _ in prompts]
    # ragged prefill of all four prompts in one call, then batched decode through the captured graph
    first = eng.step(list(zip(seqs, prompts)))
    outs = [[f[0]] for f in first]
    graphs0 = rt.graphs
    for _ in range(7):
        nxt = eng.step([(s, [o[-1]]) for s, o in zip(seqs, outs)])
        for o, n in zip(outs, nxt):
            o.append(n[0])
    assert rt.graphs == graphs0 + 1          # one capture, then replays
    rt.check_error()
    for p, o in zip(prompts, outs):
        ref = oracle.generate(p, 8)
        # greedy near-ties may flip under bf16: demand agreement of the first tokens and most of the rest
        assert o[0] == ref[0]
        assert sum(a == b for a, b in zip(o, ref)) >= 6, (o, ref)
    for s in seqs:
        eng.close(s)


def test_chunked_prefill_equals_whole(tiny):
    from kern_b200.engine import Engine

    cfg, weights, rt = tiny
    eng = Engine(rt)
    rng = np.random.default_rng(2)
    prompt = rng.integers(0, cfg.vocab, 100).tolist()
    a = eng.generate(prompt, 4)
    la = rt.tensor("logits")[0].float().clone()
    b = eng.generate(prompt, 4, chunk=33)
    lb = rt.tensor("logits")[0].float()
    assert a[0] == b[0]
    assert torch.allclose(la, lb, atol=0.06, rtol=0.05)


@pytest.mark.parametrize("lined", [False, True])
def test_integer_model_served_on_gpu_equals_twin(cuda, lined):
    """The exact integer model through the native runtime, CUDA graphs, prefix cache and state slots."""
    import random

    from kern_b200.engine import Engine
    from kern_b200.models import toy_int
    from kern_b200.runtime import Runtime
    from kern_b200.serve.scheduler import Request, Scheduler

    rt = Runtime(toy_int.build_manifest(lined), tokens=16 * 40, slots=12 if lined else 0)
    sch = Scheduler(Engine(rt), chunk=24, max_seqs=4)
    rng = random.Random(3)
    base = [rng.randrange(256) for _ in range(70)]
    waves = [[[rng.randrange(256) for _ in range(rng.randint(1, 60))] for _ in range(6)] + [base[:50]],
             [base[:50] + [1, 2, 3], base[:33], base]]
    reqs = []
    for wave in waves:
        new = [Request(id=str(len(reqs) + i), prompt=p, max_tokens=10, stop_ids=(toy_int.EOS,)) for i, p in enumerate(wave)]
        reqs += new
        for r in new:
            sch.submit(r)
        for _ in range(2000):
            if sch.idle():
                break
            sch.step()
        assert sch.idle()
    rt.check_error()
    for r in reqs:
        assert [t for t in r.out if t != toy_int.EOS] == toy_int.generate(r.prompt, 10, lined), r.id
    assert rt.graphs >= 1


def test_guard_bands_stay_clean_and_report_an_overrun(cuda):
    """Test mode: canary bands around every device allocation. A whole prefill + decode of the tiny decoder leaves them
    intact; a byte written past the end of a workspace (from the host, inside the runtime's own allocation) is named."""
    from kern_b200.engine import Engine
    from kern_b200.models import dense
    from kern_b200.runtime import Runtime, _CudaView

    cfg = dense.TINY
    weights = dense.random_weights(cfg, seed=0, std=0.05)
    rt = Runtime(dense.build_manifest(cfg), tokens=cfg.page_size * 32, slots=4, guard_bands=True)
    rt.load_tensors(lambda name: weights[name].cuda())
    rt.once()
    eng = Engine(rt)
    s = eng.open(64)
    tok = eng.step([(s, list(range(1, 40)))])[0][0]
    for _ in range(4):
        tok = eng.step([(s, [tok])])[0][0]
    rt.check_error()
    assert rt.check_guards() == []
    ptr, nbytes = rt.region("xn")
    past = torch.as_tensor(_CudaView(ptr + nbytes, (1,), "|u1"), device="cuda:0")     # first byte of the trailing band
    past.fill_(7)
    torch.cuda.synchronize()
    assert rt.check_guards() == ["xn (after)"]


def test_kernel_activity_trace_names_our_kernels(tiny, tmp_path):
    """CUPTI activity records of a prefill and a few graph-replayed decode steps: our entry points by name, positive
    durations, launch shapes; folded by kernel and written as Parquet."""
    import pyarrow.parquet as pq
    from kern_b200.engine import Engine
    from kern_b200.trace import KernelTrace

    cfg, weights, rt = tiny
    eng = Engine(rt)
    s = eng.open(64)
    try:
        probe = KernelTrace()
        probe.__enter__()
        probe.__exit__(None, None, None)
    except RuntimeError as e:      # no CUPTI on this machine, or another tool holds it
        pytest.skip(f"kernel activity tracing is not available here: {e}")
    with KernelTrace() as kt:
        tok = eng.step([(s, list(range(1, 30)))])[0][0]
        for _ in range(3):
            tok = eng.step([(s, [tok])])[0][0]
        torch.cuda.synchronize()
        first = kt.collect()
    eng.close(s)
    assert first and len(kt.records) >= len(first)
    names = {r["name"] for r in kt.records}
    assert any(n.startswith("kern_rms_norm") or n.startswith("kern_fused_add_rms_norm") for n in names), sorted(names)[:20]
    assert any(n.startswith("kern_gemm_bf16") or n.startswith("kern_gemv_bf16") for n in names)
    assert all(r["end_ns"] > r["start_ns"] and r["block"][0] >= 1 for r in kt.records)
    top = kt.by_kernel()
    assert sum(d["launches"] for d in top.values()) == len(kt.records)
    kt.write(tmp_path / "kernels.parquet")
    assert pq.ParquetFile(tmp_path / "kernels.parquet").read().num_rows == len(kt.records)


def test_mark_gate_hold_and_fetch(cuda):
    """The runtime's stream-ordered signals: a program issued behind a `hold` does not run until the host opens the
    gate; a `mark` tells the host when the stream got there without a stream synchronisation; `fetch` reads an output
    behind the work issued so far; and a gate nobody opens makes the hold give up after its limit with an error code,
    leaving the context usable."""
    import time

    from kern_b200.models import toy_int
    from kern_b200.runtime import Runtime
    from kern_b200.engine import Engine

    rt = Runtime(toy_int.build_manifest(False), tokens=16 * 40)
    eng = Engine(rt)
    seq = eng.open(64)
    prompt = list(range(3, 20))
    gate = rt.gate()
    rt.hold(gate, 1, timeout_s=20.0)
    toks = eng.step([(seq, prompt)], read=False)           # queued behind the hold
    m = rt.mark()
    time.sleep(0.05)
    assert not m.done()                                    # the stream is parked on the gate
    f = rt.fetch("next_token", 1)
    gate.open()
    m.wait(10.0)
    assert int(f.get(10.0)[0]) == toy_int.generate(prompt, 1)[0]
    rt.check_error()
    # a gate nobody opens: the hold gives up after 5 ms, sets the error word and the stream goes on
    rt.hold(rt.gate(), 1, timeout_s=0.005, code=777)
    rt.mark().wait(10.0)
    with pytest.raises(RuntimeError, match="777"):
        rt.check_error()
    rt.tensor("error").zero_()
    torch.cuda.synchronize()
    eng.step([(seq, [5])])
    rt.check_error()


@pytest.mark.gpu
def test_push_dealt_rows_and_slot_parts_between_two_runtimes(cuda):
    """`Runtime.push_rows` / `push_slot_part` as strided device copies: a prefill runtime's paged rows dealt over a
    two-member decode group by position, and its state slot sharded by heads, land where the plan says (the decode
    side's pools are plain device pointers here: both runtimes live in this process)."""
    from kern_b200.models import toy_int
    from kern_b200.runtime import Runtime
    from kern_b200.serve import pd

    doc = toy_int.build_manifest(lined=True)
    p_rt = Runtime(doc, tokens=16 * 8, slots=4)
    ranks = [Runtime(doc, tokens=16 * 8, slots=4) for _ in range(2)]
    unit = p_rt.page_unit if hasattr(p_rt, "page_unit") else 16
    paged = [n for n, s in doc["states"].items() if s.get("bytes_per_token")]
    slotted = [n for n, s in doc["states"].items() if s.get("bytes_per_seq")]
    torch.manual_seed(3)
    for n in paged + slotted:
        t = p_rt.tensor(n)
        t.copy_(torch.randint(0, 256, t.shape, device=cuda, dtype=torch.uint8))
    length, src_pages, src_slot = unit * 2 + 5, [3, 1, 6], 2
    seats = [{"pages": [2, 5], "slot": 1}, {"pages": [4, 0], "slot": 3}]
    mirrors = pd.Mirrors.__new__(pd.Mirrors)
    mirrors.rt, mirrors.mapped, mirrors.sizes = p_rt, [{n: r.region(n)[0] for n in doc["states"]} for r in ranks], [r.state_bytes() for r in ranks]
    assert mirrors.push(pd.group_moves(src_pages, seats, length, unit, src_slot, by_position=True)) > 0
    p_rt.synchronize()
    for name in paged:
        row = doc["states"][name]["bytes_per_token"]
        src_t = p_rt.tensor(name)
        for m, (rt, seat) in enumerate(zip(ranks, seats)):
            dst_t = rt.tensor(name)
            for j, pos in enumerate(range(m, length, 2)):
                s0 = (src_pages[pos // unit] * unit + pos % unit) * row
                d0 = (seat["pages"][j // unit] * unit + j % unit) * row
                assert torch.equal(dst_t[d0:d0 + row], src_t[s0:s0 + row]), (name, m, pos)
    name = slotted[0]
    nb = doc["states"][name]["bytes_per_seq"]
    halves = [torch.zeros(4 * nb // 2, dtype=torch.uint8, device=cuda) for _ in range(2)]
    for m in range(2):
        p_rt.push_slot_part(name, halves[m].data_ptr(), halves[m].numel(), src_slot, 3, [(2, nb // 2)], 2, m)
    p_rt.synchronize()
    whole = p_rt.tensor(name)[src_slot * nb:(src_slot + 1) * nb].view(2, 2, nb // 4)
    for m in range(2):
        assert torch.equal(halves[m][3 * nb // 2:4 * nb // 2].view(2, nb // 4), whole[:, m])
    with pytest.raises(RuntimeError):
        p_rt.push_rows(paged[0], ranks[0].region(paged[0])[0], 64, [(0, 2, 0, 4)], doc["states"][paged[0]]["bytes_per_token"])


@pytest.mark.gpu
def test_native_runner_executes_manifests_without_python(cuda, tmp_path):
    """`kern_b200/bin/kern-run` (C++ only: manifest, pool and runtime behind a single-sequence caller) produces the tokens
    of the exact integer model's Python twin, with and without a per-sequence state, and of the dense toy decoder served
    by the Python engine from the same safetensors checkpoint."""
    import json
    import os
    import subprocess

    from safetensors.torch import save_file

    from kern_b200.engine import Engine
    from kern_b200.models import dense, toy_int
    from kern_b200.runtime import Runtime

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = os.path.join(root, "kern_b200", "bin", "kern-run")
    kernels = os.path.join(root, "kern_b200", "kernels")
    assert os.path.exists(exe), "the native runner was not built"

    def run(manifest, prompt, steps, extra=()):
        p = subprocess.run([exe, str(manifest), "--kernels", kernels, "--prompt", ",".join(map(str, prompt)), "--steps", str(steps), *extra],
                           capture_output=True, text=True, timeout=120)
        assert p.returncode == 0, p.stderr[-2000:]
        return json.loads(p.stdout.strip().splitlines()[-1])

    prompt = [11, 12, 13, 14, 15, 16, 17]          # a prompt whose continuation does not start with the model's stop token
    for lined in (False, True):
        path = tmp_path / f"toy_int_{int(lined)}.json"
        path.write_text(json.dumps(toy_int.build_manifest(lined=lined)))
        got = run(path, prompt, 6, ("--chunk", "4"))
        assert got["tokens"] == toy_int.generate(prompt, 6, lined), (lined, got)
        assert got["launches"] > 0
    cfg = dense.TINY
    w = dense.random_weights(cfg, seed=3, std=0.08)
    save_file({k: v.contiguous() for k, v in w.items()}, str(tmp_path / "model.safetensors"))
    doc = dense.build_manifest(cfg)
    (tmp_path / "dense.json").write_text(json.dumps(doc))
    rt = Runtime(doc, tokens=cfg.page_size * 16)
    rt.load_tensors(lambda name: w[name].to(cuda))
    rt.once()
    want = Engine(rt).generate(prompt, 5)
    got = run(tmp_path / "dense.json", prompt, 5, ("--weights", str(tmp_path / "model.safetensors")))
    assert got["tokens"] == want and got["graphs"] >= 1
