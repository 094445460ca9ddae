"""Serving logic on the host-memory executor: continuous batching, bucket padding, chunked prefill,
prefix cache hits, eviction under pressure, aborts, and the OpenAI-style HTTP surface.

The gates are exact: a request served in a batch, after a prefix hit, or in chunks must produce the tokens
the same request produces alone (`conc1_equals_run`, `repeat_hit`, `turn2`, `concurrent`, `abort`,
`slot_pressure` of the reference's e2e driver: tools/e2e/e2e.py, tools/e2e/README.md)."""
import json
import urllib.request

import numpy as np
import pytest

from kern_b200.cpu import CpuRuntime
from kern_b200.engine import Engine
from kern_b200.models import dense
from kern_b200.serve.scheduler import Request, Scheduler, bucket_for
from kern_b200.serve.server import Server


@pytest.fixture(scope="module")
def toy():
    cfg = dense.TOY
    weights = dense.random_weights(cfg, seed=0, std=0.05)
    doc = dense.build_manifest(cfg)

    def make(tokens=cfg.page_size * 24):
        rt = CpuRuntime(doc, weights=weights, tokens=tokens)
        rt.once()
        return Engine(rt)

    return cfg, make


def alone(make, prompt, n):
    return make().generate(prompt, n)


def test_buckets():
    assert [bucket_for(n, 256) for n in (1, 3, 5, 9, 17, 100, 256)] == [1, 4, 8, 16, 24, 128, 256]
    assert bucket_for(5, 6) == 5      # no bucket fits under the limit: the exact size


def test_concurrent_requests_equal_single_runs(toy):
    cfg, make = toy
    rng = np.random.default_rng(0)
    prompts = [rng.integers(1, cfg.vocab, n).tolist() for n in (5, 16, 17, 30)]
    want = [alone(make, p, 6) for p in prompts]
    s = Scheduler(make(), chunk=24)          # forces chunked prefill and mixed calls
    reqs = [Request(id=f"r{i}", prompt=p, max_tokens=6) for i, p in enumerate(prompts)]
    for r in reqs:
        s.submit(r)
    s.run_until_idle(200)
    assert all(r.finished == "length" for r in reqs)
    assert [r.out for r in reqs] == want
    assert s.pool.free_pages + sum(1 for _ in range(0)) <= s.pool.total_pages


def test_repeat_prompt_hits_prefix_cache_and_matches(toy):
    cfg, make = toy
    rng = np.random.default_rng(1)
    prompt = rng.integers(1, cfg.vocab, 40).tolist()
    want = alone(make, prompt, 5)
    s = Scheduler(make())
    a = Request(id="a", prompt=prompt, max_tokens=5)
    s.submit(a)
    s.run_until_idle(100)
    b = Request(id="b", prompt=prompt, max_tokens=5)
    s.submit(b)
    s.run_until_idle(100)
    assert a.out == want and b.out == want
    assert b.cached == 32 and s.stats.prefix_hits == 1          # two whole pages of 16 reused
    # second turn: the first answer becomes part of the next prompt
    turn2 = prompt + a.out + rng.integers(1, cfg.vocab, 7).tolist()
    c = Request(id="c", prompt=turn2, max_tokens=4)
    s.submit(c)
    s.run_until_idle(100)
    assert c.cached >= 32 and c.out == alone(make, turn2, 4)


def test_eviction_makes_room_and_abort_frees_seats(toy):
    cfg, make = toy
    rng = np.random.default_rng(2)
    s = Scheduler(make(tokens=cfg.page_size * 5))           # five pages in all
    first = Request(id="x", prompt=rng.integers(1, cfg.vocab, 40).tolist(), max_tokens=4)
    s.submit(first)
    s.run_until_idle(100)
    assert len(s.prefix) == 1 and s.pool.free_pages < s.pool.total_pages
    big = Request(id="y", prompt=rng.integers(1, cfg.vocab, 44).tolist(), max_tokens=20)   # needs four pages, three are free
    s.submit(big)
    s.step()
    assert s.stats.evictions >= 1 and big in s.running
    assert s.abort("y") and big.finished == "abort"
    assert s.pool.free_pages == s.pool.total_pages
    with pytest.raises(ValueError):
        s.submit(Request(id="z", prompt=[1] * 200, max_tokens=10))


def test_stop_token_finishes_early(toy):
    cfg, make = toy
    prompt = list(range(1, 12))
    ref = alone(make, prompt, 8)
    s = Scheduler(make())
    r = Request(id="s", prompt=prompt, max_tokens=8, stop_ids=(ref[2],))
    s.submit(r)
    s.run_until_idle(50)
    assert r.finished == "stop" and r.out == ref[:ref.index(ref[2]) + 1]


def test_http_completions_stream_and_metrics(toy):
    cfg, make = toy
    srv = Server(Scheduler(make()), model_name="toy", port=0).start()
    base = f"http://127.0.0.1:{srv.port}"
    try:
        def post(path, body):
            req = urllib.request.Request(base + path, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
            return urllib.request.urlopen(req, timeout=60)

        prompt = list(range(3, 25))
        want = alone(make, prompt, 5)
        out = json.load(post("/v1/completions", {"prompt": prompt, "max_tokens": 5, "return_token_ids": True, "ignore_eos": True}))
        assert out["choices"][0]["token_ids"] == want and out["usage"]["completion_tokens"] == 5
        assert out["usage"]["prompt_tokens_details"]["cached_tokens"] == 0
        again = json.load(post("/v1/completions", {"prompt": prompt, "max_tokens": 5, "return_token_ids": True, "ignore_eos": True}))
        assert again["choices"][0]["token_ids"] == want and again["usage"]["prompt_tokens_details"]["cached_tokens"] == 16
        chunks = post("/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4, "stream": True,
                                               "return_token_ids": True, "ignore_eos": True}).read().decode()
        events = [json.loads(l[6:]) for l in chunks.splitlines() if l.startswith("data: {")]
        ids = [t for e in events for t in e["choices"][0].get("token_ids", [])]
        assert len(ids) == 4 and chunks.rstrip().endswith("data: [DONE]") and events[-1]["choices"][0]["finish_reason"] == "length"
        models = json.load(urllib.request.urlopen(base + "/v1/models", timeout=10))
        assert models["data"][0]["id"] == "toy"
        metrics = urllib.request.urlopen(base + "/kern/metrics", timeout=10).read().decode()
        assert 'kern_device_seconds_total{class="compute"}' in metrics and "kern_prefix_cache_hits_total 1" in metrics
        with pytest.raises(urllib.error.HTTPError):
            post("/v1/completions", {"prompt": "", "max_tokens": 1})
    finally:
        srv.stop()


def test_a_failed_step_answers_503_at_once(toy):
    """Once the driver thread has died on a failed step, /health says so and a new request gets 503 immediately
    instead of waiting in an inbox nobody reads."""
    import time
    import urllib.error

    cfg, make = toy
    sched = Scheduler(make())
    srv = Server(sched, model_name="toy", port=0).start()
    base = f"http://127.0.0.1:{srv.port}"
    try:
        def post(body, timeout=20):
            req = urllib.request.Request(base + "/v1/completions", data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
            return urllib.request.urlopen(req, timeout=timeout)

        def boom(*a, **k):
            raise RuntimeError("injected step failure")

        sched.eng.step = boom                      # the failure is made on the host: the next call raises
        with pytest.raises(urllib.error.HTTPError) as e1:
            post({"prompt": [1, 2, 3], "max_tokens": 2})
        assert e1.value.code >= 500
        t0 = time.monotonic()
        with pytest.raises(urllib.error.HTTPError) as e2:
            post({"prompt": [4, 5, 6], "max_tokens": 2})
        assert e2.value.code == 503 and time.monotonic() - t0 < 5
        with pytest.raises(urllib.error.HTTPError) as e3:
            urllib.request.urlopen(base + "/health", timeout=10)
        assert e3.value.code == 503
    finally:
        srv.stop()


def test_agent_traffic_replay_reuses_prefixes_and_is_exact(toy):
    """Agent-style sessions (shared family prefix, growing conversation, a new suffix per turn) replayed in a closed
    loop: every request is served, most prompt tokens come from the prefix cache from the second turn on, and the
    answers equal the same requests served alone."""
    from kern_b200.testing import agent_traffic as T

    cfg, make = toy
    sessions = T.generate(seed=5, sessions=6, turns=3, prefix=(16, 28), suffix=(2, 4), output=(2, 4), vocab=cfg.vocab,
                          families=2, shared=0.5)      # the toy's context is 64 tokens: 28 + 3 x (4 + 4) fits
    a, b = sessions[0], sessions[2]
    assert a.family == b.family and a.prefix[:8] == b.prefix[:8] and a.prefix != b.prefix
    again = T.generate(seed=5, sessions=6, turns=3, prefix=(16, 28), suffix=(2, 4), output=(2, 4), vocab=cfg.vocab, families=2)
    assert [s.prefix for s in again] == [s.prefix for s in sessions]                 # one seed, one workload
    sched = Scheduler(make(tokens=cfg.page_size * 96), chunk=32)
    res = T.replay(sched, sessions, concurrent=3, deadline_s=60)
    assert res["requests_served"] == 18 and res["unfinished"] == 0
    assert res["prefix_cache_share"] > 0.3, res                                      # turns 2 and 3 find their history
    assert res["ttft_ms_p50"] is not None and res["output_tokens"] > 0
    # exactness: the last turn of a session, alone on a fresh engine, gives the same answer
    s0 = sessions[0]
    turn = s0.turns[-1]
    # rebuild the last request: history before the last answer = prompt of the last turn
    # (history = prompt + out of the last turn)
    n_out = None
    for n in range(1, turn.max_tokens + 1):
        prompt = s0.history[: len(s0.history) - n]
        if prompt[-len(turn.suffix):] == turn.suffix:
            n_out = n
            break
    assert n_out is not None
    prompt = s0.history[: len(s0.history) - n_out]
    assert alone(make, prompt, n_out) == s0.history[len(prompt):]


@pytest.mark.parametrize("front", [False, True])
def test_http_front_over_prefill_and_decode_tiers(toy, front):
    """The OpenAI-style front over `launch_pd`: completions come out of the decode tier, token for token those of one
    engine; a repeated prompt hits the prefill tier's prefix cache; the metrics page carries the tiers' counters."""
    from kern_b200.serve import launch

    cfg, make = toy
    weights = dense.random_weights(cfg, seed=0, std=0.05)
    spec = {"manifest": dense.build_manifest(cfg), "cpu": True, "weights": weights, "tokens": cfg.page_size * 24}
    tier, worker = launch.launch_pd(spec, dict(spec, tokens=cfg.page_size * 12), chunk=16, max_seqs=3, decode_max_seqs=2, timeout=60,
                                    front=front)
    srv = Server(tier, model_name="toy-pd", port=0).start()
    base = f"http://127.0.0.1:{srv.port}"
    try:
        def post(path, body):
            req = urllib.request.Request(base + path, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
            return urllib.request.urlopen(req, timeout=60)

        prompt = list(range(3, 40))
        want = alone(make, prompt, 6)
        out = json.load(post("/v1/completions", {"prompt": prompt, "max_tokens": 6, "return_token_ids": True, "ignore_eos": True}))
        assert out["choices"][0]["token_ids"] == want and out["usage"]["completion_tokens"] == 6
        again = json.load(post("/v1/completions", {"prompt": prompt, "max_tokens": 6, "return_token_ids": True, "ignore_eos": True}))
        assert again["choices"][0]["token_ids"] == want and again["usage"]["prompt_tokens_details"]["cached_tokens"] == 32
        chunks = post("/v1/completions", {"prompt": prompt[:9], "max_tokens": 4, "stream": True, "return_token_ids": True,
                                          "ignore_eos": True}).read().decode()
        events = [json.loads(l[6:]) for l in chunks.splitlines() if l.startswith("data: {")]
        ids = [t for e in events for t in e["choices"][0].get("token_ids", [])]
        assert ids == alone(make, prompt[:9], 4) and chunks.rstrip().endswith("data: [DONE]")
        assert tier.metrics()["pd"]["decoding"] == 0 and tier.idle()
    finally:
        srv.stop()
        launch.shutdown_pd(tier, worker)
    assert not worker.is_alive()
