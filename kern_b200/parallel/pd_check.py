"""Prefill/decode disaggregation across two GPU processes: rank 0 is the prefill tier, rank 1 the decode tier, each
with its own runtime, pool and engine on its own GPU. The decode tier exports its state pools once; the prefill tier
maps them, reserves seats before it prefills, pushes the pages and the state slot of a finished prompt into the seats
(device copies over NVLink, `Runtime.push`), and hands over with the first token; tokens stream back. The model is the
exact integer serving model, so every request's tokens must equal its CPU twin's.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m kern_b200.parallel.pd_check

The messages are the state machines of `serve/pd.py`; each loop the two ranks swap message lists as objects over the
process group (any transport would do). Reference: crates/kern-serve/src/pd/mod.rs:74-329, crates/kern-runtime/src/push.rs:70-137.
"""
from __future__ import annotations

import argparse
import json
import os
import random

import torch
import torch.distributed as dist


def swap(mine: list, src: int) -> list:
    box = [mine]
    dist.broadcast_object_list(box, src=src)
    return box[0]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--lined", action="store_true", help="the model variant with a per-sequence state slot")
    ap.add_argument("--requests", type=int, default=6)
    a = ap.parse_args(argv)
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    assert world == 2, "one prefill rank and one decode rank"
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    from ..engine import Engine
    from ..models import toy_int
    from ..runtime import Runtime
    from ..serve import pd

    doc = toy_int.build_manifest(a.lined)
    is_p = rank == 0
    rt = Runtime(doc, gpu=local, tokens=16 * (30 if is_p else 12), slots=(6 if is_p else 3) if a.lined else 0)
    rt.once()
    eng = Engine(rt)
    rng = random.Random(5)
    prompts = {f"r{i}": [rng.randrange(256) for _ in range(rng.randint(5, 60))] for i in range(a.requests)}
    max_tokens = 7
    hello = swap([pd.pools_message(doc, rt.page_unit, 1, 256), rt.export_states()] if not is_p else [], src=1)
    ok, busy_seen, out = True, False, {r: [] for r in prompts}
    if is_p:
        why = pd.cover(doc, rt.page_unit, hello[0])
        assert why == [], why
        mapped = rt.map_pool(hello[1])
        hand, relay, done = pd.Handoffs(rt.page_unit), pd.Relay(), set()
        for r in prompts:
            relay.watch(r, lambda tok, last, r=r: (out[r].append(tok), done.add(r) if last else None))
        to_d = [hand.ask(r, len(p) + max_tokens) for r, p in prompts.items()]
    else:
        dec = pd.Decoder(eng, max_seqs=3, stop_ids=(toy_int.EOS,))
    for _ in range(400):
        to_d = swap(to_d if is_p else [], src=0)
        if to_d and isinstance(to_d[0], dict) and to_d[0].get("quit"):
            break
        to_p = []
        if not is_p:
            for m in to_d:
                to_p += dec.handle(m)
            to_p += dec.step()
            rt.check_error()
        to_p = swap(to_p, src=1)
        if is_p:
            to_d = []
            for m in to_p:
                busy_seen |= "busy" in m
                events = hand.told(m)
                relay.deliver(events)
                for kind, req, val in events:
                    if kind == "granted":
                        s = eng.open(len(prompts[req]))
                        first = eng.step([(s, prompts[req])])[0][0]
                        for plan in hand.prefilled(req, s.lease, len(prompts[req])):
                            rt.push(mapped, plan)
                        rt.synchronize()          # the pages are in the decode tier's pool before Start leaves
                        out[req].append(first)
                        to_d.append(hand.pushed(req, first, len(prompts[req]), max_tokens - 1, stop_ids=(toy_int.EOS,)))
                        eng.close(s)
            if len(done) == len(prompts):
                to_d = [{"quit": True}]
    if is_p:
        rt.check_error()
        for r, p in prompts.items():
            want = toy_int.generate(p, max_tokens, a.lined)
            got = [t for t in out[r] if t != toy_int.EOS]
            ok = ok and got == want
        ok = ok and len(done) == len(prompts)
        print(json.dumps({"check": "prefill_decode_two_processes", "lined": a.lined, "requests": len(prompts),
                          "busy_seen": busy_seen, "ok": ok}), flush=True)
    else:
        ok = eng.pool.free_pages == eng.pool.total_pages and not dec.seats
    flag = torch.tensor([int(ok)], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.barrier()
    dist.destroy_process_group()
    return 0 if flag.item() else 1


if __name__ == "__main__":
    raise SystemExit(main())
