"""Prefill/decode disaggregation on CPU: a prefill engine and a decode engine (two runtimes of the exact integer
model), seats reserved before prefill, pages and the state slot pushed by the plan, tokens streamed back."""
import random

import pytest

from kern_b200.cpu import CpuRuntime
from kern_b200.engine import Engine
from kern_b200.models import toy_int
from kern_b200.serve import pd


def push(plan, p_rt, d_rt):
    """Execute a push plan between two host-memory runtimes (on GPUs: copies into the mapped peer pools)."""
    for name, s in p_rt.doc["states"].items():
        src, dst = p_rt.states[name], d_rt.states[name]
        if s.get("bytes_per_token"):
            n = s["bytes_per_token"] * p_rt.page_unit
            for a, b in plan["pages"]:
                dst[b * n:(b + 1) * n] = src[a * n:(a + 1) * n]
        elif s.get("bytes_per_seq") and plan["slot"] is not None:
            n = s["bytes_per_seq"]
            a, b = plan["slot"]
            dst[b * n:(b + 1) * n] = src[a * n:(a + 1) * n]


@pytest.mark.parametrize("lined", [False, True])
def test_handoff_matches_twin(lined):
    doc = toy_int.build_manifest(lined)
    p_rt = CpuRuntime(doc, tokens=16 * 30, slots=6 if lined else 0)
    d_rt = CpuRuntime(doc, tokens=16 * 12, slots=3 if lined else 0)        # a small decode tier: it will say Busy
    p_eng, d_eng = Engine(p_rt), Engine(d_rt)
    assert pd.cover(p_rt.doc, p_rt.page_unit, pd.pools_message(d_rt.doc, d_rt.page_unit, 1, 256)) == []
    dec = pd.Decoder(d_eng, max_seqs=3, stop_ids=(toy_int.EOS,))
    hand = pd.Handoffs(p_rt.page_unit)
    relay = pd.Relay()
    rng = random.Random(5)
    prompts = {f"r{i}": [rng.randrange(256) for _ in range(rng.randint(5, 60))] for i in range(6)}
    out = {r: [] for r in prompts}
    done = set()
    for r in prompts:
        relay.watch(r, lambda tok, last, r=r: (out[r].append(tok), done.add(r) if last else None))
    max_tokens = 7
    to_d = [hand.ask(r, len(p) + max_tokens) for r, p in prompts.items()]
    seqs = {}
    busy_seen = False
    for _ in range(400):
        to_p = []
        for m in to_d:
            to_p += dec.handle(m)
        to_p += dec.step()
        to_d = []
        for m in to_p:
            busy_seen |= "busy" in m
            events = hand.told(m)
            relay.deliver(events)
            for kind, req, val in events:
                if kind == "granted":
                    # prefill on P (whole prompt, one call), push, hand over with the first token
                    s = p_eng.open(len(prompts[req]))
                    first = p_eng.step([(s, prompts[req])])[0][0]
                    for plan in hand.prefilled(req, s.lease, len(prompts[req])):
                        push(plan, p_rt, d_rt)
                    out[req].append(first)
                    to_d.append(hand.pushed(req, first, len(prompts[req]), max_tokens - 1, stop_ids=(toy_int.EOS,)))
                    p_eng.close(s)
        if len(done) == len(prompts):
            break
    assert len(done) == len(prompts) and busy_seen
    for r, p in prompts.items():
        want = toy_int.generate(p, max_tokens, lined)
        got = [t for t in out[r] if t != toy_int.EOS]
        assert got == want, r
    assert d_eng.pool.free_pages == d_eng.pool.total_pages and not dec.seats


def test_cover_names_every_mismatch_and_moves_checks_room():
    a, b = toy_int.build_manifest(False), toy_int.build_manifest(True)
    errs = pd.cover(a, 16, pd.pools_message(b, 8, 1, 256))
    assert any("line" in e for e in errs) and any("page of 16" in e for e in errs)
    assert pd.moves([5, 6, 7], {"pages": [1, 2], "slot": 4}, 20, 16, src_slot=2) == {"pages": [[5, 1], [6, 2]], "slot": [2, 4]}
    with pytest.raises(ValueError):
        pd.moves([5], {"pages": [1, 2], "slot": -1}, 20, 16)


def test_refuse_and_abort_and_two_choices():
    doc = toy_int.build_manifest(False)
    d_eng = Engine(CpuRuntime(doc, tokens=16 * 4))
    dec = pd.Decoder(d_eng)
    assert "refuse" in dec.handle({"reserve": {"req": "big", "tokens": 16 * 40}})[0]
    g = dec.handle({"reserve": {"req": "a", "tokens": 16 * 4}})[0]["grant"]
    assert len(g["seats"][0]["pages"]) == 4
    assert "busy" in dec.handle({"reserve": {"req": "b", "tokens": 16}})[0]
    replies = dec.handle({"abort": {"req": "a"}})
    assert "grant" in replies[0] and replies[0]["grant"]["req"] == "b" and "room" in replies[1]
    t = pd.Tiers(3, seed=1)
    t.report(0, {"seqs": 50, "free_pages": 1, "total_pages": 100})
    t.report(1, {"seqs": 0, "free_pages": 100, "total_pages": 100})
    t.report(2, {"seqs": 50, "free_pages": 1, "total_pages": 100})
    picks = [t.pick() for _ in range(200)]
    assert picks.count(1) > 100 and t.pick(busy={0, 1, 2}) is None and t.pick(busy={0, 2}) == 1


def test_dealt_rows_and_slot_parts_as_copies():
    """The shapes of a push that is not whole pages or slots: a deal's runs cut into strided copies of at most 64 KiB,
    and a slot sharded by heads as one strided copy per row of each segment; over all members the parts tile the slot."""
    from kern_b200 import _native as n

    runs = n.deal([3, 4, 5], 16, [7, 8], 16, 4, 1, 40)          # positions 1, 5, 9, ... of 40, member 1 of 4
    assert runs == [(3 * 16 + 1, 4, 7 * 16, 10)]
    assert n.dealt_copies(runs, 1024) == [((3 * 16 + 1) * 1024, 7 * 16 * 1024, 1024, 4096, 1024, 10)]
    big = n.dealt_copies([(0, 2, 0, 100)], 4096)                # 16 rows of 4 KiB per 64 KiB piece
    assert [c[5] for c in big] == [16] * 6 + [4] and big[1][0] == 16 * 2 * 4096 and big[1][1] == 16 * 4096
    assert n.dealt_copies([(0, 2, 0, 3)], 1 << 20)[0][5] == 1   # a row above the piece size travels alone
    segs, of, lines = [(1, 64 * 4), (3, 16 * 4)], 4, 2          # a [heads=4, 64] block and a 3-tap window of [heads=4, 16]
    line = n.split_line(segs, of)
    assert line == 256 + 192
    covered, dst_seen = set(), {}
    for part in range(of):
        for (s0, d0, w, sp, dp, rows) in n.split_copies(segs, of, lines, part):
            assert sp == line and dp == line // of and rows == lines
            for r in range(rows):
                src = range(s0 + r * sp, s0 + r * sp + w)
                assert not covered & set(src)
                covered |= set(src)
                for i, b in enumerate(src):
                    dst_seen[(part, d0 + r * dp + i)] = b
    assert covered == set(range(line * lines))                  # the members' sources tile the slot
    for part in range(of):                                      # and each member's destinations tile its own slot
        assert sorted(d for (p, d) in dst_seen if p == part) == list(range(line * lines // of))
    with pytest.raises(ValueError):
        n.split_copies([(1, 10)], 4, 1, 0)                      # a width the members do not divide


def test_mirrors_push_dealt_rows_and_parts_between_host_runtimes():
    """A prefill runtime pushing one request into a two-rank decode group held in host memory: by position (each rank
    gets every second row of the paged state, the slot whole) and by heads (each rank gets its columns of the slot)."""
    import torch

    from kern_b200.cpu import CpuRuntime
    from kern_b200.models import toy_int

    doc = toy_int.build_manifest(lined=True)
    p_rt = CpuRuntime(doc, tokens=16 * 8, slots=4)
    ranks = [CpuRuntime(doc, tokens=16 * 8, slots=4) for _ in range(2)]
    unit = p_rt.page_unit
    paged = [n for n, s in doc["states"].items() if s.get("bytes_per_token")]
    slotted = [n for n, s in doc["states"].items() if s.get("bytes_per_seq")]
    assert paged and slotted
    g = torch.Generator().manual_seed(1)
    for n in paged + slotted:
        p_rt.states[n].copy_(torch.randint(0, 256, p_rt.states[n].shape, generator=g, dtype=torch.uint8))
    length, src_pages, src_slot = unit * 2 + 5, [3, 1, 6], 2
    mirrors = pd.Mirrors(p_rt, [r.export_states() for r in ranks], [r.state_bytes() for r in ranks])
    seats = [{"pages": [2, 5], "slot": 1}, {"pages": [4, 0], "slot": 3}]
    # by position
    n_copies = mirrors.push(pd.group_moves(src_pages, seats, length, unit, src_slot, by_position=True))
    assert n_copies > 0
    for name in paged:
        row = doc["states"][name]["bytes_per_token"]
        for m, (rt, seat) in enumerate(zip(ranks, seats)):
            for j, pos in enumerate(range(m, length, 2)):
                src = (src_pages[pos // unit] * unit + pos % unit) * row
                dst = (seat["pages"][j // unit] * unit + j % unit) * row
                assert torch.equal(rt.states[name][dst:dst + row], p_rt.states[name][src:src + row]), (name, m, pos)
    for name in slotted:
        nb = doc["states"][name]["bytes_per_seq"]
        for rt, seat in zip(ranks, seats):
            assert torch.equal(rt.states[name][seat["slot"] * nb:(seat["slot"] + 1) * nb], p_rt.states[name][src_slot * nb:(src_slot + 1) * nb])
    # by heads: a group whose slots are half the size takes its columns of every row
    name = slotted[0]
    nb = doc["states"][name]["bytes_per_seq"]
    assert nb % 4 == 0
    segs = [(2, nb // 2)]                                        # two rows per line, each split over the two members
    halves = [torch.zeros(4 * nb // 2, dtype=torch.uint8) for _ in range(2)]
    for m in range(2):
        p_rt.push_slot_part(name, halves[m], halves[m].numel(), src_slot, 3, segs, 2, m)
    whole = p_rt.states[name][src_slot * nb:(src_slot + 1) * nb].view(2, 2, nb // 4)      # [row, member, bytes]
    for m in range(2):
        assert torch.equal(halves[m][3 * nb // 2:4 * nb // 2].view(2, nb // 4), whole[:, m])
    with pytest.raises(ValueError):
        p_rt.push_rows(paged[0], ranks[0].states[paged[0]], 64, [(0, 2, 0, 4)], doc["states"][paged[0]]["bytes_per_token"])
