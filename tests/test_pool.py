"""Pool, prefix index and position dealing against reference models.

Byte-level property test: random sequences of lease / write / checkpoint / restore / fork / retire against a
"position -> stamp" model (a sequence's content is the stamps written at each position; a restored or forked
lease must read back exactly the stamps of the prefix it was made from, after the copies the pool asked for
are executed on a byte array). Radix-style prefix lookups against a linear scan. `deal` against a row-by-row model.
Model for the shape of this suite: crates/kern-pool/tests/{pool,prefix,deal}.rs.
"""
import random

import pytest

from kern_b200 import _native as N


class Memory:
    """One byte-ish cell per (page, offset) and per slot: what the device would hold."""

    def __init__(self, pages, unit, slots):
        self.unit = unit
        self.cells = [[None] * unit for _ in range(pages)]
        self.slots = [None] * (slots + 1)

    def run(self, copies):
        for a, b in copies["pages"]:
            self.cells[b] = list(self.cells[a])
        if copies["slot"] is not None:
            a, b = copies["slot"]
            self.slots[b] = self.slots[a]

    def write(self, lease, pos, stamp):
        s = lease.slot_of(pos)
        self.cells[s // self.unit][s % self.unit] = stamp

    def read(self, pages, pos):
        return self.cells[pages[pos // self.unit]][pos % self.unit]


@pytest.mark.parametrize("seed", range(25))
def test_random_operations_against_stamp_model(seed):
    rng = random.Random(seed)
    unit, pages, slots = rng.choice([1, 4, 16]), 64, rng.choice([0, 12])
    pool = N.Pool(unit, pages, slots)
    mem = Memory(pages, unit, slots)
    live = []      # (lease, stamps list, filled)
    kept = []      # (checkpoint, stamps prefix)
    stamp = 0
    for _ in range(300):
        op = rng.choice(["lease", "write", "write", "checkpoint", "restore", "fork", "retire", "release", "drop"])
        try:
            if op == "lease":
                n = rng.randint(1, 5 * unit)
                l = pool.lease(n)
                if l.slot >= 0:
                    mem.slots[l.slot] = ("zero",)
                live.append([l, [], n])
            elif op == "write" and live:
                e = rng.choice(live)
                l, st, cap = e
                if len(st) < l.capacity:
                    stamp += 1
                    mem.write(l, len(st), stamp)
                    st.append(stamp)
                    if l.slot >= 0:
                        mem.slots[l.slot] = ("state", tuple(st))
            elif op == "checkpoint" and live:
                l, st, _ = rng.choice(live)
                if st:
                    n = rng.randint(1, len(st))
                    if slots and n != len(st):
                        n = len(st)          # a state snapshot is "exactly after these tokens"
                    c, cp = pool.checkpoint(l, n)
                    mem.run(cp)
                    kept.append((c, list(st[:n])))
            elif op == "restore" and kept:
                c, st = rng.choice(kept)
                n = c.len if (c.has_slot or rng.random() < 0.5) else (rng.randint(0, c.len // unit) * unit or c.len)
                l, cp = pool.restore(c, n, n + rng.randint(0, 2 * unit))
                mem.run(cp)
                assert [mem.read(l.pages, p) for p in range(n)] == st[:n]
                if c.has_slot:
                    assert mem.slots[l.slot] == ("state", tuple(st[:n]))
                live.append([l, list(st[:n]), l.capacity])
            elif op == "fork" and live:
                l, st, _ = rng.choice(live)
                if st:
                    n = len(st) if slots else rng.randint(1, len(st))
                    child, cp = pool.fork(l, n, n + unit)
                    mem.run(cp)
                    assert [mem.read(child.pages, p) for p in range(n)] == st[:n]
                    live.append([child, list(st[:n]), child.capacity])
            elif op == "retire" and live:
                e = live.pop(rng.randrange(len(live)))
                l, st, _ = e
                if st:
                    c = pool.retire(l, len(st))
                    assert [mem.read(c.page_ids(), p) for p in range(len(st))] == st
                    kept.append((c, list(st)))
                else:
                    l.release()
            elif op == "release" and live:
                live.pop(rng.randrange(len(live)))[0].release()
            elif op == "drop" and kept:
                kept.pop(rng.randrange(len(kept)))
        except N.Denied:
            pass
        # every kept prefix still reads back its stamps: nothing a lease wrote later leaked into a frozen page
        for c, st in kept:
            ids = c.page_ids()
            assert [mem.read(ids, p) for p in range(c.len)] == st[:c.len]
        for l, st, _ in live:
            assert [mem.read(l.pages, p) for p in range(len(st))] == st
    for e in live:
        e[0].release()
    live.clear()
    kept.clear()
    c = l = child = e = st = None     # the loop's last holders
    assert pool.free_pages == pages and pool.free_slots == slots


def test_lease_refuses_pages_it_sealed_and_denials():
    pool = N.Pool(4, 8, 2, 4)
    l = pool.lease(10)
    c, cp = pool.checkpoint(l, 8)
    assert cp["pages"] == [] and c.pages == 2 and l.shared_pages == 2
    with pytest.raises(Exception):
        l.slot_of(3)                       # a frozen page is never written again, not even by its lease
    assert l.slot_of(8) == l.pages[2] * 4
    with pytest.raises(N.Denied) as e:
        pool.lease(17)
    assert e.value.args[1] == "exceeds_row"
    with pytest.raises(N.Denied) as e:
        N.Pool(4, 8, 0).lease(100)
    assert e.value.args[1] == "exceeds_pool"
    p2 = N.Pool(4, 2, 0)
    a = p2.lease(8)
    with pytest.raises(N.Denied) as e:
        p2.lease(1)
    assert e.value.args[1] == "busy"
    a.release()
    assert p2.free_pages == 2


@pytest.mark.parametrize("seed", range(10))
def test_prefix_lookup_equals_linear_scan(seed):
    rng = random.Random(seed)
    unit = rng.choice([2, 4, 8])
    px = N.Prefix(unit)
    entries = {}
    base = [[rng.randrange(4) for _ in range(40)] for _ in range(4)]
    for _ in range(60):
        src = rng.choice(base)
        n = rng.randint(1, 40)
        key = src[:n] if rng.random() < 0.7 else src[: n // 2] + [rng.randrange(4) for _ in range(n - n // 2)]
        slot = rng.random() < 0.3
        px.insert(key, ("kept", tuple(key), slot), slot, len(key))
        entries[tuple(key)] = slot

    def scan(prompt, at_most):
        best = 0
        for key, slot in entries.items():
            common = 0
            lim = min(len(key), len(prompt), at_most)
            while common < lim and key[common] == prompt[common]:
                common += 1
            if common == len(key):
                usable = common
            elif slot:
                usable = 0
            else:
                usable = common // unit * unit
            best = max(best, usable)
        return best

    for _ in range(200):
        src = rng.choice(base)
        prompt = src[: rng.randint(1, 40)] + [rng.randrange(4) for _ in range(rng.randint(0, 5))]
        at_most = rng.choice([len(prompt), len(prompt) - 1, 10**9])
        got = px.lookup(prompt, at_most)
        want = scan(prompt, at_most)
        assert (got[0] if got else 0) == want
        if got:
            kept = got[1]
            assert list(kept[1][:got[0]]) == prompt[:got[0]]
    n = len(px)
    for _ in range(n):
        assert px.evict()
    assert len(px) == 0 and px.evict() == []


@pytest.mark.parametrize("seed", range(30))
def test_deal_against_row_by_row_model(seed):
    rng = random.Random(seed)
    for _ in range(100):
        w = rng.randint(1, 8)
        su, du = rng.choice([1, 4, 16, 64]), rng.choice([1, 4, 8, 64])
        length = rng.randint(0, 300)
        m = rng.randrange(w)
        il = N.Interleave(w)
        mine = il.len(length, m)
        assert sum(il.len(length, k) for k in range(w)) == length
        src = rng.sample(range(1000), -(-length // su) + 1)
        dst = rng.sample(range(1000), -(-mine // du) + 1)
        runs = N.deal(src, su, dst, du, w, m, length)
        placed = {}
        for s_row, s_stride, d_row, rows in runs:
            for i in range(rows):
                placed[d_row + i] = s_row + i * s_stride
        want = {}
        for j in range(mine):
            p = j * w + m
            assert il.owner(p) == m and il.local(p) == j
            want[dst[j // du] * du + j % du] = src[p // su] * su + p % su
        assert placed == want
        for a, b in zip(runs, runs[1:]):        # maximal: neighbours cannot be merged
            assert not (b[2] == a[2] + a[3] and b[0] == a[0] + a[3] * a[1] and (b[3] == 1 or b[1] == a[1]) and a[3] > 1)
    with pytest.raises(Exception):
        N.deal([0], 4, [0], 4, 2, 2, 4)
