"""Packages written for the reference run here unmodified: its toy manifests (tools/toy/gen.py) and its toy.cu cubin,
served by this package's runtime and scheduler, must give the tokens of the reference's own oracle
(tools/toy/model.py) — paged state, a per-sequence line, speculative rounds, and both together. Needs the copy that
`python baseline/install_ref.py --reference <checkout>` leaves under baseline/_ref; skipped without it."""
import json
import random

import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("target", ["toy-paged", "toy-stateful", "toy-spec", "toy-stateful-spec"])
def test_reference_toy_package_serves_the_oracles_tokens(cuda, target):
    from kern_b200.engine import Engine
    from kern_b200.runtime import Runtime
    from kern_b200.serve.scheduler import Request, Scheduler
    from kern_b200.testing import bench_toy

    if not bench_toy.available():
        pytest.skip("baseline/_ref/toy_pkg is not installed")
    pkg = bench_toy.PKG
    doc = json.loads((pkg / f"{target}.json").read_text())
    rt = Runtime(json.dumps(doc), kernels=pkg / "kernels", weights=[pkg / "model" / "toy.safetensors"], tokens=16 * 600, slots=12)
    rt.once()
    sch = Scheduler(Engine(rt), chunk=256, max_seqs=6)
    rng = random.Random(11)
    prompts = [[rng.randrange(256) for _ in range(n)] for n in (1, 9, 130, 300, 47, 700, 16, 33)]
    model = bench_toy.oracle()
    reqs = [Request(id=str(i), prompt=p, max_tokens=12, stop_ids=(model.EOS,)) for i, p in enumerate(prompts)]
    for r in reqs:
        sch.submit(r)
    sch.run_until_idle(5000)
    rt.check_error()
    assert sch.idle()
    for r in reqs:
        want = model.generate(r.prompt, 12, doc)
        got = [t for t in r.out if t != model.EOS]
        assert got == want, (target, r.id, got, want)
    # a second turn over the kept prefix: the history of request 3 plus new tokens
    turn2 = Request(id="t2", prompt=prompts[3] + [t for t in reqs[3].out if t != model.EOS] + [5, 6, 7], max_tokens=6,
                    stop_ids=(model.EOS,))
    sch.submit(turn2)
    sch.run_until_idle(500)
    rt.check_error()
    assert [t for t in turn2.out if t != model.EOS] == model.generate(turn2.prompt, 6, doc)
