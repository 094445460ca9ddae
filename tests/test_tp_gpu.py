"""Tensor parallelism over NVLink peer memory: the fused all-reduce + residual + RMSNorm kernel and the
tensor-parallel decoder, as one process per GPU; plus the bounded wait of the peer barrier on one GPU
(a flag that nothing sets makes the wait run out and the kernel report which rank is missing)."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_peer_barrier_wait_runs_out_and_names_the_missing_rank(cuda):
    from kern_b200.ops.launcher import Kernels, i32, i64, ptr
    import struct

    k = Kernels.get(cuda)
    flags = torch.zeros(8, dtype=torch.int32, device=cuda)
    epoch = torch.zeros(1, dtype=torch.int32, device=cuda)
    err = torch.zeros(1, dtype=torch.int32, device=cuda)
    # a "group" of 3 whose other two members never launch: every flag pointer is this rank's own array, so
    # rank 0's own arrival shows up and ranks 1 and 2 never do
    peers = torch.tensor([flags.data_ptr()] * 3, dtype=torch.int64, device=cuda)
    k.launch("tp_allreduce_norm", "kern_peer_barrier", (1,), (32,),
             [ptr(flags), ptr(peers), ptr(epoch), ptr(err), i32(0), i32(3), i64(2_000_000)])   # 2 ms
    torch.cuda.synchronize()
    assert int(err.item()) in (201, 202)
    assert int(epoch.item()) == 1 and int(flags[0].item()) == 1
    # the context is still usable and a complete group passes
    err.zero_()
    peers1 = torch.tensor([flags.data_ptr()], dtype=torch.int64, device=cuda)
    k.launch("tp_allreduce_norm", "kern_peer_barrier", (1,), (32,),
             [ptr(flags), ptr(peers1), ptr(epoch), ptr(err), i32(0), i32(1), i64(2_000_000)])
    torch.cuda.synchronize()
    assert int(err.item()) == 0 and int(epoch.item()) == 2


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tp_allreduce_and_model(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29500 + world), "-m", "kern_b200.parallel.tp_check", "--rows", "1", "8", "64", "65", "300", "1000"]
    p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    lines = [json.loads(l) for l in p.stdout.splitlines() if l.startswith("{")]
    assert p.returncode == 0, (p.stdout[-3000:], p.stderr[-3000:])
    ar = next(l for l in lines if l["check"] == "allreduce_residual_norm")
    assert all(r["ok"] for r in ar["results"]) and len(ar["results"]) == 12
    model = next(l for l in lines if l["check"] == "tp_model")
    assert model["ok"], model


def test_collective_externs_group_of_one(cuda):
    """`extern:nccl_*` launches on one rank: no communicator, every collective is a device copy (eager and captured)."""
    from kern_b200.parallel import coll_check

    assert coll_check.main(["--sizes", "1", "1000"]) == 0


@pytest.mark.parametrize("world", [2, 4])
def test_collective_externs(world):
    """All-reduce, all-gather, reduce-scatter and all-to-all built-ins over NCCL, one process per GPU; the communicator
    id travels in rank 0's offer."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29520 + world), "-m", "kern_b200.parallel.coll_check"]
    p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, (p.stdout[-3000:], p.stderr[-3000:])
    line = next(json.loads(l) for l in p.stdout.splitlines() if l.startswith("{"))
    assert line["world"] == world and all(r["ok"] for r in line["results"]), line


def test_decode_context_parallel_one_rank(cuda):
    """The dealt-position path with a group of one: local lengths, partial slots, merge over ranks."""
    from kern_b200.parallel import dcp_check

    assert dcp_check.main(["--lens", "1", "65", "300", "--model"]) == 0


@pytest.mark.parametrize("world", [2, 4])
def test_decode_context_parallel(world):
    """Positions dealt over the ranks, per-rank partial attention, all-gather over NVLink, one merge."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29540 + world), "-m", "kern_b200.parallel.dcp_check", "--model"]
    p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, (p.stdout[-3000:], p.stderr[-3000:])
    lines = [json.loads(l) for l in p.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 2 and all(l["ok"] and l["world"] == world for l in lines), lines


@pytest.mark.parametrize("lined", [False, True])
def test_prefill_decode_two_gpu_processes(lined):
    """A prefill process and a decode process on two GPUs: seats reserved, pages and the state slot pushed into the
    decode tier's exported pools by device copies, tokens equal to the exact model's twin."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(29560 + int(lined)), "-m", "kern_b200.parallel.pd_check"] + (["--lined"] if lined else [])
    p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, (p.stdout[-3000:], p.stderr[-3000:])
    line = next(json.loads(l) for l in p.stdout.splitlines() if l.startswith("{"))
    assert line["ok"] and line["busy_seen"], line


@pytest.mark.parametrize("world", [2, 4])
def test_pipeline_with_a_process_per_stage(world):
    """`cut` stage manifests on their own GPUs and processes; crossing workspaces pushed into the next stage's exported
    landing buffers; tokens equal the uncut model's."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29570 + world), "-m", "kern_b200.parallel.pp_check"]
    p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, (p.stdout[-3000:], p.stderr[-3000:])
    line = next(json.loads(l) for l in p.stdout.splitlines() if l.startswith("{"))
    assert line["ok"] and line["stages"] == world and line["crossing_bytes"] > 0, line


def test_allgather_gemm_one_rank(cuda):
    """The all-gather GEMM with a group of one: no rows to pull, every counter still moves by the grid size per launch
    (row counts change between launches, then a captured replay)."""
    from kern_b200.parallel import ag_gemm_check

    assert ag_gemm_check.main(["--rows", "128", "512", "256", "--n", "512", "--k", "1024"]) == 0


@pytest.mark.parametrize("world", [2, 4])
def test_allgather_gemm_fused(world):
    """Rows sharded over the ranks; one kernel pulls the peers' slices over NVLink while the tensor cores run the local
    ones; the product equals the GEMM over all rows (whatever was not pulled would be NaN)."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29580 + world), "-m", "kern_b200.parallel.ag_gemm_check"]
    p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, (p.stdout[-3000:], p.stderr[-3000:])
    line = next(json.loads(l) for l in p.stdout.splitlines() if l.startswith("{"))
    assert line["world"] == world and all(r["ok"] for r in line["results"]), line


def test_expert_parallel_all_to_all_one_rank(cuda):
    """The sharded-token expert-parallel layer with a group of one: dispatch and return go through the peer tables
    (which hold this rank's own addresses)."""
    from kern_b200.parallel import ep_check

    assert ep_check.main(["--rows", "8", "130"]) == 0


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_all_to_all(world):
    """Tokens and experts sharded over the ranks: ids all-gathered, rows pulled from their home ranks by the gather that
    feeds the grouped GEMMs, results pushed back into per-(token, choice) slots; equals the dense mixture."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29600 + world), "-m", "kern_b200.parallel.ep_check"]
    p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, (p.stdout[-3000:], p.stderr[-3000:])
    line = next(json.loads(l) for l in p.stdout.splitlines() if l.startswith("{"))
    assert line["world"] == world and all(r["ok"] for r in line["results"]), line


@pytest.mark.parametrize("form", ["bf16", "mx"])
def test_expert_parallel_fused_one_rank(cuda, form):
    """Dispatch inside FC1, combine inside FC2, with a group of one (every pull and slot store goes through the peer
    tables, which hold this rank's own addresses): the layer against the dense mixture at three sizes and as a graph,
    then the MoE decoder over it. `mx`: MXFP4 expert weights, MXFP8 activations (the block-scaled tcgen05 pair)."""
    from kern_b200.parallel import ep_check

    assert ep_check.main(["--fused", "--model", "--rows", "8", "200", "64"] + (["--mx"] if form == "mx" else [])) == 0


@pytest.mark.parametrize("form", ["bf16", "mx"])
@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_fused(world, form):
    """The fused dispatch / combine layer and the sharded-token decoder on 2 and 4 ranks: rows cross NVLink inside the
    routed GEMMs (peer loads in FC1's gather warps, peer stores in FC2's epilogue), no barrier kernel, no NCCL call in
    the layer; guard bands around every allocation stay intact."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29620 + world), "-m", "kern_b200.parallel.ep_check", "--fused", "--model"]
    p = subprocess.run(cmd + (["--mx"] if form == "mx" else []), cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, (p.stdout[-3000:], p.stderr[-3000:])
    lines = [json.loads(l) for l in p.stdout.splitlines() if l.startswith("{")]
    assert lines[0]["world"] == world and all(r["ok"] for r in lines[0]["results"]), lines[0]
    assert lines[1]["ok"], lines[1]


@pytest.mark.parametrize("shape", ["pd", "pd-dcp", "pp"])
def test_deployments_from_the_launcher(shape):
    """`serve/launch.py` on two GPUs: a prefill tier in the launching process with a decode tier as a spawned process
    (pools exported and mapped, pages pushed by device copies); the same with the decode tier a context-parallel group
    of two rank processes (the prompt's rows dealt into both members' mapped pools); and a pipeline with a process per
    stage. All under the scheduler, token for token the output of one engine (the context-parallel group: the first
    token of every request exactly, the rest up to rounding in the merge of partial attention)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "kern_b200.serve.launch"] + {"pd": ["--pd"], "pd-dcp": ["--pd", "--dcp", "2"], "pp": ["--stages", "2"]}[shape]
    p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, (p.stdout[-3000:], p.stderr[-3000:])
    line = json.loads([l for l in p.stdout.splitlines() if l.startswith("{")][-1])
    assert line["ok"] and line["tokens"] == 20, line
