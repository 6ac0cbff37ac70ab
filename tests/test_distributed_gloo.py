"""World-size-2 checks of the multi-GPU plumbing on CPU (gloo): sharding, gradient averaging, max-over-ranks timing."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mlcg_b200.distributed import allreduce_gradients, max_over_ranks, shard_range


def test_shard_ranges_partition_the_structures():
    for B, W in [(512, 8), (10, 4), (3, 8), (1024, 3)]:
        spans = [shard_range(B, r, W) for r in range(W)]
        assert spans[0][0] == 0 and spans[-1][1] == B
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [hi - lo for lo, hi in spans]
        assert max(sizes) - min(sizes) <= 1


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(0)                                   # same model on every rank
    model = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.Tanh(), torch.nn.Linear(5, 1))
    data = torch.arange(8 * 6, dtype=torch.float32).view(8, 6) / 10
    lo, hi = shard_range(8, rank, world)
    model(data[lo:hi]).sum().backward()                    # each rank: its own shard of structures
    allreduce_gradients(model.parameters())
    ref = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.Tanh(), torch.nn.Linear(5, 1))
    ref.load_state_dict(model.state_dict())
    (ref(data).sum() / world).backward()                   # gradient of the mean over ranks of per-shard sums
    ok = all(torch.allclose(p.grad, q_.grad, atol=1e-6) for p, q_ in zip(model.parameters(), ref.parameters()))
    slowest = max_over_ranks(1.0 + rank, torch.device("cpu"))
    q.put((rank, ok, slowest))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_gradient_average_and_timing():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _ in results)
    assert all(slowest == 2.0 for _, _, slowest in results)


def test_reference_arm_under_two_ranks_prints_one_line():
    """`bench.py --impl reference` launched the way the multi-GPU runs are: rank 0 alone times the CPU arm and prints the JSON
    line, the other rank exits 0 without work."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    port = 31500 + os.getpid() % 2000
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(root, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "1"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=root)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["n_gpus"] == 2 and line["value"] > 0
    from oracle import mlcg_loader
    # mlcg's own modules where oracle/build_ref.py has installed them, else the restatement
    assert line["cpu_baseline"]["kind"] == ("reference" if mlcg_loader.available() else "port") and line["e2e"]["h2d_bytes_per_step"] == 0
