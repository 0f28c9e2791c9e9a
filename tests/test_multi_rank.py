"""The N > 1 arrangement of the benchmark is data-parallel replicas: no data-path collective, one barrier and
a MAX over the ranks' device times, whole-job throughput = ranks x units / slowest rank.  Checked here with two
gloo ranks on CPU (the GPU run uses the same code with the nccl backend)."""
import os
import subprocess
import sys
import textwrap

from tests.util import free_port

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent(
    """
    import os, sys
    sys.path.insert(0, %r)
    import torch
    import torch.distributed as dist
    import bench

    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    ms = 10.0 * (rank + 1)                      # rank 1 is the slow one
    agg_ms = bench.max_over_ranks(ms, dist, device="cpu")
    value = bench.whole_job_rate(world, steps=2, units_per_step=5, ms=agg_ms)
    assert agg_ms == 20.0, agg_ms
    assert abs(value - world * 2 * 5 / 0.020) < 1e-6, value
    dist.barrier()
    dist.destroy_process_group()
    print("ok", rank)
    """
) % ROOT


def test_replica_aggregation_two_gloo_ranks(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(free_port()), WORLD_SIZE="2", GLOO_SOCKET_IFNAME="lo")
    procs = []
    for rank in range(2):
        e = dict(env, RANK=str(rank), LOCAL_RANK=str(rank))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=e, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=120)[0] for p in procs]
    for rank, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, out
        assert f"ok {rank}" in out
