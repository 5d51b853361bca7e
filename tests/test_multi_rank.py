"""Host-side logic of the multi-GPU paths, on CPU: the contiguous row split used by the sharded
predictor, and the per-rank bookkeeping of the benchmark (row shards per rank, max-over-ranks time,
whole-job throughput) with two `gloo` ranks."""
import os
import socket
import subprocess
import sys

import pytest

from cuml_b200.fil.multi_gpu import shard_rows
from tests.conftest import ROOT


@pytest.mark.parametrize("n,g", [(0, 1), (1, 8), (7, 3), (100, 8), (10_000_000, 8), (13, 13)])
def test_shard_rows_cover_every_row_once(n, g):
    shards = shard_rows(n, g)
    assert len(shards) == g
    assert shards[0][0] == 0 and shards[-1][1] == n
    for (b0, e0), (b1, e1) in zip(shards, shards[1:]):
        assert e0 == b1 and b0 <= e0
    sizes = [e - b for b, e in shards]
    assert max(sizes) - min(sizes) <= 1


def test_shard_rows_rejects_bad_arguments():
    with pytest.raises(ValueError):
        shard_rows(10, 0)
    with pytest.raises(ValueError):
        shard_rows(-1, 2)


WORKER = r"""
import os, sys, json
sys.path.insert(0, sys.argv[1])
import torch, torch.distributed as dist
import bench
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
# every rank owns its rows; the job's time is the slowest rank's and the throughput counts all rows
ms = torch.tensor([10.0 + 5.0 * rank], dtype=torch.float64)
total = bench.max_over_ranks(ms, world)
value = bench.whole_job_rows_per_s(1000, world, total)
ok = abs(total - 15.0) < 1e-12 and abs(value - 2000 / 15e-3) < 1e-6
print(json.dumps({"rank": rank, "ok": ok, "total": total, "value": value}))
dist.destroy_process_group()
"""


def test_two_gloo_ranks_reduce_time_and_throughput(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, OMP_NUM_THREADS="1")
    for attempt in range(3):  # a freshly probed port can be taken by the time torchrun binds it
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node",
               "2", "--master-addr", "127.0.0.1", "--master-port", str(port), str(script), ROOT]
        out = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)
        if out.returncode == 0:
            break
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 2
    import json

    assert all(json.loads(ln)["ok"] for ln in lines)
