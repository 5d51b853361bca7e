"""Host-side logic of the multi-GPU paths, on CPU: the contiguous row split used by the sharded
predictor, and the per-rank bookkeeping of the benchmark (row shards per rank, max-over-ranks time,
whole-job throughput) with two `gloo` ranks."""
import os
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
rank, world = int(sys.argv[3]), 2
# a file store needs no network port
dist.init_process_group("gloo", init_method="file://" + sys.argv[2], rank=rank, world_size=world)
# every rank owns its rows; the job's time is the slowest rank's and the throughput counts all rows
ms = torch.tensor([10.0 + 5.0 * rank], dtype=torch.float64)
total = bench.max_over_ranks(ms, world)
value = bench.whole_job_rows_per_s(1000, world, total)
ok = abs(total - 15.0) < 1e-12 and abs(value - 2000 / 15e-3) < 1e-6
print(json.dumps({"rank": rank, "ok": ok, "total": total, "value": value}))
dist.destroy_process_group()
"""


def test_two_gloo_ranks_reduce_time_and_throughput(tmp_path):
    import json

    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    store = tmp_path / "store"
    env = dict(os.environ, OMP_NUM_THREADS="1")
    procs = [subprocess.Popen([sys.executable, str(script), ROOT, str(store), str(r)],
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env)
             for r in range(2)]
    outs = [p.communicate(timeout=240) for p in procs]
    for p, (out, err) in zip(procs, outs):
        assert p.returncode == 0, err[-2000:]
    lines = [ln for out, _ in outs for ln in out.splitlines() if ln.startswith("{")]
    assert len(lines) == 2
    assert all(json.loads(ln)["ok"] for ln in lines)
