"""Benchmark of the forest-inference hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the configuration the headline metric is quoted on): a synthetic gradient-boosted binary
forest of 1000 complete depth-8 trees over 256 fp32 features (feature ~ U{0..255}, threshold ~
N(0,1), leaves ~ N(0, 0.1), sigmoid), predicting probabilities for 10,000,000 seed-generated
N(0,1) rows per GPU.  One step = one prediction pass over the whole batch.  With N > 1 (launched
by torchrun, one rank per GPU) the forest is replicated and every rank predicts its own 10 M rows:
no collective is on the data path, weak scaling.

Prints ONE JSON line (rank 0).  `value` is rows/s with rows resident in HBM; `e2e` is rows/s through
`ForestInference.predict_proba` on pinned HOST arrays (copies inside the timed region), with the
bare host-to-device copy rate of the same buffers (`h2d_only_GBps`, the ceiling of that path) and
the figure for pageable host arrays beside it; `roofline` relates the kernel to the measured HBM
copy bandwidth through the algorithmic bytes per row (256 * 4 read + 2 * 4 written = 1032 B), the
kernel names come from the library (`b2fil_last_variant`); `cpu_baseline` is the CPU oracle on this
box's cores.

`sharded` is the product's own multi-GPU path on the scale-out configuration: ONE process (rank 0;
the other ranks have freed their memory and wait on a CPU barrier) drives all N GPUs through
`ShardedForestInference` / `b2fil_predict_sharded` - forest of 2000 depth-10 trees over 512
features replicated by peer copies, 100,000,000 rows in total split into contiguous shards
(strong scaling), results gathered on GPU 0 by peer copies.  100 M x 512 fp32 rows (205 GB) do
not fit the GPUs that a small N offers, so every GPU keeps one resident buffer of 12.5 M rows and
predicts it once per pass until its share of the 100 M rows is done (8 passes at N = 1, one at
N = 8).  The same run also times one GPU alone, which gives the efficiency.

At N = 1 `other_configs` adds the remaining benchmark configurations (one line each from
bench_configs.py: rows/s, roofline fraction, CPU figures, parity of a row sample).

`--impl reference` times the CPU implementation (the oracle port: the reference's own CPU code for
this path is not in its tree) on a bounded row sample with all host threads.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_TREES, DEPTH, N_FEATURES = 1000, 8, 256
ROWS_PER_GPU = 10_000_000
BYTES_PER_ROW = N_FEATURES * 4 + 2 * 4
WORKLOAD = "gbdt_1000x_depth8_256f_fp32_sigmoid_10M_rows"
# dram__bytes_read.sum + dram__bytes_write.sum per row of the two kernels of a prediction, from
# the ncu captures of a 1 M-row case summarised under profiles/ (quantise 1560 B + dense_q 525 B;
# the rank image of a chunk is larger than L2 and goes through HBM); traffic grows in proportion to
# the rows, so it is scaled to the batch
NCU_TRAFFIC_BYTES_PER_ROW = 2085
NCU_TRAFFIC_KERNELS = "quantise_kernel<float> + dense_q_top_kernel<float,scalar,NT=6,DEPTH=8>"


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms",
                 "200", "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, v in zip(names, parts[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def max_over_ranks(t, world: int) -> float:
    """Largest value of a one-element tensor over all ranks (the job ends with its slowest rank)."""
    if world > 1:
        import torch.distributed as dist

        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def whole_job_rows_per_s(rows_per_rank: int, world: int, ms_per_step: float) -> float:
    """Rows all ranks processed in one step over the time of the slowest rank."""
    return rows_per_rank * world / (ms_per_step * 1e-3)


def build_forest_desc():
    from cuml_b200.fil import synthetic_complete_forest

    return synthetic_complete_forest(N_TREES, DEPTH, N_FEATURES, seed=2)


def cpu_rows_per_s(desc, seconds_target: float, seed: int = 3):
    """Rows/s of the CPU oracle with all host threads on a sample sized for ~seconds_target."""
    import numpy as np

    from cuml_b200.fil._desc import INFER_PROBA2
    from oracle import oracle

    cores = os.cpu_count() or 1
    rng = np.random.default_rng(seed)
    probe = rng.standard_normal((4096, N_FEATURES)).astype(np.float32)
    # the packed walk of the oracle: same results as the plain walk the tests use, several times
    # faster (one record per node, eight rows side by side)
    oracle.predict(desc, probe[:256], INFER_PROBA2, "single", n_threads=cores, packed=True)
    t0 = time.perf_counter()
    oracle.predict(desc, probe, INFER_PROBA2, "single", n_threads=cores, packed=True)
    rate = probe.shape[0] / (time.perf_counter() - t0)
    n = int(min(ROWS_PER_GPU, max(4096, rate * seconds_target)))
    X = rng.standard_normal((n, N_FEATURES)).astype(np.float32)
    t0 = time.perf_counter()
    oracle.predict(desc, X, INFER_PROBA2, "single", n_threads=cores, packed=True)
    dt = time.perf_counter() - t0
    return n / dt, cores, n


def run_reference(args):
    """CPU arm: the oracle port with all host threads, each step a bounded row sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np

    from cuml_b200.fil._desc import INFER_PROBA2
    from oracle import oracle

    desc = build_forest_desc()
    cores = os.cpu_count() or 1
    rate, _, _ = cpu_rows_per_s(desc, 2.0)
    budget = 120.0 / max(1, args.steps + args.warmup)  # whole run within a few minutes
    n = int(min(ROWS_PER_GPU, max(4096, rate * min(10.0, budget))))
    X = np.random.default_rng(3).standard_normal((n, N_FEATURES)).astype(np.float32)
    for _ in range(args.warmup):
        oracle.predict(desc, X, INFER_PROBA2, "single", n_threads=cores, packed=True)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.predict(desc, X, INFER_PROBA2, "single", n_threads=cores, packed=True)
    dt = (time.perf_counter() - t0) / args.steps
    value = n / dt
    sample = (f"{n} of {ROWS_PER_GPU} rows per step, same forest, {cores} OpenMP threads, packed "
              "node records, eight rows side by side")
    print(json.dumps({
        "impl": "reference", "metric": "rows/sec (1000-tree depth-8 fp32)", "value": value,
        "unit": "rows/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "rows_per_step": n},
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "note": "reference FIL CPU backend (nvForest) is not in the reference tree and not "
                "installed; this arm times the CPU oracle port"}))


def measure_latency(fi, X, dev, batches=(1, 1024, 65536), calls=300):
    """p50 / p99 wall-clock latency (ms) of one `predict_proba` call on device rows, synchronised."""
    import torch

    res = {}
    for b in batches:
        xb = X[:b]
        ob = torch.empty((b, 2), device=dev, dtype=torch.float32)
        for _ in range(20):
            fi.predict_proba(xb, preds=ob)
        torch.cuda.synchronize(dev)
        ts = []
        for _ in range(calls):
            t0 = time.perf_counter()
            fi.predict_proba(xb, preds=ob)
            torch.cuda.synchronize(dev)
            ts.append((time.perf_counter() - t0) * 1e3)
        ts.sort()
        res[str(b)] = {"p50_ms": ts[len(ts) // 2], "p99_ms": ts[min(len(ts) - 1, int(len(ts) * 0.99))]}
    return res


def gpu_numa_node(local: int):
    """NUMA node of the GPU's PCIe slot and the CPUs of that node, from sysfs (None if unknown)."""
    try:
        import torch

        p = torch.cuda.get_device_properties(local)
        bus = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as fh:
            node = int(fh.read().strip())
        if node < 0:
            return None, None
        with open(f"/sys/devices/system/node/node{node}/cpulist") as fh:
            cpus = set()
            for part in fh.read().strip().split(","):
                a, _, b = part.partition("-")
                cpus.update(range(int(a), int(b or a) + 1))
        return node, cpus
    except Exception:
        return None, None


def n_numa_nodes() -> int:
    try:
        return len([d for d in os.listdir("/sys/devices/system/node") if d.startswith("node")])
    except Exception:
        return 1


def measure_e2e(fi, X, out, n, world, dev, barrier, args):
    """Rows/s through `predict_proba` on pinned host arrays: copies inside the timed region."""
    import numpy as np
    import psutil
    import torch
    import torch.distributed as dist

    # Host placement: on a box with several NUMA nodes the pinned buffer is allocated (first
    # touch) and fed from the node the GPU hangs on.
    node, cpus = gpu_numa_node(dev.index)
    nodes = n_numa_nodes()
    bound = False
    if nodes > 1 and cpus:
        try:
            allowed = os.sched_getaffinity(0) & cpus
            if allowed:
                os.sched_setaffinity(0, allowed)
                bound = True
        except Exception:
            pass
    # every rank pins its own host copy: keep it below a quarter of the rank's share of free RAM
    e2e_rows = n
    need = e2e_rows * N_FEATURES * 4
    avail = psutil.virtual_memory().available / max(1, world)
    while need * 4 > avail and e2e_rows > 100_000:
        e2e_rows //= 2
        need = e2e_rows * N_FEATURES * 4
    if world > 1:  # every rank times the same number of rows
        agreed = torch.tensor([e2e_rows], device=dev, dtype=torch.int64)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        e2e_rows = int(agreed.item())
    Xh = torch.empty((e2e_rows, N_FEATURES), dtype=torch.float32, pin_memory=True)
    Xh.copy_(X[:e2e_rows])
    oh = torch.empty((e2e_rows, 2), dtype=torch.float32, pin_memory=True)
    Xh_np, oh_np = Xh.numpy(), oh.numpy()
    e2e_steps = max(1, min(args.steps, 3))
    fi.predict_proba(Xh_np, preds=oh_np)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        fi.predict_proba(Xh_np, preds=oh_np)
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    e2e_s = max_over_ranks(torch.tensor([e2e_s], device=dev, dtype=torch.float64), world)
    e2e_ok = bool(np.allclose(oh_np[:1000], out[:1000].cpu().numpy(), rtol=1e-6, atol=1e-7))

    # the ceiling of that path: the same pinned buffer copied to the device and nothing else
    dst = X[:e2e_rows]
    dst.copy_(Xh, non_blocking=True)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        dst.copy_(Xh, non_blocking=True)
    torch.cuda.synchronize(dev)
    h2d_s = (time.perf_counter() - t0) / e2e_steps
    h2d_s = max_over_ranks(torch.tensor([h2d_s], device=dev, dtype=torch.float64), world)
    h2d_gbps = e2e_rows * N_FEATURES * 4 * world / h2d_s / 1e9

    # pageable host memory: what a user who passes an ordinary NumPy array gets
    pg_rows = min(e2e_rows, 2_000_000)
    Xp = np.empty((pg_rows, N_FEATURES), np.float32)
    Xp[:] = Xh_np[:pg_rows]
    op = np.empty((pg_rows, 2), np.float32)
    fi.predict_proba(Xp, preds=op)
    barrier()
    t0 = time.perf_counter()
    for _ in range(2):
        fi.predict_proba(Xp, preds=op)
    pg_s = (time.perf_counter() - t0) / 2
    pg_s = max_over_ranks(torch.tensor([pg_s], device=dev, dtype=torch.float64), world)
    del Xh, oh, Xh_np, oh_np, Xp, op

    return {"value": e2e_rows * world / e2e_s, "unit": "rows/s",
            "h2d_bytes_per_step": e2e_rows * N_FEATURES * 4,
            "d2h_bytes_per_step": e2e_rows * 2 * 4, "rows_per_step": e2e_rows,
            "matches_device_path": e2e_ok,
            "GBps_host_to_device": e2e_rows * N_FEATURES * 4 * world / e2e_s / 1e9,
            "h2d_only_GBps": h2d_gbps,
            "fraction_of_h2d_only": (e2e_rows * N_FEATURES * 4 * world / e2e_s / 1e9) / h2d_gbps,
            "pageable": {"value": pg_rows * world / pg_s, "unit": "rows/s",
                         "rows_per_step": pg_rows},
            "host": {"numa_nodes": nodes, "gpu_numa_node_rank0": node,
                     "bound_to_gpu_node": bound, "cpus_allowed": len(os.sched_getaffinity(0))}}


C5_TREES, C5_DEPTH, C5_FEATURES = 2000, 10, 512
C5_TOTAL_ROWS = 100_000_000
C5_BUFFER_ROWS = 12_500_000
C5_BYTES_PER_ROW = C5_FEATURES * 4 + 2 * 4


def measure_sharded(n_dev: int, steps: int, total_rows: int = C5_TOTAL_ROWS,
                    buffer_rows: int = C5_BUFFER_ROWS):
    """The product's single-process multi-GPU path on the scale-out configuration (strong
    scaling): one device alone, then all `n_dev` devices, same total row count."""
    import torch

    from cuml_b200.fil import ForestInference, _lib, synthetic_complete_forest
    from cuml_b200.fil.multi_gpu import ShardedForestInference

    desc = synthetic_complete_forest(C5_TREES, C5_DEPTH, C5_FEATURES, seed=6)
    fi = ForestInference.load_from_treelite_model(desc, device_id=0)
    peak, peak_kind = measured_peak()
    records = {}
    shards = {}
    for nd in sorted({1, n_dev}):
        sh = ShardedForestInference(fi, list(range(nd)))
        per_dev = total_rows // nd
        buf = min(per_dev, buffer_rows)
        passes = -(-per_dev // buf)
        for d in range(nd):
            if d not in shards or shards[d].shape[0] != buf:
                g = torch.Generator(device=f"cuda:{d}")
                g.manual_seed(7 + d)
                x = torch.empty((buf, C5_FEATURES), device=f"cuda:{d}", dtype=torch.float32)
                for b in range(0, buf, 2_500_000):
                    e = min(buf, b + 2_500_000)
                    x[b:e] = torch.randn((e - b, C5_FEATURES), generator=g, device=f"cuda:{d}")
                shards[d] = x
        xs = [shards[d] for d in range(nd)]
        out = torch.empty((nd * buf, 2), device="cuda:0", dtype=torch.float32)
        sh.predict_proba(xs, preds=out)  # warm-up: pools, kernel attributes, peer mappings
        variant = _lib.last_variant()
        sh.predict_proba(xs, preds=out)
        wall = compute = gather = 0.0
        direct = 1
        for _ in range(steps):
            for _ in range(passes):
                sh.predict_proba(xs, preds=out)
                t = sh.last_timing()
                wall += t["wall_ms"]
                compute += t["compute_ms"]
                gather += t["gather_ms"]
                direct &= t["gather_direct"]
        wall /= steps
        rows = passes * buf * nd
        # the sharded result of device 0's rows equals what device 0 predicts on its own
        alone = fi.predict_proba(xs[0][:100_000])
        same = bool(torch.equal(alone, out[:100_000]))
        records[nd] = {
            "n_devices": nd, "rows_total": rows, "passes_per_step": passes,
            "rows_per_device_per_pass": buf, "wall_ms_per_step": wall,
            "rows_per_s": rows / (wall * 1e-3),
            "compute_ms_per_step": compute / steps, "gather_ms_per_step": gather / steps,
            "gather_direct": bool(direct), "gather_bytes_per_step": (nd - 1) * buf * passes * 8,
            "hbm_frac": rows / (wall * 1e-3) * C5_BYTES_PER_ROW / 1e9 / (peak * nd),
            "matches_single_device": same, "kernel": variant}
        del sh, out
    one = records[1]
    rec = dict(records[n_dev])
    rec.update({
        "workload": "gbdt_2000x_depth10_512f_fp32_sigmoid_100M_rows_row_sharded",
        "scaling": "strong", "driver": "one process, b2fil_predict_sharded",
        "resident_rows_note": "each GPU predicts one resident 12.5 M-row buffer once per pass "
                              "(100 M x 512 fp32 = 205 GB does not fit a small N)",
        "one_device_rows_per_s": one["rows_per_s"],
        "efficiency_vs_one_device": rec["rows_per_s"] / (n_dev * one["rows_per_s"]),
        "hbm_peak": peak_kind, "algorithmic_bytes_per_row": C5_BYTES_PER_ROW})
    del shards
    for d in range(n_dev):
        with torch.cuda.device(d):
            torch.cuda.empty_cache()
    return rec


def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    from cuml_b200.fil import ForestInference, _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: there is no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    cpu_group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        # waits that must leave the GPUs idle (the sharded leg) use a CPU barrier
        cpu_group = dist.new_group(backend="gloo")
    lib = _lib.load()
    desc = build_forest_desc()
    fi = ForestInference.load_from_treelite_model(desc, device_id=local)
    n = args.rows
    g = torch.Generator(device=dev)
    g.manual_seed(3 + rank)
    X = torch.randn((n, N_FEATURES), generator=g, device=dev, dtype=torch.float32)
    out = torch.empty((n, 2), device=dev, dtype=torch.float32)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()  # samples cover the warm-up and the timed steps (both under load)
    for _ in range(max(3, args.warmup)):
        fi.predict_proba(X, preds=out)
    barrier()
    launches0 = lib.b2fil_kernel_launches()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
          for _ in range(args.steps)]
    barrier()
    t_start = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    t_start.record()
    for a, b in ev:
        a.record()
        fi.predict_proba(X, preds=out)
        b.record()
    t_end.record()
    barrier()
    launches = lib.b2fil_kernel_launches() - launches0
    variant = _lib.last_variant()
    fi.check_status()
    clocks = sampler.stop() if rank == 0 else None
    total_ms = t_start.elapsed_time(t_end)
    kernel_ms = [a.elapsed_time(b) for a, b in ev]
    total_ms = max_over_ranks(torch.tensor([total_ms], device=dev, dtype=torch.float64), world)
    ms_per_step = total_ms / args.steps
    value = whole_job_rows_per_s(n, world, ms_per_step)

    e2e = None
    if not args.no_e2e:
        e2e = measure_e2e(fi, X, out, n, world, dev, barrier, args)

    latency = None
    if rank == 0 and world == 1 and not args.no_latency:
        latency = measure_latency(fi, X, dev)

    # The sharded leg: every rank frees its rows, rank 0 alone drives all GPUs, the others wait
    # on the CPU (a NCCL barrier would keep a kernel spinning on their GPUs).
    sharded = None
    if not args.no_sharded:
        del X, out
        torch.cuda.empty_cache()
        barrier()
        if rank == 0:
            try:
                sharded = measure_sharded(world, max(1, min(args.steps, 2)))
            except Exception as e:  # noqa: BLE001 - the headline line must still be printed
                sharded = {"error": f"{type(e).__name__}: {e}"}
        if world > 1:
            dist.barrier(group=cpu_group)

    if rank == 0:
        peak, peak_kind = measured_peak()
        k_ms = statistics.mean(kernel_ms)
        achieved = n * BYTES_PER_ROW / (k_ms * 1e-3) / 1e9
        line = {
            "metric": "rows/sec (1000-tree depth-8 fp32)", "value": value, "unit": "rows/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "rows_per_gpu": n, "n_trees": N_TREES,
                       "depth": DEPTH, "n_features": N_FEATURES, "storage": "dense",
                       "l2": "inputs (10.24 GB per GPU) are larger than L2",
                       "sharding": f"rows x{world}, forest replicated, no collective"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_kind": peak_kind,
                         "traffic": (NCU_TRAFFIC_BYTES_PER_ROW * n
                                     if NCU_TRAFFIC_BYTES_PER_ROW else None),
                         "kernel": variant,
                         "kernel_ms": k_ms, "algorithmic_bytes_per_row": BYTES_PER_ROW},
            "e2e": e2e,
            "gpu_launches": int(launches),
            "clocks": clocks,
        }
        if not variant.startswith(NCU_TRAFFIC_KERNELS):
            line["roofline"]["traffic"] = None  # the ncu figure belongs to another kernel pair
        if sharded is not None:
            line["sharded"] = sharded
        if latency is not None:
            line["latency"] = latency
        if world == 1 and not args.no_configs:
            import bench_configs

            others = []
            for cfg in args.configs:
                try:
                    others.extend(bench_configs.run(cfg, 3, 1.0, cpu=not args.no_cpu, emit=None))
                except Exception as e:  # noqa: BLE001
                    others.append({"config": cfg, "error": f"{type(e).__name__}: {e}"})
                torch.cuda.empty_cache()
            line["other_configs"] = others
        if world == 1 and not args.no_cpu:
            v, cores, sample_n = cpu_rows_per_s(desc, 15.0)
            line["cpu_baseline"] = {
                "value": v, "unit": "rows/s", "cores": cores, "kind": "port",
                "sample": f"{sample_n} of {n} rows, same forest, {cores} OpenMP threads, packed "
                          "node records, eight rows side by side"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rows", type=int, default=ROWS_PER_GPU, help="rows per GPU")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling)")
    ap.add_argument("--no-latency", action="store_true", help="skip the small-batch latency leg")
    ap.add_argument("--no-sharded", action="store_true",
                    help="skip the single-process multi-GPU leg on the scale-out configuration")
    ap.add_argument("--no-configs", action="store_true",
                    help="skip the other benchmark configurations (N = 1 only)")
    ap.add_argument("--configs", nargs="+", default=["c1", "c3", "c4", "c5"],
                    help="which other configurations to add at N = 1")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
