"""Benchmark of the forest-inference hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the configuration the headline metric is quoted on): a synthetic gradient-boosted binary
forest of 1000 complete depth-8 trees over 256 fp32 features (feature ~ U{0..255}, threshold ~
N(0,1), leaves ~ N(0, 0.1), sigmoid), predicting probabilities for 10,000,000 seed-generated
N(0,1) rows per GPU.  One step = one prediction pass over the whole batch.  With N > 1 (launched
by torchrun, one rank per GPU) the forest is replicated and every rank predicts its own 10 M rows:
no collective is on the data path, weak scaling.

Prints ONE JSON line (rank 0).  `value` is rows/s with rows resident in HBM; `e2e` is rows/s through
`ForestInference.predict_proba` on pinned HOST arrays (copies inside the timed region);
`roofline` relates the kernel to the measured HBM copy bandwidth through the algorithmic bytes per
row (256 * 4 read + 2 * 4 written = 1032 B); `cpu_baseline` is the CPU oracle on this box's cores.
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
    oracle.predict(desc, probe[:256], INFER_PROBA2, "single", n_threads=cores)
    t0 = time.perf_counter()
    oracle.predict(desc, probe, INFER_PROBA2, "single", n_threads=cores)
    rate = probe.shape[0] / (time.perf_counter() - t0)
    n = int(min(ROWS_PER_GPU, max(4096, rate * seconds_target)))
    X = rng.standard_normal((n, N_FEATURES)).astype(np.float32)
    t0 = time.perf_counter()
    oracle.predict(desc, X, INFER_PROBA2, "single", n_threads=cores)
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
        oracle.predict(desc, X, INFER_PROBA2, "single", n_threads=cores)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.predict(desc, X, INFER_PROBA2, "single", n_threads=cores)
    dt = (time.perf_counter() - t0) / args.steps
    value = n / dt
    sample = f"{n} of {ROWS_PER_GPU} rows per step, same forest, {cores} OpenMP threads"
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


def measure_e2e(fi, X, out, n, world, dev, barrier, args):
    """Rows/s through `predict_proba` on pinned host arrays: copies inside the timed region."""
    import numpy as np
    import psutil
    import torch
    import torch.distributed as dist

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

    return {"value": e2e_rows * world / e2e_s, "unit": "rows/s",
            "h2d_bytes_per_step": e2e_rows * N_FEATURES * 4,
            "d2h_bytes_per_step": e2e_rows * 2 * 4, "rows_per_step": e2e_rows,
            "matches_device_path": e2e_ok}


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
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
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
    clocks = sampler.stop() if rank == 0 else None
    total_ms = t_start.elapsed_time(t_end)
    kernel_ms = [a.elapsed_time(b) for a, b in ev]
    total_ms = max_over_ranks(torch.tensor([total_ms], device=dev, dtype=torch.float64), world)
    ms_per_step = total_ms / args.steps
    value = whole_job_rows_per_s(n, world, ms_per_step)

    e2e = None
    if not args.no_e2e:
        e2e = measure_e2e(fi, X, out, n, world, dev, barrier, args)

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
                         "kernel": "quantise_kernel<float> + dense_q_top_kernel<float,MODE_SCALAR,6,8>",
                         "kernel_ms": k_ms, "algorithmic_bytes_per_row": BYTES_PER_ROW},
            "e2e": e2e,
            "gpu_launches": int(launches),
            "clocks": clocks,
        }
        if world == 1 and not args.no_latency:
            line["latency"] = measure_latency(fi, X, dev)
        if world == 1 and not args.no_cpu:
            v, cores, sample_n = cpu_rows_per_s(desc, 15.0)
            line["cpu_baseline"] = {
                "value": v, "unit": "rows/s", "cores": cores, "kind": "port",
                "sample": f"{sample_n} of {n} rows, same forest, {cores} OpenMP threads"}
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
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
