"""Throughput of the five benchmark configurations on one GPU, each checked against the CPU
oracle in the run that times it.

    python bench_configs.py [--config c1 c2 c3 c4 c5 sweep] [--steps K] [--rows-scale S] [--no-cpu]
                            [--plain-sparse]

Prints one JSON line per configuration and call: rows/s with device-resident rows (CUDA events on
the launching stream), the algorithmic bytes per row (features read once + outputs written once),
the fraction of the measured HBM copy bandwidth that the row stream reaches, the kernels that ran
(as the library reports them), and a `cpu` record: the CPU oracle (all host threads) timed on a
bounded row sample of the same workload, whose outputs are also what the GPU results of that
sample are compared with (`parity`: scores within rtol 1e-5 / atol 1e-6 in fp32, rtol 1e-12 in
fp64; leaf ids bit-exact), plus scikit-learn with `n_jobs=-1` where scikit-learn trained the model.
`bench.py` measures the headline configuration (c2) under the full reporting contract and embeds
the other lines; this file is the quick way to run one shape (e.g. under a profiler).

  c1  scikit-learn RandomForestClassifier, 100 trees, depth <= 8, 32 fp32 features, 2 classes,
      predict_proba on 1 M rows
  c2  1000 complete depth-8 trees, 256 fp32 features, sigmoid, 10 M rows
  c3  scikit-learn RandomForestRegressor, 200 unpruned trees (depth <= 20) fit on 100 k rows of 64
      fp64 features; fp64 predict and apply on 5 M rows
  c4  10-class boosted forest, 5000 depth-6 trees, 128 fp32 features (8 categorical x 32
      categories), 5 % NaN, softmax, 20 M rows
  c5  2000 complete depth-10 trees, 512 fp32 features; 20 M rows per pass (100 M x 512 fp32 does
      not fit one GPU's memory)
  sweep  the c2 forest at batch sizes 1 ... 10 M: back-to-back GPU time per call
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HBM_GBS_FALLBACK = 6650.0


def _peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return HBM_GBS_FALLBACK, "fallback"


def _time(fn, steps):
    import torch

    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    from cuml_b200.fil import _lib

    _time.variant = _lib.last_variant()  # the kernels of the call that was just timed
    return a.elapsed_time(b) / steps


def _randn_rows(n, f, dtype, seed, chunk=2_000_000):
    import torch

    g = torch.Generator(device="cuda:0")
    g.manual_seed(seed)
    X = torch.empty((n, f), device="cuda:0", dtype=dtype)
    for b in range(0, n, chunk):
        e = min(n, b + chunk)
        X[b:e] = torch.randn((e - b, f), generator=g, device="cuda:0", dtype=dtype)
    return X


def _cpu_and_parity(desc, Xd, gpu_out, kind, precision, sample_rows, seconds=4.0, ids_out=None):
    """CPU baseline leg: run the oracle with all host threads on a bounded sample of the timed
    rows (sized for about `seconds` of CPU work, at most `sample_rows`), report its rows/s, and
    compare the GPU results of the same rows with it."""
    from cuml_b200.fil._desc import INFER_LEAF_ID
    from oracle import oracle

    cores = os.cpu_count() or 1
    n = int(Xd.shape[0])
    probe = Xd[:min(n, 2048)].cpu().numpy()
    oracle.predict(desc, probe[:64], kind, precision, n_threads=cores, packed=True)
    t0 = time.perf_counter()
    oracle.predict(desc, probe, kind, precision, n_threads=cores, packed=True)
    rate = probe.shape[0] / max(1e-9, time.perf_counter() - t0)
    m = int(max(256, min(n, sample_rows, rate * seconds)))
    # evenly spread rows, first and last included
    idx = np.unique(np.linspace(0, n - 1, m).astype(np.int64))
    import torch

    sel = torch.as_tensor(idx, device=Xd.device)
    Xs = Xd[sel].cpu().numpy()
    # timed: the packed walk (one record per node, eight rows side by side); checked against
    # the plain walk, which is the one the tests pin, on the head of the sample
    t0 = time.perf_counter()
    want = oracle.predict(desc, Xs, kind, precision, n_threads=cores, packed=True)
    dt = time.perf_counter() - t0
    head = min(idx.size, 2000)
    walks_agree = bool(np.array_equal(
        want[:head], oracle.predict(desc, Xs[:head], kind, precision, n_threads=cores)))
    got = gpu_out[sel].cpu().numpy()
    tol = dict(rtol=1e-5, atol=1e-6) if precision == "single" else dict(rtol=1e-12, atol=1e-12)
    if precision == "double":
        tol["atol"] *= max(1.0, float(np.abs(want).max()))
    ok = bool(np.allclose(got, want, **tol))
    rec = {"cpu": {"value": idx.size / dt, "unit": "rows/s", "cores": cores, "kind": "port",
                   "sample": f"{idx.size} of {n} rows, same forest, {cores} OpenMP threads, "
                             "packed node records", "agrees_with_plain_walk": walks_agree},
           "parity": {"rows_checked": int(idx.size), "scores_within_tolerance": ok,
                      "max_abs_diff": float(np.abs(got.astype(np.float64) - want).max())}}
    if ids_out is not None:
        k = min(idx.size, 2000)
        want_ids = oracle.predict(desc, Xs[:k], INFER_LEAF_ID, precision, n_threads=cores)
        rec["parity"]["leaf_ids_exact"] = bool(
            np.array_equal(ids_out[sel[:k]].cpu().numpy().astype(np.uint32), want_ids))
        rec["parity"]["leaf_id_rows_checked"] = int(k)
    return rec


def _print_line(line):
    print(json.dumps(line), flush=True)


def run(config: str, steps: int, scale: float, cpu: bool = True, emit=_print_line,
        c3_options=None):
    c3_options = c3_options or {}
    import torch

    from cuml_b200.fil import ForestInference, _lib, synthetic_complete_forest
    from cuml_b200.fil._desc import INFER_DEFAULT, INFER_PROBA2

    peak, peak_kind = _peak()
    lines = []

    def report(name, what, n, ms, bytes_per_row, fi, extra=None):
        rows_s = n / (ms * 1e-3)
        d = fi.describe()
        line = {"config": name, "call": what, "rows": n, "ms": ms, "rows_per_s": rows_s,
                "algorithmic_bytes_per_row": bytes_per_row,
                "row_stream_GBps": rows_s * bytes_per_row / 1e9,
                "hbm_frac": rows_s * bytes_per_row / 1e9 / peak, "hbm_peak": peak_kind,
                "kernel": getattr(_time, "variant", ""),
                "forest": {k: d[k] for k in
                           ("storage", "node_bytes", "max_depth", "n_trees", "row_quantization",
                            "device_bytes")}}
        if extra:
            line.update(extra)
        if emit:
            emit(line)
        lines.append(line)

    if config == "c1":
        from sklearn.datasets import make_classification
        from sklearn.ensemble import RandomForestClassifier

        X, y = make_classification(n_samples=10_000, n_features=32, n_informative=16, n_classes=2,
                                   random_state=0)
        m = RandomForestClassifier(n_estimators=100, max_depth=8, random_state=0,
                                   n_jobs=-1).fit(X.astype(np.float32), y)
        n = int(1_000_000 * scale)
        Xt = make_classification(n_samples=n, n_features=32, n_informative=16, n_classes=2,
                                 random_state=1)[0].astype(np.float32)
        fi = ForestInference.load_from_sklearn(m)
        Xd = torch.as_tensor(Xt, device="cuda:0")
        out = torch.empty((n, 2), device="cuda:0", dtype=torch.float32)
        ms = _time(lambda: fi.predict_proba(Xd, preds=out), steps)
        extra = {}
        if cpu:
            extra = _cpu_and_parity(fi._desc, Xd, out, INFER_DEFAULT, "single", 500_000,
                                    ids_out=fi.apply(Xd))
            k = min(n, 200_000)
            t0 = time.perf_counter()
            sk = m.predict_proba(Xt[:k])
            extra["cpu_sklearn"] = {"value": k / (time.perf_counter() - t0), "unit": "rows/s",
                                    "cores": os.cpu_count(), "kind": "scikit-learn n_jobs=-1",
                                    "sample": f"{k} of {n} rows"}
            extra["parity"]["matches_sklearn"] = bool(
                np.allclose(out[:k].cpu().numpy(), sk, rtol=1e-5, atol=1e-6))
        report("c1", "predict_proba", n, ms, 32 * 4 + 2 * 4, fi, extra)
    elif config == "c2":
        n = int(10_000_000 * scale)
        desc = synthetic_complete_forest(1000, 8, 256, 2)
        fi = ForestInference.load_from_treelite_model(desc)
        Xd = _randn_rows(n, 256, torch.float32, 3)
        out = torch.empty((n, 2), device="cuda:0", dtype=torch.float32)
        ms = _time(lambda: fi.predict_proba(Xd, preds=out), steps)
        extra = _cpu_and_parity(desc, Xd, out, INFER_PROBA2, "single", 200_000) if cpu else None
        report("c2", "predict_proba", n, ms, 256 * 4 + 2 * 4, fi, extra)
    elif config == "c3":
        from sklearn.datasets import make_regression
        from sklearn.ensemble import RandomForestRegressor

        X, y = make_regression(n_samples=100_000, n_features=64, noise=0.1, random_state=0)
        m = RandomForestRegressor(n_estimators=200, max_depth=20, min_samples_leaf=1,
                                  random_state=0, n_jobs=-1).fit(X, y)
        n = int(5_000_000 * scale)
        fi = ForestInference.load_from_sklearn(m, precision="double", **c3_options)
        Xd = _randn_rows(n, 64, torch.float64, 1)
        out = torch.empty((n, 1), device="cuda:0", dtype=torch.float64)
        ms = _time(lambda: fi.predict(Xd, preds=out), steps)
        variant_predict = _time.variant
        ids = torch.empty((n, 200), device="cuda:0", dtype=torch.int32)
        ms_apply = _time(lambda: fi.apply(Xd, preds=ids), steps)
        variant_apply = _time.variant
        extra = {"kernel": variant_predict}
        if cpu:
            extra.update(_cpu_and_parity(fi._desc, Xd, out, INFER_DEFAULT, "double", 200_000,
                                         ids_out=ids))
            k = min(n, 100_000)
            X32 = Xd[:k].float().cpu().numpy()  # scikit-learn predicts on fp32 inputs
            t0 = time.perf_counter()
            m.predict(X32)
            extra["cpu_sklearn"] = {"value": k / (time.perf_counter() - t0), "unit": "rows/s",
                                    "cores": os.cpu_count(), "kind": "scikit-learn n_jobs=-1",
                                    "sample": f"{k} of {n} rows"}
        report("c3", "predict", n, ms, 64 * 8 + 8, fi, extra)
        report("c3", "apply", n, ms_apply, 64 * 8 + 200 * 4, fi, {"kernel": variant_apply})
    elif config == "c4":
        n = int(20_000_000 * scale)
        desc = synthetic_complete_forest(5000, 6, 128, seed=4, n_classes=10, n_categorical=8,
                                         n_categories=32)
        fi = ForestInference.load_from_treelite_model(desc)
        Xd = _randn_rows(n, 128, torch.float32, 5)
        g = torch.Generator(device="cuda:0")
        g.manual_seed(6)
        for b in range(0, n, 2_000_000):
            e = min(n, b + 2_000_000)
            Xd[b:e, :8] = torch.randint(0, 32, (e - b, 8), generator=g, device="cuda:0").float()
            Xd[b:e][torch.rand((e - b, 128), generator=g, device="cuda:0") < 0.05] = float("nan")
        out = torch.empty((n, 10), device="cuda:0", dtype=torch.float32)
        ms = _time(lambda: fi.predict_proba(Xd, preds=out), steps)
        extra = _cpu_and_parity(desc, Xd, out, INFER_DEFAULT, "single", 100_000) if cpu else None
        report("c4", "predict_proba", n, ms, 128 * 4 + 10 * 4, fi, extra)
    elif config == "c5":
        n = int(20_000_000 * scale)
        desc = synthetic_complete_forest(2000, 10, 512, 6)
        fi = ForestInference.load_from_treelite_model(desc)
        Xd = _randn_rows(n, 512, torch.float32, 7)
        out = torch.empty((n, 2), device="cuda:0", dtype=torch.float32)
        ms = _time(lambda: fi.predict_proba(Xd, preds=out), steps)
        extra = _cpu_and_parity(desc, Xd, out, INFER_PROBA2, "single", 100_000) if cpu else None
        report("c5", "predict_proba", n, ms, 512 * 4 + 2 * 4, fi, extra)
    elif config == "sweep":
        fi = ForestInference.load_from_treelite_model(synthetic_complete_forest(1000, 8, 256, 2))
        big = int(10_000_000 * scale)
        Xd = _randn_rows(big, 256, torch.float32, 3)
        out = torch.empty((big, 2), device="cuda:0", dtype=torch.float32)
        for n in (1, 8, 64, 512, 1024, 4096, 32768, 65536, 262144, 1_000_000, big):
            n = min(n, big)
            # rotate through the resident rows so that small batches do not re-read L2-hot rows
            starts = [(i * n) % max(1, big - n + 1) for i in range(64)]
            state = {"i": 0}

            def call():
                b = starts[state["i"] % len(starts)]
                state["i"] += 1
                fi.predict_proba(Xd[b:b + n], preds=out[:n])

            ms = _time(call, max(steps, 200 if n <= 65536 else steps))
            report("sweep", f"predict_proba batch {n}", n, ms, 256 * 4 + 2 * 4, fi)
    else:
        raise ValueError(f"unknown config {config}")
    return lines


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", nargs="+", default=["c1", "c2", "c3", "c4", "c5"])
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--rows-scale", type=float, default=1.0,
                    help="multiply every configuration's row count (smaller runs)")
    ap.add_argument("--no-cpu", action="store_true",
                    help="skip the CPU baseline / parity leg (profiling runs)")
    ap.add_argument("--plain-sparse", action="store_true",
                    help="c3: build the forest without the compact image (plain sparse kernel)")
    args = ap.parse_args()
    for c in args.config:
        run(c, args.steps, args.rows_scale, cpu=not args.no_cpu,
            c3_options={"compact_nodes": False} if args.plain_sparse else None)
        import torch

        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
