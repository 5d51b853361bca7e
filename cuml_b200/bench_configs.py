"""Throughput of the five benchmark configurations on one GPU.

    python -m cuml_b200.bench_configs [--config c1 c2 c3 c4 c5] [--steps K] [--rows-scale S]

Prints one JSON line per configuration: rows/s with device-resident rows (CUDA events on the
launching stream), the algorithmic bytes per row (features read once + outputs written once) and
the fraction of the measured HBM copy bandwidth that the row stream reaches.  `bench.py` at the
repository root measures the headline configuration (c2) under the full reporting contract; this
module is the quick way to see the other shapes.

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
import time

import numpy as np

HBM_GBS_FALLBACK = 6650.0


def _peak():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                        "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
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


def run(config: str, steps: int, scale: float):
    import torch

    from .fil import ForestInference, synthetic_complete_forest

    peak, peak_kind = _peak()
    lines = []

    def report(name, what, n, ms, bytes_per_row, fi, extra=None):
        rows_s = n / (ms * 1e-3)
        line = {"config": name, "call": what, "rows": n, "ms": ms, "rows_per_s": rows_s,
                "algorithmic_bytes_per_row": bytes_per_row,
                "row_stream_GBps": rows_s * bytes_per_row / 1e9,
                "hbm_frac": rows_s * bytes_per_row / 1e9 / peak, "hbm_peak": peak_kind,
                "forest": {k: fi.describe()[k] for k in
                           ("storage", "node_bytes", "max_depth", "n_trees", "row_quantization",
                            "device_bytes")}}
        if extra:
            line.update(extra)
        print(json.dumps(line), flush=True)
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
        t0 = time.perf_counter()
        m.predict_proba(Xt[:200_000])
        sk = 200_000 / (time.perf_counter() - t0)
        report("c1", "predict_proba", n, ms, 32 * 4 + 2 * 4, fi,
               {"sklearn_rows_per_s": sk, "cores": os.cpu_count()})
    elif config == "c2":
        n = int(10_000_000 * scale)
        fi = ForestInference.load_from_treelite_model(synthetic_complete_forest(1000, 8, 256, 2))
        Xd = _randn_rows(n, 256, torch.float32, 3)
        out = torch.empty((n, 2), device="cuda:0", dtype=torch.float32)
        ms = _time(lambda: fi.predict_proba(Xd, preds=out), steps)
        report("c2", "predict_proba", n, ms, 256 * 4 + 2 * 4, fi)
    elif config == "c3":
        from sklearn.datasets import make_regression
        from sklearn.ensemble import RandomForestRegressor

        X, y = make_regression(n_samples=100_000, n_features=64, noise=0.1, random_state=0)
        m = RandomForestRegressor(n_estimators=200, max_depth=20, min_samples_leaf=1,
                                  random_state=0, n_jobs=-1).fit(X, y)
        n = int(5_000_000 * scale)
        fi = ForestInference.load_from_sklearn(m, precision="double")
        Xd = _randn_rows(n, 64, torch.float64, 1)
        out = torch.empty((n, 1), device="cuda:0", dtype=torch.float64)
        ms = _time(lambda: fi.predict(Xd, preds=out), steps)
        report("c3", "predict", n, ms, 64 * 8 + 8, fi)
        del out
        ids = torch.empty((n, 200), device="cuda:0", dtype=torch.int32)
        ms = _time(lambda: fi.apply(Xd, preds=ids), steps)
        report("c3", "apply", n, ms, 64 * 8 + 200 * 4, fi)
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
        report("c4", "predict_proba", n, ms, 128 * 4 + 10 * 4, fi)
    elif config == "c5":
        n = int(20_000_000 * scale)
        fi = ForestInference.load_from_treelite_model(synthetic_complete_forest(2000, 10, 512, 6))
        Xd = _randn_rows(n, 512, torch.float32, 7)
        out = torch.empty((n, 2), device="cuda:0", dtype=torch.float32)
        ms = _time(lambda: fi.predict_proba(Xd, preds=out), steps)
        report("c5", "predict_proba", n, ms, 512 * 4 + 2 * 4, fi)
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
    args = ap.parse_args()
    for c in args.config:
        run(c, args.steps, args.rows_scale)
        import torch

        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
