"""The allocation-free entry point, `b2fil_predict_fixed_scratch`, against the ordinary
`b2fil_predict` and against the CPU oracle, through the C ABI.

Who needs it: a caller that may not allocate device memory while it predicts - for instance a
process that handed all GPU memory to its own allocator at start-up, or a latency-bound serving
loop that cannot take the allocator's lock in the middle of a request.  The ordinary call keeps the
16-bit rank image of the batch in pool memory; this one keeps it in a fixed 32 MiB array inside
the library, shared by all calls on a GPU, which still holds the previous call's contents.

The first test runs two calls back to back on one stream.  The first batch contains NaNs (its
tiles raise their "has NaN" flags in the shared array), the second has none and a different size:
if the second call did not clear what it must, or read stale ranks, its leaf ids would differ.
The second test checks the property the entry point exists for: once a warm-up call has made the
CUDA runtime load the kernels, a call changes neither the free memory of the device nor the
forest's scratch pool.  The third walks up to the documented size limit.  The file name sorts
last so that a run that stops at the first failure has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

from cuml_b200.fil import ForestInference
from cuml_b200.fil._desc import INFER_DEFAULT, INFER_LEAF_ID, INFER_PROBA2
from oracle import oracle
from tests.helpers import random_forest_desc, random_rows

pytestmark = pytest.mark.gpu

FIXED_SCRATCH_BYTES = 33554432  # B2FIL_FIXED_SCRATCH_BYTES of include/b2fil.h


def _both(lib, fi, kind, X, shape, dtype):
    """Run the ordinary and the fixed-scratch entry point on the same device rows."""
    import torch

    out_a = torch.zeros(shape, dtype=dtype, device="cuda:0")
    out_b = torch.zeros(shape, dtype=dtype, device="cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    n = X.shape[0]
    rc = lib.b2fil_predict(fi.forest.handle, kind, X.data_ptr(), n, X.stride(0), out_a.data_ptr(),
                           0, 0.5, stream)
    assert rc == 0, lib.b2fil_last_error()
    rc = lib.b2fil_predict_fixed_scratch(fi.forest.handle, kind, X.data_ptr(), n, X.stride(0),
                                         out_b.data_ptr(), 0, 0.5, stream)
    assert rc == 0, lib.b2fil_last_error()
    torch.cuda.synchronize()
    return out_a.cpu().numpy(), out_b.cpu().numpy()


def test_fixed_scratch_matches_ordinary_path_and_oracle_on_two_calls_in_a_row(lib):
    import torch

    desc = random_forest_desc(71, n_trees=60, n_features=12, max_depth=7, postproc="sigmoid")
    fi = ForestInference.load_from_treelite_model(desc, storage="dense")
    assert fi.describe()["row_quantization"] == 1  # this forest predicts on rank scratch
    first_h = random_rows(1, 5000, 12, np.float32, nan_frac=0.2)
    second_h = random_rows(2, 3111, 12, np.float32, nan_frac=0.0)
    for Xh in (first_h, second_h):  # two calls in a row share the array
        X = torch.as_tensor(Xh, device="cuda:0")
        n = X.shape[0]
        ids_a, ids_b = _both(lib, fi, INFER_LEAF_ID, X, (n, 60), torch.int32)
        assert np.array_equal(ids_a, ids_b)
        assert np.array_equal(ids_b.astype(np.uint32),
                              oracle.predict(desc, Xh, INFER_LEAF_ID, "single"))
        p_a, p_b = _both(lib, fi, INFER_PROBA2, X, (n, 2), torch.float32)
        np.testing.assert_allclose(p_b, p_a, rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(p_b, oracle.predict(desc, Xh, INFER_PROBA2, "single"),
                                   rtol=1e-5, atol=1e-6)
        s_a, s_b = _both(lib, fi, INFER_DEFAULT, X, (n, 1), torch.float32)
        np.testing.assert_allclose(s_b, s_a, rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(s_b, oracle.predict(desc, Xh, INFER_DEFAULT, "single"),
                                   rtol=1e-5, atol=1e-6)


def test_fixed_scratch_call_allocates_nothing_once_warmed_up(lib):
    """After one warm-up call per (forest shape, kind) a call leaves the device's free memory and
    the forest's scratch pool exactly as it found them; the ordinary entry point, by contrast,
    grows the pool."""
    import torch

    desc = random_forest_desc(74, n_trees=40, n_features=16, max_depth=6, postproc="sigmoid")
    fi = ForestInference.load_from_treelite_model(desc, storage="dense")
    n = 40_000
    Xh = random_rows(4, n, 16, np.float32, nan_frac=0.01)
    X = torch.as_tensor(Xh, device="cuda:0")
    outs = {INFER_PROBA2: torch.zeros((n, 2), dtype=torch.float32, device="cuda:0"),
            INFER_LEAF_ID: torch.zeros((n, 40), dtype=torch.int32, device="cuda:0")}
    stream = torch.cuda.current_stream().cuda_stream

    def call(kind):
        rc = lib.b2fil_predict_fixed_scratch(fi.forest.handle, kind, X.data_ptr(), n, 16,
                                             outs[kind].data_ptr(), 0, 0.5, stream)
        assert rc == 0, lib.b2fil_last_error()

    for kind in outs:  # warm-up: kernels get loaded, shared-memory limits raised
        call(kind)
    torch.cuda.synchronize()
    assert fi.describe()["scratch_pool_bytes"] == 0  # this forest has only used the fixed array
    free_before, _ = torch.cuda.mem_get_info(0)
    for _ in range(3):
        for kind in outs:
            call(kind)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(0)
    assert free_after == free_before
    assert fi.describe()["scratch_pool_bytes"] == 0
    np.testing.assert_allclose(outs[INFER_PROBA2].cpu().numpy(),
                               oracle.predict(desc, Xh, INFER_PROBA2, "single"),
                               rtol=1e-5, atol=1e-6)
    # the ordinary entry point takes its rank scratch from the forest's pool
    rc = lib.b2fil_predict(fi.forest.handle, INFER_PROBA2, X.data_ptr(), n, 16,
                           outs[INFER_PROBA2].data_ptr(), 0, 0.5, stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert fi.describe()["scratch_pool_bytes"] >= n * 16 * 2


def test_fixed_scratch_size_limit_is_exact(lib):
    """The largest batch that fits uses the array to its end (the NaN flags sit behind the rank
    image); one more row tile is refused with B2FIL_ERR_TOO_LARGE and the numbers in the message."""
    import torch

    desc = random_forest_desc(72, n_trees=5, n_features=64, max_depth=4)
    fi = ForestInference.load_from_treelite_model(desc, storage="dense")
    # chunk_size 8 asks for 256-row tiles: a tile of ranks is 64 features x 256 rows x 2 bytes =
    # 32 KiB plus 4 bytes of flags, so 1023 tiles fit 32 MiB and 1024 do not
    tile_rows, tile_bytes = 256, 64 * 256 * 2
    n_tiles = max(t for t in range(1, 2048)
                  if t * tile_bytes + (t * 4 + 255) // 256 * 256 <= FIXED_SCRATCH_BYTES)
    assert n_tiles == 1023
    n_fit = n_tiles * tile_rows
    Xh = random_rows(5, n_fit + 1, 64, np.float32, nan_frac=0.0)
    Xh[-300:-1][:, 3] = np.nan  # NaN in the last tile that fits: its flag is the array's last word
    X = torch.as_tensor(Xh, device="cuda:0")
    out = torch.zeros((n_fit + 1, 5), dtype=torch.int32, device="cuda:0")
    rc = lib.b2fil_predict_fixed_scratch(fi.forest.handle, INFER_LEAF_ID, X.data_ptr(), n_fit, 64,
                                         out.data_ptr(), 8, 0.5, None)
    assert rc == 0, lib.b2fil_last_error()
    torch.cuda.synchronize()
    tail = slice(n_fit - 2000, n_fit)
    assert np.array_equal(out[tail].cpu().numpy().astype(np.uint32),
                          oracle.predict(desc, Xh[tail], INFER_LEAF_ID, "single"))
    head = slice(0, 2000)
    assert np.array_equal(out[head].cpu().numpy().astype(np.uint32),
                          oracle.predict(desc, Xh[head], INFER_LEAF_ID, "single"))
    rc = lib.b2fil_predict_fixed_scratch(fi.forest.handle, INFER_LEAF_ID, X.data_ptr(), n_fit + 1,
                                         64, out.data_ptr(), 8, 0.5, None)
    assert rc == -6  # B2FIL_ERR_TOO_LARGE
    msg = lib.b2fil_last_error().decode()
    assert "fixed scratch" in msg and "rows" in msg and str(FIXED_SCRATCH_BYTES) in msg
    # the ordinary entry point takes the same batch
    rc = lib.b2fil_predict(fi.forest.handle, INFER_LEAF_ID, X.data_ptr(), n_fit + 1, 64,
                           out.data_ptr(), 8, 0.5, None)
    assert rc == 0
    torch.cuda.synchronize()


def test_fixed_scratch_forwards_forests_that_need_no_scratch(lib):
    import torch

    desc = random_forest_desc(73, n_trees=9, n_features=6, max_depth=5, categorical=True)
    fi = ForestInference.load_from_treelite_model(desc, storage="sparse")
    Xh = random_rows(3, 700, 6, np.float32, categories=22)
    X = torch.as_tensor(Xh, device="cuda:0")
    a, b = _both(lib, fi, INFER_LEAF_ID, X, (700, 9), torch.int32)
    assert np.array_equal(a, b)
    assert np.array_equal(b.astype(np.uint32), oracle.predict(desc, Xh, INFER_LEAF_ID, "single"))
