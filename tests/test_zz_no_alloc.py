"""The allocation-free entry point, `b2fil_predict_fixed_scratch`, against the ordinary
`b2fil_predict` through the C ABI.

Who needs it: a caller that may not allocate device memory while it predicts - for instance a
process that handed all GPU memory to its own allocator at start-up, or a latency-bound serving
loop that cannot take the allocator's lock in the middle of a request.  The ordinary call keeps the
16-bit rank image of the batch in pool memory; this one keeps it in a fixed 32 MiB array inside
the library, shared by all calls on a GPU, which still holds the previous call's contents.

The test runs two calls back to back on one stream.  The first batch contains NaNs (its tiles raise
their "has NaN" flags in the shared array), the second has none and a different size: if the second
call did not clear what it must, or read stale ranks, its leaf ids would differ.  The file name
sorts last so that a run that stops at the first failure has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

from cuml_b200.fil import ForestInference
from cuml_b200.fil._desc import INFER_DEFAULT, INFER_LEAF_ID, INFER_PROBA2
from tests.helpers import random_forest_desc, random_rows

pytestmark = pytest.mark.gpu


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


def test_fixed_scratch_matches_ordinary_path_on_two_calls_in_a_row(lib):
    import torch

    desc = random_forest_desc(71, n_trees=60, n_features=12, max_depth=7, postproc="sigmoid")
    fi = ForestInference.load_from_treelite_model(desc, storage="dense")
    assert fi.describe()["row_quantization"] == 1  # this forest predicts on rank scratch
    first = torch.as_tensor(random_rows(1, 5000, 12, np.float32, nan_frac=0.2), device="cuda:0")
    second = torch.as_tensor(random_rows(2, 3111, 12, np.float32, nan_frac=0.0), device="cuda:0")
    for X in (first, second):  # two calls in a row share the array
        n = X.shape[0]
        ids_a, ids_b = _both(lib, fi, INFER_LEAF_ID, X, (n, 60), torch.int32)
        assert np.array_equal(ids_a, ids_b)
        p_a, p_b = _both(lib, fi, INFER_PROBA2, X, (n, 2), torch.float32)
        np.testing.assert_allclose(p_b, p_a, rtol=1e-5, atol=1e-6)
        s_a, s_b = _both(lib, fi, INFER_DEFAULT, X, (n, 1), torch.float32)
        np.testing.assert_allclose(s_b, s_a, rtol=1e-5, atol=1e-6)


def test_fixed_scratch_rejects_batches_beyond_the_array(lib):
    import torch

    desc = random_forest_desc(72, n_trees=5, n_features=64, max_depth=4)
    fi = ForestInference.load_from_treelite_model(desc, storage="dense")
    n = 400_000  # 400k rows x 64 features x 2 bytes = 51 MB of ranks > 32 MiB
    X = torch.zeros((n, 64), dtype=torch.float32, device="cuda:0")
    out = torch.zeros((n, 1), dtype=torch.float32, device="cuda:0")
    rc = lib.b2fil_predict_fixed_scratch(fi.forest.handle, INFER_DEFAULT, X.data_ptr(), n, 64,
                                         out.data_ptr(), 0, 0.5, None)
    assert rc == -6  # B2FIL_ERR_TOO_LARGE
    msg = lib.b2fil_last_error().decode()
    assert "fixed scratch" in msg and "rows" in msg
    # the ordinary entry point takes the same batch
    rc = lib.b2fil_predict(fi.forest.handle, INFER_DEFAULT, X.data_ptr(), n, 64, out.data_ptr(),
                           0, 0.5, None)
    assert rc == 0
    torch.cuda.synchronize()


def test_fixed_scratch_forwards_forests_that_need_no_scratch(lib):
    import torch

    desc = random_forest_desc(73, n_trees=9, n_features=6, max_depth=5, categorical=True)
    fi = ForestInference.load_from_treelite_model(desc, storage="sparse")
    X = torch.as_tensor(random_rows(3, 700, 6, np.float32, categories=22), device="cuda:0")
    a, b = _both(lib, fi, INFER_LEAF_ID, X, (700, 9), torch.int32)
    assert np.array_equal(a, b)
