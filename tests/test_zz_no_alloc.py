"""The no-allocation decode entry point against the regular one.

production_mul_mat_q4_k_decode_noalloc exists for hosts that may not allocate device memory once they
are running (their own pool owns the device, or allocations are frozen after start-up): it stages
host-side activations and outputs through a fixed 1 MiB array inside the library instead of an arena
grown on demand.  It must give exactly what production_mul_mat_q4_k_decode gives, on consecutive calls
that reuse the same scratch, and must refuse what does not fit.  Collected last on purpose.
"""
from __future__ import annotations

import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_noalloc_matches_regular_entry_point_twice(oracle):
    import torch

    if not torch.cuda.is_available():
        pytest.fail("this test needs a CUDA device")
    from weft_b200.build import ensure_built

    lib = ctypes.CDLL(str(ensure_built()))
    lib.weft_b200_noalloc_last_error.restype = ctypes.c_char_p
    lib.weft_b200_last_error.restype = ctypes.c_char_p
    sig = [ctypes.c_void_p] * 4 + [ctypes.c_size_t] * 3
    noalloc, regular = lib.production_mul_mat_q4_k_decode_noalloc, lib.production_mul_mat_q4_k_decode
    noalloc.argtypes = regular.argtypes = sig

    n, k = 3000, 4096
    rng = np.random.default_rng(42)
    w = oracle.quantize(oracle.Q4_K, (rng.standard_normal((n, k)) * 0.02).astype(np.float32))
    w_dev = torch.from_numpy(w).cuda()                      # weights resident on the device, as the entry point requires
    xq_bytes = oracle.row_bytes(oracle.Q8_K, k)
    for call in range(2):                                    # the second call reuses the scratch the first one left behind
        m = 2 - call
        x = (rng.standard_normal((m, k)) * (1 + call)).astype(np.float32)
        y_a, y_b = np.full((m, n), np.nan, dtype=np.float32), np.full((m, n), np.nan, dtype=np.float32)
        xq_a, xq_b = np.zeros((m, xq_bytes), dtype=np.uint8), np.ones((m, xq_bytes), dtype=np.uint8)
        assert noalloc(w_dev.data_ptr(), x.ctypes.data, xq_a.ctypes.data, y_a.ctypes.data, n, k, m) == 0, lib.weft_b200_noalloc_last_error()
        assert regular(w_dev.data_ptr(), x.ctypes.data, xq_b.ctypes.data, y_b.ctypes.data, n, k, m) == 0, lib.weft_b200_last_error()
        assert np.array_equal(xq_a, xq_b)
        err = np.linalg.norm(y_a.astype(np.float64) - y_b) / np.linalg.norm(y_b.astype(np.float64))
        assert err <= 1e-5 and np.array_equal(y_a, y_b)
        want, _ = oracle.mul_mat(oracle.Q4_K, w, x, n, k, m, rule=1)
        assert np.linalg.norm(y_a.astype(np.float64) - want) / np.linalg.norm(want.astype(np.float64)) <= 1e-5

    # a call whose staging does not fit the fixed array is refused, with a message, and nothing is written
    big_m = 80                                               # 80 x 4096 fp32 activations alone exceed 1 MiB
    x = np.zeros((big_m, k), dtype=np.float32)
    y = np.full((big_m, n), 7.0, dtype=np.float32)
    xq = np.zeros((big_m, xq_bytes), dtype=np.uint8)
    assert noalloc(w_dev.data_ptr(), x.ctypes.data, xq.ctypes.data, y.ctypes.data, n, k, big_m) != 0
    assert b"fixed scratch" in lib.weft_b200_noalloc_last_error() and (y == 7.0).all()
    # host weights are refused too
    y1 = np.zeros((1, n), dtype=np.float32)
    assert noalloc(w.ctypes.data, x.ctypes.data, xq.ctypes.data, y1.ctypes.data, n, k, 1) != 0
    assert b"device memory" in lib.weft_b200_noalloc_last_error()
