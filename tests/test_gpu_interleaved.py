"""GPU parity of the persistent interleaved layout Q4K_I[16]: the ``_W_pack`` artifact function (bit-exact
against the oracle's statement of the documented rule), ``q4_k_q8_k_gemv`` and
``production_mul_mat_q4_k_persistent`` (<= 1e-5 relative L2 against the oracle's Q4_K x Q8_K mul_mat on the
same records: the float op tree per 256-block is the plain vec_dot's)."""
from __future__ import annotations

import numpy as np
import pytest

from helpers import activations, reference_tolerance_ok, rel_l2, weights

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device; there is no CPU fallback to test")
    return torch


@pytest.mark.parametrize("rows_k", [(16, 256), (48, 768), (160, 4096), (1024, 2048)])
@pytest.mark.parametrize("host", [False, True])
def test_pack_bit_exact(torch, oracle, rows_k, host):
    from weft_b200 import artifacts
    from weft_b200.kernels import gemv

    rows, k = rows_k
    rng = np.random.default_rng(rows + k)
    w = rng.integers(0, 256, size=(rows, k // 256 * 144), dtype=np.uint8)
    assert artifacts.packed_size(gemv.q4_k_q8_k_gemv, rows, k) == w.size
    assert artifacts.packed_size(gemv.q4_k_q8_k_gemv, rows + 1, k) == 0      # not whole cohorts
    if host:
        out = np.zeros(w.size, dtype=np.uint8)
        artifacts.pack(gemv.q4_k_q8_k_gemv, w, out, rows, k)
        got = out
    else:
        out = torch.zeros(w.size, dtype=torch.uint8, device="cuda")
        artifacts.pack(gemv.q4_k_q8_k_gemv, torch.from_numpy(w).cuda(), out, rows, k)
        got = out.cpu().numpy()
    assert np.array_equal(got, oracle.interleave(oracle.Q4_K, w, k).reshape(-1))


def test_pack_refuses_a_tail_cohort(torch):
    from weft_b200 import artifacts
    from weft_b200.kernels import gemv

    w = torch.zeros(40 * 144, dtype=torch.uint8, device="cuda")
    with pytest.raises((ValueError, RuntimeError)):
        artifacts.pack(gemv.q4_k_q8_k_gemv, w, torch.zeros_like(w), 40, 256)


@pytest.mark.parametrize("mk", [(16, 256), (48, 768), (160, 4096), (4096, 4096), (2368, 4096), (64, 14336), (336, 8192 + 256)])
def test_gemv_interleaved(torch, oracle, mk):
    import weft_b200 as weft
    from weft_b200 import artifacts
    from weft_b200.kernels import gemv
    from weft_b200.runtime import Buffer

    m, k = mk
    rng = np.random.default_rng(m * 7 + k)
    w = weights(oracle.Q4_K, rng, m, k)
    x = activations(rng, 1, k)
    xq = oracle.quantize(oracle.Q8_K, x, rule=1)
    packed = torch.zeros(w.size, dtype=torch.uint8, device="cuda")
    artifacts.pack(gemv.q4_k_q8_k_gemv, torch.from_numpy(w).cuda(), packed, m, k)
    y = torch.full((m,), float("nan"), device="cuda")
    weft.compile(gemv.q4_k_q8_k_gemv)(Buffer(packed, shape=(m, k), encoding="Q4K_I[16]"),
                                       Buffer(torch.from_numpy(xq.reshape(-1)).cuda(), shape=(k,), encoding="Q8_K"), y)
    got = y.cpu().numpy()
    want, _ = oracle.mul_mat(oracle.Q4_K, w, None, m, k, 1, xq=xq)
    assert np.isfinite(got).all()
    assert rel_l2(got, want.reshape(-1)) <= 1e-5
    assert reference_tolerance_ok(got, want.reshape(-1))


@pytest.mark.parametrize("mnk", [(1, 64, 1024), (3, 208, 2048), (5, 1024, 4096)])
def test_mul_mat_persistent(torch, oracle, mnk):
    import weft_b200 as weft
    from weft_b200 import artifacts
    from weft_b200.kernels import mul_mat
    from weft_b200.runtime import Buffer

    m, n, k = mnk
    rng = np.random.default_rng(sum(mnk))
    w = weights(oracle.Q4_K, rng, n, k)
    x = activations(rng, m, k)
    packed = torch.zeros(w.size, dtype=torch.uint8, device="cuda")
    artifacts.pack(mul_mat.production_mul_mat_q4_k_persistent, torch.from_numpy(w).cuda(), packed, n, k)
    xq = torch.zeros((m, oracle.row_bytes(oracle.Q8_K, k)), dtype=torch.uint8, device="cuda")
    y = torch.full((m, n), float("nan"), device="cuda")
    weft.compile(mul_mat.production_mul_mat_q4_k_persistent)(
        Buffer(packed, shape=(n, k), encoding="Q4K_I[16]"), torch.from_numpy(x).cuda(), Buffer(xq, shape=(m, k), encoding="Q8_K"), y)
    want_xq = oracle.quantize(oracle.Q8_K, x, rule=1)
    assert np.array_equal(xq.cpu().numpy(), want_xq)
    want, _ = oracle.mul_mat(oracle.Q4_K, w, None, n, k, m, xq=want_xq)
    got = y.cpu().numpy()
    assert rel_l2(got, want) <= 1e-5
    assert reference_tolerance_ok(got, want)


def test_interleaved_matches_plain_gemv(torch, oracle):
    """The same weights through the plain Q4_K decode kernel and through the interleaved one."""
    import weft_b200 as weft
    from weft_b200 import artifacts
    from weft_b200.kernels import gemv, rows
    from weft_b200.runtime import Buffer

    m, k = 512, 4096
    rng = np.random.default_rng(11)
    w = torch.from_numpy(weights(oracle.Q4_K, rng, m, k)).cuda()
    xq = torch.from_numpy(oracle.quantize(oracle.Q8_K, activations(rng, 1, k), rule=1).reshape(-1)).cuda()
    packed = torch.zeros_like(w.reshape(-1))
    artifacts.pack(gemv.q4_k_q8_k_gemv, w, packed, m, k)
    a = torch.zeros(m, device="cuda")
    b = torch.zeros(m, device="cuda")
    weft.compile(gemv.q4_k_q8_k_gemv)(Buffer(packed, shape=(m, k), encoding="Q4K_I[16]"), Buffer(xq, shape=(k,), encoding="Q8_K"), a)
    weft.compile(rows.quantized_vec_dot_q4_k_q8_k_rows)(Buffer(w, shape=(m, k), encoding="Q4_K"), Buffer(xq, shape=(k,), encoding="Q8_K"), b)
    assert rel_l2(a.cpu().numpy(), b.cpu().numpy()) <= 1e-5
