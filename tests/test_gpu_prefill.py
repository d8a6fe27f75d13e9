"""GPU parity of the tensor-core prefill path (production_mul_mat_q4_k_staged, production_mul_mat_tq1_0)
against the CPU oracle.

Bound: 1e-5 relative L2.  The integer part (int8 MMAs, int32 / exact-f16 accumulation) is exact; only
the per-block fp32 combine is rounded, in the reference's own order.
"""
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


def _run(torch, oracle, m, n, k, seed, column_ranges=None):
    import weft_b200 as weft
    from weft_b200.kernels import mul_mat
    from weft_b200.runtime import Buffer

    rng = np.random.default_rng(seed)
    w = weights(oracle.Q4_K, rng, n, k)
    x = activations(rng, m, k)
    xq = torch.zeros((m, oracle.row_bytes(oracle.Q8_K, k)), dtype=torch.uint8, device="cuda")
    y = torch.full((m, n), float("nan"), device="cuda")
    weft.compile(mul_mat.production_mul_mat_q4_k_staged)(
        Buffer(torch.from_numpy(w).cuda(), shape=(n, k), encoding="Q4_K"), torch.from_numpy(x).cuda(),
        Buffer(xq, shape=(m, k), encoding="Q8_K"), y)
    got = y.cpu().numpy()
    want_xq = oracle.quantize(oracle.Q8_K, x, rule=1)
    assert np.array_equal(xq.cpu().numpy(), want_xq)
    assert np.isfinite(got).all()
    for lo, hi in (column_ranges or [(0, n)]):
        want, _ = oracle.mul_mat(oracle.Q4_K, w, None, n, k, m, xq=want_xq, rows=(lo, hi))
        err = rel_l2(got[:, lo:hi], want[:, lo:hi])
        assert err <= 1e-5, (m, n, k, lo, hi, err)
        assert reference_tolerance_ok(got[:, lo:hi], want[:, lo:hi])


def test_prefill_q4_k_one_tile(torch, oracle):
    _run(torch, oracle, 128, 128, 256, seed=1)


@pytest.mark.parametrize("mnk", [(128, 128, 1024), (130, 200, 512), (512, 384, 1024), (32, 128, 4096), (200, 1000, 2048), (512, 4736, 1024),
                                 (300, 77, 768), (257, 1001, 1280), (129, 16, 256)])
def test_prefill_q4_k_shapes(torch, oracle, mnk):
    """Up to 128 tokens the single-CTA kernel (K a multiple of 1024; the GEMV per token row otherwise); above, the CTA-pair kernel
    on activation planes with tiles of 256 tokens x 16..80 weights, for every K that is a multiple of 256; ragged N and M."""
    m, n, k = mnk
    _run(torch, oracle, m, n, k, seed=sum(mnk))


@pytest.mark.parametrize("nk", [(4096, 4096), (14336, 4096), (4096, 14336)])
def test_prefill_q4_k_benchmark_shapes(torch, oracle, nk):
    """Config 4: M = 512 tokens on the three Llama-3-8B-shaped layers; three column bands against the oracle."""
    n, k = nk
    _run(torch, oracle, 512, n, k, seed=n + k, column_ranges=[(0, 128), (n // 2 - 60, n // 2 + 70), (n - 128, n)])


def test_prefill_matches_decode_path(torch, oracle):
    """The tensor-core contraction and the GEMV kernels are two implementations of the same function."""
    import weft_b200 as weft
    from weft_b200.kernels import mul_mat
    from weft_b200.runtime import Buffer

    m, n, k = 64, 512, 2048
    rng = np.random.default_rng(3)
    w = torch.from_numpy(weights(oracle.Q4_K, rng, n, k)).cuda()
    x = torch.from_numpy(activations(rng, m, k)).cuda()
    outs = []
    for definition in (mul_mat.production_mul_mat_q4_k_staged, mul_mat.production_mul_mat_q4_k_decode):
        xq = torch.zeros((m, oracle.row_bytes(oracle.Q8_K, k)), dtype=torch.uint8, device="cuda")
        y = torch.zeros((m, n), device="cuda")
        weft.compile(definition)(Buffer(w, shape=(n, k), encoding="Q4_K"), x, Buffer(xq, shape=(m, k), encoding="Q8_K"), y)
        outs.append(y.cpu().numpy())
    assert rel_l2(outs[0], outs[1]) <= 1e-5


@pytest.mark.parametrize("m", [64, 300])
def test_prefill_q4_k_saturated_records(torch, oracle, m):
    """Every weight nibble 15, every 6-bit scale and min 63, every activation code +-127: the largest sums a block can
    produce (limb sums of 3.4 million, min-term sums of 2 million), through the single-CTA (64 tokens) and the
    CTA-pair (300 tokens) kernels.  The integer part must still be exact."""
    import weft_b200 as weft
    from weft_b200.kernels import mul_mat
    from weft_b200.runtime import Buffer

    n, k = 176, 2048
    record = np.full(144, 0xFF, dtype=np.uint8)
    record[0:2] = np.frombuffer(np.float16(0.5).tobytes(), dtype=np.uint8)
    record[2:4] = np.frombuffer(np.float16(0.25).tobytes(), dtype=np.uint8)
    w = np.tile(record, (n, k // 256))
    # rows of all-positive, all-negative and alternating extremes; the block maximum sits on every element
    x = np.empty((m, k), dtype=np.float32)
    x[0::3] = 3.0
    x[1::3] = -3.0
    x[2::3] = np.where(np.arange(k) % 2 == 0, 3.0, -3.0)
    xq = torch.zeros((m, oracle.row_bytes(oracle.Q8_K, k)), dtype=torch.uint8, device="cuda")
    y = torch.full((m, n), float("nan"), device="cuda")
    weft.compile(mul_mat.production_mul_mat_q4_k_staged)(
        Buffer(torch.from_numpy(w).cuda(), shape=(n, k), encoding="Q4_K"), torch.from_numpy(x).cuda(),
        Buffer(xq, shape=(m, k), encoding="Q8_K"), y)
    want_xq = oracle.quantize(oracle.Q8_K, x, rule=1)
    assert np.array_equal(xq.cpu().numpy(), want_xq)
    codes = want_xq.reshape(m, k // 256, 292)[:, :, 4:260].view(np.int8)
    assert int(np.abs(codes).min()) == 127
    want, _ = oracle.mul_mat(oracle.Q4_K, w, None, n, k, m, xq=want_xq)
    got = y.cpu().numpy()
    assert rel_l2(got, want) <= 1e-6, rel_l2(got, want)
    assert reference_tolerance_ok(got, want)


def _run_tq1_0(torch, oracle, m, n, k, seed, column_ranges=None):
    import weft_b200 as weft
    from weft_b200.kernels import mul_mat
    from weft_b200.runtime import Buffer

    rng = np.random.default_rng(seed)
    w = weights(oracle.TQ1_0, rng, n, k)
    x = activations(rng, m, k)
    xq = torch.zeros((m, oracle.row_bytes(oracle.Q8_K, k)), dtype=torch.uint8, device="cuda")
    y = torch.full((m, n), float("nan"), device="cuda")
    powers = torch.tensor([1, 3, 9, 27, 81], dtype=torch.int32, device="cuda")
    weft.compile(mul_mat.production_mul_mat_tq1_0)(
        Buffer(torch.from_numpy(w).cuda(), shape=(n, k), encoding="TQ1_0"), torch.from_numpy(x).cuda(),
        Buffer(xq, shape=(m, k), encoding="Q8_K"), Buffer(powers, shape=(5,), encoding="dense.u32"), y)
    got = y.cpu().numpy()
    want_xq = oracle.quantize(oracle.Q8_K, x, rule=1)
    assert np.array_equal(xq.cpu().numpy(), want_xq)
    assert np.isfinite(got).all()
    for lo, hi in (column_ranges or [(0, n)]):
        want, _ = oracle.mul_mat(oracle.TQ1_0, w, None, n, k, m, xq=want_xq, rows=(lo, hi))
        err = rel_l2(got[:, lo:hi], want[:, lo:hi])
        assert err <= 1e-5, (m, n, k, lo, hi, err)
        assert reference_tolerance_ok(got[:, lo:hi], want[:, lo:hi])


@pytest.mark.parametrize("mnk", [(128, 128, 1024), (130, 200, 2048), (512, 384, 1024), (32, 130, 4096), (200, 1001, 3072), (512, 4736, 1024),
                                 (300, 77, 4096), (512, 1000, 2048), (256, 160, 2048), (129, 33, 6144), (700, 2000, 4096)])
def test_prefill_tq1_0_shapes(torch, oracle, mnk):
    """K a multiple of 1024 takes the tensor-core kernels (above 128 tokens and with K a multiple of 2048 the CTA-pair
    kernel, whose tiles are 32 to 160 weights wide); odd N exercises 2-byte-aligned weight rows and ragged last tiles."""
    m, n, k = mnk
    _run_tq1_0(torch, oracle, m, n, k, seed=sum(mnk))


def test_prefill_tq1_0_benchmark_shape(torch, oracle):
    """Config 5b: M = 512 tokens, (N, K) = (28672, 8192); three column bands against the oracle."""
    n, k = 28672, 8192
    _run_tq1_0(torch, oracle, 512, n, k, seed=5, column_ranges=[(0, 128), (n // 2 - 60, n // 2 + 70), (n - 128, n)])


def test_prefill_tq1_0_given_records_and_plane_reuse(torch, oracle):
    """The CTA-pair kernel reads planes that a kernel of its own makes of the Q8_K records.  With flags bit 0 the records
    are the caller's (X is not read); a small call after a large one reuses the larger plane allocation.  Every result
    must equal, bit for bit, what the same call computes when it quantizes X itself."""
    import ctypes

    from weft_b200.runtime.driver import Toolchain, last_error, load_library

    lib = load_library(Toolchain().resolve().compiler)
    assert lib.weft_b200_init(0) == 0, last_error(lib)
    fn = lib.weft_b200_mul_mat_shard
    fn.argtypes = [ctypes.c_int, ctypes.c_int] + [ctypes.c_void_p] * 7 + [ctypes.c_size_t] * 4 + [ctypes.c_uint]
    powers = torch.tensor([1, 3, 9, 27, 81], dtype=torch.int32, device="cuda")
    for m, n, k in [(512, 640, 4096), (130, 96, 2048), (300, 333, 2048)]:
        rng = np.random.default_rng(m + n + k)
        w = torch.from_numpy(weights(oracle.TQ1_0, rng, n, k)).cuda()
        x_host = activations(rng, m, k)
        x = torch.from_numpy(x_host).cuda()
        xq = torch.zeros((m, oracle.row_bytes(oracle.Q8_K, k)), dtype=torch.uint8, device="cuda")
        y0 = torch.full((m, n), float("nan"), device="cuda")
        y1 = torch.full((m, n), float("nan"), device="cuda")
        assert fn(oracle.TQ1_0, 1, w.data_ptr(), x.data_ptr(), xq.data_ptr(), None, None, powers.data_ptr(), y0.data_ptr(), n, k, m, n, 0) == 0, last_error(lib)
        given = torch.from_numpy(oracle.quantize(oracle.Q8_K, x_host, rule=1)).cuda()
        assert torch.equal(given, xq)
        assert fn(oracle.TQ1_0, 1, w.data_ptr(), None, given.data_ptr(), None, None, powers.data_ptr(), y1.data_ptr(), n, k, m, n, 1) == 0, last_error(lib)
        torch.cuda.synchronize()
        assert torch.isfinite(y0).all()
        assert torch.equal(y0, y1), (m, n, k)
        want, _ = oracle.mul_mat(oracle.TQ1_0, w.cpu().numpy(), None, n, k, m, xq=given.cpu().numpy())
        assert rel_l2(y1.cpu().numpy(), want) <= 1e-5
