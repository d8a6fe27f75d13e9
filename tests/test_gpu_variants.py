"""GPU parity of the symbols the reference exports under more than one name, and of the prefill-form
symbols of the 32-element and codebook formats, against the CPU oracle.

The reference states some kernels several times for different vector plans of its target
(examples/kernels/vec_dot/tq1_0_q8_k_lane16.py, mul_mat/tq1_0_lane16_decode.py, gemv/q4_k_groups4.py,
gemv/q4_k_contract.py, mul_mat/q3_k_predecoded_scales[_decode].py); the integer sums and the float op tree
are the same in every statement, so each name must give the oracle's result.  Bound: 1e-5 relative L2 and
the reference harnesses' own |a - e| <= 1e-4 + 2e-3 |e|; the written Xq workspace bit-exact.
"""
from __future__ import annotations

import numpy as np
import pytest

from helpers import TQ1_POWERS, activations, reference_tolerance_ok, rel_l2, tables, weights

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device; there is no CPU fallback to test")
    return torch


def _mul_mat(torch, oracle, golden, symbol, fmt_name, m, n, k, seed):
    import weft_b200 as weft
    from weft_b200.kernels import mul_mat
    from weft_b200.runtime import Buffer

    fmt = oracle.FORMAT_IDS[fmt_name]
    act_fmt = oracle.ACTIVATION[fmt]
    act = "Q8_0" if act_fmt == oracle.Q8_0 else "Q8_K"
    rng = np.random.default_rng(seed)
    w = weights(fmt, rng, n, k)
    x = activations(rng, m, k)
    grid, signs = tables(golden)
    want, want_xq = oracle.mul_mat(fmt, w, x, n, k, m, rule=1, grid=grid, signs=signs)
    extra = []
    if fmt_name == "IQ2_XXS":
        extra = [Buffer(torch.from_numpy(grid).cuda(), shape=(256, 8), encoding="I8X8"),
                 Buffer(torch.from_numpy(signs).cuda(), shape=(128, 8), encoding="I8X8")]
    elif fmt_name == "TQ1_0":
        extra = [Buffer(torch.from_numpy(TQ1_POWERS.view(np.int32)).cuda().view(torch.int32), shape=(5,), encoding="dense.u32")]
    xq = torch.zeros((m, oracle.row_bytes(act_fmt, k)), dtype=torch.uint8, device="cuda")
    y = torch.full((m, n), float("nan"), device="cuda")
    weft.compile(getattr(mul_mat, symbol))(Buffer(torch.from_numpy(w).cuda(), shape=(n, k), encoding=fmt_name),
                                           torch.from_numpy(x).cuda(), Buffer(xq, shape=(m, k), encoding=act), *extra, y)
    got = y.cpu().numpy()
    assert np.array_equal(xq.cpu().numpy(), want_xq), symbol
    assert np.isfinite(got).all()
    assert rel_l2(got, want) <= 1e-5, (symbol, m, n, k, rel_l2(got, want))
    assert reference_tolerance_ok(got, want)


@pytest.mark.parametrize("symbol,fmt", [("production_mul_mat_q4_0", "Q4_0"), ("production_mul_mat_q8_0", "Q8_0"),
                                        ("production_mul_mat_iq2_xxs_staged", "IQ2_XXS")])
@pytest.mark.parametrize("mnk", [(3, 200, 1024), (128, 384, 2048), (128, 1000, 1024), (40, 64, 256), (512, 1000, 2048), (300, 77, 3072)])
def test_prefill_form_of_small_block_and_codebook_formats(torch, oracle, golden, symbol, fmt, mnk):
    """examples/kernels/mul_mat/q4_0.py:9-30, q8_0.py:9-29, iq2_xxs_staged.py:9-97: token batches below the tensor-core
    threshold (32 tokens: row-by-row GEMV) and above it (one contraction per 32-element block or group), token and
    weight counts that are not whole tiles, K = 256 (one unit; the codebook format then takes the row-by-row path,
    its activation rows are whole 16-byte multiples only for K % 1024 = 0)."""
    m, n, k = mnk
    _mul_mat(torch, oracle, golden, symbol, fmt, m, n, k, seed=sum(mnk) + len(symbol))


@pytest.mark.parametrize("symbol,fmt", [("production_mul_mat_q4_0", "Q4_0"), ("production_mul_mat_q8_0", "Q8_0"),
                                        ("production_mul_mat_iq2_xxs_staged", "IQ2_XXS")])
def test_prefill_form_reference_harness_shape(torch, oracle, golden, symbol, fmt):
    """The shape the reference's own harness runs: N = K = 4096, M = 128 (examples/repro/weft/mul_mat_runtime.cpp:668-676)."""
    _mul_mat(torch, oracle, golden, symbol, fmt, 128, 4096, 4096, seed=4096)


@pytest.mark.parametrize("symbol,fmt,mnk", [
    ("production_mul_mat_tq1_0_lane16_decode", "TQ1_0", (1, 512, 1024)),
    ("production_mul_mat_tq1_0_lane16_decode", "TQ1_0", (3, 200, 2048)),
    ("production_mul_mat_q3_k_predecoded_scales_decode", "Q3_K", (1, 512, 1024)),
    ("production_mul_mat_q3_k_predecoded_scales_decode", "Q3_K", (2, 130, 2048)),
    ("production_mul_mat_q3_k_predecoded_scales", "Q3_K", (5, 256, 1024)),
])
def test_mul_mat_under_the_reference_other_names(torch, oracle, golden, symbol, fmt, mnk):
    m, n, k = mnk
    _mul_mat(torch, oracle, golden, symbol, fmt, m, n, k, seed=sum(mnk))


def test_vec_dot_tq1_0_lane16(torch, oracle, golden):
    """Known-answer record of the reference harness (vec_dot_runtime.cpp:385-434) and a seeded row, both names."""
    import weft_b200 as weft
    from weft_b200.kernels import vec_dot
    from weft_b200.runtime import Buffer

    powers = Buffer(torch.from_numpy(TQ1_POWERS.view(np.int32)).cuda().view(torch.int32), shape=(5,), encoding="dense.u32")
    k = 4096
    w_row = np.tile(golden["kat_vd_w_tq1_0"], k // 256)
    x_row = np.tile(golden["kat_vd_x_tq1_0"], k // 256)
    rng = np.random.default_rng(21)
    w_rnd = weights(oracle.TQ1_0, rng, 1, k)[0]
    x_rnd = oracle.quantize(oracle.Q8_K, activations(rng, 1, k))[0]
    want_rnd, _ = oracle.mul_mat(oracle.TQ1_0, w_rnd[None], None, 1, k, 1, xq=x_rnd[None])
    for w, x, want in [(w_row, x_row, float(golden["kat_vd_row_tq1_0"])), (w_rnd, x_rnd, float(want_rnd[0, 0]))]:
        results = []
        for definition in (vec_dot.quantized_vec_dot_tq1_0_q8_k_lane16, vec_dot.quantized_vec_dot_tq1_0_q8_k):
            y = torch.zeros(1, device="cuda")
            weft.compile(definition)(Buffer(torch.from_numpy(w).cuda(), shape=(k,), encoding="TQ1_0"),
                                     Buffer(torch.from_numpy(x).cuda(), shape=(k,), encoding="Q8_K"), powers, y)
            results.append(float(y.cpu()[0]))
        assert results[0] == results[1]
        assert abs(results[0] - want) <= 1e-5 * abs(want) + 1e-6


@pytest.mark.parametrize("name", ["q4_k_q8_k_gemv_groups4", "q4_k_q8_k_gemv_contract"])
@pytest.mark.parametrize("mk", [(48, 768), (2368, 4096)])
def test_interleaved_gemv_under_the_reference_other_names(torch, oracle, name, mk):
    """examples/repro/weft/q4_k_gemv_runtime.cpp:12-25: each name has its own _W_packed_size / _W_pack / kernel triple."""
    import weft_b200 as weft
    from weft_b200 import artifacts
    from weft_b200.kernels import gemv
    from weft_b200.runtime import Buffer

    definition = getattr(gemv, name)
    m, k = mk
    rng = np.random.default_rng(m + k)
    w = weights(oracle.Q4_K, rng, m, k)
    xq = oracle.quantize(oracle.Q8_K, activations(rng, 1, k), rule=1)
    assert artifacts.packed_size(definition, m, k) == w.size
    packed = torch.zeros(w.size, dtype=torch.uint8, device="cuda")
    artifacts.pack(definition, torch.from_numpy(w).cuda(), packed, m, k)
    assert np.array_equal(packed.cpu().numpy(), oracle.interleave(oracle.Q4_K, w, k).reshape(-1))
    y = torch.full((m,), float("nan"), device="cuda")
    weft.compile(definition)(Buffer(packed, shape=(m, k), encoding="Q4K_I[16]"),
                             Buffer(torch.from_numpy(xq.reshape(-1)).cuda(), shape=(k,), encoding="Q8_K"), y)
    want, _ = oracle.mul_mat(oracle.Q4_K, w, None, m, k, 1, xq=xq)
    got = y.cpu().numpy()
    assert rel_l2(got, want.reshape(-1)) <= 1e-5
    assert reference_tolerance_ok(got, want.reshape(-1))
