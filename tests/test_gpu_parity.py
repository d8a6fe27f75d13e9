"""GPU parity: the CUDA path, called through the C ABI, against the CPU oracle on the same inputs.

Bars: dequantize and activation quantize bit-exact; dot products and mul_mat within 1e-5 relative
L2 (fp32 accumulation in a different summation order than the scalar oracle), and inside the
reference harnesses' own bound |a - e| <= 1e-4 + 2e-3 |e|.
"""
from __future__ import annotations

import ctypes

import numpy as np
import pytest

from helpers import TQ1_POWERS, activations, random_iq2_xxs, reference_tolerance_ok, rel_l2, tables, weights

pytestmark = pytest.mark.gpu

DECODE_FORMATS = ["q4_0", "q8_0", "q4_k", "iq2_xxs", "tq1_0", "q6_k", "q5_k", "q2_k", "q3_k"]   # have a production_mul_mat_<fmt>_decode
FORMATS = DECODE_FORMATS + ["iq2_xs", "iq3_xxs", "iq2_s", "iq3_s", "iq1_s", "iq1_m"]
CODEBOOKS = {"iq2_xxs": (256, 8, "I8X8"), "iq2_xs": (512, 8, "I8X8"), "iq3_xxs": (256, 4, "I8X4"), "iq2_s": (1024, 8, "I8X8"), "iq3_s": (512, 4, "I8X4"),
             "iq1_s": (2048, 8, "I8X8"), "iq1_m": (2048, 8, "I8X8")}
SIGN_TABLE = ("iq2_xxs", "iq2_xs", "iq3_xxs")     # the other codebook formats carry their sign bits in the record
REL_L2_BOUND = 1e-5


@pytest.fixture(scope="module")
def torch():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device; there is no CPU fallback to test")
    return torch


@pytest.fixture(scope="module")
def weft():
    import weft_b200

    return weft_b200


def dev(torch, array):
    return torch.from_numpy(np.ascontiguousarray(array)).cuda()


def _fmt(oracle, name):
    return oracle.FORMAT_IDS[name.upper()]


def _table_args(torch, golden, name):
    grid, signs = tables(golden, name)
    if name == "iq1_m":      # the reference passes the f16 -> f32 conversion as a table of 65536 floats
        f16_bits = np.arange(65536, dtype=np.uint16).view(np.float16).astype(np.float32)
        return [dev(torch, grid), dev(torch, f16_bits)]
    if name in CODEBOOKS:
        return [dev(torch, grid), dev(torch, signs)] if name in SIGN_TABLE else [dev(torch, grid)]
    if name == "tq1_0":
        return [dev(torch, TQ1_POWERS.view(np.int32)).view(torch.int32)]
    return []


def _wrap_tables(weft, name, tensors, dequant=False):
    from weft_b200.runtime import Buffer

    if name in CODEBOOKS:
        if dequant:
            return tensors
        entries, width, encoding = CODEBOOKS[name]
        wrapped = [Buffer(tensors[0], shape=(entries, width), encoding=encoding)]
        if name == "iq1_m":
            return wrapped + [tensors[1]]
        return wrapped + ([Buffer(tensors[1], shape=(128, 8), encoding="I8X8")] if name in SIGN_TABLE else [])
    if name == "tq1_0":
        return [Buffer(tensors[0], shape=(5,), encoding="dense.u32")]
    return []


def _definition(module, symbol):
    return getattr(module, symbol)


# ------------------------------------------------------------------ dequantize

@pytest.mark.parametrize("name", FORMATS)
def test_row_dequantize_bit_exact(torch, weft, oracle, golden, name):
    from weft_b200.kernels import dequantize, rows
    from weft_b200.runtime import Buffer

    fmt = _fmt(oracle, name)
    grid, signs = tables(golden, name)
    rng = np.random.default_rng(100 + fmt)
    cases = [
        (golden[f"rnd_w_{name}"], 8, 1024),                                              # reference-made golden bytes
        (np.tile(golden[f"deq_rec_{name}"], (64, 4096 // oracle.RECORD_ELEMENTS[fmt])), 64, 4096),  # random-byte record replicated
        (weights(fmt, rng, 300, 2048), 300, 2048),                                        # seeded N(0, 0.02)
        (weights(fmt, rng, 1, 256), 1, 256),                                              # one record row
    ]
    kernel = weft.compile(_definition(rows, f"row_dequantize_{name}_rows"))
    for w, n, k in cases:
        w = np.ascontiguousarray(w).reshape(n, -1)
        want = oracle.dequantize(fmt, w, k, grid, signs)
        y = torch.full((n, k), float("nan"), device="cuda")
        kernel(Buffer(dev(torch, w), shape=(n, k), encoding=name.upper()),
               *_wrap_tables(weft, name, _table_args(torch, golden, name), dequant=True), y)
        assert np.array_equal(y.cpu().numpy().view(np.uint32), want.view(np.uint32)), (name, n, k)
    # the reference's per-row symbol
    row_kernel = weft.compile(_definition(dequantize, f"row_dequantize_{name}"))
    w, n, k = cases[2]
    y = torch.empty(k, device="cuda")
    row_kernel(Buffer(dev(torch, w[5]), shape=(k,), encoding=name.upper()),
               *_wrap_tables(weft, name, _table_args(torch, golden, name), dequant=True), y)
    assert np.array_equal(y.cpu().numpy().view(np.uint32), oracle.dequantize(fmt, w[5], k, grid, signs)[0].view(np.uint32))


def test_row_dequantize_q4_k_full_size(torch, weft, oracle):
    """Config 2 of the benchmark: 14336 x 4096 Q4_K, bit-exact over all 58.7 M values."""
    from weft_b200.kernels import rows
    from weft_b200.runtime import Buffer

    n, k = 14336, 4096
    rng = np.random.default_rng(2)
    base = weights(oracle.Q4_K, rng, 512, k)                     # 512 distinct rows, tiled with a row rotation
    w = np.concatenate([np.roll(base, shift, axis=0) for shift in range(n // 512)], axis=0)
    want = oracle.dequantize(oracle.Q4_K, w, k)
    y = torch.empty((n, k), device="cuda")
    weft.compile(rows.row_dequantize_q4_k_rows)(Buffer(dev(torch, w), shape=(n, k), encoding="Q4_K"), y)
    got = y.cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_row_dequantize_unaligned_views(torch, weft, oracle):
    """Record alignment is 2 bytes (Q4_K) and fp32 alignment 4: odd offsets must still be exact."""
    from weft_b200.kernels import rows
    from weft_b200.runtime import Buffer

    rng = np.random.default_rng(9)
    n, k = 7, 512
    w = weights(oracle.Q4_K, rng, n, k)
    want = oracle.dequantize(oracle.Q4_K, w, k)
    raw = torch.zeros(w.size + 64, dtype=torch.uint8, device="cuda")
    raw[2:2 + w.size] = dev(torch, w.reshape(-1))
    out = torch.zeros(n * k + 8, device="cuda")
    kernel = weft.compile(rows.row_dequantize_q4_k_rows)
    kernel(Buffer(raw[2:2 + w.size], shape=(n, k), encoding="Q4_K"), Buffer(out[1:1 + n * k], shape=(n, k)))
    assert np.array_equal(out[1:1 + n * k].cpu().numpy().view(np.uint32), want.reshape(-1).view(np.uint32))
    assert out[0] == 0 and out[1 + n * k] == 0


def test_q6_k_at_an_odd_address(torch, weft, oracle):
    """The reference's Q6_K Encoding states no alignment: a weight view may start at any byte."""
    from weft_b200.kernels import mul_mat, rows
    from weft_b200.runtime import Buffer

    rng = np.random.default_rng(19)
    n, k = 37, 1024
    w = weights(oracle.Q6_K, rng, n, k)
    x = activations(rng, 2, k)
    raw = torch.zeros(w.size + 16, dtype=torch.uint8, device="cuda")
    raw[1:1 + w.size] = dev(torch, w.reshape(-1))
    view = Buffer(raw[1:1 + w.size], shape=(n, k), encoding="Q6_K")
    y = torch.empty((n, k), device="cuda")
    weft.compile(rows.row_dequantize_q6_k_rows)(view, y)
    assert np.array_equal(y.cpu().numpy().view(np.uint32), oracle.dequantize(oracle.Q6_K, w, k).view(np.uint32))
    want, want_xq = oracle.mul_mat(oracle.Q6_K, w, x, n, k, 2, rule=1)
    xq = torch.zeros((2, oracle.row_bytes(oracle.Q8_K, k)), dtype=torch.uint8, device="cuda")
    out = torch.empty((2, n), device="cuda")
    weft.compile(mul_mat.production_mul_mat_q6_k)(view, dev(torch, x), Buffer(xq, shape=(2, k), encoding="Q8_K"), out)
    assert np.array_equal(xq.cpu().numpy(), want_xq) and rel_l2(out.cpu().numpy(), want) <= REL_L2_BOUND


# ------------------------------------------------------------------ activation quantize

@pytest.mark.parametrize("act", ["q8_0", "q8_1", "q8_K"])
def test_activation_quantize_bit_exact(torch, weft, oracle, golden, act):
    from weft_b200.kernels import quantize, rows
    from weft_b200.runtime import Buffer

    fmt = {"q8_0": oracle.Q8_0, "q8_1": oracle.Q8_1, "q8_K": oracle.Q8_K}[act]
    enc = act.upper()
    rng = np.random.default_rng(31)
    i = np.arange(128 * 14336, dtype=np.int64)
    mod31 = (((i % 31) - 15).astype(np.float32) / np.float32(16.0)).reshape(128, 14336)   # q8_quantize_runtime.cpp:163-166
    special = np.zeros((4, 512), dtype=np.float32)
    special[1, 3] = 5.0; special[1, 300] = -5.0                  # exact +a/-a tie
    special[2] = np.linspace(-2.5, 2.5, 512, dtype=np.float32)    # exact .5 products
    special[3, :256] = 1e-30
    cases = [mod31, activations(rng, 16, 4096), special, activations(rng, 1, 256) * 1e4]
    kernel = weft.compile(getattr(rows, f"{act}_quantize_rows"))
    for x in cases:
        m, k = x.shape
        want = oracle.quantize(fmt, x, rule=1)                    # the Weft rule
        y = torch.full((m, oracle.row_bytes(fmt, k)), 0xA5, dtype=torch.uint8, device="cuda")
        kernel(dev(torch, x), Buffer(y, shape=(m, k), encoding=enc))
        assert np.array_equal(y.cpu().numpy(), want)
    # no exact ties in N(0,1) data: identical to GGML's quantize_row_*_ref as well
    x = cases[1]
    y = torch.empty((16, oracle.row_bytes(fmt, 4096)), dtype=torch.uint8, device="cuda")
    kernel(dev(torch, x), Buffer(y, shape=(16, 4096), encoding=enc))
    assert np.array_equal(y.cpu().numpy(), oracle.quantize(fmt, x, rule=0))
    # per-row reference symbol
    row = weft.compile(getattr(quantize, f"{act}_quantize"))
    y1 = torch.empty(oracle.row_bytes(fmt, 4096), dtype=torch.uint8, device="cuda")
    row(dev(torch, x[3]), Buffer(y1, shape=(4096,), encoding=enc))
    assert np.array_equal(y1.cpu().numpy(), oracle.quantize(fmt, x[3:4], rule=1)[0])


# ------------------------------------------------------------------ vec_dot

@pytest.mark.parametrize("name", FORMATS)
def test_vec_dot_closed_form_known_answer(torch, weft, oracle, golden, name):
    """examples/repro/weft/vec_dot_runtime.cpp:385-434: one valid record replicated over K = 4096."""
    from weft_b200.kernels import vec_dot
    from weft_b200.runtime import Buffer

    fmt = _fmt(oracle, name)
    act = "Q8_0" if name in ("q4_0", "q8_0") else "Q8_K"
    reps = 4096 // oracle.RECORD_ELEMENTS[fmt]
    w_row = np.tile(golden[f"kat_vd_w_{name}"], reps)
    x_row = np.tile(golden[f"kat_vd_x_{name}"], reps)
    symbol = f"quantized_vec_dot_{name}_{act.lower()}"
    kernel = weft.compile(getattr(vec_dot, symbol))
    y = torch.zeros(1, device="cuda")
    kernel(Buffer(dev(torch, w_row), shape=(4096,), encoding=name.upper()), Buffer(dev(torch, x_row), shape=(4096,), encoding=act),
           *_wrap_tables(weft, name, _table_args(torch, golden, name)), y)
    want = float(golden[f"kat_vd_row_{name}"])
    got = float(y.cpu()[0])
    assert reference_tolerance_ok(np.array([got]), np.array([want]))
    assert abs(got - want) <= 1e-5 * abs(want) + 1e-6


@pytest.mark.parametrize("name", FORMATS)
@pytest.mark.parametrize("shape", [(64, 256), (333, 1024), (4096, 4096), (130, 14336), (96, 8192)])
def test_vec_dot_rows_against_oracle(torch, weft, oracle, golden, name, shape):
    from weft_b200.kernels import rows
    from weft_b200.runtime import Buffer

    fmt = _fmt(oracle, name)
    act_fmt = oracle.ACTIVATION[fmt]
    act = "Q8_0" if act_fmt == oracle.Q8_0 else "Q8_K"
    n, k = shape
    rng = np.random.default_rng(1000 * fmt + n + k)
    w = weights(fmt, rng, n, k)
    xq = oracle.quantize(act_fmt, activations(rng, 1, k))
    grid, signs = tables(golden, name)
    want, _ = oracle.mul_mat(fmt, w, None, n, k, 1, xq=xq, grid=grid, signs=signs)
    kernel = weft.compile(getattr(rows, f"quantized_vec_dot_{name}_{act.lower()}_rows"))
    y = torch.full((n,), float("nan"), device="cuda")
    kernel(Buffer(dev(torch, w), shape=(n, k), encoding=name.upper()), Buffer(dev(torch, xq[0]), shape=(k,), encoding=act),
           *_wrap_tables(weft, name, _table_args(torch, golden, name)), y)
    got = y.cpu().numpy()
    assert rel_l2(got, want[0]) <= REL_L2_BOUND, (name, shape, rel_l2(got, want[0]))
    assert reference_tolerance_ok(got, want[0])


# ------------------------------------------------------------------ mul_mat (decode)

@pytest.mark.parametrize("symbol", ["production_mul_mat_iq2_xs", "production_mul_mat_iq2_xs_staged", "production_mul_mat_iq3_xxs", "production_mul_mat_iq2_xxs",
                                    "production_mul_mat_iq2_s", "production_mul_mat_iq2_s_staged", "production_mul_mat_iq3_s",
                                    "production_mul_mat_iq1_s", "production_mul_mat_iq1_s_decode", "production_mul_mat_iq1_m",
                                    "production_mul_mat_iq1_m_decode", "production_mul_mat_iq1_m_lane16_decode"])
@pytest.mark.parametrize("mnk", [(1, 512, 2048), (3, 200, 1024), (40, 96, 4096), (1, 4096, 4096)])
def test_mul_mat_codebook_formats(torch, weft, oracle, golden, symbol, mnk):
    """The mul_mat symbols of IQ2_XS, IQ3_XXS and the unstaged IQ2_XXS name: K = 1024 leaves rows that are not whole
    16-byte multiples (per-warp copies), K = 2048 and 4096 take the ring kernel with bank-striped tables."""
    from weft_b200.kernels import mul_mat
    from weft_b200.runtime import Buffer

    name = symbol[len("production_mul_mat_"):].removesuffix("_staged").removesuffix("_decode").removesuffix("_lane16")
    fmt = _fmt(oracle, name)
    m, n, k = mnk
    rng = np.random.default_rng(11 * fmt + m + n + k)
    w = weights(fmt, rng, n, k)
    x = activations(rng, m, k)
    grid, signs = tables(golden, name)
    want, want_xq = oracle.mul_mat(fmt, w, x, n, k, m, rule=1, grid=grid, signs=signs)
    xq = torch.zeros((m, oracle.row_bytes(oracle.Q8_K, k)), dtype=torch.uint8, device="cuda")
    y = torch.full((m, n), float("nan"), device="cuda")
    table_tensors = _table_args(torch, golden, name)
    wrapped = table_tensors if symbol.endswith(("iq2_xs_staged", "iq2_s_staged")) else _wrap_tables(weft, name, table_tensors)   # flat int8 arrays there
    weft.compile(getattr(mul_mat, symbol))(Buffer(dev(torch, w), shape=(n, k), encoding=name.upper()), dev(torch, x),
                                           Buffer(xq, shape=(m, k), encoding="Q8_K"), *wrapped, y)
    assert np.array_equal(xq.cpu().numpy(), want_xq)
    got = y.cpu().numpy()
    assert rel_l2(got, want) <= REL_L2_BOUND, (symbol, mnk, rel_l2(got, want))
    assert reference_tolerance_ok(got, want)


@pytest.mark.parametrize("name", DECODE_FORMATS)
@pytest.mark.parametrize("mnk", [(1, 512, 1024), (3, 200, 2048), (1, 4096, 4096)])
def test_mul_mat_decode(torch, weft, oracle, golden, name, mnk):
    from weft_b200.kernels import mul_mat
    from weft_b200.runtime import Buffer

    fmt = _fmt(oracle, name)
    act_fmt = oracle.ACTIVATION[fmt]
    act = "Q8_0" if act_fmt == oracle.Q8_0 else "Q8_K"
    m, n, k = mnk
    rng = np.random.default_rng(7 * fmt + m + n + k)
    w = weights(fmt, rng, n, k)
    x = activations(rng, m, k)
    grid, signs = tables(golden)
    want, want_xq = oracle.mul_mat(fmt, w, x, n, k, m, rule=1, grid=grid, signs=signs)
    kernel = weft.compile(getattr(mul_mat, f"production_mul_mat_{name}_decode"))
    xq = torch.zeros((m, oracle.row_bytes(act_fmt, k)), dtype=torch.uint8, device="cuda")
    y = torch.full((m, n), float("nan"), device="cuda")
    kernel(Buffer(dev(torch, w), shape=(n, k), encoding=name.upper()), dev(torch, x), Buffer(xq, shape=(m, k), encoding=act),
           *_wrap_tables(weft, name, _table_args(torch, golden, name)), y)
    assert np.array_equal(xq.cpu().numpy(), want_xq)          # the written workspace has the reference byte layout
    got = y.cpu().numpy()
    assert rel_l2(got, want) <= REL_L2_BOUND, (name, mnk, rel_l2(got, want))
    assert reference_tolerance_ok(got, want)


def test_mul_mat_q4_k_decode_benchmark_shapes(torch, weft, oracle):
    """Config 3: Llama-3-8B-shaped layers at batch 1, full size, against the oracle."""
    from weft_b200.kernels import mul_mat
    from weft_b200.runtime import Buffer

    kernel = weft.compile(mul_mat.production_mul_mat_q4_k_decode)
    for n, k in [(4096, 4096), (14336, 4096), (4096, 14336)]:
        rng = np.random.default_rng(n + k)
        w = weights(oracle.Q4_K, rng, n, k)
        x = activations(rng, 1, k)
        want, want_xq = oracle.mul_mat(oracle.Q4_K, w, x, n, k, 1, rule=1)
        xq = torch.zeros((1, oracle.row_bytes(oracle.Q8_K, k)), dtype=torch.uint8, device="cuda")
        y = torch.empty((1, n), device="cuda")
        kernel(Buffer(dev(torch, w), shape=(n, k), encoding="Q4_K"), dev(torch, x), Buffer(xq, shape=(1, k), encoding="Q8_K"), y)
        assert np.array_equal(xq.cpu().numpy(), want_xq)
        assert rel_l2(y.cpu().numpy(), want) <= REL_L2_BOUND


def test_low_bit_70b_shaped_decode(torch, weft, oracle, golden):
    """Config 5a shape (N = 28672, K = 8192) for IQ2_XXS; random valid records stand in for quantized weights."""
    from weft_b200.kernels import mul_mat
    from weft_b200.runtime import Buffer

    n, k = 28672, 8192
    rng = np.random.default_rng(5)
    w = random_iq2_xxs(rng, n, k)
    x = activations(rng, 1, k)
    grid, signs = tables(golden)
    want, _ = oracle.mul_mat(oracle.IQ2_XXS, w, x, n, k, 1, rule=1, grid=grid, signs=signs)
    xq = torch.zeros((1, oracle.row_bytes(oracle.Q8_K, k)), dtype=torch.uint8, device="cuda")
    y = torch.empty((1, n), device="cuda")
    weft.compile(mul_mat.production_mul_mat_iq2_xxs_decode)(
        Buffer(dev(torch, w), shape=(n, k), encoding="IQ2_XXS"), dev(torch, x), Buffer(xq, shape=(1, k), encoding="Q8_K"),
        *_wrap_tables(weft, "iq2_xxs", _table_args(torch, golden, "iq2_xxs")), y)
    assert rel_l2(y.cpu().numpy(), want) <= REL_L2_BOUND


# ------------------------------------------------------------------ host pointers through the raw C ABI

def test_c_abi_with_host_buffers(torch, weft, oracle):
    """The literal drop-in call: every pointer is host memory, exactly what the reference's FFI passes."""
    from weft_b200.runtime.driver import Toolchain, load_library

    lib = load_library(Toolchain().resolve().compiler)
    n, k = 1024, 2048
    rng = np.random.default_rng(77)
    w = weights(oracle.Q4_K, rng, n, k)
    x = activations(rng, 1, k)
    want, want_xq = oracle.mul_mat(oracle.Q4_K, w, x, n, k, 1, rule=1)
    xq = np.zeros_like(want_xq)
    y = np.full((1, n), np.nan, dtype=np.float32)
    fn = lib.production_mul_mat_q4_k_decode
    fn.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_size_t] * 3
    fn.restype = ctypes.c_int
    assert fn(w.ctypes.data, x.ctypes.data, xq.ctypes.data, y.ctypes.data, n, k, 1) == 0, lib.weft_b200_last_error()
    assert np.array_equal(xq, want_xq) and rel_l2(y, want) <= REL_L2_BOUND
    # resident weights: the second call finds the uploaded copy by address
    assert lib.weft_b200_weights_resident(w.ctypes.data, w.nbytes) == 0
    y2 = np.zeros_like(y)
    assert fn(w.ctypes.data, x.ctypes.data, xq.ctypes.data, y2.ctypes.data, n, k, 1) == 0
    assert np.array_equal(y2, y)
    assert lib.weft_b200_weights_release(w.ctypes.data) == 0
    # dequantize with host pointers
    out = np.empty((n, k), dtype=np.float32)
    dq = lib.row_dequantize_q4_k_rows
    dq.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_size_t]
    assert dq(w.ctypes.data, out.ctypes.data, n, k) == 0
    assert np.array_equal(out.view(np.uint32), oracle.dequantize(oracle.Q4_K, w, k).view(np.uint32))
    # errors come back as a status and a message, never as a crash
    assert fn(w.ctypes.data, x.ctypes.data, xq.ctypes.data, y.ctypes.data, n, 100, 1) != 0
    assert b"records" in lib.weft_b200_last_error()


def test_c_abi_with_pinned_host_buffers(torch, weft, oracle):
    """Pinned (mapped) host arguments are moved by a copy kernel rather than the copy engine: same results, also
    for sizes that are not whole 16-byte words and for buffers at odd offsets."""
    from weft_b200.runtime.driver import Toolchain, load_library

    lib = load_library(Toolchain().resolve().compiler)
    fn = lib.production_mul_mat_q4_k_decode
    fn.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_size_t] * 3
    fn.restype = ctypes.c_int
    rng = np.random.default_rng(78)
    # the larger cases: every CTA collects several rounds of rows and a ragged tail before it stores them to the host;
    # the last one has more rows per CTA than the kernel collects, so every row is stored as it completes
    for n, k, m, shift in [(1024, 2048, 1, 0), (333, 768, 3, 4), (64, 256, 1, 4), (14336, 4096, 1, 0), (5003, 1024, 2, 4), (90000, 256, 1, 0)]:
        w = weights(oracle.Q4_K, rng, n, k)
        x = activations(rng, m, k)
        want, want_xq = oracle.mul_mat(oracle.Q4_K, w, x, n, k, m, rule=1)
        w_dev = dev(torch, w)
        x_pin = torch.zeros(m * k + 8).pin_memory()
        x_pin[shift // 4: shift // 4 + m * k] = torch.from_numpy(x.reshape(-1))
        xq_pin = torch.zeros(want_xq.size + 16, dtype=torch.uint8).pin_memory()
        y_pin = torch.full((m * n + 8,), float("nan")).pin_memory()
        x_ptr, xq_ptr, y_ptr = x_pin.data_ptr() + shift, xq_pin.data_ptr() + shift, y_pin.data_ptr() + shift
        assert fn(w_dev.data_ptr(), x_ptr, xq_ptr, y_ptr, n, k, m) == 0, lib.weft_b200_last_error()
        got_xq = xq_pin.numpy()[shift: shift + want_xq.size].reshape(want_xq.shape)
        got = y_pin.numpy()[shift // 4: shift // 4 + m * n].reshape(m, n)
        assert np.array_equal(got_xq, want_xq) and rel_l2(got, want) <= REL_L2_BOUND, (n, k, m)
        assert np.isnan(y_pin.numpy()[shift // 4 + m * n:]).all() and (xq_pin.numpy()[shift + want_xq.size:] == 0).all()


def test_ragged_and_empty_shapes(torch, weft, oracle):
    """32-element formats whose K is not a multiple of 256, a single row, and empty extents through the C ABI."""
    from weft_b200.runtime.driver import Toolchain, load_library

    lib = load_library(Toolchain().resolve().compiler)
    rng = np.random.default_rng(90)
    for name, fmt in (("q4_0", oracle.Q4_0), ("q8_0", oracle.Q8_0)):
        fn = getattr(lib, f"production_mul_mat_{name}_decode")
        fn.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_size_t] * 3
        fn.restype = ctypes.c_int
        for n, k, m in [(5, 96, 1), (37, 288, 2), (1, 32, 1), (130, 4128, 1)]:
            w = weights(fmt, rng, n, k)
            x = activations(rng, m, k)
            want, want_xq = oracle.mul_mat(fmt, w, x, n, k, m, rule=1)
            xq = torch.zeros((m, oracle.row_bytes(oracle.Q8_0, k)), dtype=torch.uint8, device="cuda")
            y = torch.full((m, n), float("nan"), device="cuda")
            assert fn(dev(torch, w).data_ptr(), dev(torch, x).data_ptr(), xq.data_ptr(), y.data_ptr(), n, k, m) == 0, lib.weft_b200_last_error()
            assert np.array_equal(xq.cpu().numpy(), want_xq) and rel_l2(y.cpu().numpy(), want) <= REL_L2_BOUND, (name, n, k, m)
    # empty extents: success, nothing written
    fn = lib.production_mul_mat_q4_k_decode
    fn.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_size_t] * 3
    fn.restype = ctypes.c_int
    w = dev(torch, weights(oracle.Q4_K, rng, 4, 256))
    x = dev(torch, activations(rng, 1, 256))
    xq = torch.full((292,), 7, dtype=torch.uint8, device="cuda")
    y = torch.full((4,), 5.0, device="cuda")
    for n, k, m in [(0, 256, 1), (4, 0, 1), (4, 256, 0)]:
        assert fn(w.data_ptr(), x.data_ptr(), xq.data_ptr(), y.data_ptr(), n, k, m) == 0, lib.weft_b200_last_error()
    assert bool((y == 5.0).all()) and bool((xq == 7).all())
    dq = lib.row_dequantize_q4_k_rows
    dq.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_size_t]
    assert dq(w.data_ptr(), y.data_ptr(), 0, 256) == 0 and bool((y == 5.0).all())
    assert dq(w.data_ptr(), y.data_ptr(), 1, 100) != 0 and b"records" in lib.weft_b200_last_error()


def test_runtime_errors_match_the_reference(torch, weft, oracle):
    from weft_b200.kernels import rows
    from weft_b200.runtime import Buffer

    kernel = weft.compile(rows.row_dequantize_q4_k_rows)
    assert weft.compile(rows.row_dequantize_q4_k_rows) is kernel
    w = torch.zeros(144 * 4, dtype=torch.uint8, device="cuda")
    y = torch.zeros((1, 1024), device="cuda")
    with pytest.raises(TypeError):
        kernel(Buffer(w, shape=(1, 1024), encoding="Q8_K"), y)
    with pytest.raises(ValueError):
        kernel(Buffer(w, shape=(1, 1000), encoding="Q4_K"), torch.zeros((1, 1000), device="cuda"))
    with pytest.raises(ValueError):
        kernel(Buffer(w, shape=(2, 1024), encoding="Q4_K"), torch.zeros((2, 1024), device="cuda"))   # storage too short
    overlap = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    with pytest.raises(ValueError):
        kernel(Buffer(overlap[:576], shape=(1, 1024), encoding="Q4_K"), Buffer(overlap, shape=(1, 1024), encoding="dense.f32"))
    from weft_b200.runtime import CompileOptions
    other = weft.compile(rows.row_dequantize_q4_k_rows, options=CompileOptions(unroll=2))
    assert other is not kernel
    other.close(); other.close()
    with pytest.raises(RuntimeError):
        other(Buffer(w, shape=(1, 1024), encoding="Q4_K"), y)
