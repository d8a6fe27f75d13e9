"""The CPU oracle port against golden vectors made by the reference's own GGML C.

tests/golden/golden.npz comes from tests/golden/make_golden.py, which runs the reference sources
compiled in place.  These tests pin the port (oracle/weft_oracle.c) to it bit for bit; when the
compiled reference is present they also compare the two live on fresh seeded inputs.
"""
from __future__ import annotations

import numpy as np
import pytest

FORMATS = ["q4_0", "q8_0", "q4_k", "iq2_xxs", "tq1_0", "q6_k", "q5_k", "q2_k", "q3_k", "iq2_xs", "iq3_xxs", "iq2_s", "iq3_s", "iq1_s", "iq1_m"]


def _tables(golden, name):
    grid = {"iq2_xs": "iq2xs_grid", "iq3_xxs": "iq3xxs_grid", "iq2_s": "iq2s_grid", "iq3_s": "iq3s_grid", "iq1_s": "iq1s_grid", "iq1_m": "iq1s_grid"}.get(name, "iq2xxs_grid")
    return golden[grid], golden["iq2xxs_signs"]
K = 1024


def _fmt(oracle, name):
    return oracle.FORMAT_IDS[name.upper()]


def _bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def test_half_float_conversions(oracle):
    lib = oracle.port()
    halves = np.arange(65536, dtype=np.uint16)
    want = halves.view(np.float16).astype(np.float32)
    got = np.array([lib.wo_f16_to_f32(int(h)) for h in halves], dtype=np.float32)
    finite = ~np.isnan(want)
    assert np.array_equal(_bits(got[finite]), _bits(want[finite]))
    rng = np.random.default_rng(3)
    xs = np.concatenate([rng.standard_normal(4000).astype(np.float32) * s for s in (1e-8, 1e-6, 1e-3, 1, 300, 7e4)]
                        + [want[finite], np.array([65519.9, 65520, 65504, 2.9802322e-8, 8.9e-8], dtype=np.float32)])
    with np.errstate(over="ignore"):
        expect = xs.astype(np.float16).view(np.uint16)
    got16 = np.array([lib.wo_f32_to_f16(float(v)) for v in xs], dtype=np.uint16)
    assert np.array_equal(got16, expect)


def test_sign_table_is_seven_bits_plus_parity(oracle, golden):
    assert np.array_equal(oracle.sign_table(), golden["iq2xxs_signs"])
    grid = golden["iq2xxs_grid"]
    assert grid.shape == (2048,) and set(np.unique(grid)) <= {8, 25, 43}
    assert golden["iq2xs_grid"].shape == (4096,) and set(np.unique(golden["iq2xs_grid"])) <= {8, 25, 43}
    assert golden["iq3xxs_grid"].shape == (1024,) and int(golden["iq3xxs_grid"].min()) >= 4 and int(golden["iq3xxs_grid"].max()) <= 62


@pytest.mark.parametrize("name", ["q4_0", "q8_0", "q4_k", "tq1_0"])
def test_weight_quantizers_match_reference_bytes(oracle, golden, name):
    got = oracle.quantize(_fmt(oracle, name), golden[f"rnd_wsrc_{name}"])
    assert np.array_equal(got, golden[f"rnd_w_{name}"])


@pytest.mark.parametrize("act", ["q8_0", "q8_k", "q8_1"])
def test_activation_quantizers_match_reference_bytes(oracle, golden, act):
    fmt = _fmt(oracle, act)
    assert np.array_equal(oracle.quantize(fmt, golden["rnd_x"]), golden[f"rnd_xq_{act}"])
    i = np.arange(4 * 2048, dtype=np.int64)
    x31 = (((i % 31) - 15).astype(np.float32) / np.float32(16.0)).reshape(4, 2048)
    assert np.array_equal(oracle.quantize(fmt, x31), golden[f"{act}_mod31"])


def test_weft_activation_rule_differs_only_by_sign_on_ties(oracle):
    # q8_quantize_runtime.cpp:163-166 input: +15/16 and -15/16 tie in every block
    i = np.arange(2048, dtype=np.int64)
    x31 = (((i % 31) - 15).astype(np.float32) / np.float32(16.0))[None, :]
    ggml = oracle.quantize(oracle.Q8_K, x31, rule=0).reshape(-1, 292)
    weft = oracle.quantize(oracle.Q8_K, x31, rule=1).reshape(-1, 292)
    for a, b in zip(ggml, weft):
        da, db = a[:4].view(np.float32)[0], b[:4].view(np.float32)[0]
        qa, qb = a[4:260].view(np.int8).astype(int), b[4:260].view(np.int8).astype(int)
        assert db > 0 or da == db               # a tie keeps the negative extreme, so d = extreme / -127 > 0
        assert (da == db and np.array_equal(qa, qb)) or (da == -db and np.array_equal(qa, -qb))
    rng = np.random.default_rng(5)
    x = rng.standard_normal((4, 2048)).astype(np.float32)
    for fmt in (oracle.Q8_0, oracle.Q8_K):      # no ties in N(0,1) data: both rules agree
        assert np.array_equal(oracle.quantize(fmt, x, rule=0), oracle.quantize(fmt, x, rule=1))


@pytest.mark.parametrize("name", FORMATS)
def test_dequantize_bit_exact(oracle, golden, name):
    fmt = _fmt(oracle, name)
    grid, signs = _tables(golden, name)
    got = oracle.dequantize(fmt, golden[f"rnd_w_{name}"], K, grid, signs)
    assert np.array_equal(_bits(got), _bits(golden[f"rnd_deq_{name}"]))
    # the reference's random-byte record (row_dequantize_runtime.cpp:145-164)
    elems = oracle.RECORD_ELEMENTS[fmt]
    got = oracle.dequantize(fmt, golden[f"deq_rec_{name}"], elems, grid, signs)[0]
    assert np.array_equal(_bits(got), _bits(golden[f"deq_out_{name}"]))


@pytest.mark.parametrize("name", FORMATS)
def test_mul_mat_bit_exact(oracle, golden, name):
    fmt = _fmt(oracle, name)
    grid, signs = _tables(golden, name)
    y, xq = oracle.mul_mat(fmt, golden[f"rnd_w_{name}"], golden["rnd_x"], 8, K, 3, grid=grid, signs=signs)
    act = "q8_0" if name in ("q4_0", "q8_0") else "q8_k"
    assert np.array_equal(xq, golden[f"rnd_xq_{act}"])
    assert np.array_equal(_bits(y), _bits(golden[f"rnd_y_{name}"]))


@pytest.mark.parametrize("name", FORMATS)
@pytest.mark.parametrize("tag", ["vd", "mm"])
def test_closed_form_known_answers(oracle, golden, name, tag):
    """vec_dot_runtime.cpp:385-434 / mul_mat_runtime.cpp:762-794: one valid record replicated over K = 4096."""
    fmt = _fmt(oracle, name)
    reps = 4096 // oracle.RECORD_ELEMENTS[fmt]
    w_row = np.tile(golden[f"kat_{tag}_w_{name}"], reps)
    x_rec = golden[f"kat_{tag}_x_{name}"]
    x_row = np.tile(x_rec, reps) if tag == "vd" else x_rec
    got = oracle.vec_dot(fmt, w_row, x_row, 4096, *_tables(golden, name))
    assert np.float32(got).view(np.uint32) == golden[f"kat_{tag}_row_{name}"].view(np.uint32)
    assert np.isfinite(got)


@pytest.mark.parametrize("name", FORMATS)
def test_live_against_compiled_reference(oracle, golden, name):
    if not oracle.ref_available():
        pytest.skip("compiled reference (oracle/_ref) not present")
    fmt = _fmt(oracle, name)
    rng = np.random.default_rng(77 + fmt)
    n, k, m = 12, 2048, 2
    src = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    if name == "tq1_0":
        src = (rng.integers(-1, 2, size=(n, k)) * np.float32(0.031)).astype(np.float32)
    w = oracle.ref_quantize_weights(fmt, src)
    if name not in ("iq2_xxs", "q6_k", "q5_k", "q2_k", "q3_k", "iq2_xs", "iq3_xxs", "iq2_s", "iq3_s", "iq1_s", "iq1_m"):   # the port has no quantizer for these weight formats
        assert np.array_equal(oracle.quantize(fmt, src), w)
    grid, signs = oracle.ref_iq2xxs_tables()
    assert np.array_equal(grid, golden["iq2xxs_grid"])
    assert np.array_equal(oracle.ref_iq2xs_grid(), golden["iq2xs_grid"]) and np.array_equal(oracle.ref_iq3xxs_grid(), golden["iq3xxs_grid"])
    assert np.array_equal(oracle.ref_iq2s_grid(), golden["iq2s_grid"]) and np.array_equal(oracle.ref_iq3s_grid(), golden["iq3s_grid"])
    assert np.array_equal(oracle.ref_iq1s_grid(), golden["iq1s_grid"])
    grid, signs = _tables(golden, name)
    x = rng.standard_normal((m, k)).astype(np.float32)
    assert np.array_equal(_bits(oracle.dequantize(fmt, w, k, grid, signs)), _bits(oracle.ref_dequantize(fmt, w, k)))
    y, xq = oracle.mul_mat(fmt, w, x, n, k, m, grid=grid, signs=signs)
    yr, xqr = oracle.ref_mul_mat(fmt, w, x, n, k, m)
    assert np.array_equal(xq, xqr) and np.array_equal(_bits(y), _bits(yr))


def test_interleave_follows_the_documented_rule(oracle):
    """doc/dsl/encoding-and-artifacts.md:209: for every cohort of R rows and every record, byte b of the R rows
    in row order, then byte b + 1.  Checked against an independent numpy statement of the rule, and that the
    mul_mat over the unpacked object equals the mul_mat over the source."""
    rng = np.random.default_rng(7)
    rows, k, R = 48, 768, 16
    blocks = k // 256
    w = rng.integers(0, 256, size=(rows, blocks * 144), dtype=np.uint8)
    packed = oracle.interleave(oracle.Q4_K, w, k, R)
    want = w.reshape(rows // R, R, blocks, 144).transpose(0, 2, 3, 1)          # [cohort][block][byte][row]
    assert np.array_equal(packed.reshape(-1), np.ascontiguousarray(want).reshape(-1))
    assert np.array_equal(oracle.interleave(oracle.Q4_K, packed, k, R, inverse=True), w)
    with pytest.raises(ValueError):
        oracle.interleave(oracle.Q4_K, w[:40], k, R)                            # no tail cohort
