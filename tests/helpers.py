"""Shared input builders for the parity tests (test infrastructure)."""
from __future__ import annotations

import numpy as np

import oracle as o

TQ1_POWERS = np.array([1, 3, 9, 27, 81], dtype=np.uint32)


def rel_l2(got: np.ndarray, want: np.ndarray) -> float:
    got64, want64 = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    denom = np.linalg.norm(want64)
    return float(np.linalg.norm(got64 - want64) / denom) if denom else float(np.linalg.norm(got64))


def reference_tolerance_ok(got: np.ndarray, want: np.ndarray) -> bool:
    """|a - e| <= 1e-4 + 2e-3 |e| and finite: the reference harnesses' bound (vec_dot_runtime.cpp:23-38)."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    return bool(np.isfinite(got).all() and (np.abs(got - want) <= 1e-4 + 2e-3 * np.abs(want)).all())


def random_iq2_xxs(rng: np.random.Generator, n: int, k: int) -> np.ndarray:
    """Random but valid IQ2_XXS records: any grid index, sign index and 4-bit scale is legal; d is a small f16."""
    nb = k // 256
    rec = rng.integers(0, 256, size=(n, nb, 66), dtype=np.uint8)
    d = (np.abs(rng.standard_normal((n, nb))) * 0.01 + 1e-3).astype(np.float16)
    rec[:, :, 0:2] = d.view(np.uint8).reshape(n, nb, 2)
    return rec.reshape(n, nb * 66)


def random_iq2_xs(rng: np.random.Generator, n: int, k: int) -> np.ndarray:
    """Random but valid IQ2_XS records: any 9-bit grid index, sign index and scale nibble is legal; d is a small f16."""
    nb = k // 256
    rec = rng.integers(0, 256, size=(n, nb, 74), dtype=np.uint8)
    d = (np.abs(rng.standard_normal((n, nb))) * 0.01 + 1e-3).astype(np.float16)
    rec[:, :, 0:2] = d.view(np.uint8).reshape(n, nb, 2)
    return rec.reshape(n, nb * 74)


def random_codebook_records(rng: np.random.Generator, n: int, k: int, record_bytes: int) -> np.ndarray:
    """Random but valid IQ2_S / IQ3_S records: every index, sign and scale bit pattern is legal; d (the first two bytes) is a small f16."""
    nb = k // 256
    rec = rng.integers(0, 256, size=(n, nb, record_bytes), dtype=np.uint8)
    d = (np.abs(rng.standard_normal((n, nb))) * 0.01 + 1e-3).astype(np.float16)
    rec[:, :, 0:2] = d.view(np.uint8).reshape(n, nb, 2)
    return rec.reshape(n, nb * record_bytes)


def random_iq3_xxs(rng: np.random.Generator, n: int, k: int) -> np.ndarray:
    """Random but valid IQ3_XXS records: any grid index byte, sign index and 4-bit scale is legal; d is a small f16."""
    nb = k // 256
    rec = rng.integers(0, 256, size=(n, nb, 98), dtype=np.uint8)
    d = (np.abs(rng.standard_normal((n, nb))) * 0.01 + 1e-3).astype(np.float16)
    rec[:, :, 0:2] = d.view(np.uint8).reshape(n, nb, 2)
    return rec.reshape(n, nb * 98)


def random_q6_k(rng: np.random.Generator, n: int, k: int) -> np.ndarray:
    """Random but valid Q6_K records: any ql / qh byte and any int8 scale is legal; d is a small f16."""
    nb = k // 256
    rec = rng.integers(0, 256, size=(n, nb, 210), dtype=np.uint8)
    d = (np.abs(rng.standard_normal((n, nb))) * 1e-4 + 1e-5).astype(np.float16)
    rec[:, :, 208:210] = d.view(np.uint8).reshape(n, nb, 2)
    return rec.reshape(n, nb * 210)


def random_k_records(rng: np.random.Generator, n: int, k: int, record_bytes: int, scales_at: int, scales: int) -> np.ndarray:
    """Random but valid K-family records: every bit pattern is legal once the f16 super-scales are small finite numbers."""
    nb = k // 256
    rec = rng.integers(0, 256, size=(n, nb, record_bytes), dtype=np.uint8)
    d = (np.abs(rng.standard_normal((n, nb, scales))) * 1e-3 + 1e-4).astype(np.float16)
    rec[:, :, scales_at:scales_at + 2 * scales] = d.view(np.uint8).reshape(n, nb, 2 * scales)
    return rec.reshape(n, nb * record_bytes)


def random_q5_k(rng: np.random.Generator, n: int, k: int) -> np.ndarray:
    """Random but valid Q5_K records: every scale / min / bit pattern is legal; d and dmin are small f16."""
    nb = k // 256
    rec = rng.integers(0, 256, size=(n, nb, 176), dtype=np.uint8)
    d = (np.abs(rng.standard_normal((n, nb, 2))) * 1e-3 + 1e-4).astype(np.float16)
    rec[:, :, 0:4] = d.view(np.uint8).reshape(n, nb, 4)
    return rec.reshape(n, nb * 176)


def weights(fmt: int, rng: np.random.Generator, n: int, k: int) -> np.ndarray:
    """Seeded weights of the benchmark distributions, quantized: N(0, 0.02) (scale * {-1,0,+1} for TQ1_0).

    IQ2_XXS, Q2_K, Q3_K, Q5_K and Q6_K go through the compiled reference quantizer when it is present and fall back to
    random valid records otherwise (the port has no quantizer for them)."""
    if fmt == o.TQ1_0:
        src = (rng.integers(-1, 2, size=(n, k)) * np.float32(0.02)).astype(np.float32)
        return o.quantize(fmt, src)
    if fmt == o.IQ2_XXS:
        if o.ref_available() and n * k <= 1 << 22:
            return o.ref_quantize_weights(fmt, (rng.standard_normal((n, k)) * 0.02).astype(np.float32))
        return random_iq2_xxs(rng, n, k)
    if fmt in (o.IQ2_XS, o.IQ3_XXS, o.IQ2_S, o.IQ3_S, o.IQ1_S, o.IQ1_M):
        if o.ref_available() and n * k <= 1 << 21:
            return o.ref_quantize_weights(fmt, (rng.standard_normal((n, k)) * 0.02).astype(np.float32))
        if fmt == o.IQ1_M:          # the f16 scale is spread over the top nibbles of the last eight bytes: 0x2xxx is a small normal number
            rec = rng.integers(0, 256, size=(n, k // 256, 56), dtype=np.uint8)
            rec[:, :, 55] = (rec[:, :, 55] & 0x0f) | 0x20
            return rec.reshape(n, -1)
        if fmt in (o.IQ2_S, o.IQ3_S, o.IQ1_S):
            return random_codebook_records(rng, n, k, o.RECORD_BYTES[fmt])
        return random_iq2_xs(rng, n, k) if fmt == o.IQ2_XS else random_iq3_xxs(rng, n, k)
    if fmt in (o.Q2_K, o.Q3_K, o.Q5_K, o.Q6_K):
        if o.ref_available() and n * k <= 1 << 22:
            return o.ref_quantize_weights(fmt, (rng.standard_normal((n, k)) * 0.02).astype(np.float32))
        if fmt == o.Q2_K:
            return random_k_records(rng, n, k, 84, 80, 2)
        if fmt == o.Q3_K:
            return random_k_records(rng, n, k, 110, 108, 1)
        return random_q5_k(rng, n, k) if fmt == o.Q5_K else random_q6_k(rng, n, k)
    return o.quantize(fmt, (rng.standard_normal((n, k)) * 0.02).astype(np.float32))


def activations(rng: np.random.Generator, m: int, k: int) -> np.ndarray:
    return rng.standard_normal((m, k)).astype(np.float32)


def tables(golden: dict, name: str = "iq2_xxs"):
    """The codebook and the sign table a format's kernels take as arguments (the sign table is the same for all three)."""
    grid = {"iq2_xs": "iq2xs_grid", "iq3_xxs": "iq3xxs_grid", "iq2_s": "iq2s_grid", "iq3_s": "iq3s_grid", "iq1_s": "iq1s_grid", "iq1_m": "iq1s_grid"}.get(name.lower(), "iq2xxs_grid")
    return golden[grid], golden["iq2xxs_signs"]
