"""Regenerates tests/golden/golden.npz from the reference's own GGML C code.

Run in a checkout that has the reference tree, after ``make -C oracle ref``:

    python tests/golden/make_golden.py

Every array is produced by ``oracle/_ref/libweft_ref.so`` (the reference sources compiled in
place), never by this repository's restatement.  The inputs restate the reference harnesses'
input policies:

* ``kat_*``  -- the closed-form sequences of examples/repro/weft/vec_dot_runtime.cpp:385-434 and
  mul_mat_runtime.cpp:762-776: w[i] = ((19 i + 7 fmt) mod 127 - 63) / 13 over one weight record,
  x[i] = ((37 i) mod 251 - 125) / 17, one valid record replicated over a K = 4096 row;
* ``deq_*``  -- the random-byte record of row_dequantize_runtime.cpp:145-164: std::mt19937 seeded
  with 0x57454654 + fmt, one byte from the top 8 bits of each draw, retried until every
  dequantized value is finite;
* ``q8_*``   -- the activation-quantize input of q8_quantize_runtime.cpp:163-166,
  x[i] = ((i mod 31) - 15) / 16;
* ``rnd_*``  -- seeded N(0, 0.02) weights (scale * {-1, 0, +1} for TQ1_0) and N(0, 1) activations.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
import oracle as o  # noqa: E402

# new formats go last: the seeded generator is consumed in this order
FORMATS = {"q4_0": o.Q4_0, "q8_0": o.Q8_0, "q4_k": o.Q4_K, "iq2_xxs": o.IQ2_XXS, "tq1_0": o.TQ1_0, "q6_k": o.Q6_K, "q5_k": o.Q5_K, "q2_k": o.Q2_K, "q3_k": o.Q3_K, "iq2_xs": o.IQ2_XS, "iq3_xxs": o.IQ3_XXS, "iq2_s": o.IQ2_S, "iq3_s": o.IQ3_S, "iq1_s": o.IQ1_S, "iq1_m": o.IQ1_M}
VEC_DOT_IDS = {"q4_0": 1, "q8_0": 5, "q4_k": 8, "iq2_xxs": 15, "tq1_0": 20, "q6_k": 10, "q5_k": 9, "q2_k": 6, "q3_k": 7, "iq2_xs": 14, "iq3_xxs": 17, "iq2_s": 13, "iq3_s": 16, "iq1_s": 11, "iq1_m": 12}    # vec_dot / dequantize harness ids
MUL_MAT_IDS = {"q4_0": 2, "q8_0": 6, "q4_k": 9, "iq2_xxs": 16, "tq1_0": 21, "q6_k": 11, "q5_k": 10, "q2_k": 7, "q3_k": 8, "iq2_xs": 15, "iq3_xxs": 18, "iq2_s": 14, "iq3_s": 17, "iq1_s": 12, "iq1_m": 13}    # mul_mat harness ids


def closed_form_weights(count: int, fmt_id: int) -> np.ndarray:
    i = np.arange(count, dtype=np.uint64)
    return (((i * 19 + fmt_id * 7) % 127).astype(np.int64) - 63).astype(np.float32) / np.float32(13.0)


def closed_form_activations(count: int) -> np.ndarray:
    i = np.arange(count, dtype=np.uint64)
    return (((i * 37) % 251).astype(np.int64) - 125).astype(np.float32) / np.float32(17.0)


def mt19937_bytes(seed: int, count: int) -> np.ndarray:
    gen = np.random.MT19937()
    gen._legacy_seeding(seed)
    return (gen.random_raw(count) >> 24).astype(np.uint8)


def main() -> None:
    assert o.ref_available(), "build oracle/_ref first (make -C oracle ref)"
    out: dict[str, np.ndarray] = {}
    grid, signs = o.ref_iq2xxs_tables()
    out["iq2xxs_grid"] = grid
    out["iq2xxs_signs"] = signs
    out["iq2xs_grid"] = o.ref_iq2xs_grid()
    out["iq3xxs_grid"] = o.ref_iq3xxs_grid()
    out["iq2s_grid"] = o.ref_iq2s_grid()
    out["iq3s_grid"] = o.ref_iq3s_grid()
    out["iq1s_grid"] = o.ref_iq1s_grid()
    check = np.random.MT19937(); check._legacy_seeding(5489)
    assert int(check.random_raw(1)[0]) == 3499211612

    rng = np.random.default_rng(20240607)
    K = 1024
    x_rnd = rng.standard_normal((3, K)).astype(np.float32)
    out["rnd_x"] = x_rnd
    out["rnd_xq_q8_0"] = o.ref_quantize_activations(o.Q8_0, x_rnd)
    out["rnd_xq_q8_k"] = o.ref_quantize_activations(o.Q8_K, x_rnd)

    for name, fmt in FORMATS.items():
        elems = o.RECORD_ELEMENTS[fmt]
        act = o.ACTIVATION[fmt]
        # closed-form known-answer records
        for tag, ids in (("vd", VEC_DOT_IDS), ("mm", MUL_MAT_IDS)):
            w_src = closed_form_weights(elems, ids[name])
            w_rec = o.ref_quantize_weights(fmt, w_src[None, :])[0]
            x_src = closed_form_activations(elems if tag == "vd" else 4096)
            x_rec = o.ref_quantize_activations(act, x_src[None, :])[0]
            out[f"kat_{tag}_w_{name}"] = w_rec
            out[f"kat_{tag}_x_{name}"] = x_rec
            reps = 4096 // elems
            w_row = np.tile(w_rec, reps)
            x_row = np.tile(x_rec, reps) if tag == "vd" else x_rec
            out[f"kat_{tag}_row_{name}"] = np.float32(o.ref_vec_dot(fmt, w_row, x_row, 4096))
        # random-byte dequantize record
        seed = 0x57454654 + VEC_DOT_IDS[name]
        stream = mt19937_bytes(seed, 4096 * o.RECORD_BYTES[fmt])
        for attempt in range(4096):
            rec = stream[attempt * o.RECORD_BYTES[fmt]:(attempt + 1) * o.RECORD_BYTES[fmt]].copy()
            deq = o.ref_dequantize(fmt, rec, elems)
            if np.isfinite(deq).all():
                break
        else:
            raise SystemExit(f"no finite record for {name}")
        out[f"deq_rec_{name}"] = rec
        out[f"deq_out_{name}"] = deq[0]
        # seeded random matrices
        n = 8
        if name == "tq1_0":
            w_src = (rng.integers(-1, 2, size=(n, K)) * np.float32(0.02)).astype(np.float32)
        else:
            w_src = (rng.standard_normal((n, K)) * 0.02).astype(np.float32)
        w = o.ref_quantize_weights(fmt, w_src)
        out[f"rnd_wsrc_{name}"] = w_src
        out[f"rnd_w_{name}"] = w
        out[f"rnd_deq_{name}"] = o.ref_dequantize(fmt, w, K)
        y, xq = o.ref_mul_mat(fmt, w, x_rnd, n, K, 3)
        assert np.array_equal(xq, out["rnd_xq_q8_0" if act == o.Q8_0 else "rnd_xq_q8_k"])
        out[f"rnd_y_{name}"] = y

    # activation-quantize KAT input, GGML rule (the Weft rule is checked against the oracle port)
    i = np.arange(4 * 2048, dtype=np.int64)
    x31 = ((i % 31) - 15).astype(np.float32) / np.float32(16.0)
    x31 = x31.reshape(4, 2048)
    out["q8_0_mod31"] = o.ref_quantize_activations(o.Q8_0, x31)
    out["q8_k_mod31"] = o.ref_quantize_activations(o.Q8_K, x31)
    out["q8_1_mod31"] = o.ref_quantize_activations(o.Q8_1, x31)
    out["rnd_xq_q8_1"] = o.ref_quantize_activations(o.Q8_1, x_rnd)

    path = Path(__file__).with_name("golden.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path} ({path.stat().st_size} bytes, {len(out)} arrays)")


if __name__ == "__main__":
    main()
