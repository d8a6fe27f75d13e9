"""ctypes access to the CPU checkers -- TEST INFRASTRUCTURE ONLY.

Two libraries live beside this file:

* ``libweft_oracle.so`` -- this repository's plain-C restatement (``weft_oracle.c``) of the
  GGML-semantics algorithms the reference uses as its own correctness oracle;
* ``_ref/libweft_ref.so`` -- the reference's own GGML C sources compiled in place
  (``make ref``; only where the reference tree is available, the built file travels).

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may
import this package.  The product package never does.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent

Q4_0, Q8_0, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, IQ1_S, IQ1_M, IQ2_S, IQ2_XS, IQ2_XXS, IQ3_S, IQ3_XXS, TQ1_0, Q8_K, Q8_1 = 1, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15, 16, 17, 20, 100, 101
FORMAT_IDS = {"Q4_0": Q4_0, "Q8_0": Q8_0, "Q2_K": Q2_K, "Q3_K": Q3_K, "Q4_K": Q4_K, "Q5_K": Q5_K, "Q6_K": Q6_K, "IQ2_XXS": IQ2_XXS, "IQ2_XS": IQ2_XS, "IQ3_XXS": IQ3_XXS, "IQ2_S": IQ2_S, "IQ3_S": IQ3_S, "IQ1_S": IQ1_S, "IQ1_M": IQ1_M, "TQ1_0": TQ1_0, "Q8_K": Q8_K, "Q8_1": Q8_1}
RECORD_BYTES = {Q4_0: 18, Q8_0: 34, Q2_K: 84, Q3_K: 110, Q4_K: 144, Q5_K: 176, Q6_K: 210, IQ2_XXS: 66, IQ2_XS: 74, IQ3_XXS: 98, IQ2_S: 82, IQ3_S: 110, IQ1_S: 50, IQ1_M: 56, TQ1_0: 54, Q8_K: 292, Q8_1: 36}
RECORD_ELEMENTS = {Q4_0: 32, Q8_0: 32, Q2_K: 256, Q3_K: 256, Q4_K: 256, Q5_K: 256, Q6_K: 256, IQ2_XXS: 256, IQ2_XS: 256, IQ3_XXS: 256, IQ2_S: 256, IQ3_S: 256, IQ1_S: 256, IQ1_M: 256, TQ1_0: 256, Q8_K: 256, Q8_1: 32}
ACTIVATION = {Q4_0: Q8_0, Q8_0: Q8_0, Q2_K: Q8_K, Q3_K: Q8_K, Q4_K: Q8_K, Q5_K: Q8_K, Q6_K: Q8_K, IQ2_XXS: Q8_K, IQ2_XS: Q8_K, IQ3_XXS: Q8_K, IQ2_S: Q8_K, IQ3_S: Q8_K, IQ1_S: Q8_K, IQ1_M: Q8_K, TQ1_0: Q8_K}

_u8p = ctypes.POINTER(ctypes.c_uint8)
_i8p = ctypes.POINTER(ctypes.c_int8)
_f32p = ctypes.POINTER(ctypes.c_float)
_i64 = ctypes.c_int64


def build(ref: bool = True) -> None:
    """Compile the port (always) and the reference build (when its sources are present)."""
    targets = ["port"] + (["ref"] if ref else [])
    subprocess.run(["make", "-s", "-C", str(HERE), "-f", str(HERE / "Makefile"), *targets], check=True)


def row_bytes(fmt: int, k: int) -> int:
    return k // RECORD_ELEMENTS[fmt] * RECORD_BYTES[fmt]


def _ptr(array: np.ndarray | None, kind):
    if array is None:
        return ctypes.cast(None, kind)
    assert array.flags.c_contiguous
    return array.ctypes.data_as(kind)


_port = None
_ref = None


def port() -> ctypes.CDLL:
    global _port
    if _port is None:
        path = HERE / "libweft_oracle.so"
        if not path.exists():
            build(ref=False)
        lib = ctypes.CDLL(str(path))
        lib.wo_quantize_rows.argtypes = [ctypes.c_int, ctypes.c_int, _f32p, _u8p, _i64, _i64]
        lib.wo_dequantize_rows.argtypes = [ctypes.c_int, _u8p, _i8p, _i8p, _f32p, _i64, _i64]
        lib.wo_vec_dot.argtypes = [ctypes.c_int, _u8p, _u8p, _i8p, _i8p, _i64, _f32p]
        lib.wo_mul_mat.argtypes = [ctypes.c_int, ctypes.c_int, _u8p, _f32p, _u8p, _i8p, _i8p, _f32p,
                                   _i64, _i64, _i64, _i64, _i64, ctypes.c_int]
        lib.wo_iq2_sign_table.argtypes = [_i8p]
        lib.wo_f16_to_f32.argtypes = [ctypes.c_uint16]
        lib.wo_f16_to_f32.restype = ctypes.c_float
        lib.wo_f32_to_f16.argtypes = [ctypes.c_float]
        lib.wo_f32_to_f16.restype = ctypes.c_uint16
        lib.wo_interleave_pack.argtypes = [_u8p, _u8p, ctypes.c_size_t, _i64, _i64, _i64]
        lib.wo_interleave_unpack.argtypes = [_u8p, _u8p, ctypes.c_size_t, _i64, _i64, _i64]
        lib.wo_max_threads.restype = ctypes.c_int
        lib.wo_set_threads.argtypes = [ctypes.c_int]
        _port = lib
    return _port


def ref_available() -> bool:
    return (HERE / "_ref" / "libweft_ref.so").exists()


def ref() -> ctypes.CDLL:
    global _ref
    if _ref is None:
        lib = ctypes.CDLL(str(HERE / "_ref" / "libweft_ref.so"))
        lib.weft_ref_row_bytes.argtypes = [ctypes.c_int, _i64]
        lib.weft_ref_row_bytes.restype = ctypes.c_size_t
        lib.weft_ref_quantize_weights.argtypes = [ctypes.c_int, _f32p, ctypes.c_void_p, _i64, _i64]
        lib.weft_ref_quantize_q8_0.argtypes = [_f32p, ctypes.c_void_p, _i64]
        lib.weft_ref_quantize_q8_K.argtypes = [_f32p, ctypes.c_void_p, _i64]
        lib.weft_ref_quantize_q8_1.argtypes = [_f32p, ctypes.c_void_p, _i64]
        lib.weft_ref_dequantize.argtypes = [ctypes.c_int, ctypes.c_void_p, _f32p, _i64]
        lib.weft_ref_vec_dot.argtypes = [ctypes.c_int, _i64, _f32p, ctypes.c_void_p, ctypes.c_void_p]
        lib.weft_ref_mul_mat.argtypes = [ctypes.c_int, ctypes.c_void_p, _f32p, ctypes.c_void_p, _f32p,
                                         _i64, _i64, _i64, _i64, _i64, ctypes.c_int]
        lib.weft_ref_iq2xxs_tables.argtypes = [_i8p, _i8p]
        lib.weft_ref_iq2xs_grid.argtypes = [_i8p]
        lib.weft_ref_iq3xxs_grid.argtypes = [_i8p]
        lib.weft_ref_iq2s_grid.argtypes = [_i8p]
        lib.weft_ref_iq3s_grid.argtypes = [_i8p]
        lib.weft_ref_iq1s_grid.argtypes = [_i8p]
        _ref = lib
    return _ref


# ---------------------------------------------------------------- port wrappers

def sign_table() -> np.ndarray:
    out = np.empty(1024, dtype=np.int8)
    port().wo_iq2_sign_table(_ptr(out, _i8p))
    return out


def quantize(fmt: int, x: np.ndarray, rule: int = 0) -> np.ndarray:
    """Rows of fp32 ``x`` (nrows, k) -> packed records (nrows, row_bytes) uint8. rule: 0 GGML, 1 Weft."""
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, x.shape[-1])
    nrows, k = x.shape
    out = np.zeros((nrows, row_bytes(fmt, k)), dtype=np.uint8)
    if port().wo_quantize_rows(fmt, rule, _ptr(x, _f32p), _ptr(out, _u8p), nrows, k):
        raise ValueError(f"the oracle port has no quantizer for format {fmt}")
    return out


def dequantize(fmt: int, w: np.ndarray, k: int, grid=None, signs=None) -> np.ndarray:
    w = np.ascontiguousarray(w, dtype=np.uint8).reshape(-1, row_bytes(fmt, k))
    out = np.empty((w.shape[0], k), dtype=np.float32)
    if port().wo_dequantize_rows(fmt, _ptr(w, _u8p), _ptr(grid, _i8p), _ptr(signs, _i8p),
                                 _ptr(out, _f32p), w.shape[0], k):
        raise ValueError(f"no dequantizer for format {fmt}")
    return out


def vec_dot(fmt: int, w: np.ndarray, x: np.ndarray, k: int, grid=None, signs=None) -> float:
    out = ctypes.c_float()
    w = np.ascontiguousarray(w, dtype=np.uint8)
    x = np.ascontiguousarray(x, dtype=np.uint8)
    if port().wo_vec_dot(fmt, _ptr(w, _u8p), _ptr(x, _u8p), _ptr(grid, _i8p), _ptr(signs, _i8p), k,
                         ctypes.byref(out)):
        raise ValueError(f"no dot product for format {fmt}")
    return out.value


def mul_mat(fmt: int, w: np.ndarray, x: np.ndarray | None, n: int, k: int, m: int, *, xq=None, rule: int = 0,
            grid=None, signs=None, rows: tuple[int, int] | None = None):
    """Y (m, n) fp32 and the activation records used.  Pass fp32 ``x`` to quantize it, or ready ``xq``."""
    act = ACTIVATION[fmt]
    quantize_x = xq is None
    if quantize_x:
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(m, k)
        xq = np.zeros((m, row_bytes(act, k)), dtype=np.uint8)
    else:
        xq = np.ascontiguousarray(xq, dtype=np.uint8)
    w = np.ascontiguousarray(w, dtype=np.uint8)
    y = np.zeros((m, n), dtype=np.float32)
    n0, n1 = rows if rows is not None else (0, n)
    status = port().wo_mul_mat(fmt, rule, _ptr(w, _u8p), _ptr(x if quantize_x else None, _f32p), _ptr(xq, _u8p),
                               _ptr(grid, _i8p), _ptr(signs, _i8p), _ptr(y, _f32p), n, k, m, n0, n1,
                               int(quantize_x))
    if status:
        raise ValueError(f"no mul_mat for format {fmt}")
    return y, xq


# ----------------------------------------------------------- reference wrappers

def ref_quantize_weights(fmt: int, x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, x.shape[-1])
    nrows, k = x.shape
    out = np.zeros((nrows, row_bytes(fmt, k)), dtype=np.uint8)
    if ref().weft_ref_quantize_weights(fmt, _ptr(x, _f32p), out.ctypes.data, nrows, k):
        raise ValueError(f"reference cannot quantize format {fmt}")
    return out


def ref_quantize_activations(fmt: int, x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, x.shape[-1])
    nrows, k = x.shape
    out = np.zeros((nrows, row_bytes(fmt, k)), dtype=np.uint8)
    fn = {Q8_0: ref().weft_ref_quantize_q8_0, Q8_1: ref().weft_ref_quantize_q8_1, Q8_K: ref().weft_ref_quantize_q8_K}[fmt]
    for r in range(nrows):
        fn(_ptr(x[r], _f32p), out[r].ctypes.data, k)
    return out


def ref_dequantize(fmt: int, w: np.ndarray, k: int) -> np.ndarray:
    w = np.ascontiguousarray(w, dtype=np.uint8).reshape(-1, row_bytes(fmt, k))
    out = np.empty((w.shape[0], k), dtype=np.float32)
    for r in range(w.shape[0]):
        if ref().weft_ref_dequantize(fmt, w[r].ctypes.data, _ptr(out[r], _f32p), k):
            raise ValueError(f"reference cannot dequantize format {fmt}")
    return out


def ref_vec_dot(fmt: int, w: np.ndarray, x: np.ndarray, k: int) -> float:
    out = ctypes.c_float()
    w = np.ascontiguousarray(w, dtype=np.uint8)
    x = np.ascontiguousarray(x, dtype=np.uint8)
    ref().weft_ref_vec_dot(fmt, k, ctypes.byref(out), w.ctypes.data, x.ctypes.data)
    return out.value


def ref_mul_mat(fmt: int, w: np.ndarray, x: np.ndarray, n: int, k: int, m: int):
    act = ACTIVATION[fmt]
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(m, k)
    w = np.ascontiguousarray(w, dtype=np.uint8)
    xq = np.zeros((m, row_bytes(act, k)), dtype=np.uint8)
    y = np.zeros((m, n), dtype=np.float32)
    ref().weft_ref_mul_mat(fmt, w.ctypes.data, _ptr(x, _f32p), xq.ctypes.data, _ptr(y, _f32p), n, k, m, 0, n, 1)
    return y, xq


def ref_iq2xxs_tables():
    grid = np.empty(2048, dtype=np.int8)
    signs = np.empty(1024, dtype=np.int8)
    ref().weft_ref_iq2xxs_tables(_ptr(grid, _i8p), _ptr(signs, _i8p))
    return grid, signs


def ref_iq2xs_grid():
    grid = np.empty(4096, dtype=np.int8)
    ref().weft_ref_iq2xs_grid(_ptr(grid, _i8p))
    return grid


def ref_iq3xxs_grid():
    grid = np.empty(1024, dtype=np.int8)
    ref().weft_ref_iq3xxs_grid(_ptr(grid, _i8p))
    return grid


def ref_iq2s_grid():
    grid = np.empty(8192, dtype=np.int8)
    ref().weft_ref_iq2s_grid(_ptr(grid, _i8p))
    return grid


def ref_iq3s_grid():
    grid = np.empty(2048, dtype=np.int8)
    ref().weft_ref_iq3s_grid(_ptr(grid, _i8p))
    return grid


def ref_iq1s_grid():
    grid = np.empty(16384, dtype=np.int8)
    ref().weft_ref_iq1s_grid(_ptr(grid, _i8p))
    return grid


def interleave(fmt: int, w: np.ndarray, k: int, rows_per_cohort: int = 16, *, inverse: bool = False) -> np.ndarray:
    """The persistent interleaved layout ``Family[rows_per_cohort]`` of the (rows, row_bytes) records ``w``
    (doc/dsl/encoding-and-artifacts.md:209), or back to plain records with ``inverse``.  Same shape and size."""
    w = np.ascontiguousarray(w, dtype=np.uint8)
    rows = w.shape[0]
    blocks = k // RECORD_ELEMENTS[fmt]
    out = np.empty_like(w)
    move = port().wo_interleave_unpack if inverse else port().wo_interleave_pack
    if move(_ptr(w, _u8p), _ptr(out, _u8p), RECORD_BYTES[fmt], rows_per_cohort, rows, blocks) != 0:
        raise ValueError(f"{rows} rows are not whole cohorts of {rows_per_cohort}")
    return out


def host_threads() -> int:
    return int(port().wo_max_threads())


def cpu_model() -> str:
    try:
        for line in Path("/proc/cpuinfo").read_text().splitlines():
            if line.startswith("model name"):
                return line.split(":", 1)[1].strip()
    except OSError:
        pass
    return os.uname().machine
