"""Row dequantizers: K packed elements -> K fp32 values, bit-exact with the reference's GGML semantics.

Signatures follow examples/kernels/dequantize/q4_0.py:9-13, q8_0.py:9-13, q4_k.py:9-20,
q2_k.py:8-17, q3_k.py:8-17, q5_k.py:9-15, q6_k.py:8-15, iq2_xxs.py:9-53 and tq1_0.py:9-46 of the reference (Y is its own alias group where the reference says so).
"""
from __future__ import annotations

from .. import formats as ggml
from .. import language as wl
from ..api import kernel


@kernel
def row_dequantize_q4_0(W: wl.View[ggml.Q4_0, (K,)], Y: wl.View[wl.f32, (K,)]):
    """Y = f32(q - 8) * f32(d)."""


@kernel
def row_dequantize_q8_0(W: wl.View[ggml.Q8_0, (K,)], Y: wl.View[wl.f32, (K,)]):
    """Y = f32(q) * f32(d)."""


@kernel(alias_groups={"Y": "output"})
def row_dequantize_q4_k(W: wl.View[ggml.Q4_K, (K,)], Y: wl.View[wl.f32, (K,)]):
    """Y = (d * sc) * q - (dmin * m), three rounded multiplies and one subtract."""


@kernel(alias_groups={"Y": "output"})
def row_dequantize_q2_k(W: wl.View[ggml.Q2_K, (K,)], Y: wl.View[wl.f32, (K,)]):
    """Y = (d * (scales & 15)) * q2 - (dmin * (scales >> 4))."""


@kernel(alias_groups={"Y": "output"})
def row_dequantize_q3_k(W: wl.View[ggml.Q3_K, (K,)], Y: wl.View[wl.f32, (K,)]):
    """Y = (d * (scale - 32)) * (q2 + 4 * hmask - 4)."""


@kernel(alias_groups={"Y": "output"})
def row_dequantize_q5_k(W: wl.View[ggml.Q5_K, (K,)], Y: wl.View[wl.f32, (K,)]):
    """Y = (d * sc) * q5 - (dmin * m)."""


@kernel
def row_dequantize_q6_k(W: wl.View[ggml.Q6_K, (K,)], Y: wl.View[wl.f32, (K,)]):
    """Y = (d * f32(scale)) * f32(q - 32), two rounded multiplies."""


@kernel(alias_groups={"Y": "output"})
def row_dequantize_iq2_xxs(W: wl.View[ggml.IQ2_XXS, (K,)], grid: wl.View[wl.i8, (2048,)],
                           signs: wl.View[wl.i8, (1024,)], Y: wl.View[wl.f32, (K,)]):
    """Y = (d * (0.5 + s) * 0.25) * (grid[idx] * signs[sidx])."""


@kernel
def row_dequantize_iq2_xs(W: wl.View[ggml.IQ2_XS, (K,)], grid: wl.View[wl.i8, (4096,)],
                          signs: wl.View[wl.i8, (1024,)], Y: wl.View[wl.f32, (K,)]):
    """Y = (d * (0.5 + s) * 0.25) * (grid[idx] * signs[sidx]), s per 16 elements (examples/kernels/dequantize/iq2_xs.py:9-68)."""


@kernel(alias_groups={"Y": "output"})
def row_dequantize_iq3_xxs(W: wl.View[ggml.IQ3_XXS, (K,)], grid: wl.View[wl.i8, (1024,)],
                           signs: wl.View[wl.i8, (1024,)], Y: wl.View[wl.f32, (K,)]):
    """Y = (d * (0.5 + s) * 0.5) * (grid[idx] * signs[sidx]) (examples/kernels/dequantize/iq3_xxs.py:9-14)."""


@kernel(alias_groups={"Y": "output"})
def row_dequantize_iq2_s(W: wl.View[ggml.IQ2_S, (K,)], grid: wl.View[wl.i8, (8192,)], Y: wl.View[wl.f32, (K,)]):
    """Y = (d * (0.5 + s) * 0.25) * (grid[idx] * sign), s per 16 elements (examples/kernels/dequantize/iq2_s.py:9-13)."""


@kernel(alias_groups={"Y": "output"})
def row_dequantize_iq3_s(W: wl.View[ggml.IQ3_S, (K,)], grid: wl.View[wl.i8, (2048,)], Y: wl.View[wl.f32, (K,)]):
    """Y = (d * (1 + 2 s)) * (grid[idx] * sign), s per 32 elements (examples/kernels/dequantize/iq3_s.py:9-13)."""


@kernel(alias_groups={"Y": "output"})
def row_dequantize_iq1_s(W: wl.View[ggml.IQ1_S, (K,)], grid: wl.View[wl.i8, (16384,)], Y: wl.View[wl.f32, (K,)]):
    """Y = (d * (2 s + 1)) * (grid[idx] + delta), delta = +-0.125 per 32 elements (examples/kernels/dequantize/iq1_s.py:9-13)."""


@kernel(alias_groups={"Y": "output"})
def row_dequantize_iq1_m(W: wl.View[ggml.IQ1_M, (K,)], grid: wl.View[wl.i8, (16384,)], f16_bits: wl.View[wl.f32, (65536,)],
                         Y: wl.View[wl.f32, (K,)]):
    """As IQ1_S with per-16 scales, per-8 shift signs and the scale looked up in f16_bits (examples/kernels/dequantize/iq1_m.py:18-23)."""


@kernel(alias_groups={"Y": "output"})
def row_dequantize_tq1_0(W: wl.View[ggml.TQ1_0, (K,)], powers: wl.View[wl.u32, (5,)], Y: wl.View[wl.f32, (K,)]):
    """Y = f32(trit - 1) * d, digit-major within each of the record's three regions."""
