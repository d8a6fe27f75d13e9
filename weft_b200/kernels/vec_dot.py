"""Block dot products: one weight row against one activation row, one fp32 result.

Signatures follow examples/kernels/vec_dot/q4_0_q8_0.py:18-23, q8_0_q8_0.py:17-22, q4_k_q8_k.py:31-36,
q2_k_q8_k.py:28-32, q3_k_q8_k.py:46-50, q5_k_q8_k.py:34-38, q6_k_q8_k.py:39-43, iq2_xxs_q8_k.py:45-54 and tq1_0_q8_k.py:47-55 of the reference.
"""
from __future__ import annotations

from .. import formats as ggml
from .. import language as wl
from ..api import kernel


@kernel
def quantized_vec_dot_q4_0_q8_0(W: wl.View[ggml.Q4_0, (K,)], X: wl.View[ggml.Q8_0, (K,)], Y: wl.View[wl.f32, (1,)]):
    """Y[0] = sum over 32-blocks of f32(d_w) * f32(d_x) * f32(sum((q - 8) * x))."""


@kernel
def quantized_vec_dot_q8_0_q8_0(W: wl.View[ggml.Q8_0, (K,)], X: wl.View[ggml.Q8_0, (K,)], Y: wl.View[wl.f32, (1,)]):
    """Y[0] = sum over 32-blocks of f32(sum(w * x)) * (f32(d_w) * f32(d_x))."""


@kernel
def quantized_vec_dot_q4_k_q8_k(W: wl.View[ggml.Q4_K, (K,)], X: wl.View[ggml.Q8_K, (K,)], Y: wl.View[wl.f32, (1,)]):
    """Y[0] = sum over 256-blocks of x.ds * (d * sum_g sc_g * dot32_g - dmin * sum_g m_g * (bsum_2g + bsum_2g+1))."""


@kernel
def quantized_vec_dot_q2_k_q8_k(W: wl.View[ggml.Q2_K, (K,)], X: wl.View[ggml.Q8_K, (K,)], Y: wl.View[wl.f32, (1,)]):
    """Y[0] = sum over 256-blocks of x.ds * (d * sum_g (scales_g & 15) * dot16_g - dmin * sum_g (scales_g >> 4) * bsum_g)."""


@kernel
def quantized_vec_dot_q3_k_q8_k(W: wl.View[ggml.Q3_K, (K,)], X: wl.View[ggml.Q8_K, (K,)], Y: wl.View[wl.f32, (1,)]):
    """Y[0] = sum over 256-blocks of d * x.ds * f32(sum_g (scale_g - 32) * dot16_g(q3 - 4, x))."""


@kernel
def quantized_vec_dot_q5_k_q8_k(W: wl.View[ggml.Q5_K, (K,)], X: wl.View[ggml.Q8_K, (K,)], Y: wl.View[wl.f32, (1,)]):
    """As Q4_K with 5-bit weights: q = nibble | fifth bit << 4."""


@kernel
def quantized_vec_dot_q6_k_q8_k(W: wl.View[ggml.Q6_K, (K,)], X: wl.View[ggml.Q8_K, (K,)], Y: wl.View[wl.f32, (1,)]):
    """Y[0] = sum over 256-blocks of d * x.ds * f32(sum_g scales_g * dot16_g(q - 32, x))."""


@kernel
def quantized_vec_dot_iq2_xxs_q8_k(W: wl.View[ggml.IQ2_XXS, (K,)], X: wl.View[ggml.Q8_K, (K,)],
                                   grid: wl.View[ggml.I8X8, (256, 8)], signs: wl.View[ggml.I8X8, (128, 8)],
                                   Y: wl.View[wl.f32, (1,)]):
    """Y[0] = 0.125 * sum over 256-blocks of d * x.ds * sum_g (2 s_g + 1) * dot(grid[idx] * signs[sidx], x)."""


@kernel
def quantized_vec_dot_iq2_xs_q8_k(W: wl.View[ggml.IQ2_XS, (K,)], X: wl.View[ggml.Q8_K, (K,)],
                                  grid: wl.View[ggml.I8X8, (512, 8)], signs: wl.View[ggml.I8X8, (128, 8)],
                                  Y: wl.View[wl.f32, (1,)]):
    """Y[0] = 0.125 * sum over 256-blocks of d * x.ds * sum over 16-element halves (2 s + 1) * dot(grid[idx] * signs[sidx], x)
    (examples/kernels/vec_dot/iq2_xs_q8_k.py:9-39)."""


@kernel
def quantized_vec_dot_iq3_xxs_q8_k(W: wl.View[ggml.IQ3_XXS, (K,)], X: wl.View[ggml.Q8_K, (K,)],
                                   grid: wl.View[ggml.I8X4, (256, 4)], signs: wl.View[ggml.I8X8, (128, 8)],
                                   Y: wl.View[wl.f32, (1,)]):
    """Y[0] = 0.25 * sum over 256-blocks of d * x.ds * sum_g (2 s_g + 1) * dot(grid[idx] * signs[sidx], x)
    (examples/kernels/vec_dot/iq3_xxs_q8_k.py:70-76)."""


@kernel
def quantized_vec_dot_iq2_s_q8_k(W: wl.View[ggml.IQ2_S, (K,)], X: wl.View[ggml.Q8_K, (K,)],
                                 grid: wl.View[ggml.I8X8, (1024, 8)], Y: wl.View[wl.f32, (1,)]):
    """As IQ2_XS with 10-bit grid indices and sign bits stored in the record (examples/kernels/vec_dot/iq2_s_q8_k.py:68-73)."""


@kernel
def quantized_vec_dot_iq3_s_q8_k(W: wl.View[ggml.IQ3_S, (K,)], X: wl.View[ggml.Q8_K, (K,)],
                                 grid: wl.View[ggml.I8X4, (512, 4)], Y: wl.View[wl.f32, (1,)]):
    """Y[0] = sum over 256-blocks of d * x.ds * sum_g (2 s_g + 1) * dot(grid[idx] * sign, x)
    (examples/kernels/vec_dot/iq3_s_q8_k.py:67-72)."""


@kernel
def quantized_vec_dot_iq1_s_q8_k(W: wl.View[ggml.IQ1_S, (K,)], X: wl.View[ggml.Q8_K, (K,)],
                                 grid: wl.View[ggml.I8X8, (2048, 8)], Y: wl.View[wl.f32, (1,)]):
    """Y[0] = sum over 256-blocks of d * x.ds * (sum_g (2 s_g + 1) dot(grid[idx], x) + 0.125 sum_g (2 s_g + 1) (+-1) bsum32_g)
    (examples/kernels/vec_dot/iq1_s_q8_k.py:51-56)."""


@kernel
def quantized_vec_dot_iq1_m_q8_k(W: wl.View[ggml.IQ1_M, (K,)], X: wl.View[ggml.Q8_K, (K,)],
                                 grid: wl.View[ggml.I8X8, (2048, 8)], f16_bits: wl.View[wl.f32, (65536,)],
                                 Y: wl.View[wl.f32, (1,)]):
    """As IQ1_S with a scale per 16 weights, a shift sign per 8 and the record's f16 scale spread over four u16
    (examples/kernels/vec_dot/iq1_m_q8_k.py:73-79)."""


@kernel
def quantized_vec_dot_iq1_m_q8_k_lane16(W: wl.View[ggml.IQ1_M, (K,)], X: wl.View[ggml.Q8_K, (K,)],
                                        grid: wl.View[ggml.I8X8, (2048, 8)], f16_bits: wl.View[wl.f32, (65536,)],
                                        Y: wl.View[wl.f32, (1,)]):
    """The same dot product under the name of the reference's sixteen-wide plan (examples/kernels/vec_dot/iq1_m_q8_k_lane16.py:85-91)."""


@kernel
def quantized_vec_dot_tq1_0_q8_k(W: wl.View[ggml.TQ1_0, (K,)], X: wl.View[ggml.Q8_K, (K,)],
                                 powers: wl.View[wl.u32, (5,)], Y: wl.View[wl.f32, (1,)]):
    """Y[0] = sum over 256-blocks of f32(sum((trit - 1) * x)) * (d * x.ds); trits decoded with powers[]."""


@kernel
def quantized_vec_dot_tq1_0_q8_k_lane16(W: wl.View[ggml.TQ1_0, (K,)], X: wl.View[ggml.Q8_K, (K,)],
                                        powers: wl.View[wl.u32, (5,)], Y: wl.View[wl.f32, (1,)]):
    """The TQ1_0 dot product as the reference states it for sixteen-wide partial sums
    (examples/kernels/vec_dot/tq1_0_q8_k_lane16.py:9-54): the per-block integer sum is the same, so is every result."""
