"""Whole-matrix forms of the per-row kernels (no counterpart in the reference).

The reference's standalone vec_dot / dequantize / quantize symbols take one row and its harnesses
loop over rows on the host (examples/repro/weft/vec_dot_runtime.cpp:468-475,
row_dequantize_runtime.cpp:433-438).  A launch per row is meaningless on a GPU, so the same CUDA
kernels are also reachable through these (N, K) definitions.
"""
from __future__ import annotations

from .. import formats as ggml
from .. import language as wl
from ..api import kernel


@kernel
def row_dequantize_q4_0_rows(W: wl.View[ggml.Q4_0, (N, K)], Y: wl.View[wl.f32, (N, K)]): ...


@kernel
def row_dequantize_q8_0_rows(W: wl.View[ggml.Q8_0, (N, K)], Y: wl.View[wl.f32, (N, K)]): ...


@kernel(alias_groups={"Y": "output"})
def row_dequantize_q4_k_rows(W: wl.View[ggml.Q4_K, (N, K)], Y: wl.View[wl.f32, (N, K)]): ...


@kernel(alias_groups={"Y": "output"})
def row_dequantize_q2_k_rows(W: wl.View[ggml.Q2_K, (N, K)], Y: wl.View[wl.f32, (N, K)]): ...


@kernel(alias_groups={"Y": "output"})
def row_dequantize_q3_k_rows(W: wl.View[ggml.Q3_K, (N, K)], Y: wl.View[wl.f32, (N, K)]): ...


@kernel(alias_groups={"Y": "output"})
def row_dequantize_q5_k_rows(W: wl.View[ggml.Q5_K, (N, K)], Y: wl.View[wl.f32, (N, K)]): ...


@kernel
def row_dequantize_q6_k_rows(W: wl.View[ggml.Q6_K, (N, K)], Y: wl.View[wl.f32, (N, K)]): ...


@kernel(alias_groups={"Y": "output"})
def row_dequantize_iq2_xxs_rows(W: wl.View[ggml.IQ2_XXS, (N, K)], grid: wl.View[wl.i8, (2048,)],
                                signs: wl.View[wl.i8, (1024,)], Y: wl.View[wl.f32, (N, K)]): ...


@kernel
def row_dequantize_iq2_xs_rows(W: wl.View[ggml.IQ2_XS, (N, K)], grid: wl.View[wl.i8, (4096,)],
                               signs: wl.View[wl.i8, (1024,)], Y: wl.View[wl.f32, (N, K)]): ...


@kernel(alias_groups={"Y": "output"})
def row_dequantize_iq3_xxs_rows(W: wl.View[ggml.IQ3_XXS, (N, K)], grid: wl.View[wl.i8, (1024,)],
                                signs: wl.View[wl.i8, (1024,)], Y: wl.View[wl.f32, (N, K)]): ...


@kernel(alias_groups={"Y": "output"})
def row_dequantize_iq2_s_rows(W: wl.View[ggml.IQ2_S, (N, K)], grid: wl.View[wl.i8, (8192,)], Y: wl.View[wl.f32, (N, K)]): ...


@kernel(alias_groups={"Y": "output"})
def row_dequantize_iq3_s_rows(W: wl.View[ggml.IQ3_S, (N, K)], grid: wl.View[wl.i8, (2048,)], Y: wl.View[wl.f32, (N, K)]): ...


@kernel(alias_groups={"Y": "output"})
def row_dequantize_iq1_s_rows(W: wl.View[ggml.IQ1_S, (N, K)], grid: wl.View[wl.i8, (16384,)], Y: wl.View[wl.f32, (N, K)]): ...


@kernel(alias_groups={"Y": "output"})
def row_dequantize_iq1_m_rows(W: wl.View[ggml.IQ1_M, (N, K)], grid: wl.View[wl.i8, (16384,)], f16_bits: wl.View[wl.f32, (65536,)],
                              Y: wl.View[wl.f32, (N, K)]): ...


@kernel(alias_groups={"Y": "output"})
def row_dequantize_tq1_0_rows(W: wl.View[ggml.TQ1_0, (N, K)], powers: wl.View[wl.u32, (5,)],
                              Y: wl.View[wl.f32, (N, K)]): ...


@kernel
def quantized_vec_dot_q4_0_q8_0_rows(W: wl.View[ggml.Q4_0, (N, K)], X: wl.View[ggml.Q8_0, (K,)], Y: wl.View[wl.f32, (N,)]): ...


@kernel
def quantized_vec_dot_q8_0_q8_0_rows(W: wl.View[ggml.Q8_0, (N, K)], X: wl.View[ggml.Q8_0, (K,)], Y: wl.View[wl.f32, (N,)]): ...


@kernel
def quantized_vec_dot_q4_k_q8_k_rows(W: wl.View[ggml.Q4_K, (N, K)], X: wl.View[ggml.Q8_K, (K,)], Y: wl.View[wl.f32, (N,)]): ...


@kernel
def quantized_vec_dot_q2_k_q8_k_rows(W: wl.View[ggml.Q2_K, (N, K)], X: wl.View[ggml.Q8_K, (K,)], Y: wl.View[wl.f32, (N,)]): ...


@kernel
def quantized_vec_dot_q3_k_q8_k_rows(W: wl.View[ggml.Q3_K, (N, K)], X: wl.View[ggml.Q8_K, (K,)], Y: wl.View[wl.f32, (N,)]): ...


@kernel
def quantized_vec_dot_q5_k_q8_k_rows(W: wl.View[ggml.Q5_K, (N, K)], X: wl.View[ggml.Q8_K, (K,)], Y: wl.View[wl.f32, (N,)]): ...


@kernel
def quantized_vec_dot_q6_k_q8_k_rows(W: wl.View[ggml.Q6_K, (N, K)], X: wl.View[ggml.Q8_K, (K,)], Y: wl.View[wl.f32, (N,)]): ...


@kernel
def quantized_vec_dot_iq2_xxs_q8_k_rows(W: wl.View[ggml.IQ2_XXS, (N, K)], X: wl.View[ggml.Q8_K, (K,)],
                                        grid: wl.View[ggml.I8X8, (256, 8)], signs: wl.View[ggml.I8X8, (128, 8)],
                                        Y: wl.View[wl.f32, (N,)]): ...


@kernel
def quantized_vec_dot_iq2_xs_q8_k_rows(W: wl.View[ggml.IQ2_XS, (N, K)], X: wl.View[ggml.Q8_K, (K,)],
                                       grid: wl.View[ggml.I8X8, (512, 8)], signs: wl.View[ggml.I8X8, (128, 8)],
                                       Y: wl.View[wl.f32, (N,)]): ...


@kernel
def quantized_vec_dot_iq3_xxs_q8_k_rows(W: wl.View[ggml.IQ3_XXS, (N, K)], X: wl.View[ggml.Q8_K, (K,)],
                                        grid: wl.View[ggml.I8X4, (256, 4)], signs: wl.View[ggml.I8X8, (128, 8)],
                                        Y: wl.View[wl.f32, (N,)]): ...


@kernel
def quantized_vec_dot_iq2_s_q8_k_rows(W: wl.View[ggml.IQ2_S, (N, K)], X: wl.View[ggml.Q8_K, (K,)],
                                      grid: wl.View[ggml.I8X8, (1024, 8)], Y: wl.View[wl.f32, (N,)]): ...


@kernel
def quantized_vec_dot_iq3_s_q8_k_rows(W: wl.View[ggml.IQ3_S, (N, K)], X: wl.View[ggml.Q8_K, (K,)],
                                      grid: wl.View[ggml.I8X4, (512, 4)], Y: wl.View[wl.f32, (N,)]): ...


@kernel
def quantized_vec_dot_iq1_s_q8_k_rows(W: wl.View[ggml.IQ1_S, (N, K)], X: wl.View[ggml.Q8_K, (K,)],
                                      grid: wl.View[ggml.I8X8, (2048, 8)], Y: wl.View[wl.f32, (N,)]): ...


@kernel
def quantized_vec_dot_iq1_m_q8_k_rows(W: wl.View[ggml.IQ1_M, (N, K)], X: wl.View[ggml.Q8_K, (K,)],
                                      grid: wl.View[ggml.I8X8, (2048, 8)], f16_bits: wl.View[wl.f32, (65536,)],
                                      Y: wl.View[wl.f32, (N,)]): ...


@kernel
def quantized_vec_dot_tq1_0_q8_k_rows(W: wl.View[ggml.TQ1_0, (N, K)], X: wl.View[ggml.Q8_K, (K,)],
                                      powers: wl.View[wl.u32, (5,)], Y: wl.View[wl.f32, (N,)]): ...


@kernel
def q8_0_quantize_rows(X: wl.View[wl.f32, (M, K)], Y: wl.View[ggml.Q8_0, (M, K)]): ...


@kernel
def q8_1_quantize_rows(X: wl.View[wl.f32, (M, K)], Y: wl.View[ggml.Q8_1, (M, K)]): ...


@kernel
def q8_K_quantize_rows(X: wl.View[wl.f32, (M, K)], Y: wl.View[ggml.Q8_K, (M, K)]): ...
