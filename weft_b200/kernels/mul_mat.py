"""production_mul_mat_*: quantize X into the Xq workspace, then Y[m, n] = vec_dot(W[n], Xq[m]).

Signatures and alias groups follow the reference: examples/kernels/mul_mat/q4_0_decode.py:10-20,
q8_0_decode.py, q4_k_decode.py:10-20, q2_k_decode.py:10-20, q3_k_decode.py:10-20, q5_k_decode.py:10-20, q6_k_decode.py:10-20, iq2_xxs_decode.py:10-23, tq1_0_decode.py:10-21 (decode: a GEMV
per activation row) and q4_0.py:9-30, q8_0.py:9-29, q4_k_staged.py:9-37, q2_k.py:9-41, q3_k.py:9-61, q5_k.py:9-37, q6_k.py:9-37, tq1_0.py:10-64,
iq2_xxs_staged.py:9-97 (prefill: tiled contraction).  The reference's tile symbols NC/MC/MR/NR/KC are
bound through CompileOptions.meta and are not call parameters.
"""
from __future__ import annotations

from .. import formats as ggml
from .. import language as wl
from ..api import kernel


@kernel
def production_mul_mat_q4_0_decode(W: wl.View[ggml.Q4_0, (N, K)], X: wl.View[wl.f32, (M, K)],
                                   Xq: wl.View[ggml.Q8_0, (M, K)], Y: wl.View[wl.f32, (M, N)]):
    """Decode GEMV, Q4_0 weights x Q8_0 activations."""


@kernel
def production_mul_mat_q8_0_decode(W: wl.View[ggml.Q8_0, (N, K)], X: wl.View[wl.f32, (M, K)],
                                   Xq: wl.View[ggml.Q8_0, (M, K)], Y: wl.View[wl.f32, (M, N)]):
    """Decode GEMV, Q8_0 weights x Q8_0 activations."""


@kernel(alias_groups={"Xq": "workspace", "Y": "output"})
def production_mul_mat_q4_k_decode(W: wl.View[ggml.Q4_K, (N, K)], X: wl.View[wl.f32, (M, K)],
                                   Xq: wl.View[ggml.Q8_K, (M, K)], Y: wl.View[wl.f32, (M, N)]):
    """Decode GEMV, Q4_K weights x Q8_K activations."""


@kernel(alias_groups={"Xq": "workspace", "Y": "output"})
def production_mul_mat_q2_k_decode(W: wl.View[ggml.Q2_K, (N, K)], X: wl.View[wl.f32, (M, K)],
                                   Xq: wl.View[ggml.Q8_K, (M, K)], Y: wl.View[wl.f32, (M, N)]):
    """Decode GEMV, Q2_K weights x Q8_K activations."""


@kernel
def production_mul_mat_q2_k(W: wl.View[ggml.Q2_K, (N, K)], X: wl.View[wl.f32, (M, K)],
                            Xq: wl.View[ggml.Q8_K, (M, K)], Y: wl.View[wl.f32, (M, N)]):
    """Tiled contraction in the reference; here the decode GEMV per activation row."""


@kernel
def production_mul_mat_q3_k_decode(W: wl.View[ggml.Q3_K, (N, K)], X: wl.View[wl.f32, (M, K)],
                                   Xq: wl.View[ggml.Q8_K, (M, K)], Y: wl.View[wl.f32, (M, N)]):
    """Decode GEMV, Q3_K weights x Q8_K activations."""


@kernel
def production_mul_mat_q3_k(W: wl.View[ggml.Q3_K, (N, K)], X: wl.View[wl.f32, (M, K)],
                            Xq: wl.View[ggml.Q8_K, (M, K)], Y: wl.View[wl.f32, (M, N)]):
    """Tiled contraction in the reference; here the decode GEMV per activation row."""


@kernel
def production_mul_mat_q5_k_decode(W: wl.View[ggml.Q5_K, (N, K)], X: wl.View[wl.f32, (M, K)],
                                   Xq: wl.View[ggml.Q8_K, (M, K)], Y: wl.View[wl.f32, (M, N)]):
    """Decode GEMV, Q5_K weights x Q8_K activations."""


@kernel
def production_mul_mat_q5_k(W: wl.View[ggml.Q5_K, (N, K)], X: wl.View[wl.f32, (M, K)],
                            Xq: wl.View[ggml.Q8_K, (M, K)], Y: wl.View[wl.f32, (M, N)]):
    """Tiled contraction in the reference; here the decode GEMV per activation row."""


@kernel
def production_mul_mat_q6_k_decode(W: wl.View[ggml.Q6_K, (N, K)], X: wl.View[wl.f32, (M, K)],
                                   Xq: wl.View[ggml.Q8_K, (M, K)], Y: wl.View[wl.f32, (M, N)]):
    """Decode GEMV, Q6_K weights x Q8_K activations."""


@kernel(alias_groups={"Xq": "workspace", "Y": "output"})
def production_mul_mat_q6_k(W: wl.View[ggml.Q6_K, (N, K)], X: wl.View[wl.f32, (M, K)],
                            Xq: wl.View[ggml.Q8_K, (M, K)], Y: wl.View[wl.f32, (M, N)]):
    """Tiled contraction in the reference; here the decode GEMV per activation row."""


@kernel(alias_groups={"Xq": "workspace", "Y": "output"})
def production_mul_mat_iq2_xxs_decode(W: wl.View[ggml.IQ2_XXS, (N, K)], X: wl.View[wl.f32, (M, K)],
                                      Xq: wl.View[ggml.Q8_K, (M, K)], grid: wl.View[ggml.I8X8, (256, 8)],
                                      signs: wl.View[ggml.I8X8, (128, 8)], Y: wl.View[wl.f32, (M, N)]):
    """Decode GEMV, IQ2_XXS codebook weights x Q8_K activations."""


@kernel
def production_mul_mat_tq1_0_decode(W: wl.View[ggml.TQ1_0, (N, K)], X: wl.View[wl.f32, (M, K)],
                                    Xq: wl.View[ggml.Q8_K, (M, K)], powers: wl.View[wl.u32, (5,)],
                                    Y: wl.View[wl.f32, (M, N)]):
    """Decode GEMV, TQ1_0 ternary weights x Q8_K activations."""


@kernel(alias_groups={"Xq": "workspace", "Y": "output"})
def production_mul_mat_tq1_0_lane16_decode(W: wl.View[ggml.TQ1_0, (N, K)], X: wl.View[wl.f32, (M, K)],
                                           Xq: wl.View[ggml.Q8_K, (M, K)], powers: wl.View[wl.u32, (5,)],
                                           Y: wl.View[wl.f32, (M, N)]):
    """Decode GEMV over the lane16 statement of the TQ1_0 dot product
    (examples/kernels/mul_mat/tq1_0_lane16_decode.py:10-23): same function as production_mul_mat_tq1_0_decode."""


@kernel
def production_mul_mat_q3_k_predecoded_scales_decode(W: wl.View[ggml.Q3_K, (N, K)], X: wl.View[wl.f32, (M, K)],
                                                     Xq: wl.View[ggml.Q8_K, (M, K)], Y: wl.View[wl.f32, (M, N)]):
    """Decode GEMV, Q3_K x Q8_K, under the name of the reference plan that decodes a record's scales ahead of its
    inner loop (examples/kernels/mul_mat/q3_k_predecoded_scales_decode.py:10-21)."""


@kernel
def production_mul_mat_q3_k_predecoded_scales(W: wl.View[ggml.Q3_K, (N, K)], X: wl.View[wl.f32, (M, K)],
                                              Xq: wl.View[ggml.Q8_K, (M, K)], Y: wl.View[wl.f32, (M, N)]):
    """Tiled form of the same (examples/kernels/mul_mat/q3_k_predecoded_scales.py:10-61)."""


@kernel
def production_mul_mat_q4_0(W: wl.View[ggml.Q4_0, (N, K)], X: wl.View[wl.f32, (M, K)],
                            Xq: wl.View[ggml.Q8_0, (M, K)], Y: wl.View[wl.f32, (M, N)]):
    """Prefill contraction, Q4_0 x Q8_0."""


@kernel
def production_mul_mat_q8_0(W: wl.View[ggml.Q8_0, (N, K)], X: wl.View[wl.f32, (M, K)],
                            Xq: wl.View[ggml.Q8_0, (M, K)], Y: wl.View[wl.f32, (M, N)]):
    """Prefill contraction, Q8_0 x Q8_0."""


@kernel
def production_mul_mat_q4_k_staged(W: wl.View[ggml.Q4_K, (N, K)], X: wl.View[wl.f32, (M, K)],
                                   Xq: wl.View[ggml.Q8_K, (M, K)], Y: wl.View[wl.f32, (M, N)]):
    """Prefill contraction, Q4_K x Q8_K, int8 tensor cores."""


@kernel(alias_groups={"Xq": "workspace", "Y": "output"})
def production_mul_mat_tq1_0(W: wl.View[ggml.TQ1_0, (N, K)], X: wl.View[wl.f32, (M, K)],
                             Xq: wl.View[ggml.Q8_K, (M, K)], powers: wl.View[wl.u32, (5,)],
                             Y: wl.View[wl.f32, (M, N)]):
    """Prefill contraction, TQ1_0 x Q8_K, int8 tensor cores."""


@kernel(alias_groups={"Xq": "workspace", "Y": "output"})
def production_mul_mat_iq2_xxs_staged(W: wl.View[ggml.IQ2_XXS, (N, K)], X: wl.View[wl.f32, (M, K)],
                                      Xq: wl.View[ggml.Q8_K, (M, K)], grid: wl.View[ggml.I8X8, (256, 8)],
                                      signs: wl.View[ggml.I8X8, (128, 8)], Y: wl.View[wl.f32, (M, N)]):
    """Prefill form, IQ2_XXS x Q8_K."""


@kernel
def production_mul_mat_iq2_xxs(W: wl.View[ggml.IQ2_XXS, (N, K)], X: wl.View[wl.f32, (M, K)],
                               Xq: wl.View[ggml.Q8_K, (M, K)], grid: wl.View[ggml.I8X8, (256, 8)],
                               signs: wl.View[ggml.I8X8, (128, 8)], Y: wl.View[wl.f32, (M, N)]):
    """IQ2_XXS x Q8_K mul_mat (examples/kernels/mul_mat/iq2_xxs.py:10-17): the function of the staged form."""


@kernel(alias_groups={"Xq": "workspace", "Y": "output"})
def production_mul_mat_iq2_xs(W: wl.View[ggml.IQ2_XS, (N, K)], X: wl.View[wl.f32, (M, K)],
                              Xq: wl.View[ggml.Q8_K, (M, K)], grid: wl.View[ggml.I8X8, (512, 8)],
                              signs: wl.View[ggml.I8X8, (128, 8)], Y: wl.View[wl.f32, (M, N)]):
    """IQ2_XS x Q8_K mul_mat (examples/kernels/mul_mat/iq2_xs.py:26-33)."""


@kernel
def production_mul_mat_iq2_xs_staged(W: wl.View[ggml.IQ2_XS, (N, K)], X: wl.View[wl.f32, (M, K)],
                                     Xq: wl.View[ggml.Q8_K, (M, K)], grid: wl.View[wl.i8, (4096,)],
                                     signs: wl.View[wl.i8, (1024,)], Y: wl.View[wl.f32, (M, N)]):
    """The same with the tables as flat byte arrays (examples/kernels/mul_mat/iq2_xs_staged.py:29-36)."""


@kernel(alias_groups={"Xq": "workspace", "Y": "output"})
def production_mul_mat_iq3_xxs(W: wl.View[ggml.IQ3_XXS, (N, K)], X: wl.View[wl.f32, (M, K)],
                               Xq: wl.View[ggml.Q8_K, (M, K)], grid: wl.View[ggml.I8X4, (256, 4)],
                               signs: wl.View[ggml.I8X8, (128, 8)], Y: wl.View[wl.f32, (M, N)]):
    """IQ3_XXS x Q8_K mul_mat (examples/kernels/mul_mat/iq3_xxs.py:10-17)."""


@kernel
def production_mul_mat_iq2_s(W: wl.View[ggml.IQ2_S, (N, K)], X: wl.View[wl.f32, (M, K)], Xq: wl.View[ggml.Q8_K, (M, K)],
                             grid: wl.View[ggml.I8X8, (1024, 8)], Y: wl.View[wl.f32, (M, N)]):
    """IQ2_S x Q8_K mul_mat (examples/kernels/mul_mat/iq2_s.py:10-16)."""


@kernel
def production_mul_mat_iq2_s_staged(W: wl.View[ggml.IQ2_S, (N, K)], X: wl.View[wl.f32, (M, K)], Xq: wl.View[ggml.Q8_K, (M, K)],
                                    grid: wl.View[wl.i8, (8192,)], Y: wl.View[wl.f32, (M, N)]):
    """The same with the grid as a flat byte array (examples/kernels/mul_mat/iq2_s_staged.py:29-35)."""


@kernel(alias_groups={"Xq": "workspace", "Y": "output"})
def production_mul_mat_iq3_s(W: wl.View[ggml.IQ3_S, (N, K)], X: wl.View[wl.f32, (M, K)], Xq: wl.View[ggml.Q8_K, (M, K)],
                             grid: wl.View[ggml.I8X4, (512, 4)], Y: wl.View[wl.f32, (M, N)]):
    """IQ3_S x Q8_K mul_mat (examples/kernels/mul_mat/iq3_s.py:10-16)."""


@kernel(alias_groups={"Xq": "workspace", "Y": "output"})
def production_mul_mat_iq1_s(W: wl.View[ggml.IQ1_S, (N, K)], X: wl.View[wl.f32, (M, K)], Xq: wl.View[ggml.Q8_K, (M, K)],
                             grid: wl.View[ggml.I8X8, (2048, 8)], Y: wl.View[wl.f32, (M, N)]):
    """IQ1_S x Q8_K mul_mat (examples/kernels/mul_mat/iq1_s.py:9-15)."""


@kernel(alias_groups={"Xq": "workspace", "Y": "output"})
def production_mul_mat_iq1_s_decode(W: wl.View[ggml.IQ1_S, (N, K)], X: wl.View[wl.f32, (M, K)], Xq: wl.View[ggml.Q8_K, (M, K)],
                                    grid: wl.View[ggml.I8X8, (2048, 8)], Y: wl.View[wl.f32, (M, N)]):
    """Decode GEMV, IQ1_S (examples/kernels/mul_mat/iq1_s_decode.py:10-16)."""


@kernel
def production_mul_mat_iq1_m(W: wl.View[ggml.IQ1_M, (N, K)], X: wl.View[wl.f32, (M, K)], Xq: wl.View[ggml.Q8_K, (M, K)],
                             grid: wl.View[ggml.I8X8, (2048, 8)], f16_bits: wl.View[wl.f32, (65536,)], Y: wl.View[wl.f32, (M, N)]):
    """IQ1_M x Q8_K mul_mat (examples/kernels/mul_mat/iq1_m.py:10-17)."""


@kernel(alias_groups={"Xq": "workspace", "Y": "output"})
def production_mul_mat_iq1_m_decode(W: wl.View[ggml.IQ1_M, (N, K)], X: wl.View[wl.f32, (M, K)], Xq: wl.View[ggml.Q8_K, (M, K)],
                                    grid: wl.View[ggml.I8X8, (2048, 8)], f16_bits: wl.View[wl.f32, (65536,)], Y: wl.View[wl.f32, (M, N)]):
    """Decode GEMV, IQ1_M (examples/kernels/mul_mat/iq1_m_decode.py:10-17)."""


@kernel
def production_mul_mat_iq1_m_lane16_decode(W: wl.View[ggml.IQ1_M, (N, K)], X: wl.View[wl.f32, (M, K)], Xq: wl.View[ggml.Q8_K, (M, K)],
                                           grid: wl.View[ggml.I8X8, (2048, 8)], f16_bits: wl.View[wl.f32, (65536,)], Y: wl.View[wl.f32, (M, N)]):
    """The same under the name of the reference's sixteen-wide plan (examples/kernels/mul_mat/iq1_m_lane16_decode.py:10-17)."""


@kernel
def production_mul_mat_q4_k_persistent(W: wl.View[ggml.Q4K_I[16], (N, K)], X: wl.View[wl.f32, (M, K)],
                                       Xq: wl.View[ggml.Q8_K, (M, K)], Y: wl.View[wl.f32, (M, N)]):
    """Q4_K x Q8_K over the persistent interleaved layout (examples/kernels/mul_mat/q4_k_persistent.py:9-30).
    The C symbol takes its extents as (M, K, N): the derived Encoding's builder declares M and K first
    (examples/repro/weft/mul_mat_runtime.cpp:337-348)."""
