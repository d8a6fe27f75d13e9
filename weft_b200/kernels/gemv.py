"""q4_k_q8_k_gemv: Y[m] = quantized_vec_dot_q4_k_q8_k(W[m], X) over the persistent interleaved weight
layout ``Q4K_I[16]`` (examples/kernels/gemv/q4_k.py:8-26).  Rows are computed in cohorts of 16; the float
op tree per 256-block is ``x.ds * (w.d * i32_acc - w.dmin * min_term)`` as in the plain vec_dot.
C symbol and artifact functions (examples/repro/weft/q4_k_gemv_runtime.cpp:28-32):
``q4_k_q8_k_gemv(W, X, Y, M, K)``, ``q4_k_q8_k_gemv_W_packed_size(M, K)``, ``q4_k_q8_k_gemv_W_pack(source, target, M, K)``.
"""
from __future__ import annotations

from .. import formats as ggml
from .. import language as wl
from ..api import kernel


@kernel
def q4_k_q8_k_gemv(W: wl.View[ggml.Q4K_I[16], (M, K)], X: wl.View[ggml.Q8_K, (K,)], Y: wl.View[wl.f32, (M,)]):
    """GEMV, 16-row interleaved Q4_K weights x one Q8_K activation row."""


@kernel
def q4_k_q8_k_gemv_groups4(W: wl.View[ggml.Q4K_I[16], (M, K)], X: wl.View[ggml.Q8_K, (K,)], Y: wl.View[wl.f32, (M,)]):
    """The same GEMV with four 16-bit partial groups per sub-block in the reference's vector plan
    (examples/kernels/gemv/q4_k_groups4.py:8-27): identical integer sums and float op tree, one CUDA kernel for both."""


@kernel
def q4_k_q8_k_gemv_contract(W: wl.View[ggml.Q4K_I[16], (M, K)], X: wl.View[ggml.Q8_K, (K,)], Y: wl.View[wl.f32, (M,)]):
    """The same GEMV with one 32-bit contraction per sub-block, the form the reference gives its matrix unit
    (examples/kernels/gemv/q4_k_contract.py:8-27): identical results, one CUDA kernel for all three names."""
