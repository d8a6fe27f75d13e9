"""Activation quantizers (examples/kernels/quantize/q8_0.py:20-23, q8_1.py:28-30, q8_k.py:32-35 of the reference)."""
from __future__ import annotations

from .. import formats as ggml
from .. import language as wl
from ..api import kernel


@kernel
def q8_0_quantize(X: wl.View[wl.f32, (K,)], Y: wl.View[ggml.Q8_0, (K,)]):
    """Per 32: d = amax / 127 (f16), q = rne(x / d) clamped to int8."""


@kernel
def q8_1_quantize(X: wl.View[wl.f32, (K,)], Y: wl.View[ggml.Q8_1, (K,)]):
    """Q8_0 plus s = f16(f32(sum of the 32 codes) * d) stored after d."""


@kernel
def q8_K_quantize(X: wl.View[wl.f32, (K,)], Y: wl.View[ggml.Q8_K, (K,)]):
    """Per 256: extreme = |max| > |min| ? max : min; q = rne(x * (-127 / extreme)); bsum per 16; ds = extreme / -127."""
