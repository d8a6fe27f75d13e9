"""``@weft.kernel`` definitions of the quantized matrix path, one per exported C symbol.

The names, parameter names, View annotations and alias groups are those of the reference's kernel
files (examples/kernels/{vec_dot,dequantize,quantize,mul_mat,gemv}/*.py), so either set of definitions
can be handed to ``weft.compile``.  The bodies here are documentation only: the arithmetic lives in
the CUDA kernels under ``weft_b200/csrc`` and is selected by symbol and signature.
"""
from . import dequantize, gemv, mul_mat, quantize, rows, vec_dot  # noqa: F401
