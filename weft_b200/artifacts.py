"""Artifact functions of kernels that take a derived (persistent) Encoding.

For a kernel with a ``Family[p]`` parameter the reference emits, next to the kernel itself,
``<kernel>_<param>_packed_size(rows, K)`` and ``<kernel>_<param>_pack(source, target, rows, K)``
(lib/Target/Emission/Emitter.h:231-272); a model loader calls them once and keeps the packed object
(examples/repro/weft/q4_k_gemv_runtime.cpp:243-247).  Its Python runtime has no wrapper for them; this
module is the thin one this build adds.  Source and target may be host or device buffers.
"""
from __future__ import annotations

import ctypes

from .api import KernelDefinition
from .registry import resolve
from .runtime.buffer import Buffer
from .runtime.driver import Toolchain, last_error, load_library


def _functions(definition: KernelDefinition, parameter: str):
    metadata = resolve(definition)
    argument = next((a for a in metadata["arguments"] if a["name"] == parameter), None)
    if argument is None or "[" not in argument["encoding"]:
        raise TypeError(f"{metadata['symbol']} has no derived-Encoding parameter {parameter}")
    lib = load_library(Toolchain().resolve().compiler)
    size = getattr(lib, f"{metadata['symbol']}_{parameter}_packed_size")
    pack = getattr(lib, f"{metadata['symbol']}_{parameter}_pack")
    size.argtypes = [ctypes.c_size_t, ctypes.c_size_t]
    size.restype = ctypes.c_size_t
    pack.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_size_t]
    pack.restype = ctypes.c_int
    return lib, size, pack, argument


def packed_size(definition: KernelDefinition, rows: int, k: int, parameter: str = "W") -> int:
    """Bytes of the packed object for a (rows, k) source; 0 when the shape has no packed form."""
    _, size, _, _ = _functions(definition, parameter)
    return int(size(rows, k))


def pack(definition: KernelDefinition, source: object, target: object, rows: int, k: int, parameter: str = "W") -> None:
    """Write the persistent layout of the (rows, k) base-Encoding records ``source`` into ``target``."""
    lib, size, pack_fn, _ = _functions(definition, parameter)
    need = int(size(rows, k))
    if need == 0 and rows and k:
        raise ValueError(f"({rows}, {k}) has no packed form: rows must be whole cohorts and K whole records")
    src = source if isinstance(source, Buffer) else Buffer(source)
    dst = target if isinstance(target, Buffer) else Buffer(target)
    if src.nbytes < need or dst.nbytes < need:
        raise ValueError(f"packing ({rows}, {k}) needs {need} bytes of source and of target")
    if dst.readonly:
        raise TypeError("the pack target must be writable")
    if pack_fn(src.address, dst.address, rows, k):
        raise RuntimeError(f"pack failed: {last_error(lib)}")
