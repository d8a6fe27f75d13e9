"""Which kernel definitions this build can execute, and how each maps onto its C symbol.

The reference lowers any DSL body; this build carries hand-written CUDA for a fixed set of kernels
and refuses everything else explicitly (NotImplementedError) -- there is no generic or CPU fallback.
A definition is accepted when its name is known and its signature is the known one up to renaming of
shape symbols: same argument count and order, same Encoding identities and record geometry, same
ranks, and the same pattern of shared extents.
"""
from __future__ import annotations

from . import kernels
from .api import KernelDefinition
from .signature import kernel_abi

_MODULES = (kernels.vec_dot, kernels.dequantize, kernels.quantize, kernels.mul_mat, kernels.gemv, kernels.rows)

#: C symbols whose trailing size_t extents are not in first-appearance order of the signature: the builder of a
#: derived Encoding declares its own extents first (examples/repro/weft/mul_mat_runtime.cpp:337-348)
_C_ORDER = {"production_mul_mat_q4_k_persistent": ["M", "K", "N"]}


def _access(symbol: str, name: str) -> str:
    if name == "Y":
        return "readwrite" if symbol == "production_mul_mat_q4_k_staged" else "write"
    if name == "Xq":
        return "readwrite"
    return "read"


def _canonical() -> dict[str, dict]:
    table = {}
    for module in _MODULES:
        for value in vars(module).values():
            if isinstance(value, KernelDefinition):
                abi = kernel_abi(value)
                for argument in abi["arguments"]:
                    argument["access"] = _access(abi["symbol"], argument["name"])
                    argument["writable"] = argument["access"] != "read"
                table[abi["symbol"]] = abi
    return table


CANONICAL = _canonical()


def supported_symbols() -> list[str]:
    return sorted(CANONICAL)


def resolve(definition: KernelDefinition) -> dict:
    """Kernel metadata for ``definition`` (arguments with access modes, shape parameters in the
    definition's own order, ``c_dimension_order`` naming them in the C symbol's order)."""
    symbol = definition.__name__
    known = CANONICAL.get(symbol)
    if known is None:
        raise NotImplementedError(
            f"kernel {symbol} has no sm_100a implementation in this build; supported: {', '.join(supported_symbols())}")
    given = kernel_abi(definition)
    if len(given["arguments"]) != len(known["arguments"]):
        raise TypeError(f"{symbol} takes {len(known['arguments'])} arguments, the definition declares {len(given['arguments'])}")
    rename: dict[str, str] = {}
    for mine, theirs in zip(known["arguments"], given["arguments"]):
        if theirs["encoding"] != mine["encoding"]:
            raise TypeError(f"{symbol}: parameter {theirs['name']} is {theirs['encoding']}, the kernel takes {mine['encoding']}")
        if (theirs["storage_bytes"], theirs["record_elements"]) != (mine["storage_bytes"], mine["record_elements"]):
            raise TypeError(f"{symbol}: Encoding {theirs['encoding']} of {theirs['name']} has a different record geometry")
        if len(theirs["shape"]) != len(mine["shape"]):
            raise TypeError(f"{symbol}: parameter {theirs['name']} has rank {len(theirs['shape'])}, the kernel takes {len(mine['shape'])}")
        for a, b in zip(mine["shape"], theirs["shape"]):
            if a.isdecimal() or b.isdecimal():
                if a != b:
                    raise TypeError(f"{symbol}: parameter {theirs['name']} has extent {b} where the kernel takes {a}")
            elif rename.setdefault(a, b) != b:
                raise TypeError(f"{symbol}: extent {b} of {theirs['name']} breaks the kernel's shape pattern")
    if len(set(rename.values())) != len(rename):
        raise TypeError(f"{symbol}: distinct kernel extents are tied together in the definition")
    arguments = []
    for mine, theirs in zip(known["arguments"], given["arguments"]):
        merged = dict(theirs)
        merged["alignment"] = max(theirs["alignment"], 1)
        merged["writable"] = mine["writable"]
        merged["access"] = mine["access"]
        arguments.append(merged)
    return {"symbol": symbol, "arguments": arguments, "shape_parameters": given["shape_parameters"],
            "c_dimension_order": [rename[name] for name in _C_ORDER.get(symbol, known["shape_parameters"])]}
