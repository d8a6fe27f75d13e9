"""From a ``@weft.kernel`` definition to the call ABI the runtime validates against.

The reference derives this from its canonical IR (python/weft/frontend/compiler.py:299-389,448-533)
and the emitter's ABI table (lib/Target/Emission/Emitter.h:274-343,491-512).  The rules kept here:

* arguments in signature order, each ``View[Encoding, shape]``;
* an Encoding's identity is its declared name (``Q4_K``), ``dense.<dtype>`` for a dtype, or
  ``Family[p, ...]`` for a derived Encoding (compiler.py:480,497-503,760);
* shape symbols become ``size_t`` parameters in first-appearance order across the annotations;
  integer literals stay literals;
* alias set 0 is the default may-alias group; named groups are numbered from 1 in the order their
  first parameter appears (compiler.py:342-361);
* dense arguments: storage_bytes = max(8, bits)/8, record_elements = 1, alignment = storage_bytes
  (Emitter.h:310-318).
"""
from __future__ import annotations

import ast
import json
import math

from . import language as wl
from .api import DerivedEncodingInstance, EncodingDefinition, KernelDefinition
from .diagnostics import FrontendError

_C_TYPES = {"f32": "float", "f64": "double", "f16": "_Float16", "bf16": "uint16_t", "i1": "uint8_t",
            "i8": "int8_t", "i16": "int16_t", "i32": "int32_t", "i64": "int64_t",
            "u8": "uint8_t", "u16": "uint16_t", "u32": "uint32_t", "u64": "uint64_t"}


class _Symbols(dict):
    """Evaluation namespace in which an unknown name is a shape symbol, not an error."""

    def __missing__(self, key: str):
        return _Symbol(key)


class _Symbol:
    def __init__(self, name: str) -> None:
        self.name = name


def encoding_facts(enc: EncodingDefinition) -> tuple[int, int, int]:
    """(storage bytes, logical elements, alignment) of a declared record, from its field annotations."""
    cls = enc.python_class
    namespace = dict(enc.bindings)
    bits = 0
    for name, annotation in getattr(cls, "__annotations__", {}).items():
        spec = eval(annotation, namespace) if isinstance(annotation, str) else annotation
        if isinstance(spec, wl.DType):
            bits += spec.bits
        elif isinstance(spec, wl.ArraySpec):
            bits += spec.dtype.bits * math.prod(int(extent) for extent in spec.shape)
        elif isinstance(spec, wl.PaddingSpec):
            bits += 8 * spec.bytes
        elif _duck_bits(spec) is not None:
            bits += _duck_bits(spec)
        else:
            raise FrontendError(f"field {name} of encoding {enc.__name__} has no storage type")
    if bits % 8:
        raise FrontendError(f"encoding {enc.__name__} does not fill whole bytes")
    return bits // 8, int(getattr(cls, "elements", 1)), int(getattr(cls, "alignment", 1))


def _duck_bits(spec: object) -> int | None:
    # declarations made with another module that offers the same vocabulary (the reference's own)
    dtype = getattr(spec, "dtype", spec)
    width = getattr(dtype, "bits", None)
    if width is None:
        return None
    shape = getattr(spec, "shape", ())
    return width * math.prod(int(extent) for extent in shape)


def _identity(enc: object) -> tuple[str, int, int, int, str]:
    """(identity, storage_bytes, record_elements, alignment, c_type)."""
    if isinstance(enc, EncodingDefinition) or (hasattr(enc, "python_class") and hasattr(enc, "bindings")):
        storage, elements, alignment = encoding_facts(enc)
        return enc.__name__, storage, elements, alignment, "uint8_t"
    if isinstance(enc, DerivedEncodingInstance) or (hasattr(enc, "family") and hasattr(enc, "parameters")):
        spelling = f"{enc.family.__name__}[{', '.join(map(str, enc.parameters))}]"
        # a derived Encoding keeps the record geometry of its base family (Emitter.h:321-333)
        storage, elements, alignment = _derived_base_facts(enc.family)
        return spelling, storage, elements, alignment, "uint8_t"
    name, width = getattr(enc, "name", None), getattr(enc, "bits", None)
    if isinstance(name, str) and isinstance(width, int):
        storage = max(8, width) // 8
        return "dense." + name, storage, 1, storage, _C_TYPES.get(name, "uint8_t")
    raise FrontendError(f"{enc!r} is not an Encoding or dtype")


def _derived_base_facts(family: object) -> tuple[int, int, int]:
    function = getattr(family, "python_function", None)
    if function is None:
        raise FrontendError(f"derived encoding {getattr(family, '__name__', family)!r} has no builder")
    parameters = list(family.signature.parameters.values())
    if not parameters or parameters[0].annotation is parameters[0].empty:
        raise FrontendError(f"derived encoding {family.__name__} needs a View[base Encoding, shape] source parameter")
    namespace = dict(function.__globals__)
    namespace.setdefault(family.__name__, family)
    base, _ = _view_parts(parameters[0].annotation, namespace)
    _, storage, elements, alignment, _ = _identity(base)
    if not storage or not elements:
        raise FrontendError(f"derived encoding {family.__name__} has no closed storage record")
    return storage, elements, alignment


def _view_parts(annotation: object, namespace: dict) -> tuple[object, tuple]:
    if isinstance(annotation, str):
        tree = ast.parse(annotation.strip(), mode="eval").body
        if not (isinstance(tree, ast.Subscript) and isinstance(tree.slice, ast.Tuple) and len(tree.slice.elts) == 2):
            raise FrontendError(f"kernel parameters are View[Encoding, shape]; got {annotation!r}")
        head = eval(compile(ast.Expression(tree.value), "<annotation>", "eval"), namespace)
        if getattr(head, "__name__", "") != "View":
            raise FrontendError(f"kernel parameters are View[Encoding, shape]; got {annotation!r}")
        enc_node, shape_node = tree.slice.elts
        enc = eval(compile(ast.Expression(enc_node), "<annotation>", "eval"), _Symbols(namespace))
        elements = shape_node.elts if isinstance(shape_node, ast.Tuple) else [shape_node]
        shape = []
        for node in elements:
            if isinstance(node, ast.Name):
                shape.append(node.id)
            elif isinstance(node, ast.Constant) and type(node.value) is int and node.value >= 0:
                shape.append(str(node.value))
            else:
                raise FrontendError(f"shape extents are symbols or non-negative integers; got {ast.unparse(node)}")
        return enc, tuple(shape)
    if hasattr(annotation, "encoding") and hasattr(annotation, "shape"):
        shape = tuple(str(e.name if isinstance(e, _Symbol) else e) for e in annotation.shape)
        return annotation.encoding, shape
    raise FrontendError(f"kernel parameters are View[Encoding, shape]; got {annotation!r}")


def kernel_abi(definition: KernelDefinition) -> dict:
    """Arguments (without access modes) and shape parameters of a kernel definition."""
    function = definition.python_function
    namespace = dict(function.__globals__)
    parameters = list(definition.signature.parameters.values())
    unknown = set(definition.alias_groups) - {p.name for p in parameters}
    if unknown:
        raise FrontendError("kernel alias_groups names unknown parameters: " + ", ".join(sorted(unknown)))
    alias_ids: dict[str, int] = {}
    arguments, symbols = [], []
    for parameter in parameters:
        if parameter.annotation is parameter.empty:
            raise FrontendError(f"kernel parameter {parameter.name} needs a View annotation")
        enc, shape = _view_parts(parameter.annotation, namespace)
        identity, storage, elements, alignment, c_type = _identity(enc)
        for extent in shape:
            if not extent.isdecimal() and extent not in symbols:
                symbols.append(extent)
        group = definition.alias_groups.get(parameter.name)
        alias = 0 if group is None else alias_ids.setdefault(group, len(alias_ids) + 1)
        arguments.append({"name": parameter.name, "c_type": c_type, "encoding": identity, "shape": list(shape),
                          "storage_bytes": storage, "record_elements": elements, "alignment": alignment,
                          "alias_set": alias})
    return {"symbol": definition.__name__, "arguments": arguments, "shape_parameters": symbols}


def describe(definition: KernelDefinition) -> str:
    """Canonical text of a definition's ABI; stands where the reference uses its canonical IR as cache key."""
    return json.dumps(kernel_abi(definition), sort_keys=True, indent=1)
