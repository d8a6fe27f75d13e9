"""The DSL vocabulary kernel files import as ``wl``: dtypes, ``View``, field layouts, intrinsics.

Same names as the reference's ``weft.language`` (python/weft/language/__init__.py:1-113,
dtypes.py:43-61, annotations.py:39-123, builtins.py:41-63).  Everything here is declarative: dtypes
and layout helpers build small immutable descriptions, and every intrinsic raises LanguageUseError
when called, because kernel bodies are specifications that are never executed (builtins.py:12-15).
"""
from __future__ import annotations

from .diagnostics import LanguageUseError

# ------------------------------------------------------------------ dtypes


class DType:
    __slots__ = ("name", "category", "bits", "signedness")

    def __init__(self, name: str, category: str, bits: int | None, signedness: str | None = None) -> None:
        self.name, self.category, self.bits, self.signedness = name, category, bits, signedness

    def __call__(self, value: object):
        raise LanguageUseError(f"W.{self.name}(...) is valid only while lowering a Weft definition")

    def __getitem__(self, shape: object) -> "ArraySpec":
        return ArraySpec(self, shape if isinstance(shape, tuple) else (shape,))

    def __matmul__(self, packing: object) -> "ArraySpec":
        return ArraySpec(self, ()) @ packing

    def __repr__(self) -> str:
        return "W." + self.name


def _ints(signedness: str, prefix: str, widths) -> dict:
    return {f"{prefix}{w}": DType(f"{prefix}{w}", "integer", w, signedness) for w in widths}


_TABLE = {"i1": DType("i1", "bool", 1), "index": DType("index", "index", None)}
_TABLE.update(_ints("signed", "i", (4, 8, 16, 32, 64)))
_TABLE.update(_ints("unsigned", "u", (1, 2, 4, 6, 8, 16, 32, 64)))
_TABLE.update({"f16": DType("f16", "float", 16), "bf16": DType("bf16", "bfloat", 16),
               "f32": DType("f32", "float", 32), "f64": DType("f64", "float", 64)})
globals().update(_TABLE)

# ------------------------------------------------------------------ layout annotations


class LayoutAtom:
    __slots__ = ("category", "value")

    def __init__(self, category: str, value: str) -> None:
        self.category, self.value = category, value

    def __repr__(self) -> str:
        return f"{self.category}.{self.value}"


class _Orders:
    def __init__(self, category: str, *values: str) -> None:
        for value in values:
            setattr(self, value, LayoutAtom(category, value))


bitorder = _Orders("bit_order", "lsb_first", "msb_first")
byteorder = _Orders("byte_order", "little", "big")
lo_first, hi_first = "lo_first", "hi_first"


class FieldLayoutSpec:
    __slots__ = ("kind", "size", "order", "fields", "low_bits")

    def __init__(self, kind: str, size: int, order: str = "", fields: int = 0, low_bits: int = 0) -> None:
        self.kind, self.size, self.order, self.fields, self.low_bits = kind, size, order, fields, low_bits


def _positive(name: str, value: object, what: str) -> int:
    if type(value) is not int or value <= 0:
        raise TypeError(f"{name} expects a positive {what}")
    return value


def _order(name: str, order: object) -> str:
    if order not in (lo_first, hi_first):
        raise TypeError(f"{name} order must be lo_first or hi_first")
    return order


def grouped(*, elements: int) -> FieldLayoutSpec:
    return FieldLayoutSpec("grouped", _positive("grouped", elements, "logical element count"))


def bit_layers(*, elements: int, order: str) -> FieldLayoutSpec:
    return FieldLayoutSpec("layered", _positive("bit_layers", elements, "logical layer extent"), _order("bit_layers", order))


def pack_fields(*, group: int, fields: int, low_bits: int, order: str) -> FieldLayoutSpec:
    for label, value in (("group", group), ("fields", fields), ("low_bits", low_bits)):
        _positive(f"pack_fields {label}", value, "integer")
    return FieldLayoutSpec("joined", group, _order("pack_fields", order), fields, low_bits)


class PaddingSpec:
    __slots__ = ("bytes", "value")

    def __init__(self, bytes: int, value: int = 0) -> None:
        self.bytes, self.value = bytes, value


def padding(bytes: int, value: int = 0) -> PaddingSpec:
    _positive("padding", bytes, "byte count")
    if type(value) is not int or not 0 <= value <= 255:
        raise TypeError("padding fill must be a byte")
    return PaddingSpec(bytes, value)


class ArraySpec:
    __slots__ = ("dtype", "shape", "layouts")

    def __init__(self, dtype: DType, shape: tuple, layouts: tuple = ()) -> None:
        self.dtype, self.shape, self.layouts = dtype, shape, layouts

    def __matmul__(self, layout: object) -> "ArraySpec":
        if not isinstance(layout, FieldLayoutSpec):
            raise TypeError("encoding field @ annotation must be a field layout")
        return ArraySpec(self.dtype, self.shape, self.layouts + (layout,))


class ViewSpec:
    __slots__ = ("encoding", "shape")

    def __init__(self, encoding: object, shape: tuple) -> None:
        self.encoding, self.shape = encoding, shape


class View:
    """``View[Encoding, shape]``: a logical tensor of ``shape`` elements stored as ``Encoding`` records."""

    def __class_getitem__(cls, parameters: object) -> ViewSpec:
        if not (isinstance(parameters, tuple) and len(parameters) == 2):
            raise TypeError("View expects View[Encoding, shape]")
        enc, shape = parameters
        return ViewSpec(enc, shape if isinstance(shape, tuple) else (shape,))


class static:
    """``static[int]``: marks a build-time parameter of a derived Encoding."""

    def __class_getitem__(cls, parameter: object) -> object:
        return parameter


class AutoSpec:
    __slots__ = ("choices",)

    def __init__(self, choices: tuple) -> None:
        self.choices = choices

    @property
    def spelling(self) -> str:
        return "|".join(map(str, self.choices))


def auto(*choices: object) -> AutoSpec:
    if not choices:
        raise TypeError("auto expects at least one candidate or one symbolic parameter")
    return AutoSpec(choices)

# ------------------------------------------------------------------ intrinsics


class Intrinsic:
    __slots__ = ("name",)

    def __init__(self, name: str) -> None:
        self.name = name

    def __call__(self, *args, **kwargs):
        raise LanguageUseError(f"wl.{self.name} is valid only while lowering a Weft definition")


class LevelConstructor:
    __slots__ = ("relation",)

    def __init__(self, relation: str) -> None:
        self.relation = relation

    def __call__(self, *args, **kwargs):
        raise LanguageUseError("Weft levels exist only while lowering a kernel")


class _Levels:
    rows, cols, tiles = LevelConstructor("rows"), LevelConstructor("cols"), LevelConstructor("tiles")
    blocks, subtiles = LevelConstructor("blocks"), LevelConstructor("subs")


level = _Levels()

_INTRINSICS = ("state arange stage load store subview reshape mac_pairs mac_groups widen narrow reduce "
               "sum_pairs dot reduce_dot lookup interleave maximum minimum abs exp").split()
globals().update({name: Intrinsic(name) for name in _INTRINSICS})

__all__ = (["View", "auto", "bit_layers", "bitorder", "byteorder", "grouped", "hi_first", "lo_first", "level",
            "pack_fields", "padding", "static"] + _INTRINSICS + list(_TABLE))
