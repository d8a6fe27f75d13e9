"""Definition capture: ``@kernel``, ``@encoding``, ``@derive``, ``overloads``.

Mirrors the reference's decorator surface (python/weft/api/definitions.py:36-205) so that kernel
files written for it import and decorate unchanged.  A definition is inert data: its body is never
run (calling it raises LanguageUseError, as in the reference); ``weft.compile`` resolves it to a
hand-written CUDA kernel by name and signature instead of lowering the body.
"""
from __future__ import annotations

import inspect
import sys
import textwrap
from types import FunctionType
from typing import Callable, Mapping

from .diagnostics import DefinitionError, LanguageUseError


class DefinitionSource:
    """Where a definition was written and its dedented text."""

    __slots__ = ("filename", "first_line", "text")

    def __init__(self, filename: str, first_line: int, text: str) -> None:
        self.filename, self.first_line, self.text = filename, first_line, text

    @classmethod
    def of(cls, obj: object, noun: str) -> "DefinitionSource":
        try:
            lines, first = inspect.getsourcelines(obj)
            filename = inspect.getsourcefile(obj) or "<unknown>"
        except (OSError, TypeError) as error:
            raise DefinitionError(f"the source of this {noun} cannot be read back; definitions must live in a file") from error
        return cls(filename, first, textwrap.dedent("".join(lines)))


def _copy_identity(target: object, function: FunctionType) -> None:
    for attribute in ("__name__", "__qualname__", "__module__", "__doc__"):
        setattr(target, attribute, getattr(function, attribute))
    target.__wrapped__ = function


class KernelDefinition:
    """One ``@weft.kernel`` function: signature, alias groups and source, nothing executable."""

    def __init__(self, function: Callable, *, alias_groups: Mapping[str, str] | None = None) -> None:
        if not isinstance(function, FunctionType):
            raise DefinitionError("@kernel goes on a plain Python function (got something else)")
        if alias_groups is not None and not isinstance(alias_groups, Mapping):
            raise DefinitionError("alias_groups= takes a mapping {parameter name: group name}")
        groups = dict(alias_groups or {})
        for parameter, group in groups.items():
            if not (isinstance(parameter, str) and parameter and isinstance(group, str) and group):
                raise DefinitionError("alias_groups= needs non-empty strings for both the parameter and its group")
        self.python_function = function
        self.alias_groups = groups
        self.source = DefinitionSource.of(function, "decorated DSL kernel")
        _copy_identity(self, function)

    @property
    def signature(self) -> inspect.Signature:
        return inspect.signature(self.python_function, eval_str=False)

    def source_text(self) -> str:
        return self.source.text

    def lower(self) -> str:
        from .signature import describe

        return describe(self)

    def __call__(self, *args, **kwargs):
        raise LanguageUseError(
            f"{self.__name__} only describes a kernel and has no Python behaviour; run it through weft.compile(...) or weft.jit(...)")

    def __repr__(self) -> str:
        return f"<weft kernel {self.__module__}.{self.__qualname__}>"


class EncodingDefinition:
    """One ``@weft.encoding`` class: a named record layout."""

    def __init__(self, declaration: type, bindings: dict) -> None:
        if not isinstance(declaration, type):
            raise DefinitionError("@encoding goes on a class that declares a record layout")
        self.python_class = declaration
        self.bindings = bindings
        self.source = DefinitionSource.of(declaration, "encoding class")
        self.__name__ = declaration.__name__
        self.__qualname__ = declaration.__qualname__
        self.__module__ = declaration.__module__

    def __repr__(self) -> str:
        return f"<weft encoding {self.__module__}.{self.__qualname__}>"


class DerivedEncodingInstance:
    __slots__ = ("family", "parameters")

    def __init__(self, family: "DerivedEncodingDefinition", parameters: tuple) -> None:
        self.family, self.parameters = family, parameters

    def __eq__(self, other: object) -> bool:
        return (isinstance(other, DerivedEncodingInstance) and other.family is self.family
                and other.parameters == self.parameters)

    def __hash__(self) -> int:
        return hash((id(self.family), self.parameters))


class DerivedEncodingDefinition:
    """One ``@weft.derive`` generator; ``Family[16]`` names a member of the family."""

    def __init__(self, function: Callable) -> None:
        if not isinstance(function, FunctionType):
            raise DefinitionError("@derive goes on a plain Python function")
        self.python_function = function
        self.source = DefinitionSource.of(function, "derived encoding definition")
        _copy_identity(self, function)

    @property
    def signature(self) -> inspect.Signature:
        return inspect.signature(self.python_function, eval_str=False)

    def __call__(self, *args, **kwargs):
        raise LanguageUseError(f"{self.__name__} names a family of derived Encodings; index it (Family[rows]) instead of calling it")

    def __getitem__(self, parameters: object) -> DerivedEncodingInstance:
        values = parameters if isinstance(parameters, tuple) else (parameters,)
        if not values or not all(type(value) is int for value in values):
            raise TypeError("a derived Encoding is selected by integer constants, e.g. Family[16]")
        return DerivedEncodingInstance(self, values)


class InlineDefinition:
    __slots__ = ("python_function", "source")

    def __init__(self, python_function: FunctionType, source: DefinitionSource) -> None:
        self.python_function, self.source = python_function, source

    @classmethod
    def capture(cls, function: Callable) -> "InlineDefinition":
        if not isinstance(function, FunctionType):
            raise DefinitionError("an overload candidate has to be a plain Python function")
        return cls(function, DefinitionSource.of(function, "inline function"))

    @property
    def signature(self) -> inspect.Signature:
        return inspect.signature(self.python_function, eval_str=False)

    @property
    def name(self) -> str:
        return self.python_function.__name__


class OverloadSet:
    __slots__ = ("name", "definitions")

    def __init__(self, name: str, definitions: tuple) -> None:
        self.name, self.definitions = name, definitions

    def __call__(self, *args, **kwargs):
        raise LanguageUseError(f"{self.name} is a set of overloads for use inside kernel bodies; it cannot be called from Python")


def kernel(function: Callable | None = None, *, alias_groups: Mapping[str, str] | None = None):
    if function is not None:
        return KernelDefinition(function, alias_groups=alias_groups)

    def decorate(decorated: Callable) -> KernelDefinition:
        return KernelDefinition(decorated, alias_groups=alias_groups)

    return decorate


def encoding(declaration: type) -> EncodingDefinition:
    caller = sys._getframe(1)
    try:
        return EncodingDefinition(declaration, dict(caller.f_globals))
    finally:
        del caller


def derive(function: Callable) -> DerivedEncodingDefinition:
    return DerivedEncodingDefinition(function)


def overloads(name: str, *functions: Callable) -> OverloadSet:
    if not name or not functions:
        raise DefinitionError("overloads(name, f, ...) needs a name and one candidate or more")
    return OverloadSet(name, tuple(InlineDefinition.capture(function) for function in functions))
