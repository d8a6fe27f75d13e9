"""weft_b200: the reference's ``weft`` Python surface in front of hand-written sm_100a kernels.

``import weft_b200 as weft`` gives ``weft.kernel / encoding / derive / overloads / compile / jit /
lower_to_mlir`` and the error types (python/weft/__init__.py:13-46 of the reference), with
``weft.language`` and ``weft.runtime`` underneath.  ``install_as_weft()`` registers the package under
the name ``weft`` so that kernel files written for the reference (``import weft``,
``import weft.language as wl``) import unchanged.
"""
from __future__ import annotations

import sys

from . import api, language
from .api import (DerivedEncodingDefinition, EncodingDefinition, KernelDefinition, derive, encoding, kernel,
                  overloads)
from .diagnostics import DefinitionError, FrontendError, LanguageUseError, WeftError


def compile(definition, *, options=None, toolchain=None):
    from .runtime import compile as native_compile

    return native_compile(definition, options=options, toolchain=toolchain)


def jit(definition, *, options=None, toolchain=None):
    from .runtime import jit as native_jit

    return native_jit(definition, options=options, toolchain=toolchain)


def lower_to_mlir(definition: KernelDefinition) -> str:
    """The canonical ABI text of a definition.  The reference returns MLIR here; this build has no IR
    and uses the text only as a cache key and for display."""
    from .signature import describe

    return describe(definition)


def install_as_weft() -> None:
    """Make ``import weft``, ``weft.language``, ``weft.runtime``, ``weft.api`` resolve to this package."""
    from . import runtime

    sys.modules.setdefault("weft", sys.modules[__name__])
    sys.modules.setdefault("weft.language", language)
    sys.modules.setdefault("weft.api", api)
    sys.modules.setdefault("weft.runtime", runtime)
    sys.modules.setdefault("weft.diagnostics", sys.modules[__name__ + ".diagnostics"])


__all__ = ["DefinitionError", "DerivedEncodingDefinition", "EncodingDefinition", "FrontendError", "KernelDefinition",
           "LanguageUseError", "WeftError", "derive", "compile", "encoding", "kernel", "jit", "lower_to_mlir",
           "overloads", "install_as_weft"]
