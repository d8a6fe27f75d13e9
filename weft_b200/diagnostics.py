"""Public error types; same names and hierarchy as the reference (python/weft/diagnostics.py:6-33)."""
from __future__ import annotations

from typing import NamedTuple


class WeftError(Exception):
    """Root of every error this package raises on purpose."""


class DefinitionError(WeftError):
    """A decorated object cannot serve as a kernel, encoding or derived-encoding definition."""


class LanguageUseError(WeftError):
    """A definition-time-only object (kernel, dtype, intrinsic) was executed as ordinary Python."""


class SourceLocation(NamedTuple):
    filename: str
    line: int
    column: int

    def format(self) -> str:
        return "%s:%d:%d" % (self.filename, self.line, self.column + 1)


class FrontendError(WeftError):
    """A kernel signature or annotation could not be understood."""

    def __init__(self, message: str, location: SourceLocation | None = None) -> None:
        self.message, self.location = message, location
        super().__init__(message if location is None else location.format() + ": " + message)
