"""The native runtime surface: same names as the reference's ``weft.runtime`` (python/weft/runtime/__init__.py:1-8)."""
from .buffer import Buffer
from .compiler import CompiledKernel, CompileOptions, JITKernel, compile, jit
from .driver import CompilationError, NativeTarget, Toolchain

__all__ = ["Buffer", "CompilationError", "CompiledKernel", "CompileOptions", "JITKernel", "NativeTarget", "Toolchain",
           "compile", "jit"]
