"""Toolchain and target discovery for the CUDA build of the runtime.

Counterpart of the reference's python/weft/runtime/driver.py:22-85.  There the toolchain is the
``weft-compile`` binary plus a C compiler and the target is the RISC-V hart set found by
``--query-native-target``; here the "compiler" is the prebuilt kernel library (rebuilt with nvcc when
its sources are newer) and the target is the CUDA device the library binds to.  Field names are kept
so code that inspects ``kernel.target`` keeps working: ``march`` is the SM architecture, ``abi`` the
C calling convention of the library, ``xlen`` the pointer width, ``vlen_bits`` the SIMT width in
bits (32 lanes x 32 bits) and ``cpus`` the set of visible device ordinals.
"""
from __future__ import annotations

import ctypes
import os
import shutil
import sys
import threading
from dataclasses import dataclass, field
from pathlib import Path

from ..diagnostics import WeftError

PACKAGE = Path(__file__).resolve().parents[1]
DEFAULT_LIBRARY = PACKAGE / "libweft_b200.so"


class CompilationError(WeftError):
    pass


@dataclass(frozen=True)
class Toolchain:
    compiler: str = str(DEFAULT_LIBRARY)          # the kernel library (the reference: weft-compile)
    cc: tuple[str, ...] = ("nvcc",)               # used only to rebuild a stale library
    cflags: tuple[str, ...] = ()

    def __post_init__(self) -> None:
        object.__setattr__(self, "cc", tuple(self.cc))
        object.__setattr__(self, "cflags", tuple(self.cflags))
        if not self.compiler or not self.cc:
            raise ValueError("the kernel library and the CUDA compiler must be explicit")

    def resolve(self) -> "Toolchain":
        library = Path(self.compiler)
        if library == DEFAULT_LIBRARY:
            from .. import build

            if build.stale():
                if shutil.which(self.cc[0]) is None and not Path("/usr/local/cuda/bin/nvcc").exists():
                    raise CompilationError(f"native toolchain is unavailable: library={library}, CUDA compiler={self.cc[0]}")
                try:
                    build.ensure_built(extra=list(self.cflags))   # file-locked: ranks of one job build once
                except Exception as error:  # nvcc diagnostics are in the message
                    raise CompilationError(str(error)) from error
        if not library.exists():
            raise CompilationError(f"native toolchain is unavailable: kernel library {library} does not exist")
        return Toolchain(str(library.resolve()), self.cc, self.cflags)


_libraries: dict[str, ctypes.CDLL] = {}
_libraries_lock = threading.Lock()


def load_library(path: str) -> ctypes.CDLL:
    with _libraries_lock:
        lib = _libraries.get(path)
        if lib is None:
            try:
                lib = ctypes.CDLL(path, mode=os.RTLD_LOCAL)
            except OSError as error:
                raise CompilationError(f"cannot load the kernel library {path}: {error}") from error
            lib.weft_b200_last_error.restype = ctypes.c_char_p
            lib.weft_b200_launch_count.restype = ctypes.c_ulonglong
            lib.weft_b200_set_stream.argtypes = [ctypes.c_void_p]
            lib.weft_b200_weights_resident.argtypes = [ctypes.c_void_p, ctypes.c_size_t]
            lib.weft_b200_weights_release.argtypes = [ctypes.c_void_p]
            _libraries[path] = lib
        return lib


def last_error(lib: ctypes.CDLL) -> str:
    return (lib.weft_b200_last_error() or b"").decode("utf-8", "replace")


@dataclass(frozen=True)
class NativeTarget:
    march: str
    abi: str
    xlen: int
    vlen_bits: int
    cpus: frozenset[int]
    name: str = ""
    sm_count: int = 0
    memory_bytes: int = 0
    device: int = 0
    library: str = field(default="", compare=False)

    @classmethod
    def discover(cls, toolchain: Toolchain) -> "NativeTarget":
        lib = load_library(toolchain.compiler)
        major, minor, sms = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        total = ctypes.c_size_t()
        name = ctypes.create_string_buffer(256)
        if lib.weft_b200_device_info(ctypes.byref(major), ctypes.byref(minor), ctypes.byref(sms),
                                     ctypes.byref(total), name, ctypes.c_size_t(256)):
            raise CompilationError("native discovery failed: " + last_error(lib))
        target = cls(march=f"sm_{major.value}{minor.value}a", abi="weft_b200-c", xlen=ctypes.sizeof(ctypes.c_void_p) * 8,
                     vlen_bits=32 * 32, cpus=frozenset({0}), name=name.value.decode(), sm_count=sms.value,
                     memory_bytes=total.value, device=0, library=toolchain.compiler)
        if target.sm_count <= 0:
            raise CompilationError("native discovery returned incomplete hardware facts")
        target.check_execution()
        return target

    def check_execution(self) -> None:
        if sys.platform != "linux" or sys.byteorder != "little":
            raise CompilationError("native execution requires little-endian Linux")
        if ctypes.sizeof(ctypes.c_void_p) * 8 != self.xlen:
            raise CompilationError("process pointer ABI disagrees with the compiled target")
        if self.march != "sm_100a":
            raise CompilationError(f"the kernel library carries sm_100a code; the device is {self.march}")
