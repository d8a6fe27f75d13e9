"""``compile`` / ``jit`` / ``CompiledKernel``: the call ABI in front of the CUDA kernels.

Same surface and the same argument checks, in the same order, as the reference's
python/weft/runtime/compiler.py:37-254.  What differs is what "compile" means: the reference lowers a
kernel body to RVV C and builds a shared object per kernel; here a definition is resolved by name and
signature to an ``extern "C"`` entry point of the prebuilt sm_100a library (see ``registry``), and an
unknown definition is refused with NotImplementedError instead of falling back.

Arguments may be host objects (buffer protocol), torch tensors or anything with
``__cuda_array_interface__``; wrap packed storage in ``Buffer(data, shape=..., encoding=...)``.  No
copy, repack or hidden workspace is made for device arguments; host arguments are staged by the C
library for the duration of the call.
"""
from __future__ import annotations

import ctypes
import json
import math
import threading
from collections.abc import Mapping
from dataclasses import dataclass, field
from pathlib import Path
from types import MappingProxyType

from ..api import KernelDefinition
from .. import registry
from ..signature import describe
from .buffer import Buffer
from .driver import CompilationError, NativeTarget, Toolchain, last_error, load_library

ARTIFACT_KIND = "weft-b200-artifact"


def _freeze(value):
    if isinstance(value, dict):
        return MappingProxyType({key: _freeze(item) for key, item in value.items()})
    if isinstance(value, (list, tuple)):
        return tuple(_freeze(item) for item in value)
    return value


@dataclass(frozen=True)
class CompileOptions:
    """The reference's option record (compiler.py:37-67), field for field.

    ``meta`` binds source symbols such as NC/MC/MR/NR/KC; the RVV knobs select vector-register
    grouping and software pipelining.  None of them has a CUDA meaning: they are accepted so that
    existing call sites keep working, recorded in ``metadata["bindings"]``, take part in the cache
    key (different options give a different CompiledKernel object, as in the reference) and are
    otherwise ignored.  ``matrix_extension`` other than "none" is refused, as in the reference.
    """
    meta: Mapping[str, int] = field(default_factory=dict)
    lmul_eighths: int = 8
    unroll: int = 1
    pipeline_depth: int = 1
    scalar_load_prime: int = 0
    partial_combine_policy: str = "independent-multilevel"
    record_axis_policy: str = "within-record"
    max_widening_combine_groups: int = 2
    matrix_extension: str = "none"

    def __post_init__(self) -> None:
        values = dict(self.meta)
        for name, value in values.items():
            if not isinstance(name, str) or not name.isidentifier() or type(value) is not int or value <= 0:
                raise ValueError("source bindings must be named positive integers")
        object.__setattr__(self, "meta", MappingProxyType(values))

    def __hash__(self) -> int:
        return hash(tuple(self.arguments()))

    def arguments(self) -> list[str]:
        listed = [f"--meta={name}={value}" for name, value in sorted(self.meta.items())]
        listed += [
            f"--auto-lmul-eighths={self.lmul_eighths}",
            f"--auto-unroll={self.unroll}",
            f"--auto-pipeline-depth={self.pipeline_depth}",
            f"--auto-scalar-load-prime={self.scalar_load_prime}",
            f"--partial-combine-policy={self.partial_combine_policy}",
            f"--record-axis-policy={self.record_axis_policy}",
            f"--max-widening-combine-groups={self.max_widening_combine_groups}",
            f"--matrix-extension={self.matrix_extension}",
        ]
        return listed


class CompiledKernel:
    def __init__(self, definition: KernelDefinition, artifact: dict, target: NativeTarget, options: CompileOptions) -> None:
        if artifact["kind"] != ARTIFACT_KIND or len(artifact["kernels"]) != 1:
            raise CompilationError("a callable kernel requires one resolved ABI")
        self.metadata = _freeze(artifact["kernels"][0])
        if (self.metadata["march"], self.metadata["abi"], self.metadata["vlen_bits"]) != (target.march, target.abi, target.vlen_bits):
            raise CompilationError("compiled artifact disagrees with its discovered target")
        self.target = target
        self.options = options
        self.riscv_ir = artifact["riscv_ir"]          # kept by name; holds the canonical ABI text
        self.source = artifact["intrinsic_c"]         # kept by name; holds the C prototype of the symbol
        self.library_path = Path(target.library)
        self._lock = threading.RLock()
        self._signature = definition.signature
        self._library = load_library(target.library)
        try:
            self._function = getattr(self._library, self.metadata["symbol"])
        except AttributeError as error:
            raise CompilationError(f"the kernel library does not export {self.metadata['symbol']}") from error
        self._function.argtypes = ([ctypes.c_void_p] * len(self.metadata["arguments"]) +
                                   [ctypes.c_size_t] * len(self.metadata["shape_parameters"]))
        self._function.restype = ctypes.c_int
        self.closed = False

    def __call__(self, *args: object, **kwargs: object) -> None:
        with self._lock:
            if self.closed:
                raise RuntimeError("the compiled kernel has been closed")
            self.target.check_execution()
            dimensions: dict[str, int] = {}
            for name in self.metadata["shape_parameters"]:
                if name in kwargs and name not in self._signature.parameters:
                    value = kwargs.pop(name)
                    if type(value) is not int or not 0 <= value < 1 << self.target.xlen:
                        raise ValueError(f"shape parameter {name} must fit the target unsigned index ABI")
                    dimensions[name] = value
            bound = self._signature.bind(*args, **kwargs)
            bound.apply_defaults()
            buffers, spans = [], []
            for parameter in self.metadata["arguments"]:
                value = bound.arguments[parameter["name"]]
                buffer = value if isinstance(value, Buffer) else Buffer(value)
                if buffer.encoding != parameter["encoding"]:
                    raise TypeError(f"{parameter['name']} requires {parameter['encoding']}, got {buffer.encoding}")
                if len(buffer.shape) != len(parameter["shape"]):
                    raise ValueError(f"{parameter['name']} has the wrong logical rank")
                for spelling, extent in zip(parameter["shape"], buffer.shape):
                    if extent >= 1 << self.target.xlen:
                        raise ValueError(f"{parameter['name']} extent cannot be represented by the target ABI")
                    if spelling.isdecimal():
                        expected = int(spelling)
                    elif spelling in dimensions:
                        expected = dimensions[spelling]
                    else:
                        dimensions[spelling] = expected = extent
                    if extent != expected:
                        raise ValueError(f"{parameter['name']} disagrees with extent {spelling}={expected}")
                elements = parameter["record_elements"]
                if buffer.shape and buffer.shape[-1] % elements:
                    raise ValueError(f"{parameter['name']} does not contain complete Encoding records")
                required = math.prod(buffer.shape) // elements * parameter["storage_bytes"]
                if required > buffer.nbytes:
                    raise ValueError(f"{parameter['name']} storage is shorter than its logical View")
                if required and buffer.address % parameter["alignment"]:
                    raise ValueError(f"{parameter['name']} does not meet its Encoding alignment")
                if parameter["writable"] and buffer.readonly:
                    raise TypeError(f"{parameter['name']} requires writable storage")
                for other, begin, end, alias_set in spans:
                    if required and parameter["alias_set"] != alias_set and (
                            buffer.address < end and begin < buffer.address + required):
                        raise ValueError(f"{parameter['name']} aliases {other} across declared alias groups")
                if required:
                    spans.append((parameter["name"], buffer.address, buffer.address + required, parameter["alias_set"]))
                buffers.append(buffer)
            missing = [name for name in self.metadata["shape_parameters"] if name not in dimensions]
            if missing:
                raise ValueError("shape parameters without a value: " + ", ".join(missing))
            status = self._function(*(buffer.address for buffer in buffers),
                                    *(dimensions[name] for name in self.metadata["c_dimension_order"]))
            if status:
                raise RuntimeError(f"{self.metadata['symbol']} failed: {last_error(self._library)}")

    def close(self) -> None:
        with self._lock:
            if self.closed:
                return
            self.closed = True
            self._function = None
            self._library = None


def _prototype(kernel: dict) -> str:
    pointers = [("" if a["writable"] else "const ") + a["c_type"] + " *" + a["name"] for a in kernel["arguments"]]
    dims = ["size_t " + name for name in kernel["c_dimension_order"]]
    return f"int {kernel['symbol']}({', '.join(pointers + dims)});"


class _Compiler:
    def __init__(self, toolchain: Toolchain) -> None:
        self.toolchain = toolchain
        self.target = NativeTarget.discover(toolchain)
        self._cache: dict[tuple, CompiledKernel] = {}
        self._lock = threading.RLock()

    def compile(self, definition: KernelDefinition, options: CompileOptions) -> CompiledKernel:
        if not isinstance(definition, KernelDefinition):
            raise TypeError("compile expects an @weft.kernel definition")
        if options.matrix_extension != "none":
            raise NotImplementedError("native discovery does not expose vendor matrix capabilities")
        canonical = describe(definition)
        arguments = options.arguments()
        key = (definition, canonical, tuple(arguments))
        with self._lock:
            self.target.check_execution()
            cached = self._cache.get(key)
            if cached is not None and not cached.closed:
                return cached
            kernel = registry.resolve(definition)
            kernel.update({"march": self.target.march, "abi": self.target.abi, "vlen_bits": self.target.vlen_bits,
                           "bindings": {"meta": dict(options.meta), "options": arguments}})
            artifact = {"kind": ARTIFACT_KIND, "riscv_ir": canonical, "intrinsic_c": _prototype(kernel), "kernels": [kernel]}
            json.dumps(artifact)    # the artifact stays plain data, as the reference's JSON is
            compiled = CompiledKernel(definition, artifact, self.target, options)
            self._cache[key] = compiled
            return compiled


_compilers: dict[tuple, _Compiler] = {}
_compilers_lock = threading.RLock()


def compile(definition: KernelDefinition, *, options: CompileOptions | None = None,
            toolchain: Toolchain | None = None) -> CompiledKernel:
    selected = (Toolchain() if toolchain is None else toolchain).resolve()
    stamp = Path(selected.compiler).stat()
    identity = (selected, stamp.st_dev, stamp.st_ino, stamp.st_mtime_ns, stamp.st_size)
    with _compilers_lock:
        compiler = _compilers.get(identity)
        if compiler is None:
            compiler = _compilers[identity] = _Compiler(selected)
    return compiler.compile(definition, CompileOptions() if options is None else options)


class JITKernel:
    def __init__(self, definition: KernelDefinition, options: CompileOptions, toolchain: Toolchain) -> None:
        if not isinstance(definition, KernelDefinition):
            raise TypeError("jit expects an @weft.kernel definition")
        self.definition = definition
        self.options = options
        self.toolchain = toolchain
        self.compiled: CompiledKernel | None = None
        self._lock = threading.RLock()

    def __call__(self, *args: object, **kwargs: object) -> None:
        with self._lock:
            if self.compiled is None:
                self.compiled = compile(self.definition, options=self.options, toolchain=self.toolchain)
            compiled = self.compiled
        compiled(*args, **kwargs)


def jit(definition: KernelDefinition, *, options: CompileOptions | None = None,
        toolchain: Toolchain | None = None) -> JITKernel:
    return JITKernel(definition, CompileOptions() if options is None else options,
                     Toolchain() if toolchain is None else toolchain)
