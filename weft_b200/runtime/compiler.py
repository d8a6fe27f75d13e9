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
from dataclasses import field, make_dataclass
from pathlib import Path
from types import MappingProxyType

from ..api import KernelDefinition
from .. import registry
from ..signature import describe
from .buffer import Buffer
from .driver import CompilationError, NativeTarget, Toolchain, last_error, load_library

ARTIFACT_KIND = "weft-b200-artifact"


def _freeze(value):
    """A read-only view of plain nested data (dicts become mapping proxies, sequences tuples)."""
    if isinstance(value, dict):
        return MappingProxyType({key: _freeze(item) for key, item in value.items()})
    if isinstance(value, (list, tuple)):
        return tuple(_freeze(item) for item in value)
    return value


#: (field, default, command-line spelling) of the reference's physical knobs, in the order its compiler driver
#: lists them (python/weft/runtime/compiler.py:37-67).  Kept as data: the record must have these fields and this
#: spelling so that option objects built for the reference work here and two option sets compare as they do there.
_KNOBS = (
    ("lmul_eighths", 8, "--auto-lmul-eighths"),
    ("unroll", 1, "--auto-unroll"),
    ("pipeline_depth", 1, "--auto-pipeline-depth"),
    ("scalar_load_prime", 0, "--auto-scalar-load-prime"),
    ("partial_combine_policy", "independent-multilevel", "--partial-combine-policy"),
    ("record_axis_policy", "within-record", "--record-axis-policy"),
    ("max_widening_combine_groups", 2, "--max-widening-combine-groups"),
    ("matrix_extension", "none", "--matrix-extension"),
)


def _checked_bindings(meta: Mapping[str, int]) -> MappingProxyType:
    """Source-symbol bindings (NC, MC, MR, NR, KC ...): identifier -> positive int, nothing else."""
    bindings = {}
    for name, value in dict(meta).items():
        named = isinstance(name, str) and name.isidentifier()
        positive = type(value) is int and value > 0
        if not (named and positive):
            raise ValueError(f"meta binds source symbols to positive integers; got {name!r}={value!r}")
        bindings[name] = value
    return MappingProxyType(bindings)


def _make_options_class():
    fields = [("meta", Mapping[str, int], field(default_factory=dict))]
    fields += [(name, type(default), field(default=default)) for name, default, _ in _KNOBS]

    def post_init(self) -> None:
        object.__setattr__(self, "meta", _checked_bindings(self.meta))

    def arguments(self) -> list[str]:
        """The option set as the reference's compiler driver would receive it; also the cache identity."""
        bound = [f"--meta={name}={self.meta[name]}" for name in sorted(self.meta)]
        return bound + [f"{flag}={getattr(self, name)}" for name, _, flag in _KNOBS]

    namespace = {
        "__post_init__": post_init,
        "__hash__": lambda self: hash(tuple(self.arguments())),
        "arguments": arguments,
        "__doc__": """The reference's option record, field for field.

    ``meta`` binds source symbols such as NC/MC/MR/NR/KC; the other fields select vector-register grouping
    and software pipelining on the reference's RISC-V targets.  None of them has a CUDA meaning: they are
    accepted so that existing call sites keep working, recorded in ``metadata["bindings"]``, take part in
    the cache key (different options give a different CompiledKernel object, as in the reference) and are
    otherwise ignored.  ``matrix_extension`` other than "none" is refused, as in the reference.
    """,
    }
    return make_dataclass("CompileOptions", fields, frozen=True, namespace=namespace)


CompileOptions = _make_options_class()
CompileOptions.__module__ = __name__


# ---- argument validation --------------------------------------------------------------------------------
# One function per rule.  The order in which CompiledKernel.__call__ applies them, and the exception class of
# each, is the reference's (python/weft/runtime/compiler.py:99-155): code written against it sees the same
# failure for the same mistake.

def _take_explicit_extents(shape_parameters, python_parameters, kwargs: dict, index_bits: int) -> dict[str, int]:
    """Extents passed by keyword (only names that are not also Python parameters of the kernel)."""
    given = {}
    for name in shape_parameters:
        if name in kwargs and name not in python_parameters:
            value = kwargs.pop(name)
            if type(value) is not int or value < 0 or value >> index_bits:
                raise ValueError(f"extent {name}={value!r} is not an unsigned {index_bits}-bit index")
            given[name] = value
    return given


def _check_encoding(parameter, buffer: Buffer) -> None:
    if buffer.encoding != parameter["encoding"]:
        raise TypeError(f"argument {parameter['name']} requires {parameter['encoding']} storage but holds {buffer.encoding}")


def _check_shape(parameter, buffer: Buffer, extents: dict[str, int], index_bits: int) -> None:
    """Rank, then every extent against its literal or symbol; a symbol's first use fixes its value."""
    declared = parameter["shape"]
    if len(buffer.shape) != len(declared):
        raise ValueError(f"argument {parameter['name']} has rank {len(buffer.shape)}, the kernel declares rank {len(declared)}")
    for symbol, extent in zip(declared, buffer.shape):
        if extent >> index_bits:
            raise ValueError(f"argument {parameter['name']}: extent {extent} does not fit a {index_bits}-bit index")
        expected = int(symbol) if symbol.isdecimal() else extents.setdefault(symbol, extent)
        if extent != expected:
            raise ValueError(f"argument {parameter['name']} disagrees with extent {symbol}={expected} (got {extent})")


def _storage_span(parameter, buffer: Buffer) -> int:
    """Bytes the logical View occupies; checks whole records, length and alignment on the way."""
    per_record = parameter["record_elements"]
    if buffer.shape and buffer.shape[-1] % per_record:
        raise ValueError(f"argument {parameter['name']}: the last extent must hold complete Encoding records of {per_record} elements")
    span = math.prod(buffer.shape) // per_record * parameter["storage_bytes"]
    if span > buffer.nbytes:
        raise ValueError(f"argument {parameter['name']}: {buffer.nbytes} bytes of storage are shorter than the {span} its View needs")
    if span and buffer.address % parameter["alignment"]:
        raise ValueError(f"argument {parameter['name']} breaks the {parameter['alignment']}-byte alignment of its Encoding")
    return span


def _check_writable(parameter, buffer: Buffer) -> None:
    if parameter["writable"] and buffer.readonly:
        raise TypeError(f"argument {parameter['name']} is written by the kernel and needs writable storage")


class _AliasLedger:
    """Byte ranges seen so far, each with its alias group: ranges of different groups must not overlap."""

    def __init__(self) -> None:
        self._ranges: list[tuple[str, int, int, int]] = []

    def admit(self, parameter, address: int, span: int) -> None:
        if not span:
            return
        group, stop = parameter["alias_set"], address + span
        for name, lo, hi, other_group in self._ranges:
            if other_group != group and address < hi and lo < stop:
                raise ValueError(f"argument {parameter['name']} aliases {name}, which belongs to another alias group")
        self._ranges.append((parameter["name"], address, stop, group))


class CompiledKernel:
    """A resolved kernel: frozen ABI metadata plus the bound ``extern "C"`` entry point."""

    def __init__(self, definition: KernelDefinition, artifact: dict, target: NativeTarget, options: CompileOptions) -> None:
        kernels = artifact["kernels"]
        if artifact["kind"] != ARTIFACT_KIND or len(kernels) != 1:
            raise CompilationError("a callable kernel needs an artifact of this build with exactly one kernel in it")
        self.metadata = _freeze(kernels[0])
        built_for = (self.metadata["march"], self.metadata["abi"], self.metadata["vlen_bits"])
        if built_for != (target.march, target.abi, target.vlen_bits):
            raise CompilationError(f"the artifact was resolved for {built_for}, not for the discovered target")
        self.target = target
        self.options = options
        self.riscv_ir = artifact["riscv_ir"]          # attribute name kept; holds the canonical ABI text
        self.source = artifact["intrinsic_c"]         # attribute name kept; holds the C prototype of the symbol
        self.library_path = Path(target.library)
        self._lock = threading.RLock()
        self._signature = definition.signature
        self._library = load_library(target.library)
        symbol = self.metadata["symbol"]
        self._function = getattr(self._library, symbol, None)
        if self._function is None:
            raise CompilationError(f"the kernel library does not export {symbol}")
        pointers, extents = len(self.metadata["arguments"]), len(self.metadata["shape_parameters"])
        self._function.argtypes = [ctypes.c_void_p] * pointers + [ctypes.c_size_t] * extents
        self._function.restype = ctypes.c_int
        self.closed = False

    def __call__(self, *args: object, **kwargs: object) -> None:
        with self._lock:
            if self.closed:
                raise RuntimeError("this kernel was closed and can no longer be called")
            self.target.check_execution()
            meta, bits = self.metadata, self.target.xlen
            extents = _take_explicit_extents(meta["shape_parameters"], self._signature.parameters, kwargs, bits)
            call = self._signature.bind(*args, **kwargs)
            call.apply_defaults()
            ledger, addresses = _AliasLedger(), []
            for parameter in meta["arguments"]:
                given = call.arguments[parameter["name"]]
                buffer = given if isinstance(given, Buffer) else Buffer(given)
                _check_encoding(parameter, buffer)
                _check_shape(parameter, buffer, extents, bits)
                span = _storage_span(parameter, buffer)
                _check_writable(parameter, buffer)
                ledger.admit(parameter, buffer.address, span)
                addresses.append(buffer.address)
            unbound = [name for name in meta["shape_parameters"] if name not in extents]
            if unbound:
                raise ValueError("no argument fixes these extents, pass them by keyword: " + ", ".join(unbound))
            failed = self._function(*addresses, *(extents[name] for name in meta["c_dimension_order"]))
            if failed:
                raise RuntimeError(f"{meta['symbol']} failed: {last_error(self._library)}")

    def close(self) -> None:
        """Idempotent; a closed kernel raises RuntimeError when called."""
        with self._lock:
            self.closed, self._function, self._library = True, None, None


def _prototype(kernel: dict) -> str:
    pointers = [("" if a["writable"] else "const ") + a["c_type"] + " *" + a["name"] for a in kernel["arguments"]]
    dims = ["size_t " + name for name in kernel["c_dimension_order"]]
    return f"int {kernel['symbol']}({', '.join(pointers + dims)});"


def _library_identity(toolchain: Toolchain) -> tuple:
    """What distinguishes one resolved kernel library from another on disk: rebuilt or replaced files get a new
    resolver (and new CompiledKernel objects), an unchanged file keeps its cache."""
    facts = Path(toolchain.compiler).stat()
    return (toolchain, facts.st_dev, facts.st_ino, facts.st_mtime_ns, facts.st_size)


class _Resolver:
    """Per-library cache of resolved kernels.  Identity of a cached kernel: the definition object, its canonical
    ABI text and the full option list -- equal options give the same CompiledKernel, different options another one
    (the reference's observable caching behaviour, examples/repro/weft/native_jit.py:43-48)."""

    def __init__(self, toolchain: Toolchain) -> None:
        self.toolchain = toolchain
        self.target = NativeTarget.discover(toolchain)
        self._kernels: dict[tuple, CompiledKernel] = {}
        self._lock = threading.RLock()

    def _artifact(self, definition: KernelDefinition, canonical: str, options: CompileOptions) -> dict:
        kernel = registry.resolve(definition)
        kernel["march"], kernel["abi"], kernel["vlen_bits"] = self.target.march, self.target.abi, self.target.vlen_bits
        kernel["bindings"] = {"meta": dict(options.meta), "options": options.arguments()}
        artifact = {"kind": ARTIFACT_KIND, "riscv_ir": canonical, "intrinsic_c": _prototype(kernel), "kernels": [kernel]}
        json.dumps(artifact)    # must stay plain data, like the JSON artifact of the reference's compiler
        return artifact

    def resolve(self, definition: KernelDefinition, options: CompileOptions) -> CompiledKernel:
        if not isinstance(definition, KernelDefinition):
            raise TypeError("compile expects an @weft.kernel definition")
        if options.matrix_extension != "none":
            raise NotImplementedError("this target has no vendor matrix extension to select")
        canonical = describe(definition)
        key = (definition, canonical, tuple(options.arguments()))
        with self._lock:
            self.target.check_execution()
            kernel = self._kernels.get(key)
            if kernel is None or kernel.closed:
                kernel = self._kernels[key] = CompiledKernel(definition, self._artifact(definition, canonical, options), self.target, options)
            return kernel


_resolvers: dict[tuple, _Resolver] = {}
_resolvers_lock = threading.RLock()


def compile(definition: KernelDefinition, *, options: CompileOptions | None = None,
            toolchain: Toolchain | None = None) -> CompiledKernel:
    """``weft.compile``: the kernel behind ``definition`` as a callable (python/weft/runtime/compiler.py:218-229)."""
    resolved = (toolchain or Toolchain()).resolve()
    identity = _library_identity(resolved)
    with _resolvers_lock:
        if identity not in _resolvers:
            _resolvers[identity] = _Resolver(resolved)
        resolver = _resolvers[identity]
    return resolver.resolve(definition, options or CompileOptions())


class JITKernel:
    """``weft.jit``: resolves on first call, then forwards (python/weft/runtime/compiler.py:232-248)."""

    def __init__(self, definition: KernelDefinition, options: CompileOptions, toolchain: Toolchain) -> None:
        if not isinstance(definition, KernelDefinition):
            raise TypeError("jit expects an @weft.kernel definition")
        self.definition, self.options, self.toolchain = definition, options, toolchain
        self.compiled: CompiledKernel | None = None
        self._lock = threading.RLock()

    def __call__(self, *args: object, **kwargs: object) -> None:
        with self._lock:
            if self.compiled is None:
                self.compiled = compile(self.definition, options=self.options, toolchain=self.toolchain)
            kernel = self.compiled
        kernel(*args, **kwargs)


def jit(definition: KernelDefinition, *, options: CompileOptions | None = None,
        toolchain: Toolchain | None = None) -> JITKernel:
    return JITKernel(definition, options or CompileOptions(), toolchain or Toolchain())
