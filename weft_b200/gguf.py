"""GGUF tensors as runtime Buffers: the caller side of the quantized matrix path.

A GGUF file (version 2 or 3, little endian) is: the magic ``GGUF``, a u32 version, u64 tensor and metadata
counts, the metadata key/value pairs, the tensor directory (name, dimensions innermost first, GGML type id,
offset into the data section), padding to ``general.alignment`` (default 32), and the tensor data.  The
record formats on this path are stored in GGUF exactly as the kernels read them, so a tensor becomes a
``Buffer`` over the mapped file bytes with its logical (rows, K) shape and its Encoding -- no conversion and no
repack (the reference's model-level entry reads the same files through llama.cpp: examples/run/ggml.sh:35-43).

``read`` maps a file; ``write`` produces one (used by the tests and to make synthetic models).
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

import numpy as np

from .formats import RECORDS

MAGIC = b"GGUF"
DEFAULT_ALIGNMENT = 32

#: GGML type id (ggml/include/ggml.h enum ggml_type) -> (Encoding name or dense dtype, bytes per record, elements per record)
GGML_TYPES = {
    0: ("dense.f32", 4, 1), 1: ("dense.f16", 2, 1),
    2: ("Q4_0", 18, 32), 8: ("Q8_0", 34, 32), 9: ("Q8_1", 36, 32),
    10: ("Q2_K", 84, 256), 11: ("Q3_K", 110, 256), 12: ("Q4_K", 144, 256), 13: ("Q5_K", 176, 256), 14: ("Q6_K", 210, 256),
    15: ("Q8_K", 292, 256), 16: ("IQ2_XXS", 66, 256), 17: ("IQ2_XS", 74, 256), 18: ("IQ3_XXS", 98, 256), 19: ("IQ1_S", 50, 256), 21: ("IQ3_S", 110, 256), 22: ("IQ2_S", 82, 256), 29: ("IQ1_M", 56, 256), 34: ("TQ1_0", 54, 256),
}
TYPE_IDS = {name: type_id for type_id, (name, _, _) in GGML_TYPES.items()}

# metadata value types (gguf.h enum gguf_type)
_U8, _I8, _U16, _I16, _U32, _I32, _F32, _BOOL, _STRING, _ARRAY, _U64, _I64, _F64 = range(13)
_SCALARS = {_U8: "<B", _I8: "<b", _U16: "<H", _I16: "<h", _U32: "<I", _I32: "<i", _F32: "<f", _BOOL: "<?", _U64: "<Q", _I64: "<q", _F64: "<d"}


@dataclass(frozen=True)
class TensorInfo:
    name: str
    shape: tuple[int, ...]      # outermost first: (rows, K) for a matrix
    type_id: int
    offset: int                 # from the start of the file
    nbytes: int

    @property
    def encoding(self) -> str:
        return GGML_TYPES[self.type_id][0]


class _Cursor:
    def __init__(self, data, at: int = 0) -> None:
        self.data, self.at = data, at

    def take(self, fmt: str):
        value = struct.unpack_from(fmt, self.data, self.at)
        self.at += struct.calcsize(fmt)
        return value[0]

    def string(self) -> str:
        length = self.take("<Q")
        if length > len(self.data) - self.at:
            raise ValueError("GGUF string runs past the end of the file")
        raw = bytes(self.data[self.at:self.at + length])
        self.at += length
        return raw.decode("utf-8")

    def value(self, kind: int):
        if kind in _SCALARS:
            return self.take(_SCALARS[kind])
        if kind == _STRING:
            return self.string()
        if kind == _ARRAY:
            inner, count = self.take("<I"), self.take("<Q")
            return [self.value(inner) for _ in range(count)]
        raise ValueError(f"unknown GGUF metadata type {kind}")


def tensor_nbytes(type_id: int, shape: tuple[int, ...]) -> int:
    if type_id not in GGML_TYPES:
        raise NotImplementedError(f"GGML type {type_id} is not on the quantized matrix path of this build")
    _, storage, elements = GGML_TYPES[type_id]
    if shape[-1] % elements:
        raise ValueError(f"innermost extent {shape[-1]} does not hold whole records of {elements} elements")
    return int(np.prod(shape[:-1], dtype=np.int64)) * (shape[-1] // elements) * storage


class GGUFFile:
    """A mapped GGUF file: ``metadata`` (dict), ``tensors`` (name -> TensorInfo), ``buffer(name)``."""

    def __init__(self, path) -> None:
        self.path = Path(path)
        self._file = open(self.path, "rb")
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ)
        cursor = _Cursor(self._map)
        if bytes(self._map[:4]) != MAGIC:
            raise ValueError(f"{self.path} is not a GGUF file")
        cursor.at = 4
        self.version = cursor.take("<I")
        if self.version not in (2, 3):
            raise NotImplementedError(f"GGUF version {self.version}")
        tensor_count, kv_count = cursor.take("<Q"), cursor.take("<Q")
        self.metadata: dict[str, Any] = {}
        for _ in range(kv_count):
            key = cursor.string()
            self.metadata[key] = cursor.value(cursor.take("<I"))
        directory = []
        for _ in range(tensor_count):
            name = cursor.string()
            dims = [cursor.take("<Q") for _ in range(cursor.take("<I"))]
            type_id, offset = cursor.take("<I"), cursor.take("<Q")
            directory.append((name, tuple(reversed(dims)), type_id, offset))
        alignment = int(self.metadata.get("general.alignment", DEFAULT_ALIGNMENT))
        self.data_start = (cursor.at + alignment - 1) // alignment * alignment
        self.tensors: dict[str, TensorInfo] = {}
        for name, shape, type_id, offset in directory:
            nbytes = tensor_nbytes(type_id, shape) if type_id in GGML_TYPES else 0
            if self.data_start + offset + nbytes > len(self._map):
                raise ValueError(f"tensor {name} runs past the end of the file")
            self.tensors[name] = TensorInfo(name, shape, type_id, self.data_start + offset, nbytes)

    def raw(self, name: str) -> np.ndarray:
        """The tensor's bytes as a read-only uint8 view of the mapping."""
        info = self.tensors[name]
        if info.type_id not in GGML_TYPES:
            raise NotImplementedError(f"tensor {name} has GGML type {info.type_id}, which this build does not read")
        return np.frombuffer(self._map, dtype=np.uint8, count=info.nbytes, offset=info.offset)

    def buffer(self, name: str, device=None):
        """A runtime Buffer over the tensor: host memory by default (the C ABI stages or finds it resident),
        or a copy on ``device`` (a torch device) when given."""
        from .runtime import Buffer

        info = self.tensors[name]
        storage = self.raw(name)
        if info.encoding.startswith("dense."):
            dtype = np.float32 if info.encoding == "dense.f32" else np.float16
            dense = storage.view(dtype).reshape(info.shape)
            if device is not None:
                import torch

                return torch.from_numpy(np.array(dense)).to(device)
            return Buffer(dense, shape=info.shape, encoding=info.encoding)
        if device is not None:
            import torch

            storage = torch.from_numpy(np.array(storage)).to(device)
        return Buffer(storage, shape=info.shape, encoding=info.encoding)

    def close(self) -> None:
        """Tensor views and Buffers borrow the mapping: while any is alive the mapping stays (it is released
        with the last of them), only the file handle is closed here."""
        try:
            self._map.close()
        except BufferError:
            pass
        self._file.close()

    def __enter__(self) -> "GGUFFile":
        return self

    def __exit__(self, *exc) -> None:
        self.close()


def read(path) -> GGUFFile:
    return GGUFFile(path)


def _put_string(out: bytearray, text: str) -> None:
    raw = text.encode("utf-8")
    out += struct.pack("<Q", len(raw)) + raw


def _put_value(out: bytearray, value) -> None:
    if isinstance(value, bool):
        out += struct.pack("<I?", _BOOL, value)
    elif isinstance(value, int):
        out += struct.pack("<Iq", _I64, value) if value < 0 else struct.pack("<IQ", _U64, value)
    elif isinstance(value, float):
        out += struct.pack("<If", _F32, value)
    elif isinstance(value, str):
        out += struct.pack("<I", _STRING)
        _put_string(out, value)
    elif isinstance(value, (list, tuple)) and value and all(isinstance(v, str) for v in value):
        out += struct.pack("<IIQ", _ARRAY, _STRING, len(value))
        for v in value:
            _put_string(out, v)
    else:
        raise TypeError(f"metadata value {value!r} is not supported by this writer")


def write(path, tensors: Mapping[str, tuple[str, tuple[int, ...], np.ndarray]], metadata: Mapping[str, Any] | None = None,
          alignment: int = DEFAULT_ALIGNMENT) -> None:
    """``tensors``: name -> (encoding name, logical shape outermost first, packed bytes or dense array)."""
    metadata = dict(metadata or {})
    if alignment != DEFAULT_ALIGNMENT:
        metadata["general.alignment"] = alignment
    out = bytearray(MAGIC + struct.pack("<IQQ", 3, len(tensors), len(metadata)))
    for key, value in metadata.items():
        _put_string(out, key)
        if key == "general.alignment":
            out += struct.pack("<II", _U32, value)
        else:
            _put_value(out, value)
    offset, payloads = 0, []
    for name, (encoding, shape, data) in tensors.items():
        type_id = TYPE_IDS[encoding]
        raw = np.ascontiguousarray(data).reshape(-1).view(np.uint8)
        if raw.size != tensor_nbytes(type_id, tuple(shape)):
            raise ValueError(f"tensor {name}: {raw.size} bytes for shape {tuple(shape)} of {encoding}")
        _put_string(out, name)
        out += struct.pack("<I", len(shape)) + b"".join(struct.pack("<Q", d) for d in reversed(shape))
        out += struct.pack("<IQ", type_id, offset)
        payloads.append((offset, raw))
        offset = (offset + raw.size + alignment - 1) // alignment * alignment
    out += b"\0" * (-len(out) % alignment)
    start = len(out)
    for at, raw in payloads:
        out += b"\0" * (start + at - len(out))
        out += raw.tobytes()
    Path(path).write_bytes(bytes(out))


assert all(RECORDS[name][:2] == (storage, elements) for name, storage, elements in GGML_TYPES.values() if name in RECORDS)
