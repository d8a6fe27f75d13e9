"""``Buffer``: a borrowed, contiguous storage object with an explicit logical shape and Encoding.

Same contract as the reference (python/weft/runtime/buffer.py:33-63): no copy, dense Encodings
inferred from the element format (``dense.f32`` ...), packed storage requires an explicit ``shape``
(logical elements) and ``encoding`` (layout identity such as ``"Q4_K"``).  On top of host objects
that speak the buffer protocol, device memory is accepted: anything exposing
``__cuda_array_interface__`` (CuPy, Numba) and torch tensors on either side.  Attributes:
``shape``, ``encoding``, ``address``, ``nbytes``, ``readonly`` and, new here, ``device`` (None for
host memory, the CUDA ordinal otherwise).
"""
from __future__ import annotations

from collections.abc import Sequence

_FORMAT_TO_DENSE = {"b": "i8", "B": "u8", "h": "i16", "H": "u16", "i": "i32", "I": "u32", "q": "i64", "Q": "u64",
                    "e": "f16", "f": "f32", "d": "f64", "?": "i1"}
_TYPESTR_TO_DENSE = {"i1": "i8", "u1": "u8", "i2": "i16", "u2": "u16", "i4": "i32", "u4": "u32", "i8": "i64",
                     "u8": "u64", "f2": "f16", "f4": "f32", "f8": "f64", "b1": "i1"}
_TORCH_TO_DENSE = {"torch.int8": "i8", "torch.uint8": "u8", "torch.int16": "i16", "torch.int32": "i32",
                   "torch.int64": "i64", "torch.float16": "f16", "torch.bfloat16": "bf16", "torch.float32": "f32",
                   "torch.float64": "f64", "torch.bool": "i1", "torch.uint16": "u16", "torch.uint32": "u32"}


def _dense_from_format(fmt: str, itemsize: int) -> str | None:
    spelling = fmt.lstrip("@=<")
    if spelling in ("l", "L") and itemsize in (4, 8):
        return "dense." + ("i" if spelling == "l" else "u") + str(itemsize * 8)
    if spelling in _FORMAT_TO_DENSE:
        return "dense." + _FORMAT_TO_DENSE[spelling]
    return None


class Buffer:
    """A borrowed contiguous storage object with an explicit logical Encoding."""

    def __init__(self, data: object, *, shape: Sequence[int] | None = None, encoding: str | None = None) -> None:
        inferred = None
        if _is_torch_tensor(data):
            if not data.is_contiguous():
                raise ValueError("the current kernel ABI requires contiguous Encoding storage")
            self.address = int(data.data_ptr())
            self.nbytes = int(data.numel() * data.element_size())
            self.readonly = False
            self.device = data.device.index if data.is_cuda else None
            natural = tuple(int(e) for e in data.shape)
            dense = _TORCH_TO_DENSE.get(str(data.dtype))
            inferred = None if dense is None else "dense." + dense
        elif hasattr(data, "__cuda_array_interface__"):
            iface = data.__cuda_array_interface__
            if iface.get("strides") is not None and not _c_contiguous(iface["shape"], iface["strides"], iface["typestr"]):
                raise ValueError("the current kernel ABI requires contiguous Encoding storage")
            self.address, self.readonly = int(iface["data"][0]), bool(iface["data"][1])
            itemsize = int(iface["typestr"][2:])
            natural = tuple(int(e) for e in iface["shape"])
            count = 1
            for extent in natural:
                count *= extent
            self.nbytes = count * itemsize
            self.device = _device_of(self.address)
            dense = _TYPESTR_TO_DENSE.get(iface["typestr"][1:])
            inferred = None if dense is None else "dense." + dense
        else:
            view = memoryview(data)
            if not view.c_contiguous:
                raise ValueError("the current kernel ABI requires contiguous Encoding storage")
            import ctypes

            self.readonly = bool(view.readonly)
            self.nbytes = view.nbytes
            if view.nbytes:
                flat = view.cast("B") if view.format != "B" or view.ndim != 1 else view
                self.address = ctypes.addressof(ctypes.c_char.from_buffer(flat)) if not view.readonly else _readonly_address(flat)
            else:
                self.address = 0
            self.device = None
            natural = tuple(view.shape)
            inferred = _dense_from_format(view.format, view.itemsize)
            self._view = view
        if encoding is None:
            if inferred is None:
                raise TypeError("this buffer's element format needs an explicit Encoding")
            encoding = inferred
        if not isinstance(encoding, str) or not encoding:
            raise TypeError("buffer Encoding must be a non-empty layout identity")
        logical = tuple(natural if shape is None else shape)
        if any(type(extent) is not int or extent < 0 for extent in logical):
            raise ValueError("logical buffer extents must be non-negative integers")
        self._owner = data           # keeps the storage alive for as long as the Buffer lives
        self.shape = logical
        self.encoding = encoding

    def __repr__(self) -> str:
        where = "host" if self.device is None else f"cuda:{self.device}"
        return f"Buffer({self.encoding}, shape={self.shape}, {self.nbytes} bytes, {where})"


def _is_torch_tensor(data: object) -> bool:
    cls = type(data)
    return cls.__module__.startswith("torch") and hasattr(data, "data_ptr") and hasattr(data, "element_size")


def _c_contiguous(shape, strides, typestr) -> bool:
    expected = int(typestr[2:])
    for extent, stride in zip(reversed(shape), reversed(strides)):
        if extent != 1 and stride != expected:
            return False
        expected *= extent
    return True


def _readonly_address(flat: memoryview) -> int:
    import numpy as np

    return int(np.frombuffer(flat, dtype=np.uint8).ctypes.data)


def _device_of(address: int) -> int | None:
    return 0
