"""A layer-level driver for decode: the projections of a transformer block issued as one call.

At batch 1 every projection is a GEMV of a few microseconds, so the cost of getting from one to the next
matters as much as the kernels: ``ProjectionChain`` hands the whole sequence to the C ABI in one call
(``weft_b200_mul_mat_chain``), where consecutive kernels overlap on the stream (the next one streams its first
weights while the previous one drains), and the call can be captured into a CUDA graph and replayed per token.
Only the quantized mul_mats are driven here -- attention, normalisation and activation functions are not part
of this library -- so a step's input is whatever buffer the caller binds to it.

``llama_block_steps`` lists the seven projections of a Llama-style block from a GGUF file's tensor names
(blk.<i>.attn_q / attn_k / attn_v / attn_output / ffn_gate / ffn_up / ffn_down .weight).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Sequence

from .formats import FORMAT_IDS, row_bytes

LLAMA_PROJECTIONS = ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down")


class _Step(ctypes.Structure):          # struct weft_b200_mul_mat_step of include/weft_b200.h
    _fields_ = [("format", ctypes.c_int), ("flags", ctypes.c_uint), ("W", ctypes.c_void_p), ("X", ctypes.c_void_p),
                ("Xq", ctypes.c_void_p), ("Y", ctypes.c_void_p), ("grid", ctypes.c_void_p), ("signs", ctypes.c_void_p),
                ("powers", ctypes.c_void_p), ("N", ctypes.c_size_t), ("K", ctypes.c_size_t), ("M", ctypes.c_size_t)]


@dataclass
class Projection:
    """One mul_mat of the chain.  Addresses are device (or host) pointers as the C ABI takes them."""
    encoding: str
    w: int
    x: int
    xq: int
    y: int
    n: int
    k: int
    m: int = 1
    reuse_xq: bool = False      # Xq already holds this step's quantized input (written by an earlier step)
    grid: int = 0
    signs: int = 0
    powers: int = 0

    @property
    def weight_bytes(self) -> int:
        return self.n * row_bytes(self.encoding, self.k)


class ProjectionChain:
    def __init__(self, lib, projections: Sequence[Projection]) -> None:
        self._lib = lib
        self.projections = list(projections)
        lib.weft_b200_mul_mat_chain.argtypes = [ctypes.c_void_p, ctypes.c_size_t]
        lib.weft_b200_mul_mat_chain.restype = ctypes.c_int
        self._table = (_Step * len(self.projections))()
        for slot, p in zip(self._table, self.projections):
            if p.encoding not in FORMAT_IDS:
                raise ValueError(f"{p.encoding} is not a weight format of this library")
            slot.format, slot.flags = FORMAT_IDS[p.encoding], 1 if p.reuse_xq else 0
            slot.W, slot.X, slot.Xq, slot.Y = p.w, p.x, p.xq, p.y
            slot.grid, slot.signs, slot.powers = p.grid or None, p.signs or None, p.powers or None
            slot.N, slot.K, slot.M = p.n, p.k, p.m

    @property
    def weight_bytes(self) -> int:
        return sum(p.weight_bytes for p in self.projections)

    def run(self) -> None:
        if self._lib.weft_b200_mul_mat_chain(ctypes.addressof(self._table), len(self.projections)):
            from .runtime.driver import last_error

            raise RuntimeError("weft_b200_mul_mat_chain: " + last_error(self._lib))


def llama_block_steps(model, block: int) -> list[tuple[str, str, int, int]]:
    """(tensor name, encoding, N, K) of the seven projections of block ``block`` of a mapped GGUF model."""
    steps = []
    for part in LLAMA_PROJECTIONS:
        name = f"blk.{block}.{part}.weight"
        info = model.tensors[name]
        if len(info.shape) != 2:
            raise ValueError(f"{name} is not a matrix")
        steps.append((name, info.encoding, info.shape[0], info.shape[1]))
    return steps
