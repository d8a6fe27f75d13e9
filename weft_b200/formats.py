"""The GGML record layouts on the quantized matrix path, declared with ``@weft.encoding``.

These are the hot-path encodings of the reference's examples/formats/ggml.py (Q4_0 :16-22,
Q8_0 :56-62, Q2_K :64-72, Q3_K :75-84, Q4_K :88-97, Q5_K :100-110, Q6_K :113-120, IQ1_S :123-130, IQ1_M :133-139, IQ2_S :142-151, IQ2_XS :154-161, IQ3_S :189-198, IQ2_XXS :164-170, I8X8 :173-178, I8X4 :181-186, IQ3_XXS :201-208, TQ1_0 :231-238, Q8_K :276-283), byte for
byte the block structs of ggml-common.h:184-189,241-246,266-271,317-328,361-366,371-375.  A kernel
file may use these or the reference's own declarations: ``weft.compile`` identifies an Encoding by
its name and checks the record geometry, not the declaring module.
"""
from __future__ import annotations

from . import language as wl
from .api import derive, encoding

_LE = (wl.bitorder.lsb_first, wl.byteorder.little)


@encoding
class Q4_0:                      # 18 bytes / 32 elements
    layout = _LE
    alignment = 2
    elements = 32
    d: wl.f16                    # @0
    q: wl.u4[32] @ wl.grouped(elements=32) @ wl.bit_layers(elements=16, order=wl.lo_first)   # @2: byte j = elem j | elem j+16 << 4


@encoding
class Q8_0:                      # 34 bytes / 32 elements
    layout = _LE
    alignment = 2
    elements = 32
    d: wl.f16
    q: wl.i8[32]


@encoding
class Q2_K:                      # 84 bytes / 256 elements
    layout = _LE
    alignment = 2
    elements = 256
    scales: wl.u8[16]            # @0: low nibble scale, high nibble min, one per 16 weights
    q: wl.u2[256] @ wl.grouped(elements=128) @ wl.bit_layers(elements=32, order=wl.lo_first)   # @16
    d: wl.f16                    # @80
    dmin: wl.f16                 # @82


@encoding
class Q3_K:                      # 110 bytes / 256 elements
    layout = _LE
    alignment = 2
    elements = 256
    hmask: wl.u1[256] @ wl.grouped(elements=256) @ wl.bit_layers(elements=32, order=wl.lo_first)   # @0
    q: wl.u2[256] @ wl.grouped(elements=128) @ wl.bit_layers(elements=32, order=wl.lo_first)       # @32
    scale_low: wl.u4[16] @ wl.grouped(elements=16) @ wl.bit_layers(elements=8, order=wl.lo_first)  # @96
    scale_high: wl.u2[16] @ wl.grouped(elements=16) @ wl.bit_layers(elements=4, order=wl.lo_first) # @104
    d: wl.f16                    # @108


@encoding
class Q8_1:                      # 36 bytes / 32 elements (examples/formats/ggml.py:266-273)
    layout = _LE
    alignment = 2
    elements = 32
    d: wl.f16
    s: wl.f16                    # f16(sum of codes * d)
    q: wl.i8[32]


@encoding
class Q4_K:                      # 144 bytes / 256 elements
    layout = _LE
    alignment = 2
    elements = 256
    d: wl.f16                    # @0
    dmin: wl.f16                 # @2
    sc: wl.u6[8] @ wl.pack_fields(group=4, fields=2, low_bits=4, order=wl.lo_first)   # @4, 12 bytes shared with m
    m: wl.u6[8] @ wl.pack_fields(group=4, fields=2, low_bits=4, order=wl.lo_first)
    q: wl.u4[256] @ wl.grouped(elements=64) @ wl.bit_layers(elements=32, order=wl.lo_first)   # @16


@encoding
class Q5_K:                      # 176 bytes / 256 elements
    layout = _LE
    alignment = 2
    elements = 256
    d: wl.f16                    # @0
    dmin: wl.f16                 # @2
    sc: wl.u6[8] @ wl.pack_fields(group=4, fields=2, low_bits=4, order=wl.lo_first)   # @4, 12 bytes shared with m
    m: wl.u6[8] @ wl.pack_fields(group=4, fields=2, low_bits=4, order=wl.lo_first)
    qh: wl.u1[256] @ wl.grouped(elements=256) @ wl.bit_layers(elements=32, order=wl.lo_first)   # @16
    q: wl.u4[256] @ wl.grouped(elements=64) @ wl.bit_layers(elements=32, order=wl.lo_first)     # @48


@encoding
class Q6_K:                      # 210 bytes / 256 elements; no alignment stated by the reference: any byte address
    layout = _LE
    elements = 256
    ql: wl.u4[256] @ wl.grouped(elements=128) @ wl.bit_layers(elements=64, order=wl.lo_first)   # @0, 128 bytes
    qh: wl.u2[256] @ wl.grouped(elements=128) @ wl.bit_layers(elements=32, order=wl.lo_first)   # @128, 64 bytes
    scales: wl.i8[16] @ wl.grouped(elements=16) @ wl.bit_layers(elements=16, order=wl.lo_first)  # @192
    d: wl.f16                    # @208


@encoding
class IQ2_XXS:                   # 66 bytes / 256 elements
    layout = _LE
    alignment = 2
    elements = 256
    d: wl.f16
    q: wl.u16[32]                # per 32 elements: 4 grid indices, then u32 {4 x 7-bit sign index, 4-bit scale}


@encoding
class IQ2_XS:                    # 74 bytes / 256 elements
    layout = _LE
    alignment = 2
    elements = 256
    d: wl.f16
    q: wl.u16[32]                # per 8 elements: 9-bit grid index, 7-bit sign index
    scales: wl.u8[8]             # per 32 elements: low nibble for the first 16, high nibble for the rest


@encoding
class IQ3_XXS:                   # 98 bytes / 256 elements
    layout = _LE
    alignment = 2
    elements = 256
    d: wl.f16
    q: wl.u8[64]                 # per 4 elements: a grid index
    metadata: wl.u32[8]          # per 32 elements: 4 x 7-bit sign index, 4-bit scale


@encoding
class IQ1_S:                     # 50 bytes / 256 elements
    layout = _LE
    alignment = 2
    elements = 256
    d: wl.f16
    q: wl.u8[32]                 # low 8 bits of the grid index of every 8 elements
    qh: wl.u16[8]                # per 32 elements: four 3-bit index tops, 3-bit scale, sign of the shift


@encoding
class IQ1_M:                     # 56 bytes / 256 elements, no d field
    layout = _LE
    elements = 256
    q: wl.u8[32]
    qh: wl.u8[16]                # per 16 elements: two nibbles {3 index bits, shift sign}
    scales: wl.u8[8]             # four u16: 3-bit scales per 16 elements, top nibbles form the record's f16 scale


@encoding
class IQ2_S:                     # 82 bytes / 256 elements
    layout = _LE
    alignment = 2
    elements = 256
    d: wl.f16
    q: wl.u8[32]                 # low 8 bits of the grid index of every 8 elements
    signs: wl.u1[256] @ wl.grouped(elements=8) @ wl.bit_layers(elements=1, order=wl.lo_first)   # 32 bytes
    qh: wl.u8[8]                 # per 32 elements: four 2-bit pairs, index bits 8-9
    scales: wl.u8[8]


@encoding
class IQ3_S:                     # 110 bytes / 256 elements
    layout = _LE
    alignment = 2
    elements = 256
    d: wl.f16
    q: wl.u8[64]                 # low 8 bits of the grid index of every 4 elements
    qh: wl.u1[64] @ wl.grouped(elements=8) @ wl.bit_layers(elements=1, order=wl.lo_first)       # index bit 8
    signs: wl.u1[256] @ wl.grouped(elements=8) @ wl.bit_layers(elements=1, order=wl.lo_first)
    scales: wl.u4[8] @ wl.grouped(elements=2) @ wl.bit_layers(elements=1, order=wl.lo_first)


@encoding
class I8X4:                      # one row of the IQ3_XXS codebook
    layout = _LE
    alignment = 4
    elements = 4
    values: wl.i8[4]


@encoding
class I8X8:                      # one codebook row
    layout = _LE
    alignment = 8
    elements = 8
    values: wl.i8[8]


@encoding
class TQ1_0:                     # 54 bytes / 256 elements
    layout = _LE
    alignment = 2
    elements = 256
    q: wl.u8[48]                 # 5 trits per byte: 32 bytes over 160 elements, 16 bytes over 80
    qh: wl.u8[4]                 # 4 trits per byte over the last 16 elements
    d: wl.f16                    # @52


@encoding
class Q8_K:                      # 292 bytes / 256 elements
    layout = _LE
    alignment = 4
    elements = 256
    ds: wl.f32                   # @0
    q: wl.i8[256]                # @4
    bsum: wl.i16[16]             # @260


@derive
def Q4K_I(W: wl.View[Q4_K, (M, K)], *, rows: wl.static[int]) -> wl.View[Q4K_I[rows], (M, K)]:
    """Persistent interleaved layout (examples/formats/ggml.py:286-290): every cohort of ``rows`` rows keeps
    its Q4_K records but stores them byte-major -- byte b of row r of a block at ``rows * b + r``
    (doc/dsl/encoding-and-artifacts.md:209).  ``Q4K_I[16]`` is the member this build executes; the packed
    object is produced by the kernels' ``_W_pack`` artifact functions (``weft_b200.artifacts``)."""
    return wl.interleave(W, rows=rows)


#: name -> (storage bytes per record, logical elements per record, alignment)
RECORDS = {"Q4_0": (18, 32, 2), "Q8_0": (34, 32, 2), "Q8_1": (36, 32, 2), "Q2_K": (84, 256, 2), "Q3_K": (110, 256, 2), "Q4_K": (144, 256, 2), "Q5_K": (176, 256, 2), "Q6_K": (210, 256, 1), "IQ2_XXS": (66, 256, 2), "IQ2_XS": (74, 256, 2), "IQ3_XXS": (98, 256, 2), "IQ2_S": (82, 256, 2), "IQ3_S": (110, 256, 2), "IQ1_S": (50, 256, 2), "IQ1_M": (56, 256, 1),
           "TQ1_0": (54, 256, 2), "Q8_K": (292, 256, 4), "I8X8": (8, 8, 8), "I8X4": (4, 4, 4)}

#: numbering of the reference harnesses (examples/repro/weft/vec_dot_runtime.cpp:185-344), used by the C ABI
FORMAT_IDS = {"Q4_0": 1, "Q8_0": 5, "Q2_K": 6, "Q3_K": 7, "Q4_K": 8, "Q5_K": 9, "Q6_K": 10, "IQ1_S": 11, "IQ1_M": 12, "IQ2_S": 13, "IQ2_XS": 14, "IQ2_XXS": 15, "IQ3_S": 16, "IQ3_XXS": 17, "TQ1_0": 20}

TQ1_POWERS = (1, 3, 9, 27, 81)


def row_bytes(name: str, k: int) -> int:
    storage, elements, _ = RECORDS[name]
    if k % elements:
        raise ValueError(f"K = {k} does not contain complete {name} records")
    return k // elements * storage
