// Helpers shared by the tensor-core prefill kernels: operand layouts in shared memory, packed fp32 pairs,
// shared-memory accesses by 32-bit window address.
#pragma once

#include "tcgen05.cuh"
#include "tensormap.cuh"

namespace weft {

// byte offset of (row, 16-byte chunk 0..7) inside a 128-byte-swizzled slab
__device__ __forceinline__ uint32_t sw128_offset(int row, int chunk) {
    return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4));
}
// byte offset of (row, 16-byte chunk) in an unswizzled K-major operand: 8-row groups of `chunks` core matrices
__device__ __forceinline__ uint32_t core_offset(int row, int chunk, int chunks) {
    return (uint32_t)((row >> 3) * (chunks * 128) + chunk * 128 + (row & 7) * 16);
}

// Packed pairs of fp32 (sm_100 executes add / mul / fma on two floats held in a 64-bit register pair with one
// instruction; each lane of the pair is an ordinary IEEE round-to-nearest operation).
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
// The integers of two accumulator columns as floats, exactly, on the full-rate fp32 pipe (the conversion
// unit runs at a quarter of it): |v| <= 256 * 105 * 128 < 2^22, so adding the integer to the bit pattern of
// 1.5 * 2^23 and subtracting that constant gives its exact float.
__device__ __forceinline__ uint64_t ints_to_float2(uint32_t a, uint32_t b) {
    return add2(pack2(__uint_as_float(a + 0x4b400000u), __uint_as_float(b + 0x4b400000u)), pack2(-12582912.f, -12582912.f));
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    return (uint32_t)__half_as_ushort(__float2half_rn(lo)) | ((uint32_t)__half_as_ushort(__float2half_rn(hi)) << 16);
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts_u32(uint32_t addr, uint32_t v) { asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory"); }
__device__ __forceinline__ void sts_u16(uint32_t addr, uint32_t v) { asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"((unsigned short)v) : "memory"); }
__device__ __forceinline__ void sts_u128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

}  // namespace weft
