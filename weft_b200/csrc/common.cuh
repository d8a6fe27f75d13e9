// Shared device helpers for the sm_100a quantized-matrix kernels.
//
// Record layouts are the GGML block formats of the reference
// (source/c/ggml/llama.cpp/ggml/src/ggml-common.h:184-189 Q4_0, :241-246 Q8_0,
// :266-271 TQ1_0, :317-328 Q4_K, :361-366 Q8_K, :371-375 IQ2_XXS), read in place:
// the kernels never repack weights.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace weft {

enum Format : int { F_Q4_0 = 1, F_Q8_0 = 5, F_Q2_K = 6, F_Q3_K = 7, F_Q4_K = 8, F_Q5_K = 9, F_Q6_K = 10, F_IQ1_S = 11, F_IQ1_M = 12, F_IQ2_S = 13, F_IQ2_XS = 14, F_IQ2_XXS = 15, F_IQ3_S = 16, F_IQ3_XXS = 17, F_TQ1_0 = 20, F_Q8_K = 100, F_Q8_1 = 101,
                    F_Q4_K_I16 = 1008 /* Q4_K records, 16 rows byte-interleaved (derived Encoding Q4K_I[16]) */ };

__host__ __device__ constexpr int record_bytes(int fmt) {
    return fmt == F_Q4_0 ? 18 : fmt == F_Q8_0 ? 34 : (fmt == F_Q4_K || fmt == F_Q4_K_I16) ? 144 : fmt == F_Q2_K ? 84 : fmt == F_Q3_K ? 110 : fmt == F_Q5_K ? 176 : fmt == F_Q6_K ? 210 : fmt == F_IQ2_XXS ? 66 : fmt == F_IQ2_XS ? 74 : fmt == F_IQ3_XXS ? 98 : fmt == F_IQ2_S ? 82 : fmt == F_IQ3_S ? 110 : fmt == F_IQ1_S ? 50 : fmt == F_IQ1_M ? 56
         : fmt == F_TQ1_0 ? 54 : fmt == F_Q8_K ? 292 : fmt == F_Q8_1 ? 36 : 0;
}
__host__ __device__ constexpr int record_elements(int fmt) {
    return (fmt == F_Q4_0 || fmt == F_Q8_0 || fmt == F_Q8_1) ? 32 : 256;
}
// Every kernel walks rows in units of 256 logical elements: one K-family record, or eight
// consecutive 32-element records (8*18 = 144 B, 8*34 = 272 B, both multiples of 16 bytes).
__host__ __device__ constexpr int unit_bytes(int fmt) { return record_bytes(fmt) * (256 / record_elements(fmt)); }
__host__ __device__ constexpr int activation_of(int fmt) { return (fmt == F_Q4_0 || fmt == F_Q8_0) ? F_Q8_0 : F_Q8_K; }

// Device-side status codes written to the mapped status word (first error wins).
enum Status : int { ST_OK = 0, ST_WAIT_TIMEOUT = 1, ST_TMEM_ALLOC = 2 };

__device__ __forceinline__ void report(int *status, int code) {
    if (status) atomicCAS(status, 0, code);
}

__device__ __forceinline__ float half_bits_to_float(uint32_t h) {
    return __half2float(__ushort_as_half((unsigned short)(h & 0xffffu)));
}

__device__ __forceinline__ uint32_t ld_u16(const uint8_t *p) { return *reinterpret_cast<const uint16_t *>(p); }
// 32 bits from a 2-byte aligned address
__device__ __forceinline__ uint32_t ld_u32_a2(const uint8_t *p) { return ld_u16(p) | (ld_u16(p + 2) << 16); }

// NW 32-bit words starting at a 2-byte aligned address: NW+1 aligned loads and a funnel shift.
// Reads up to 2 bytes past the last word; callers keep that slack inside their buffer.
template <int NW>
__device__ __forceinline__ void ld_words_a2(const uint8_t *p, uint32_t (&out)[NW]) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    const uint32_t *base = reinterpret_cast<const uint32_t *>(a & ~uintptr_t(3));
    const uint32_t shift = (uint32_t)(a & 3u) * 8u;
    uint32_t prev = base[0];
#pragma unroll
    for (int i = 0; i < NW; ++i) {
        const uint32_t next = base[i + 1];
        out[i] = __funnelshift_r(prev, next, shift);
        prev = next;
    }
}

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- mbarrier + bulk async copy (TMA without a tensor map: contiguous bytes, 16-byte granules) ----

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return done != 0;
}
// Bounded wait: gives up after `limit` polls (each poll itself blocks for a hardware-defined
// time slice), so a copy that never lands ends the kernel with a status code, not a hang.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t limit = 1u << 22) {
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// global -> shared, `bytes` a multiple of 16, both addresses 16-byte aligned
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_addr(dst)), "l"(src), "r"(bytes), "r"(smem_addr(bar)) : "memory");
}

// four int8 x int8 products added to c; _ss: both operands signed, _us: a unsigned, b signed
__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// The 6-bit (scale, min) pairs of a Q4_K record as four packed byte vectors
// (ggml-quants.c:822-829 get_scale_min_k4; same unpack as ggml-cpu/quants.c:688-693).
struct Q4KScales { uint32_t sc_lo, sc_hi, mn_lo, mn_hi; };   // sc[0..3], sc[4..7], m[0..3], m[4..7]
__device__ __forceinline__ Q4KScales q4k_unpack_scales(uint32_t s0, uint32_t s1, uint32_t s2) {
    Q4KScales r;
    r.sc_lo = s0 & 0x3f3f3f3fu;
    r.mn_lo = s1 & 0x3f3f3f3fu;
    r.sc_hi = (s2 & 0x0f0f0f0fu) | (((s0 >> 6) & 0x03030303u) << 4);
    r.mn_hi = ((s2 >> 4) & 0x0f0f0f0fu) | (((s1 >> 6) & 0x03030303u) << 4);
    return r;
}
__device__ __forceinline__ uint32_t byte_of(uint32_t v, int i) { return (v >> (8 * i)) & 0xffu; }

// The sixteen 6-bit scales of a Q3_K record (stored plus 32) as four packed byte vectors, scale g in byte g % 4
// of word g / 4 (ggml-quants.c:1264-1269; same unpack as ggml-cpu/quants.c:620-625).
__device__ __forceinline__ void q3k_unpack_scales(uint32_t s0, uint32_t s1, uint32_t s2, uint32_t (&out)[4]) {
    out[0] = (s0 & 0x0f0f0f0fu) | ((s2 & 0x03030303u) << 4);
    out[1] = (s1 & 0x0f0f0f0fu) | (((s2 >> 2) & 0x03030303u) << 4);
    out[2] = ((s0 >> 4) & 0x0f0f0f0fu) | (((s2 >> 4) & 0x03030303u) << 4);
    out[3] = ((s1 >> 4) & 0x0f0f0f0fu) | (((s2 >> 6) & 0x03030303u) << 4);
}

// One base-3 digit (0 = most significant) of a packed TQ1_0 byte, as -1/0/+1
// (ggml-quants.c:2369-2371; examples/functions/quantization.py:49-64). `power` is powers[digit]
// narrowed to 8 bits as the DSL does.
__device__ __forceinline__ int tq1_digit(uint32_t packed, uint32_t power) {
    const uint32_t wrapped = (packed * (power & 0xffu)) & 0xffu;
    return (int)((wrapped * 3u) >> 8) - 1;
}

// digits of four packed bytes at once: ((byte*power) & 255) * 3 >> 8, in 16-bit lanes
__device__ __forceinline__ uint32_t tq1_digits4(uint32_t q4, uint32_t power) {
    const uint32_t M = 0x00ff00ffu;
    uint32_t e = ((q4 & M) * power) & M, o = (((q4 >> 8) & M) * power) & M;
    e = ((e * 3u) >> 8) & M;
    o = ((o * 3u) >> 8) & M;
    return e | (o << 8);
}

}  // namespace weft
