// row_dequantize_<fmt>: packed records -> fp32, bit-exact with the reference's GGML semantics.
//
// HBM-bound and write-dominated (4 bytes out per 0.5..1.06 bytes in).  A weight matrix (N, K) is a
// contiguous stream of records and its fp32 image a contiguous stream of floats, so every kernel
// here is flat: one warp owns one 256-element unit per step and every lane stores whole float4s
// that are contiguous across the warp (128-byte segments, no partial sectors).
//
// Float op trees follow the reference exactly and are spelled with __fmul_rn/__fsub_rn so the
// compiler cannot contract them:
//   Q4_0/Q8_0  f32(q - zero) * f32(d)            examples/functions/quantization.py:6-7,  ggml-quants.c:401-419,495-509
//   Q4_K       (d*sc)*q - (dmin*m)               quantization.py:14-17,                   ggml-quants.c:1471-1493
//   IQ2_XXS    (d*(0.5+s)*0.25) * (grid*sign)    examples/kernels/dequantize/iq2_xxs.py:9-53, ggml-quants.c:2416-2440
//   TQ1_0      f32(trit-1) * d                   examples/kernels/dequantize/tq1_0.py:9-46,   ggml-quants.c:2356-2393
//   Q2_K       (d*sc)*q2 - (dmin*m)              examples/kernels/dequantize/q2_k.py:8-17,    ggml-quants.c:903-933
//   Q3_K       (d*(scale-32)) * (q3 - 4)         examples/kernels/dequantize/q3_k.py:8-17,    ggml-quants.c:1247-1294
//   Q5_K       (d*sc)*q5 - (dmin*m)              examples/kernels/dequantize/q5_k.py:9-15,    ggml-quants.c:1673-1698
//   Q6_K       (d*scale) * (q6 - 32)             examples/kernels/dequantize/q6_k.py:8-14,    ggml-quants.c:1881-1910
#include "common.cuh"
#include "kernels.h"

namespace weft {

template <bool A4>
__device__ __forceinline__ uint32_t ldw(const uint8_t *p) {
    if (A4) return __ldg(reinterpret_cast<const uint32_t *>(p));
    return ld_u32_a2(p);
}

__device__ __forceinline__ void st4(float *y, float a, float b, float c, float d) {
    __stcs(reinterpret_cast<float4 *>(y), make_float4(a, b, c, d));   // streaming store: output is never re-read
}

constexpr int DQ_WARPS = 8;

// ---- Q4_K: lane = (64-element group j, 4-byte slice t): low nibbles -> 64j+4t.., high -> 64j+32+4t..
template <bool A4>
__global__ void __launch_bounds__(DQ_WARPS * 32) dequant_q4_k_kernel(const uint8_t *__restrict__ w, float *__restrict__ y, long long units) {
    const int lane = threadIdx.x & 31;
    const int j = lane >> 3, t = lane & 7;
    for (long long u = (long long)blockIdx.x * DQ_WARPS + (threadIdx.x >> 5); u < units; u += (long long)gridDim.x * DQ_WARPS) {
        const uint8_t *rec = w + u * 144;
        const uint32_t dd = ldw<A4>(rec);
        const Q4KScales s = q4k_unpack_scales(ldw<A4>(rec + 4), ldw<A4>(rec + 8), ldw<A4>(rec + 12));
        const uint32_t q = ldw<A4>(rec + 16 + 32 * j + 4 * t);
        const float d = half_bits_to_float(dd), dmin = half_bits_to_float(dd >> 16);
        // scale index 2j and 2j+1
        const uint32_t scv = j < 2 ? s.sc_lo : s.sc_hi, mnv = j < 2 ? s.mn_lo : s.mn_hi;
        const int b0 = (2 * j) & 3;
        const float d1 = __fmul_rn(d, (float)byte_of(scv, b0)), m1 = __fmul_rn(dmin, (float)byte_of(mnv, b0));
        const float d2 = __fmul_rn(d, (float)byte_of(scv, b0 + 1)), m2 = __fmul_rn(dmin, (float)byte_of(mnv, b0 + 1));
        float lo[4], hi[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t b = byte_of(q, i);
            lo[i] = __fsub_rn(__fmul_rn(d1, (float)(b & 15u)), m1);
            hi[i] = __fsub_rn(__fmul_rn(d2, (float)(b >> 4)), m2);
        }
        float *out = y + u * 256 + 64 * j + 4 * t;
        st4(out, lo[0], lo[1], lo[2], lo[3]);
        st4(out + 32, hi[0], hi[1], hi[2], hi[3]);
    }
}

// ---- Q5_K (176 bytes: the Q4_K header, qh[32] fifth bits, qs[128]): same lane map as Q4_K; sub-block g of
// weight byte l takes bit g of qh[l].
template <bool A4>
__global__ void __launch_bounds__(DQ_WARPS * 32) dequant_q5_k_kernel(const uint8_t *__restrict__ w, float *__restrict__ y, long long units) {
    const int lane = threadIdx.x & 31;
    const int j = lane >> 3, t = lane & 7;
    for (long long u = (long long)blockIdx.x * DQ_WARPS + (threadIdx.x >> 5); u < units; u += (long long)gridDim.x * DQ_WARPS) {
        const uint8_t *rec = w + u * 176;
        const uint32_t dd = ldw<A4>(rec);
        const Q4KScales s = q4k_unpack_scales(ldw<A4>(rec + 4), ldw<A4>(rec + 8), ldw<A4>(rec + 12));
        const uint32_t h = ldw<A4>(rec + 16 + 4 * t) >> (2 * j);
        const uint32_t q = ldw<A4>(rec + 48 + 32 * j + 4 * t);
        const float d = half_bits_to_float(dd), dmin = half_bits_to_float(dd >> 16);
        const uint32_t scv = j < 2 ? s.sc_lo : s.sc_hi, mnv = j < 2 ? s.mn_lo : s.mn_hi;
        const int b0 = (2 * j) & 3;
        const float d1 = __fmul_rn(d, (float)byte_of(scv, b0)), m1 = __fmul_rn(dmin, (float)byte_of(mnv, b0));
        const float d2 = __fmul_rn(d, (float)byte_of(scv, b0 + 1)), m2 = __fmul_rn(dmin, (float)byte_of(mnv, b0 + 1));
        float lo[4], hi[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t b = byte_of(q, i), hb = byte_of(h, i);
            lo[i] = __fsub_rn(__fmul_rn(d1, (float)((b & 15u) | ((hb & 1u) << 4))), m1);
            hi[i] = __fsub_rn(__fmul_rn(d2, (float)((b >> 4) | ((hb & 2u) << 3))), m2);
        }
        float *out = y + u * 256 + 64 * j + 4 * t;
        st4(out, lo[0], lo[1], lo[2], lo[3]);
        st4(out + 32, hi[0], hi[1], hi[2], hi[3]);
    }
}

// ---- Q2_K (84 bytes: scales[16], qs[64], f16 d, f16 dmin) and Q3_K (110 bytes: hmask[32], qs[64], scales[12], f16 d):
// both keep the low two bits of weight 128 n + 32 j + l in bits 2j, 2j+1 of qs[32 n + l].  lane = (n, byte pair):
// a lane writes two consecutive floats in each of the four bit planes; sixteen lanes cover 128 contiguous bytes.
template <int FMT>
__global__ void __launch_bounds__(DQ_WARPS * 32) dequant_q23_k_kernel(const uint8_t *__restrict__ w, float *__restrict__ y, long long units) {
    constexpr int RB = FMT == F_Q2_K ? 84 : 110, QS = FMT == F_Q2_K ? 16 : 32;
    const int lane = threadIdx.x & 31;
    const int n = lane >> 4, li = lane & 15;
    for (long long u = (long long)blockIdx.x * DQ_WARPS + (threadIdx.x >> 5); u < units; u += (long long)gridDim.x * DQ_WARPS) {
        const uint8_t *rec = w + u * RB;
        const uint32_t q = ld_u16(rec + QS + 32 * n + 2 * li);
        float *out = y + u * 256 + 128 * n + 2 * li;
        if (FMT == F_Q2_K) {
            const float d = half_bits_to_float(ld_u16(rec + 80)), dmin = half_bits_to_float(ld_u16(rec + 82));
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t sc = rec[8 * n + 2 * j + (li >> 3)];
                const float dl = __fmul_rn(d, (float)(sc & 15u)), ml = __fmul_rn(dmin, (float)(sc >> 4));
                const float v0 = __fsub_rn(__fmul_rn(dl, (float)((q >> (2 * j)) & 3u)), ml);
                const float v1 = __fsub_rn(__fmul_rn(dl, (float)((q >> (8 + 2 * j)) & 3u)), ml);
                __stcs(reinterpret_cast<float2 *>(out + 32 * j), make_float2(v0, v1));
            }
        } else {
            const float d = half_bits_to_float(ld_u16(rec + 108));
            const uint32_t hm = ld_u16(rec + 2 * li) >> (4 * n);
            uint32_t sc4[4];
            q3k_unpack_scales(ld_u32_a2(rec + 96), ld_u32_a2(rec + 100), ld_u32_a2(rec + 104), sc4);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int g = 8 * n + 2 * j + (li >> 3);
                const float dl = __fmul_rn(d, (float)((int)byte_of(sc4[g >> 2], g & 3) - 32));
                const int q0 = (int)((q >> (2 * j)) & 3u) - (((hm >> j) & 1u) ? 0 : 4);
                const int q1 = (int)((q >> (8 + 2 * j)) & 3u) - (((hm >> (8 + j)) & 1u) ? 0 : 4);
                __stcs(reinterpret_cast<float2 *>(out + 32 * j), make_float2(__fmul_rn(dl, (float)q0), __fmul_rn(dl, (float)q1)));
            }
        }
    }
}

// ---- Q4_0: a warp covers 8 records; lane = (record b, 4-byte slice s)
__global__ void __launch_bounds__(DQ_WARPS * 32) dequant_q4_0_kernel(const uint8_t *__restrict__ w, float *__restrict__ y, long long records) {
    const int lane = threadIdx.x & 31;
    const int b = lane >> 2, s = lane & 3;
    const long long groups = (records + 7) / 8;
    for (long long g = (long long)blockIdx.x * DQ_WARPS + (threadIdx.x >> 5); g < groups; g += (long long)gridDim.x * DQ_WARPS) {
        const long long r = g * 8 + b;
        if (r >= records) continue;
        const uint8_t *rec = w + r * 18;
        const float d = half_bits_to_float(ld_u16(rec));
        const uint32_t q = ld_u32_a2(rec + 2 + 4 * s);
        float lo[4], hi[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int v = (int)byte_of(q, i);
            lo[i] = __fmul_rn((float)((v & 15) - 8), d);
            hi[i] = __fmul_rn((float)((v >> 4) - 8), d);
        }
        float *out = y + r * 32 + 4 * s;
        st4(out, lo[0], lo[1], lo[2], lo[3]);
        st4(out + 16, hi[0], hi[1], hi[2], hi[3]);
    }
}

// ---- Q8_0: a warp covers 8 records; lane = (record b, 8-byte slice s)
__global__ void __launch_bounds__(DQ_WARPS * 32) dequant_q8_0_kernel(const uint8_t *__restrict__ w, float *__restrict__ y, long long records) {
    const int lane = threadIdx.x & 31;
    const int b = lane >> 2, s = lane & 3;
    const long long groups = (records + 7) / 8;
    for (long long g = (long long)blockIdx.x * DQ_WARPS + (threadIdx.x >> 5); g < groups; g += (long long)gridDim.x * DQ_WARPS) {
        const long long r = g * 8 + b;
        if (r >= records) continue;
        const uint8_t *rec = w + r * 34;
        const float d = half_bits_to_float(ld_u16(rec));
        const uint32_t q0 = ld_u32_a2(rec + 2 + 8 * s), q1 = ld_u32_a2(rec + 6 + 8 * s);
        float v[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[i] = __fmul_rn((float)(int)(int8_t)byte_of(q0, i), d);
            v[4 + i] = __fmul_rn((float)(int)(int8_t)byte_of(q1, i), d);
        }
        float *out = y + r * 32 + 8 * s;
        st4(out, v[0], v[1], v[2], v[3]);
        st4(out + 4, v[4], v[5], v[6], v[7]);
    }
}

// ---- IQ2_XXS: lane = (32-element group g, 8-element entry e); tables staged in shared memory
__global__ void __launch_bounds__(DQ_WARPS * 32) dequant_iq2_xxs_kernel(const uint8_t *__restrict__ w, const int8_t *__restrict__ grid,
                                                                         const int8_t *__restrict__ signs, float *__restrict__ y, long long units) {
    __shared__ __align__(8) int8_t s_grid[2048];
    __shared__ __align__(8) int8_t s_signs[1024];
    for (int i = threadIdx.x; i < 2048; i += blockDim.x) s_grid[i] = grid[i];
    for (int i = threadIdx.x; i < 1024; i += blockDim.x) s_signs[i] = signs[i];
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2, e = lane & 3;
    for (long long u = (long long)blockIdx.x * DQ_WARPS + (threadIdx.x >> 5); u < units; u += (long long)gridDim.x * DQ_WARPS) {
        const uint8_t *rec = w + u * 66;
        const float d = half_bits_to_float(ld_u16(rec));
        const uint8_t *grp = rec + 2 + 8 * g;
        const uint32_t index = rec[2 + 8 * g + e];
        const uint32_t meta = ld_u32_a2(grp + 4);
        const float db = __fmul_rn(__fmul_rn(d, __fadd_rn(0.5f, (float)(meta >> 28))), 0.25f);
        const int8_t *gv = s_grid + 8 * index;
        const int8_t *sv = s_signs + 8 * ((meta >> (7 * e)) & 127u);
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(__fmul_rn(db, (float)gv[i]), (float)sv[i]);
        float *out = y + u * 256 + 32 * g + 8 * e;
        st4(out, v[0], v[1], v[2], v[3]);
        st4(out + 4, v[4], v[5], v[6], v[7]);
    }
}

// ---- IQ2_XS (examples/kernels/dequantize/iq2_xs.py:9-68, ggml-quants.c:2444-2468): (d*(0.5+s)*0.25) * (grid*sign), s the
//      low scale nibble for the first 16 weights of a 32-group and the high nibble for the rest; lane = (group g, entry e)
__global__ void __launch_bounds__(DQ_WARPS * 32) dequant_iq2_xs_kernel(const uint8_t *__restrict__ w, const int8_t *__restrict__ grid,
                                                                        const int8_t *__restrict__ signs, float *__restrict__ y, long long units) {
    __shared__ __align__(8) int8_t s_grid[4096];
    __shared__ __align__(8) int8_t s_signs[1024];
    for (int i = threadIdx.x; i < 4096; i += blockDim.x) s_grid[i] = grid[i];
    for (int i = threadIdx.x; i < 1024; i += blockDim.x) s_signs[i] = signs[i];
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2, e = lane & 3;
    for (long long u = (long long)blockIdx.x * DQ_WARPS + (threadIdx.x >> 5); u < units; u += (long long)gridDim.x * DQ_WARPS) {
        const uint8_t *rec = w + u * 74;
        const float d = half_bits_to_float(ld_u16(rec));
        const uint32_t code = ld_u16(rec + 2 + 2 * (4 * g + e));
        const uint32_t sc = rec[66 + g];
        const float db = __fmul_rn(__fmul_rn(d, __fadd_rn(0.5f, (float)(e < 2 ? sc & 15u : sc >> 4))), 0.25f);
        const int8_t *gv = s_grid + 8 * (code & 511u);
        const int8_t *sv = s_signs + 8 * (code >> 9);
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(__fmul_rn(db, (float)gv[i]), (float)sv[i]);
        float *out = y + u * 256 + 32 * g + 8 * e;
        st4(out, v[0], v[1], v[2], v[3]);
        st4(out + 4, v[4], v[5], v[6], v[7]);
    }
}

// ---- IQ3_XXS (examples/kernels/dequantize/iq3_xxs.py, ggml-quants.c:2506-2536): (d*(0.5+s)*0.5) * (grid*sign); a grid
//      entry holds 4 weights, a sign entry 8; lane = (group g, entry e) produces 8 consecutive outputs
__global__ void __launch_bounds__(DQ_WARPS * 32) dequant_iq3_xxs_kernel(const uint8_t *__restrict__ w, const int8_t *__restrict__ grid,
                                                                         const int8_t *__restrict__ signs, float *__restrict__ y, long long units) {
    __shared__ __align__(8) int8_t s_grid[1024];
    __shared__ __align__(8) int8_t s_signs[1024];
    for (int i = threadIdx.x; i < 1024; i += blockDim.x) { s_grid[i] = grid[i]; s_signs[i] = signs[i]; }
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2, e = lane & 3;
    for (long long u = (long long)blockIdx.x * DQ_WARPS + (threadIdx.x >> 5); u < units; u += (long long)gridDim.x * DQ_WARPS) {
        const uint8_t *rec = w + u * 98;
        const float d = half_bits_to_float(ld_u16(rec));
        const uint32_t meta = ld_u32_a2(rec + 66 + 4 * g);
        const float db = __fmul_rn(__fmul_rn(d, __fadd_rn(0.5f, (float)(meta >> 28))), 0.5f);
        const uint8_t *g1 = reinterpret_cast<const uint8_t *>(s_grid) + 4 * rec[2 + 8 * g + 2 * e];
        const uint8_t *g2 = reinterpret_cast<const uint8_t *>(s_grid) + 4 * rec[2 + 8 * g + 2 * e + 1];
        const int8_t *sv = s_signs + 8 * ((meta >> (7 * e)) & 127u);
        float v[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[i] = __fmul_rn(__fmul_rn(db, (float)g1[i]), (float)sv[i]);
            v[4 + i] = __fmul_rn(__fmul_rn(db, (float)g2[i]), (float)sv[4 + i]);
        }
        float *out = y + u * 256 + 32 * g + 8 * e;
        st4(out, v[0], v[1], v[2], v[3]);
        st4(out + 4, v[4], v[5], v[6], v[7]);
    }
}

// ---- IQ2_S (examples/kernels/dequantize/iq2_s.py, GGML dequantize_row_iq2_s): as IQ2_XS with 10-bit grid indices (low
//      byte + two bits of qh) and explicit sign bits; lane = (group g, entry e).  The 8 KB grid is read through the
//      read-only cache.
__global__ void __launch_bounds__(DQ_WARPS * 32) dequant_iq2_s_kernel(const uint8_t *__restrict__ w, const int8_t *__restrict__ grid,
                                                                       float *__restrict__ y, long long units) {
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2, e = lane & 3;
    for (long long u = (long long)blockIdx.x * DQ_WARPS + (threadIdx.x >> 5); u < units; u += (long long)gridDim.x * DQ_WARPS) {
        const uint8_t *rec = w + u * 82;
        const float d = half_bits_to_float(ld_u16(rec));
        const uint32_t index = rec[2 + 4 * g + e] | (((uint32_t)rec[66 + g] << (8 - 2 * e)) & 0x300u);
        const uint32_t sb = rec[34 + 4 * g + e], sc = rec[74 + g];
        const float db = __fmul_rn(__fmul_rn(d, __fadd_rn(0.5f, (float)(e < 2 ? sc & 15u : sc >> 4))), 0.25f);
        const uint2 gv = __ldg(reinterpret_cast<const uint2 *>(grid) + index);
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float q = (float)(((i < 4 ? gv.x : gv.y) >> (8 * (i & 3))) & 0xffu);
            v[i] = __fmul_rn(__fmul_rn(db, q), (sb >> i) & 1u ? -1.f : 1.f);
        }
        float *out = y + u * 256 + 32 * g + 8 * e;
        st4(out, v[0], v[1], v[2], v[3]);
        st4(out + 4, v[4], v[5], v[6], v[7]);
    }
}

// ---- IQ3_S (examples/kernels/dequantize/iq3_s.py, GGML dequantize_row_iq3_s): (d * (1 + 2 s)) * (grid * sign), 9-bit grid
//      indices (low byte + one bit of qh), explicit sign bits; lane = (group g, entry e) produces 8 consecutive outputs
__global__ void __launch_bounds__(DQ_WARPS * 32) dequant_iq3_s_kernel(const uint8_t *__restrict__ w, const int8_t *__restrict__ grid,
                                                                       float *__restrict__ y, long long units) {
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2, e = lane & 3;
    for (long long u = (long long)blockIdx.x * DQ_WARPS + (threadIdx.x >> 5); u < units; u += (long long)gridDim.x * DQ_WARPS) {
        const uint8_t *rec = w + u * 110;
        const float d = half_bits_to_float(ld_u16(rec));
        const uint32_t high = rec[66 + g], sb = rec[74 + 4 * g + e], sc = rec[106 + (g >> 1)];
        const float db = __fmul_rn(d, (float)(1 + 2 * (int)(g & 1 ? sc >> 4 : sc & 15u)));
        const uint32_t i1 = rec[2 + 8 * g + 2 * e] | (((high >> (2 * e)) & 1u) << 8), i2 = rec[2 + 8 * g + 2 * e + 1] | (((high >> (2 * e + 1)) & 1u) << 8);
        const uint32_t g1 = __ldg(reinterpret_cast<const uint32_t *>(grid) + i1), g2 = __ldg(reinterpret_cast<const uint32_t *>(grid) + i2);
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float q = (float)(((i < 4 ? g1 : g2) >> (8 * (i & 3))) & 0xffu);
            v[i] = __fmul_rn(__fmul_rn(db, q), (sb >> i) & 1u ? -1.f : 1.f);
        }
        float *out = y + u * 256 + 32 * g + 8 * e;
        st4(out, v[0], v[1], v[2], v[3]);
        st4(out + 4, v[4], v[5], v[6], v[7]);
    }
}

// ---- IQ1_S (examples/kernels/dequantize/iq1_s.py, GGML dequantize_row_iq1_s): (d * (2 s + 1)) * (grid + delta), delta = +-0.125
//      per 32 weights; lane = (group g, entry e); the 16 KB grid (values -1, 0, +1) is read through the read-only cache
__global__ void __launch_bounds__(DQ_WARPS * 32) dequant_iq1_s_kernel(const uint8_t *__restrict__ w, const int8_t *__restrict__ grid,
                                                                       float *__restrict__ y, long long units) {
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2, e = lane & 3;
    for (long long u = (long long)blockIdx.x * DQ_WARPS + (threadIdx.x >> 5); u < units; u += (long long)gridDim.x * DQ_WARPS) {
        const uint8_t *rec = w + u * 50;
        const uint32_t qh = ld_u16(rec + 34 + 2 * g);
        const float dl = __fmul_rn(half_bits_to_float(ld_u16(rec)), (float)(int)(2u * ((qh >> 12) & 7u) + 1u));
        const float delta = qh & 0x8000u ? -0.125f : 0.125f;
        const uint2 gv = __ldg(reinterpret_cast<const uint2 *>(grid) + (rec[2 + 4 * g + e] | (((qh >> (3 * e)) & 7u) << 8)));
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(dl, __fadd_rn((float)(int)(int8_t)((i < 4 ? gv.x : gv.y) >> (8 * (i & 3))), delta));
        float *out = y + u * 256 + 32 * g + 8 * e;
        st4(out, v[0], v[1], v[2], v[3]);
        st4(out + 4, v[4], v[5], v[6], v[7]);
    }
}

// ---- IQ1_M (examples/kernels/dequantize/iq1_m.py:18-23, GGML dequantize_row_iq1_m): as IQ1_S with a scale per 16 weights, a
//      shift sign per 8 and the record's f16 scale spread over the top nibbles of four u16; f16_table is the caller's
//      float[65536] table of f16 bit patterns
__global__ void __launch_bounds__(DQ_WARPS * 32) dequant_iq1_m_kernel(const uint8_t *__restrict__ w, const int8_t *__restrict__ grid,
                                                                       const float *__restrict__ f16_table, float *__restrict__ y, long long units) {
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2, e = lane & 3;
    for (long long u = (long long)blockIdx.x * DQ_WARPS + (threadIdx.x >> 5); u < units; u += (long long)gridDim.x * DQ_WARPS) {
        const uint8_t *rec = w + u * 56;
        const uint32_t s0 = ld_u16(rec + 48), s1 = ld_u16(rec + 50), s2 = ld_u16(rec + 52), s3 = ld_u16(rec + 54);
        const float d = __ldg(f16_table + ((s0 >> 12) | ((s1 >> 8) & 0x00f0u) | ((s2 >> 4) & 0x0f00u) | (s3 & 0xf000u)));
        const uint32_t sc = ld_u16(rec + 48 + 2 * (g >> 1)), qh = rec[32 + 2 * g + (e >> 1)];
        const uint32_t nib = e & 1 ? qh >> 4 : qh & 15u;
        const float dl = __fmul_rn(d, (float)(int)(2u * ((sc >> (6 * (g & 1) + 3 * (e >> 1))) & 7u) + 1u));
        const float delta = nib & 8u ? -0.125f : 0.125f;
        const uint2 gv = __ldg(reinterpret_cast<const uint2 *>(grid) + (rec[4 * g + e] | ((nib & 7u) << 8)));
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(dl, __fadd_rn((float)(int)(int8_t)((i < 4 ? gv.x : gv.y) >> (8 * (i & 3))), delta));
        float *out = y + u * 256 + 32 * g + 8 * e;
        st4(out, v[0], v[1], v[2], v[3]);
        st4(out + 4, v[4], v[5], v[6], v[7]);
    }
}

// ---- TQ1_0: every lane produces 8 consecutive outputs; lanes 0-19 region 0 (5 digits x 32 bytes),
//      20-29 region 1 (5 digits x 16 bytes), 30-31 region 2 (4 digits x 4 bytes)
__global__ void __launch_bounds__(DQ_WARPS * 32) dequant_tq1_0_kernel(const uint8_t *__restrict__ w, const uint32_t *__restrict__ powers,
                                                                       float *__restrict__ y, long long units) {
    const int lane = threadIdx.x & 31;
    uint32_t pw[5];
#pragma unroll
    for (int i = 0; i < 5; ++i) pw[i] = __ldg(powers + i);
    for (long long u = (long long)blockIdx.x * DQ_WARPS + (threadIdx.x >> 5); u < units; u += (long long)gridDim.x * DQ_WARPS) {
        const uint8_t *rec = w + u * 54;
        const float d = half_bits_to_float(ld_u16(rec + 52));
        float v[8];
        if (lane < 30) {
            int digit, byte0;
            if (lane < 20) { digit = lane >> 2; byte0 = (lane & 3) * 8; }
            else { const int i = lane - 20; digit = i >> 1; byte0 = 32 + (i & 1) * 8; }
            const uint32_t p = digit == 0 ? pw[0] : digit == 1 ? pw[1] : digit == 2 ? pw[2] : digit == 3 ? pw[3] : pw[4];
            const uint32_t q0 = ld_u32_a2(rec + byte0), q1 = ld_u32_a2(rec + byte0 + 4);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                v[i] = __fmul_rn((float)tq1_digit(byte_of(q0, i), p), d);
                v[4 + i] = __fmul_rn((float)tq1_digit(byte_of(q1, i), p), d);
            }
        } else {
            const uint32_t qh = ld_u32_a2(rec + 48);
            const int n0 = (lane - 30) * 2;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                v[i] = __fmul_rn((float)tq1_digit(byte_of(qh, i), n0 == 0 ? pw[0] : pw[2]), d);
                v[4 + i] = __fmul_rn((float)tq1_digit(byte_of(qh, i), n0 == 0 ? pw[1] : pw[3]), d);
            }
        }
        float *out = y + u * 256 + 8 * lane;
        st4(out, v[0], v[1], v[2], v[3]);
        st4(out + 4, v[4], v[5], v[6], v[7]);
    }
}

// ---- any alignment of W and Y: one thread per output element (slow path, same op trees)
// ---- Q6_K (210 bytes, 2-byte aligned: ql[128], qh[64], int8 scales[16], f16 d): lane = (half, pair of l);
// weight 128 half + 32 p + l has low nibble ql[64 half + l + 32 (p & 1)] (>> 4 for p >= 2), high bits 2p, 2p+1
// of qh[32 half + l], scale scales[8 half + 2 p + l / 16].  A lane writes two consecutive floats in each of
// the four quadrants: sixteen lanes cover 128 contiguous bytes per store.
__global__ void __launch_bounds__(DQ_WARPS * 32) dequant_q6_k_kernel(const uint8_t *__restrict__ w, float *__restrict__ y, long long units) {
    const int lane = threadIdx.x & 31;
    const int half = lane >> 4, li = lane & 15;
    for (long long u = (long long)blockIdx.x * DQ_WARPS + (threadIdx.x >> 5); u < units; u += (long long)gridDim.x * DQ_WARPS) {
        const uint8_t *rec = w + u * 210;
        const uint32_t qa = ld_u16(rec + 64 * half + 2 * li), qb = ld_u16(rec + 64 * half + 32 + 2 * li);
        const uint32_t qh = ld_u16(rec + 128 + 32 * half + 2 * li);
        const float d = half_bits_to_float(ld_u16(rec + 208));
        float *out = y + u * 256 + 128 * half + 2 * li;
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const float ds = __fmul_rn(d, (float)(int)(int8_t)rec[192 + 8 * half + 2 * p + (li >> 3)]);
            float v[2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const uint32_t lo = ((p & 1) ? qb : qa) >> (8 * j);
                const uint32_t nib = p < 2 ? (lo & 15u) : ((lo >> 4) & 15u);
                const uint32_t hi = (qh >> (8 * j + 2 * p)) & 3u;
                v[j] = __fmul_rn(ds, (float)((int)(nib | (hi << 4)) - 32));
            }
            __stcs(reinterpret_cast<float2 *>(out + 32 * p), make_float2(v[0], v[1]));
        }
    }
}

__global__ void dequant_elementwise_kernel(int fmt, const uint8_t *__restrict__ w, const int8_t *__restrict__ grid,
                                           const int8_t *__restrict__ signs, const uint32_t *__restrict__ powers,
                                           float *__restrict__ y, long long elements) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < elements; i += (long long)gridDim.x * blockDim.x) {
        float v = 0.f;
        if (fmt == F_Q4_0) {
            const uint8_t *rec = w + (i / 32) * 18;
            const int e = (int)(i % 32);
            const int q = e < 16 ? (rec[2 + e] & 15) : (rec[2 + e - 16] >> 4);
            v = __fmul_rn((float)(q - 8), half_bits_to_float(ld_u16(rec)));
        } else if (fmt == F_Q8_0) {
            const uint8_t *rec = w + (i / 32) * 34;
            v = __fmul_rn((float)(int)(int8_t)rec[2 + i % 32], half_bits_to_float(ld_u16(rec)));
        } else if (fmt == F_Q4_K) {
            const uint8_t *rec = w + (i / 256) * 144;
            const int e = (int)(i % 256), j = e / 64, p = e % 64;
            const Q4KScales s = q4k_unpack_scales(ld_u32_a2(rec + 4), ld_u32_a2(rec + 8), ld_u32_a2(rec + 12));
            const int is = 2 * j + (p >= 32);
            const uint32_t sc = byte_of(is < 4 ? s.sc_lo : s.sc_hi, is & 3), mn = byte_of(is < 4 ? s.mn_lo : s.mn_hi, is & 3);
            const uint32_t b = rec[16 + 32 * j + (p & 31)];
            const uint32_t q = p < 32 ? (b & 15u) : (b >> 4);
            const float d1 = __fmul_rn(half_bits_to_float(ld_u16(rec)), (float)sc);
            const float m1 = __fmul_rn(half_bits_to_float(ld_u16(rec + 2)), (float)mn);
            v = __fsub_rn(__fmul_rn(d1, (float)q), m1);
        } else if (fmt == F_Q2_K) {
            const uint8_t *rec = w + (i / 256) * 84;
            const int e = (int)(i % 256);
            const uint32_t sc = rec[e >> 4];
            const uint32_t q = (rec[16 + 32 * (e >> 7) + (e & 31)] >> (2 * ((e >> 5) & 3))) & 3u;
            const float dl = __fmul_rn(half_bits_to_float(ld_u16(rec + 80)), (float)(sc & 15u));
            const float ml = __fmul_rn(half_bits_to_float(ld_u16(rec + 82)), (float)(sc >> 4));
            v = __fsub_rn(__fmul_rn(dl, (float)q), ml);
        } else if (fmt == F_Q3_K) {
            const uint8_t *rec = w + (i / 256) * 110;
            const int e = (int)(i % 256), g = e >> 4;
            uint32_t sc4[4];
            q3k_unpack_scales(ld_u32_a2(rec + 96), ld_u32_a2(rec + 100), ld_u32_a2(rec + 104), sc4);
            const int q = (int)((rec[32 + 32 * (e >> 7) + (e & 31)] >> (2 * ((e >> 5) & 3))) & 3u) - (((rec[e & 31] >> (e >> 5)) & 1u) ? 0 : 4);
            const float dl = __fmul_rn(half_bits_to_float(ld_u16(rec + 108)), (float)((int)byte_of(sc4[g >> 2], g & 3) - 32));
            v = __fmul_rn(dl, (float)q);
        } else if (fmt == F_Q5_K) {
            const uint8_t *rec = w + (i / 256) * 176;
            const int e = (int)(i % 256), g = e >> 5, l = e & 31;
            const Q4KScales s = q4k_unpack_scales(ld_u32_a2(rec + 4), ld_u32_a2(rec + 8), ld_u32_a2(rec + 12));
            const uint32_t sc = byte_of(g < 4 ? s.sc_lo : s.sc_hi, g & 3), mn = byte_of(g < 4 ? s.mn_lo : s.mn_hi, g & 3);
            const uint32_t b = rec[48 + 32 * (g >> 1) + l];
            const uint32_t q = ((g & 1) ? (b >> 4) : (b & 15u)) | (((rec[16 + l] >> g) & 1u) << 4);
            const float d1 = __fmul_rn(half_bits_to_float(ld_u16(rec)), (float)sc);
            const float m1 = __fmul_rn(half_bits_to_float(ld_u16(rec + 2)), (float)mn);
            v = __fsub_rn(__fmul_rn(d1, (float)q), m1);
        } else if (fmt == F_Q6_K) {
            const uint8_t *rec = w + (i / 256) * 210;
            const int e = (int)(i % 256), half = e >> 7, p = (e >> 5) & 3, l = e & 31;
            const uint32_t lo = rec[64 * half + l + 32 * (p & 1)];
            const uint32_t nib = p < 2 ? (lo & 15u) : (lo >> 4);
            const uint32_t hi = (rec[128 + 32 * half + l] >> (2 * p)) & 3u;
            const float ds = __fmul_rn(half_bits_to_float(ld_u16(rec + 208)), (float)(int)(int8_t)rec[192 + (e >> 4)]);
            v = __fmul_rn(ds, (float)((int)(nib | (hi << 4)) - 32));
        } else if (fmt == F_IQ2_XXS) {
            const uint8_t *rec = w + (i / 256) * 66;
            const int e = (int)(i % 256), g = e / 32, en = (e % 32) / 8, l = e % 8;
            const uint32_t meta = ld_u32_a2(rec + 2 + 8 * g + 4);
            const float db = __fmul_rn(__fmul_rn(half_bits_to_float(ld_u16(rec)), __fadd_rn(0.5f, (float)(meta >> 28))), 0.25f);
            const int gv = grid[8 * rec[2 + 8 * g + en] + l], sv = signs[8 * ((meta >> (7 * en)) & 127u) + l];
            v = __fmul_rn(__fmul_rn(db, (float)gv), (float)sv);
        } else if (fmt == F_IQ2_XS) {
            const uint8_t *rec = w + (i / 256) * 74;
            const int e = (int)(i % 256), g = e / 32, en = (e % 32) / 8, l = e % 8;
            const uint32_t code = ld_u16(rec + 2 + 2 * (4 * g + en)), sc = rec[66 + g];
            const float db = __fmul_rn(__fmul_rn(half_bits_to_float(ld_u16(rec)), __fadd_rn(0.5f, (float)(en < 2 ? sc & 15u : sc >> 4))), 0.25f);
            const int gv = grid[8 * (code & 511u) + l], sv = signs[8 * (code >> 9) + l];
            v = __fmul_rn(__fmul_rn(db, (float)gv), (float)sv);
        } else if (fmt == F_IQ3_XXS) {
            const uint8_t *rec = w + (i / 256) * 98;
            const int e = (int)(i % 256), g = e / 32, en = (e % 32) / 8, l = e % 8;
            const uint32_t meta = ld_u32_a2(rec + 66 + 4 * g);
            const float db = __fmul_rn(__fmul_rn(half_bits_to_float(ld_u16(rec)), __fadd_rn(0.5f, (float)(meta >> 28))), 0.5f);
            const int gv = (int)(uint8_t)grid[4 * rec[2 + 8 * g + 2 * en + (l >> 2)] + (l & 3)], sv = signs[8 * ((meta >> (7 * en)) & 127u) + l];
            v = __fmul_rn(__fmul_rn(db, (float)gv), (float)sv);
        } else if (fmt == F_IQ2_S) {
            const uint8_t *rec = w + (i / 256) * 82;
            const int e = (int)(i % 256), g = e / 32, en = (e % 32) / 8, l = e % 8;
            const uint32_t index = rec[2 + 4 * g + en] | (((uint32_t)rec[66 + g] << (8 - 2 * en)) & 0x300u), sc = rec[74 + g];
            const float db = __fmul_rn(__fmul_rn(half_bits_to_float(ld_u16(rec)), __fadd_rn(0.5f, (float)(en < 2 ? sc & 15u : sc >> 4))), 0.25f);
            v = __fmul_rn(__fmul_rn(db, (float)(int)(uint8_t)grid[8 * index + l]), (rec[34 + 4 * g + en] >> l) & 1 ? -1.f : 1.f);
        } else if (fmt == F_IQ3_S) {
            const uint8_t *rec = w + (i / 256) * 110;
            const int e = (int)(i % 256), g = e / 32, en = (e % 32) / 8, l = e % 8, ix = 2 * en + (l >> 2);
            const uint32_t sc = rec[106 + (g >> 1)];
            const float db = __fmul_rn(half_bits_to_float(ld_u16(rec)), (float)(1 + 2 * (int)(g & 1 ? sc >> 4 : sc & 15u)));
            const uint32_t index = rec[2 + 8 * g + ix] | ((((uint32_t)rec[66 + g] >> ix) & 1u) << 8);
            v = __fmul_rn(__fmul_rn(db, (float)(int)(uint8_t)grid[4 * index + (l & 3)]), (rec[74 + 4 * g + en] >> l) & 1 ? -1.f : 1.f);
        } else if (fmt == F_IQ1_S) {
            const uint8_t *rec = w + (i / 256) * 50;
            const int e = (int)(i % 256), g = e / 32, en = (e % 32) / 8, l = e % 8;
            const uint32_t qh = ld_u16(rec + 34 + 2 * g);
            const float dl = __fmul_rn(half_bits_to_float(ld_u16(rec)), (float)(int)(2u * ((qh >> 12) & 7u) + 1u));
            const int gvl = grid[8 * (rec[2 + 4 * g + en] | (((qh >> (3 * en)) & 7u) << 8)) + l];
            v = __fmul_rn(dl, __fadd_rn((float)gvl, qh & 0x8000u ? -0.125f : 0.125f));
        } else if (fmt == F_IQ1_M) {
            const uint8_t *rec = w + (i / 256) * 56;
            const int e = (int)(i % 256), g = e / 32, en = (e % 32) / 8, l = e % 8;
            const uint32_t s0 = rec[48] | (rec[49] << 8), s1 = rec[50] | (rec[51] << 8), s2 = rec[52] | (rec[53] << 8), s3 = rec[54] | (rec[55] << 8);
            const float d = reinterpret_cast<const float *>(powers)[(s0 >> 12) | ((s1 >> 8) & 0x00f0u) | ((s2 >> 4) & 0x0f00u) | (s3 & 0xf000u)];
            const uint32_t sc = rec[48 + 2 * (g >> 1)] | (rec[49 + 2 * (g >> 1)] << 8), qh = rec[32 + 2 * g + (en >> 1)];
            const uint32_t nib = en & 1 ? qh >> 4 : qh & 15u;
            const float dl = __fmul_rn(d, (float)(int)(2u * ((sc >> (6 * (g & 1) + 3 * (en >> 1))) & 7u) + 1u));
            const int gvl = grid[8 * (rec[4 * g + en] | ((nib & 7u) << 8)) + l];
            v = __fmul_rn(dl, __fadd_rn((float)gvl, nib & 8u ? -0.125f : 0.125f));
        } else if (fmt == F_TQ1_0) {
            const uint8_t *rec = w + (i / 256) * 54;
            const int e = (int)(i % 256);
            int byte, digit;
            if (e < 160) { digit = e / 32; byte = e % 32; }
            else if (e < 240) { digit = (e - 160) / 16; byte = 32 + (e - 160) % 16; }
            else { digit = (e - 240) / 4; byte = 48 + (e - 240) % 4; }
            v = __fmul_rn((float)tq1_digit(rec[byte], powers[digit]), half_bits_to_float(ld_u16(rec + 52)));
        }
        y[i] = v;
    }
}

static int dq_grid(long long warps_needed, int sm_count) {
    const long long blocks = (warps_needed + DQ_WARPS - 1) / DQ_WARPS;
    const long long cap = (long long)sm_count * 64;   // 8 resident blocks per SM, 8 waves deep
    return (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

cudaError_t launch_dequantize(int fmt, const void *w, const int8_t *grid, const int8_t *signs, const uint32_t *powers,
                              float *y, long long elements, int sm_count, cudaStream_t stream) {
    if (elements == 0) return cudaSuccess;
    const uint8_t *wb = static_cast<const uint8_t *>(w);
    if ((reinterpret_cast<uintptr_t>(y) & 15u) || (reinterpret_cast<uintptr_t>(w) & 1u)) {
        const long long blocks = (elements + 255) / 256, cap = (long long)sm_count * 32;
        dequant_elementwise_kernel<<<(int)(blocks > cap ? cap : blocks), 256, 0, stream>>>(fmt, wb, grid, signs, powers, y, elements);
        return cudaGetLastError();
    }
    const bool a4 = (reinterpret_cast<uintptr_t>(w) & 3u) == 0;
    switch (fmt) {
    case F_Q4_K: {
        const long long units = elements / 256;
        if (a4) dequant_q4_k_kernel<true><<<dq_grid(units, sm_count), DQ_WARPS * 32, 0, stream>>>(wb, y, units);
        else dequant_q4_k_kernel<false><<<dq_grid(units, sm_count), DQ_WARPS * 32, 0, stream>>>(wb, y, units);
        break;
    }
    case F_Q2_K: {
        const long long units = elements / 256;
        dequant_q23_k_kernel<F_Q2_K><<<dq_grid(units, sm_count), DQ_WARPS * 32, 0, stream>>>(wb, y, units);
        break;
    }
    case F_Q3_K: {
        const long long units = elements / 256;
        dequant_q23_k_kernel<F_Q3_K><<<dq_grid(units, sm_count), DQ_WARPS * 32, 0, stream>>>(wb, y, units);
        break;
    }
    case F_Q5_K: {
        const long long units = elements / 256;
        if (a4) dequant_q5_k_kernel<true><<<dq_grid(units, sm_count), DQ_WARPS * 32, 0, stream>>>(wb, y, units);
        else dequant_q5_k_kernel<false><<<dq_grid(units, sm_count), DQ_WARPS * 32, 0, stream>>>(wb, y, units);
        break;
    }
    case F_Q4_0: {
        const long long records = elements / 32;
        dequant_q4_0_kernel<<<dq_grid((records + 7) / 8, sm_count), DQ_WARPS * 32, 0, stream>>>(wb, y, records);
        break;
    }
    case F_Q8_0: {
        const long long records = elements / 32;
        dequant_q8_0_kernel<<<dq_grid((records + 7) / 8, sm_count), DQ_WARPS * 32, 0, stream>>>(wb, y, records);
        break;
    }
    case F_IQ2_XXS: {
        const long long units = elements / 256;
        dequant_iq2_xxs_kernel<<<dq_grid(units, sm_count), DQ_WARPS * 32, 0, stream>>>(wb, grid, signs, y, units);
        break;
    }
    case F_IQ2_XS: {
        const long long units = elements / 256;
        dequant_iq2_xs_kernel<<<dq_grid(units, sm_count), DQ_WARPS * 32, 0, stream>>>(wb, grid, signs, y, units);
        break;
    }
    case F_IQ3_XXS: {
        const long long units = elements / 256;
        dequant_iq3_xxs_kernel<<<dq_grid(units, sm_count), DQ_WARPS * 32, 0, stream>>>(wb, grid, signs, y, units);
        break;
    }
    case F_IQ2_S: {
        const long long units = elements / 256;
        dequant_iq2_s_kernel<<<dq_grid(units, sm_count), DQ_WARPS * 32, 0, stream>>>(wb, grid, y, units);
        break;
    }
    case F_IQ3_S: {
        const long long units = elements / 256;
        dequant_iq3_s_kernel<<<dq_grid(units, sm_count), DQ_WARPS * 32, 0, stream>>>(wb, grid, y, units);
        break;
    }
    case F_IQ1_S: {
        const long long units = elements / 256;
        dequant_iq1_s_kernel<<<dq_grid(units, sm_count), DQ_WARPS * 32, 0, stream>>>(wb, grid, y, units);
        break;
    }
    case F_IQ1_M: {
        const long long units = elements / 256;
        dequant_iq1_m_kernel<<<dq_grid(units, sm_count), DQ_WARPS * 32, 0, stream>>>(wb, grid, reinterpret_cast<const float *>(powers), y, units);
        break;
    }
    case F_Q6_K: {
        const long long units = elements / 256;
        dequant_q6_k_kernel<<<dq_grid(units, sm_count), DQ_WARPS * 32, 0, stream>>>(wb, y, units);
        break;
    }
    case F_TQ1_0: {
        const long long units = elements / 256;
        dequant_tq1_0_kernel<<<dq_grid(units, sm_count), DQ_WARPS * 32, 0, stream>>>(wb, powers, y, units);
        break;
    }
    default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

}  // namespace weft
