// Warp-level bodies of the activation quantizers, shared by the standalone kernels (quantize.cu)
// and by the GEMV prologue that quantizes X while the first weight rows are in flight (gemv.cu).
//
// Semantics are the reference DSL's, which its own bit-exact check restates in scalar C++
// (examples/kernels/quantize/q8_0.py:8-23, q8_k.py:8-35; examples/repro/weft/q8_quantize_runtime.cpp:85-141):
//   Q8_0: d = amax/127 (stored f16), inverse = amax == 0 ? 0 : 1/d, q = clamp_i8(rne(x*inverse))
//   Q8_1: Q8_0 with s = f16(f32(sum of codes) * d) after d (q8_1.py:8-20), codes at byte 4
//   Q8_K: extreme = |max| > |min| ? max : min, inverse = extreme == 0 ? 0 : -127/extreme,
//         d = inverse == 0 ? 0 : 1/inverse, q = clamp_i8(rne(x*inverse)), bsum[g] = sum of 16 codes
// GGML's quantize_row_q8_0_ref / quantize_row_q8_K_ref (ggml-quants.c:238-261, 2696-2733) produce the
// same bytes except on exact ties (round-half-away for Q8_0; first-occurrence extreme for Q8_K).
// Divisions are IEEE (__fdiv_rn); nothing here may be compiled with fast-math.
#pragma once

#include "common.cuh"

namespace weft {

template <bool A16>
__device__ __forceinline__ void load8(const float *x, float (&v)[8]) {
    if (A16) {
        const float4 a = __ldg(reinterpret_cast<const float4 *>(x)), b = __ldg(reinterpret_cast<const float4 *>(x) + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = __ldg(x + i);
    }
}

__device__ __forceinline__ void encode8(const float (&v)[8], float inverse, uint32_t &lo, uint32_t &hi, int &sum) {
    int q[8];
    sum = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int r = __float2int_rn(__fmul_rn(v[i], inverse));
        r = max(-128, min(127, r));
        q[i] = r;
        sum += r;
    }
    lo = (uint32_t)(q[0] & 255) | ((uint32_t)(q[1] & 255) << 8) | ((uint32_t)(q[2] & 255) << 16) | ((uint32_t)(q[3] & 255) << 24);
    hi = (uint32_t)(q[4] & 255) | ((uint32_t)(q[5] & 255) << 8) | ((uint32_t)(q[6] & 255) << 16) | ((uint32_t)(q[7] & 255) << 24);
}

// A full warp quantizes 256 floats (lane l holds elements 8l..8l+7) to one Q8_K record.
// Out: this lane's 8 codes (q0, q1), the sum of the 16 codes of lanes {l & ~1, l | 1}, and d.
__device__ __forceinline__ void q8_k_warp(const float (&v)[8], uint32_t &q0, uint32_t &q1, int &sum16, float &d) {
    float hi = v[0], lo = v[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) { hi = fmaxf(hi, v[i]); lo = fminf(lo, v[i]); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
    }
    const float extreme = fabsf(hi) > fabsf(lo) ? hi : lo;
    const float inverse = extreme == 0.0f ? 0.0f : __fdiv_rn(-127.0f, extreme);
    d = inverse == 0.0f ? 0.0f : __fdiv_rn(1.0f, inverse);
    int sum;
    encode8(v, inverse, q0, q1, sum);
    sum16 = sum + __shfl_xor_sync(0xffffffffu, sum, 1);
}

// A full warp quantizes 8 x 32 floats (lane l: block l/4, elements 8(l%4)..+7) to eight Q8_0 records.
// Out: this lane's 8 codes, the sum of its block's 32 codes, and the block's d (before f16 rounding).
__device__ __forceinline__ void q8_0_warp(const float (&v)[8], uint32_t &q0, uint32_t &q1, int &sum32, float &d) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    d = __fdiv_rn(amax, 127.0f);
    const float inverse = amax == 0.0f ? 0.0f : __fdiv_rn(1.0f, d);
    int sum;
    encode8(v, inverse, q0, q1, sum);
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum32 = sum + __shfl_xor_sync(0xffffffffu, sum, 2);
}

__device__ __forceinline__ void store_q8_k(uint8_t *rec, int lane, uint32_t q0, uint32_t q1, int sum16, float d) {
    uint32_t *codes = reinterpret_cast<uint32_t *>(rec + 4 + 8 * lane);
    codes[0] = q0;
    codes[1] = q1;
    if ((lane & 1) == 0) *reinterpret_cast<int16_t *>(rec + 260 + lane) = (int16_t)sum16;
    if (lane == 0) *reinterpret_cast<float *>(rec) = d;
}

__device__ __forceinline__ void store_q8_0(uint8_t *rec, int sub, uint32_t q0, uint32_t q1, float d) {
    uint16_t *codes = reinterpret_cast<uint16_t *>(rec + 2 + 8 * sub);
    codes[0] = (uint16_t)q0; codes[1] = (uint16_t)(q0 >> 16);
    codes[2] = (uint16_t)q1; codes[3] = (uint16_t)(q1 >> 16);
    if (sub == 0) *reinterpret_cast<__half *>(rec) = __float2half_rn(d);
}

// Q8_1 record (36 bytes, 2-byte aligned): f16 d, f16 s = f16(f32(sum32) * d) with the fp32 d, 32 codes
__device__ __forceinline__ void store_q8_1(uint8_t *rec, int sub, uint32_t q0, uint32_t q1, int sum32, float d) {
    uint16_t *codes = reinterpret_cast<uint16_t *>(rec + 4 + 8 * sub);
    codes[0] = (uint16_t)q0; codes[1] = (uint16_t)(q0 >> 16);
    codes[2] = (uint16_t)q1; codes[3] = (uint16_t)(q1 >> 16);
    if (sub == 0) {
        *reinterpret_cast<__half *>(rec) = __float2half_rn(d);
        *reinterpret_cast<__half *>(rec + 2) = __float2half_rn(__fmul_rn((float)sum32, d));
    }
}

}  // namespace weft
