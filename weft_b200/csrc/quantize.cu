// Activation quantizers q8_0_quantize / q8_K_quantize (the prologue of every production_mul_mat_*).
//
// Semantics are the reference DSL's, which its own bit-exact check restates in scalar C++
// (examples/kernels/quantize/q8_0.py:8-23, q8_k.py:8-35; examples/repro/weft/q8_quantize_runtime.cpp:85-141):
//   Q8_0: d = amax/127 (stored f16), inverse = amax == 0 ? 0 : 1/d, q = clamp_i8(rne(x*inverse))
//   Q8_K: extreme = |max| > |min| ? max : min, inverse = extreme == 0 ? 0 : -127/extreme,
//         d = inverse == 0 ? 0 : 1/inverse, q = clamp_i8(rne(x*inverse)), bsum[g] = sum of 16 codes
// GGML's quantize_row_q8_0_ref / quantize_row_q8_K_ref (ggml-quants.c:238-261, 2696-2733) produce the
// same bytes except on exact ties (round-half-away for Q8_0; first-occurrence extreme for Q8_K).
// Divisions are IEEE (__fdiv_rn); nothing here may be compiled with fast-math.
//
// HBM-bound: 4 bytes read per 1.06-1.14 bytes written; one warp per 256 elements, 32 bytes per lane.
#include "common.cuh"
#include "kernels.h"

namespace weft {

constexpr int QZ_WARPS = 8;

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

// X: `blocks` consecutive groups of 256 floats; Y: `blocks` Q8_K records of 292 bytes (4-byte aligned).
template <bool A16>
__global__ void __launch_bounds__(QZ_WARPS * 32) quantize_q8_k_kernel(const float *__restrict__ x, uint8_t *__restrict__ y, long long blocks) {
    const int lane = threadIdx.x & 31;
    for (long long b = (long long)blockIdx.x * QZ_WARPS + (threadIdx.x >> 5); b < blocks; b += (long long)gridDim.x * QZ_WARPS) {
        float v[8];
        load8<A16>(x + b * 256 + 8 * lane, v);
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
        const float d = inverse == 0.0f ? 0.0f : __fdiv_rn(1.0f, inverse);
        uint32_t q0, q1;
        int sum;
        encode8(v, inverse, q0, q1, sum);
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        uint8_t *rec = y + b * 292;
        uint32_t *codes = reinterpret_cast<uint32_t *>(rec + 4 + 8 * lane);
        codes[0] = q0;
        codes[1] = q1;
        if ((lane & 1) == 0) *reinterpret_cast<int16_t *>(rec + 260 + lane) = (int16_t)sum;
        if (lane == 0) *reinterpret_cast<float *>(rec) = d;
    }
}

// X: `blocks` groups of 32 floats; Y: Q8_0 records of 34 bytes (2-byte aligned). Four lanes per record.
template <bool A16>
__global__ void __launch_bounds__(QZ_WARPS * 32) quantize_q8_0_kernel(const float *__restrict__ x, uint8_t *__restrict__ y, long long blocks) {
    const int lane = threadIdx.x & 31;
    const int sub = lane & 3;
    const long long groups = (blocks + 7) / 8;
    for (long long g = (long long)blockIdx.x * QZ_WARPS + (threadIdx.x >> 5); g < groups; g += (long long)gridDim.x * QZ_WARPS) {
        const long long b = g * 8 + (lane >> 2);
        const bool live = b < blocks;
        float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (live) load8<A16>(x + b * 32 + 8 * sub, v);
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        const float d = __fdiv_rn(amax, 127.0f);
        const float inverse = amax == 0.0f ? 0.0f : __fdiv_rn(1.0f, d);
        uint32_t q0, q1;
        int sum;
        encode8(v, inverse, q0, q1, sum);
        if (live) {
            uint8_t *rec = y + b * 34;
            uint16_t *codes = reinterpret_cast<uint16_t *>(rec + 2 + 8 * sub);
            codes[0] = (uint16_t)q0; codes[1] = (uint16_t)(q0 >> 16);
            codes[2] = (uint16_t)q1; codes[3] = (uint16_t)(q1 >> 16);
            if (sub == 0) *reinterpret_cast<__half *>(rec) = __float2half_rn(d);
        }
    }
}

cudaError_t launch_quantize(int act_fmt, const float *x, void *y, long long rows, long long k, int sm_count, cudaStream_t stream) {
    const long long elements = rows * k;
    if (elements == 0) return cudaSuccess;
    const bool a16 = (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
    uint8_t *yb = static_cast<uint8_t *>(y);
    const long long cap = (long long)sm_count * 32;
    if (act_fmt == F_Q8_K) {
        const long long blocks = elements / 256;
        const long long want = (blocks + QZ_WARPS - 1) / QZ_WARPS;
        const int grid = (int)(want > cap ? cap : want);
        if (a16) quantize_q8_k_kernel<true><<<grid, QZ_WARPS * 32, 0, stream>>>(x, yb, blocks);
        else quantize_q8_k_kernel<false><<<grid, QZ_WARPS * 32, 0, stream>>>(x, yb, blocks);
    } else if (act_fmt == F_Q8_0) {
        const long long blocks = elements / 32;
        const long long want = ((blocks + 7) / 8 + QZ_WARPS - 1) / QZ_WARPS;
        const int grid = (int)(want > cap ? cap : want);
        if (a16) quantize_q8_0_kernel<true><<<grid, QZ_WARPS * 32, 0, stream>>>(x, yb, blocks);
        else quantize_q8_0_kernel<false><<<grid, QZ_WARPS * 32, 0, stream>>>(x, yb, blocks);
    } else {
        return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

}  // namespace weft
