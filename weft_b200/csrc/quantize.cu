// Standalone activation quantizers q8_0_quantize / q8_1_quantize / q8_K_quantize (one warp per 256 elements).
// The arithmetic lives in quantize.cuh.  HBM-bound: 4 bytes read per 1.06-1.14 bytes written.
#include "quantize.cuh"
#include "kernels.h"

namespace weft {

constexpr int QZ_WARPS = 8;

// X: `blocks` consecutive groups of 256 floats; Y: `blocks` Q8_K records of 292 bytes (4-byte aligned).
template <bool A16>
__global__ void __launch_bounds__(QZ_WARPS * 32) quantize_q8_k_kernel(const float *__restrict__ x, uint8_t *__restrict__ y, long long blocks) {
    const int lane = threadIdx.x & 31;
    for (long long b = (long long)blockIdx.x * QZ_WARPS + (threadIdx.x >> 5); b < blocks; b += (long long)gridDim.x * QZ_WARPS) {
        float v[8];
        load8<A16>(x + b * 256 + 8 * lane, v);
        uint32_t q0, q1;
        int sum16;
        float d;
        q8_k_warp(v, q0, q1, sum16, d);
        store_q8_k(y + b * 292, lane, q0, q1, sum16, d);
    }
}

// X: `blocks` groups of 32 floats; Y: Q8_0 records of 34 bytes or Q8_1 records of 36 (2-byte aligned). Four lanes per record.
template <bool A16, bool WITH_SUM>
__global__ void __launch_bounds__(QZ_WARPS * 32) quantize_q8_0_kernel(const float *__restrict__ x, uint8_t *__restrict__ y, long long blocks) {
    const int lane = threadIdx.x & 31;
    const int sub = lane & 3;
    const long long groups = (blocks + 7) / 8;
    for (long long g = (long long)blockIdx.x * QZ_WARPS + (threadIdx.x >> 5); g < groups; g += (long long)gridDim.x * QZ_WARPS) {
        const long long b = g * 8 + (lane >> 2);
        const bool live = b < blocks;
        float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (live) load8<A16>(x + b * 32 + 8 * sub, v);
        uint32_t q0, q1;
        int sum32;
        float d;
        q8_0_warp(v, q0, q1, sum32, d);
        if (live) {
            if (WITH_SUM) store_q8_1(y + b * 36, sub, q0, q1, sum32, d);
            else store_q8_0(y + b * 34, sub, q0, q1, d);
        }
    }
}

// Byte copy for small staged arguments; 16-byte words when both sides allow, whole bytes otherwise.
__global__ void __launch_bounds__(256) copy_bytes_kernel(uint8_t *__restrict__ dst, const uint8_t *__restrict__ src, size_t bytes, int vec) {
    // The kernel behind this one may start its own prologue now (programmatic dependent launch); it waits for this
    // grid to complete before it touches what is copied here.
    asm volatile("griddepcontrol.launch_dependents;");
    const size_t stride = (size_t)gridDim.x * 256, first = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (vec) {
        for (size_t i = first; i < bytes / 16; i += stride) reinterpret_cast<uint4 *>(dst)[i] = reinterpret_cast<const uint4 *>(src)[i];
        for (size_t i = (bytes & ~size_t(15)) + first; i < bytes; i += stride) dst[i] = src[i];
    } else {
        for (size_t i = first; i < bytes; i += stride) dst[i] = src[i];
    }
}

cudaError_t launch_copy_bytes(void *dst, const void *src, size_t bytes, cudaStream_t stream) {
    if (!bytes) return cudaSuccess;
    const int vec = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15u) == 0;
    size_t ctas = ((vec ? bytes / 16 : bytes) + 255) / 256;
    if (ctas > 64) ctas = 64;
    if (ctas < 1) ctas = 1;
    copy_bytes_kernel<<<(unsigned)ctas, 256, 0, stream>>>(static_cast<uint8_t *>(dst), static_cast<const uint8_t *>(src), bytes, vec);
    return cudaGetLastError();
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
    } else if (act_fmt == F_Q8_0 || act_fmt == F_Q8_1) {
        const long long blocks = elements / 32;
        const long long want = ((blocks + 7) / 8 + QZ_WARPS - 1) / QZ_WARPS;
        const int grid = (int)(want > cap ? cap : want);
        if (act_fmt == F_Q8_1) {
            if (a16) quantize_q8_0_kernel<true, true><<<grid, QZ_WARPS * 32, 0, stream>>>(x, yb, blocks);
            else quantize_q8_0_kernel<false, true><<<grid, QZ_WARPS * 32, 0, stream>>>(x, yb, blocks);
        } else if (a16) quantize_q8_0_kernel<true, false><<<grid, QZ_WARPS * 32, 0, stream>>>(x, yb, blocks);
        else quantize_q8_0_kernel<false, false><<<grid, QZ_WARPS * 32, 0, stream>>>(x, yb, blocks);
    } else {
        return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

}  // namespace weft
