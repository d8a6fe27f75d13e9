// Issue-rate measurement of the int8 tensor cores: every SM runs a bare loop of tcgen05.mma kind::i8 instructions
// (M = 128 per CTA, N = 256, K = 32) on operands that sit in shared memory, nothing else.  The result is the
// denominator for the prefill kernels' roofline fraction ("dense int8 peak as this device sustains it"), since the
// driver-measured peaks hold a bf16 figure only.  mode 0: one CTA per SM (cta_group::1); mode 1: CTA pairs
// (cta_group::2, M = 256); mode 2: kind::f16 (K = 16) with one CTA per SM, for comparison with the bf16 figure.
#include "prefill_common.cuh"
#include "kernels.h"

namespace weft {

namespace {

constexpr int MP_THREADS = 128;
constexpr int MP_SMEM = 1024 + 128 * 128 + 256 * 128;   // control + A slab (128 rows) + B slab (256 rows), 128 bytes of K each

template <int MODE>
__global__ void __launch_bounds__(MP_THREADS, 1) mma_peak_kernel(int iterations, unsigned long long *spans, int *status) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t *done = reinterpret_cast<uint64_t *>(smem);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + 64);
    const int warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < (MP_SMEM - 1024) / 4; i += MP_THREADS) reinterpret_cast<uint32_t *>(smem + 1024)[i] = 0x01010101u;
    if (threadIdx.x == 0) { mbar_init(done, 1); mbar_fence_init(); *tmem_slot = 0xffffffffu; }
    fence_proxy_async();
    __syncthreads();
    if (warp == 0) tc::tmem_alloc(tmem_slot, 512);   // per CTA, also for pairs
    tc::fence_before_sync();
    __syncthreads();
    if (MODE == 1) tc::cluster_sync_all();
    tc::fence_after_sync();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t *>(tmem_slot);
    if (tmem != 0u) { if (threadIdx.x == 0) report(status, ST_TMEM_ALLOC); return; }   // all 512 columns were asked for
    const bool issuer = threadIdx.x == 0 && (MODE != 1 || tc::cluster_ctarank() == 0);
    if (issuer) {
        const uint32_t a = smem_addr(smem + 1024), b = a + 128 * 128;
        const uint32_t idesc = MODE == 2 ? tc::idesc_f16_f32acc(128, 256) : tc::idesc_i8(MODE == 1 ? 256 : 128, 256, true, true);
        unsigned long long t0, t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        for (int it = 0; it < iterations; ++it) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint64_t ad = tc::smem_desc_sw128(a + k * 32), bd = tc::smem_desc_sw128(b + k * 32);
                const uint32_t d = tmem + (uint32_t)(it & 1) * 256;
                if (MODE == 1) tc::mma_i8_pair(d, ad, bd, idesc, 1);
                else if (MODE == 2) tc::mma_f16(d, ad, bd, idesc, 1);
                else tc::mma_i8(d, ad, bd, idesc, 1);
            }
        }
        if (MODE == 1) tc::commit_pair(smem_addr(done)); else tc::commit(done);
        if (!mbar_wait(done, 0, 1u << 26)) report(status, ST_WAIT_TIMEOUT);
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
        spans[blockIdx.x] = t1 - t0;
    }
    tc::fence_before_sync();
    __syncthreads();
    if (MODE == 1) tc::cluster_sync_all();
    if (warp == 0) tc::tmem_free(tmem, 512);
}

}  // namespace

// TOP/s (mode 0, 1: int8) or TFLOP/s (mode 2: f16) over the whole device; `spans_dev` holds sm_count 64-bit slots.
cudaError_t measure_mma_peak(int mode, int iterations, int sm_count, unsigned long long *spans_dev, int *status, cudaStream_t stream, double *ops_per_launch) {
    const int ctas = mode == 1 ? (sm_count & ~1) : sm_count;
    cudaError_t e;
    if (mode == 0) {
        e = grant_dynamic_smem(reinterpret_cast<const void *>(mma_peak_kernel<0>), MP_SMEM);
        if (e != cudaSuccess) return e;
        mma_peak_kernel<0><<<ctas, MP_THREADS, MP_SMEM, stream>>>(iterations, spans_dev, status);
    } else if (mode == 2) {
        e = grant_dynamic_smem(reinterpret_cast<const void *>(mma_peak_kernel<2>), MP_SMEM);
        if (e != cudaSuccess) return e;
        mma_peak_kernel<2><<<ctas, MP_THREADS, MP_SMEM, stream>>>(iterations, spans_dev, status);
    } else {
        e = grant_dynamic_smem(reinterpret_cast<const void *>(mma_peak_kernel<1>), MP_SMEM);
        if (e != cudaSuccess) return e;
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3((unsigned)ctas);
        config.blockDim = dim3(MP_THREADS);
        config.dynamicSmemBytes = MP_SMEM;
        config.stream = stream;
        cudaLaunchAttribute attribute[1];
        attribute[0].id = cudaLaunchAttributeClusterDimension;
        attribute[0].val.clusterDim.x = 2; attribute[0].val.clusterDim.y = 1; attribute[0].val.clusterDim.z = 1;
        config.attrs = attribute;
        config.numAttrs = 1;
        e = cudaLaunchKernelEx(&config, mma_peak_kernel<1>, iterations, spans_dev, status);
        if (e != cudaSuccess) return e;
    }
    // per issuing CTA: iterations x 4 instructions of 2 * M * N * K operations
    const double per_instruction = 2.0 * (mode == 1 ? 256.0 : 128.0) * 256.0 * (mode == 2 ? 16.0 : 32.0);
    *ops_per_launch = (double)(mode == 1 ? ctas / 2 : ctas) * iterations * 4.0 * per_instruction;
    return cudaGetLastError();
}

}  // namespace weft
