// Two-launch form of the peer all-gather: a kernel that pushes this rank's finished column block to every
// peer (flagged values or plain stores plus the ranks' barrier, see gather.cuh).  Used behind kernels that do not store to peers
// themselves (tensor-core prefill, the fallback GEMVs).
#include "kernels.h"

namespace weft {

namespace {

constexpr int GP_THREADS = 256;

__global__ void __launch_bounds__(GP_THREADS) gather_push_kernel(const GatherArgs g, long long m, long long n_local, long long ldy,
                                                                 int vec4, int *status) {
    const float *mine = g.y[g.rank];
    const int epoch = gather_epoch(g);
    const long long stride = (long long)gridDim.x * GP_THREADS;
    if (vec4 && !g.ll) {   // column blocks and pitch are multiples of four floats, buffers 16-byte aligned
        const long long per_row = n_local / 4;
        for (long long i = (long long)blockIdx.x * GP_THREADS + threadIdx.x; i < m * per_row; i += stride) {
            const size_t at = (size_t)(i / per_row) * ldy + 4 * (size_t)(i % per_row);
            const float4 v = *reinterpret_cast<const float4 *>(mine + at);
            for (int r = 0; r < g.world; ++r)
                if (r != g.rank) *reinterpret_cast<float4 *>(g.y[r] + at) = v;
        }
    } else {
        for (long long i = (long long)blockIdx.x * GP_THREADS + threadIdx.x; i < m * n_local; i += stride) {
            const long long row = i / n_local, col = i % n_local;
            gather_store(g, epoch, row, col, ldy, mine[(size_t)row * ldy + col]);
        }
    }
    const int warps = (int)gridDim.x * (GP_THREADS / 32);
    gather_receive(g, epoch, m, n_local, ldy, (int)blockIdx.x * (GP_THREADS / 32) + (threadIdx.x >> 5), warps, status);
    gather_finish(g, epoch, status, warps);
}

}  // namespace

cudaError_t launch_gather_push(const GatherArgs &g, long long m, long long n_local, long long ldy, int *status, int sm_count, cudaStream_t stream) {
    if (g.world < 2 || g.world > GATHER_MAX_RANKS || g.rank < 0 || g.rank >= g.world) return cudaErrorInvalidValue;
    bool vec4 = n_local % 4 == 0 && ldy % 4 == 0;
    for (int r = 0; r < g.world; ++r) vec4 = vec4 && (reinterpret_cast<uintptr_t>(g.y[r]) & 15u) == 0;
    const long long items = vec4 ? m * (n_local / 4) : m * n_local;
    long long ctas = (items + GP_THREADS - 1) / GP_THREADS;
    if (ctas > 2LL * sm_count) ctas = 2LL * sm_count;   // every CTA resident at once (256 threads, no shared memory): waiting warps hold nobody back
    if (ctas < 1) ctas = 1;
    gather_push_kernel<<<(unsigned)ctas, GP_THREADS, 0, stream>>>(g, m, n_local, ldy, vec4 ? 1 : 0, status);
    return cudaGetLastError();
}

}  // namespace weft
