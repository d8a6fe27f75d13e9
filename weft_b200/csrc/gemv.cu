// Decode path: Y[m, n] = quantized_vec_dot(W[n], Xq[m]) for every weight row -- the loop the
// reference's production_mul_mat_*_decode kernels spell out (examples/kernels/mul_mat/q4_k_decode.py:17-20)
// around the block dots of examples/kernels/vec_dot/{q4_0_q8_0,q8_0_q8_0,q2_k_q8_k,q3_k_q8_k,q4_k_q8_k,q5_k_q8_k,q6_k_q8_k,iq2_xxs_q8_k,tq1_0_q8_k}.py
// (GGML: ggml-cpu/quants.c:174-208, 400-428, 514-564, 566-643, 645-718, 720-798, 800-853, 855-895, 430-480).
//
// The GEMV is HBM-bound: each weight byte is read exactly once.  One persistent CTA per SM owns a
// contiguous range of weight rows.  Every warp streams whole rows from HBM into its own shared-memory
// double buffer with bulk asynchronous copies (cp.async.bulk + mbarrier: one instruction moves
// kilobytes, so the bytes in flight per SM do not depend on how many loads a thread can issue), claims
// its next rows from a shared-memory counter (so the tail is one row long, not one warp-share long),
// and computes from shared memory with packed int8 dot products (dp4a).  Activations are staged once
// per CTA into a bank-conflict-free layout.  Row sums are reduced with warp shuffles; a row is never
// split across warps or GPUs, so results do not depend on the grid.
//
// Float op trees per 256-element unit follow the DSL kernels:
//   Q4_0  acc += (d_w*d_x) * f32(sum)              Q8_0  acc += f32(sum) * (d_w*d_x)
//   Q4_K  acc += x.d * (d*f32(isum) - dmin*f32(msum))
//   IQ2_XXS acc += (d_w*x.d) * f32(bsum), result *= 0.125     TQ1_0 acc += f32(sum) * (d_w*x.d)
//   Q6_K  acc += (d_w*x.d) * f32(isum)                        Q5_K, Q2_K  as Q4_K      Q3_K  as Q6_K
#include "gemv_units.cuh"

#include <climits>
#include <cstdlib>
#include <map>
#include <mutex>
#include <utility>

namespace weft {


struct GemvParams {
    const uint8_t *w;
    const uint8_t *xq;       // activation records: read, or written by CTA column 0 when the prologue quantizes
    const float *x;          // fp32 activations (fused-quantize kernels only)
    const int8_t *grid;
    const int8_t *signs;
    const uint32_t *powers;
    float *y;
    long long n;
    int nb;            // 256-element units per row
    long long ldy;
    int lanes_per_row; // power of two, <= 32
    int stage_bytes;   // per-buffer bytes (16-byte multiple, includes slack)
    int nbuf;          // ring depth per warp (2..4)
    int *status;
};
// ------------------------------------------------------------------ the kernel

template <int FMT, int RL, bool BULK, bool QX>
__global__ void __launch_bounds__(512) gemv_kernel(const GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int UB = Unit<FMT>::BYTES;
    constexpr bool ACT_Q8_0 = (FMT == F_Q4_0 || FMT == F_Q8_0);
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb = p.nb;
    const int L = p.lanes_per_row, RPW = 32 / L, SR = RPW * RL;
    const int row_bytes = nb * UB;

    // carve shared memory
    const int NBUF = p.nbuf;
    int *s_next = reinterpret_cast<int *>(smem);
    uint64_t *s_bar = reinterpret_cast<uint64_t *>(smem + 16);          // four barriers per warp
    int *s_rows = reinterpret_cast<int *>(smem + 16 + 32 * warps);      // four claimed row offsets per warp
    uint8_t *cursor = smem + 16 + 48 * warps;
    uint8_t *s_tab0 = cursor, *s_tab1 = cursor;
    // codebook formats: the grid as given, then the sign table as byte masks (1 KB)
    constexpr int GRID_BYTES = FMT == F_IQ2_XXS ? 2048 : FMT == F_IQ2_XS ? 4096 : FMT == F_IQ3_XXS ? 1024 : FMT == F_IQ2_S ? 8192 : FMT == F_IQ3_S ? 2048 : (FMT == F_IQ1_S || FMT == F_IQ1_M) ? 16384 : 0;
    constexpr bool SIGN_TABLE = FMT == F_IQ2_XXS || FMT == F_IQ2_XS || FMT == F_IQ3_XXS;
    if (GRID_BYTES) { s_tab1 = cursor + GRID_BYTES; cursor += GRID_BYTES + (SIGN_TABLE ? 1024 : 0); }
    uint8_t *s_xq = cursor;
    cursor += nb * XQ_PITCH;
    uint8_t *s_xaux = cursor;
    cursor += nb * XAUX_BYTES;
    uint8_t *s_ring = cursor + (size_t)warp * NBUF * p.stage_bytes;

    // this CTA's rows
    const long long r_begin = p.n * blockIdx.x / gridDim.x, r_end = p.n * (blockIdx.x + 1) / gridDim.x;
    const size_t xq_row = (size_t)blockIdx.y * nb * (ACT_Q8_0 ? 272 : 292);
    const uint8_t *xq = p.xq + xq_row;
    float *y = p.y + (size_t)blockIdx.y * p.ldy;

    if (threadIdx.x == 0) {
        *s_next = 0;
        for (int i = 0; i < 4 * warps; ++i) mbar_init(s_bar + i, 1);
        mbar_fence_init();
    }
    __syncthreads();

    uint64_t *bar = s_bar + 4 * warp;
    int *my_rows = s_rows + 4 * warp;
    const long long rows_here = r_end - r_begin;

    auto claim = [&]() -> long long {
        int r = 0;
        if (lane == 0) r = atomicAdd(s_next, SR);
        return (long long)__shfl_sync(0xffffffffu, r, 0);
    };
    auto issue = [&](int buf, long long row0) {
        if (row0 >= rows_here) return;
        const long long rows = min((long long)SR, rows_here - row0);
        const uint8_t *src = p.w + (size_t)(r_begin + row0) * row_bytes;
        uint8_t *dst = s_ring + (size_t)buf * p.stage_bytes;
        const uint32_t bytes = (uint32_t)(rows * row_bytes);
        if (BULK) {
            if (lane == 0) {
                fence_proxy_async();
                mbar_expect_tx(bar + buf, bytes);
                bulk_g2s(dst, src, bytes, bar + buf);
            }
        } else {   // rows that are not 16-byte multiples: plain 2-byte copies by the whole warp
            for (uint32_t i = lane; i < bytes / 2; i += 32)
                reinterpret_cast<uint16_t *>(dst)[i] = __ldg(reinterpret_cast<const uint16_t *>(src) + i);
        }
    };

    // first copies go out before anything else is touched
    for (int b = 0; b < NBUF - 1; ++b) {
        const long long r = claim();
        if (lane == 0) my_rows[b] = (int)min(r, (long long)INT_MAX);
        issue(b, r);
    }

    // stage tables and activations
    if (GRID_BYTES) {
        for (int i = threadIdx.x; i < GRID_BYTES; i += blockDim.x) s_tab0[i] = (uint8_t)p.grid[i];
        if (SIGN_TABLE) for (int i = threadIdx.x; i < 1024; i += blockDim.x) s_tab1[i] = p.signs[i] < 0 ? 0xffu : 0u;
    }
    uint32_t pw[5] = {1, 3, 9, 27, 81};
    if (FMT == F_TQ1_0) {
#pragma unroll
        for (int i = 0; i < 5; ++i) pw[i] = __ldg(p.powers + i) & 0xffu;
    }
    if (QX) {
        uint8_t *out = blockIdx.x == 0 ? const_cast<uint8_t *>(xq) : nullptr;
        const float *x = p.x + (size_t)blockIdx.y * nb * 256;
        if (ACT_Q8_0) quantize_stage_q8_0(x, nb, s_xq, s_xaux, out); else quantize_stage_q8_k(x, nb, s_xq, s_xaux, out);
    } else {
        if (ACT_Q8_0) stage_q8_0(xq, nb, s_xq, s_xaux); else stage_q8_k(xq, nb, s_xq, s_xaux);
    }
    __syncthreads();

    const int slot = lane / L, ul = lane % L;
    uint32_t phases = 0;   // bit b = parity the next wait on buffer b expects
    int buf = 0;
    while (true) {
        __syncwarp();
        const long long cur = my_rows[buf];
        if (cur >= rows_here) break;
        {   // refill the buffer that the previous iteration finished reading
            const int spare = buf == 0 ? NBUF - 1 : buf - 1;
            const long long nxt = claim();
            if (lane == 0) my_rows[spare] = (int)min(nxt, (long long)INT_MAX);
            issue(spare, nxt);
        }
        if (BULK) {
            if (!mbar_wait(bar + buf, (phases >> buf) & 1u)) { report(p.status, ST_WAIT_TIMEOUT); return; }
            phases ^= 1u << buf;
        } else {
            __syncwarp();
        }
        const uint8_t *stage = s_ring + (size_t)buf * p.stage_bytes;
        float acc[RL];
        const uint8_t *wp[RL];
        bool live[RL];
#pragma unroll
        for (int r = 0; r < RL; ++r) {
            acc[r] = 0.f;
            live[r] = cur + slot * RL + r < rows_here;
        }
        for (int u = ul; u < nb; u += L) {
#pragma unroll
            for (int r = 0; r < RL; ++r)   // rows past the end read row 0 of the stage (always valid) and are dropped
                wp[r] = stage + (size_t)(live[r] ? slot * RL + r : 0) * row_bytes + (size_t)u * UB;
            const uint8_t *xu = s_xq + u * XQ_PITCH, *xa = s_xaux + u * XAUX_BYTES;
            if (FMT == F_Q4_K) dot_q4_k<RL>(wp, xu, xa, acc);
            else if (FMT == F_Q4_0) dot_q4_0<RL>(wp, xu, xa, acc);
            else if (FMT == F_Q8_0) dot_q8_0<RL>(wp, xu, xa, acc);
            else if (FMT == F_Q2_K) dot_q2_k<RL>(wp, xu, xa, acc);
            else if (FMT == F_Q3_K) dot_q3_k<RL>(wp, xu, xa, acc);
            else if (FMT == F_Q5_K) dot_q5_k<RL>(wp, xu, xa, acc);
            else if (FMT == F_Q6_K) dot_q6_k<RL>(wp, xu, xa, acc);
            else if (FMT == F_IQ2_XXS) dot_iq2_xxs<RL>(wp, xu, xa, s_tab0, s_tab1, acc);
            else if (FMT == F_IQ2_XS) dot_iq2_xs<RL>(wp, xu, xa, s_tab0, s_tab1, acc);
            else if (FMT == F_IQ3_XXS) dot_iq3_xxs<RL>(wp, xu, xa, s_tab0, s_tab1, acc);
            else if (FMT == F_IQ2_S) dot_iq2_s<RL>(wp, xu, xa, s_tab0, acc);
            else if (FMT == F_IQ3_S) dot_iq3_s<RL>(wp, xu, xa, s_tab0, acc);
            else if (FMT == F_IQ1_S) dot_iq1_s<RL>(wp, xu, xa, s_tab0, acc);
            else if (FMT == F_IQ1_M) dot_iq1_m<RL>(wp, xu, xa, s_tab0, reinterpret_cast<const float *>(p.powers), acc);
            else dot_tq1_0<RL>(wp, xu, xa, pw, acc);
        }
#pragma unroll
        for (int r = 0; r < RL; ++r) {
            float v = acc[r];
            for (int o = L >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (FMT == F_IQ2_XXS || FMT == F_IQ2_XS || FMT == F_IQ2_S) v *= 0.125f;
            if (FMT == F_IQ3_XXS) v *= 0.25f;
            if (ul == 0 && live[r]) y[r_begin + cur + slot * RL + r] = v;
        }
        buf = buf + 1 == NBUF ? 0 : buf + 1;
    }
}

// ------------------------------------------------------------------ 32-element formats with K % 256 != 0
// One warp per weight row, one lane per record; plain loads. Correctness path for odd shapes only.
template <int FMT>
__global__ void gemv_block32_kernel(const uint8_t *__restrict__ w, const uint8_t *__restrict__ xq, float *__restrict__ y,
                                    long long n, long long blocks, long long ldy) {
    constexpr int RB = record_bytes(FMT);
    const int lane = threadIdx.x & 31;
    const uint8_t *x = xq + (size_t)blockIdx.y * blocks * 34;
    for (long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < n; row += (long long)gridDim.x * (blockDim.x >> 5)) {
        float acc = 0.f;
        for (long long b = lane; b < blocks; b += 32) {
            const uint8_t *wr = w + ((size_t)row * blocks + b) * RB, *xr = x + (size_t)b * 34;
            const float dw = half_bits_to_float(ld_u16(wr)), dx = half_bits_to_float(ld_u16(xr));
            int s = 0;
            if (FMT == F_Q4_0) {
                for (int j = 0; j < 16; ++j) {
                    s += ((int)(wr[2 + j] & 15) - 8) * (int)(int8_t)xr[2 + j];
                    s += ((int)(wr[2 + j] >> 4) - 8) * (int)(int8_t)xr[18 + j];
                }
                acc += (dw * dx) * (float)s;
            } else {
                for (int j = 0; j < 32; ++j) s += (int)(int8_t)wr[2 + j] * (int)(int8_t)xr[2 + j];
                acc += (float)s * (dw * dx);
            }
        }
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) y[(size_t)blockIdx.y * ldy + row] = acc;
    }
}

// ------------------------------------------------------------------ launch

cudaError_t grant_dynamic_smem(const void *kernel, int bytes) {
    static std::mutex lock;
    static std::map<std::pair<const void *, int>, int> granted;
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> guard(lock);
    int &have = granted[{kernel, device}];
    if (bytes > have) {
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) return e;
        have = bytes;
    }
    return cudaSuccess;
}

// launch shape (measured on B200)
constexpr int kEnvWarps = 12;
constexpr int kEnvRowsPerLane = 1;
constexpr int kEnvRingDepth = 3;

template <int FMT>
static cudaError_t launch_fmt(const GemvArgs &a, int sm_count, cudaStream_t stream) {
    constexpr int UB = Unit<FMT>::BYTES;
    const int nb = (int)(a.k / 256);
    const long long row_bytes = (long long)nb * UB;
    int L = 1;
    while (L < 32 && L < nb) L <<= 1;
    const bool bulk = (row_bytes % 16 == 0) && ((reinterpret_cast<uintptr_t>(a.w) & 15u) == 0);
    const int smem_cap = 200 * 1024;
    int warps = kEnvWarps;
    warps = warps < 1 ? 1 : (warps > 16 ? 16 : warps);
    int rl = kEnvRowsPerLane;
    const long long x_bytes = (long long)nb * (XQ_PITCH + XAUX_BYTES) + (FMT == F_IQ2_XXS ? 3072 : FMT == F_IQ2_XS ? 5120 : FMT == F_IQ3_XXS ? 2048 : FMT == F_IQ2_S ? 8192 : FMT == F_IQ3_S ? 2048 : (FMT == F_IQ1_S || FMT == F_IQ1_M) ? 16384 : 0) + 16 + 48 * 16;
    int nbuf = kEnvRingDepth;
    nbuf = nbuf < 2 ? 2 : (nbuf > 4 ? 4 : nbuf);
    auto ring = [&](int w_, int rl_) { return (long long)w_ * nbuf * (((32 / L) * rl_ * row_bytes + 31) / 16 * 16); };
    if (FMT == F_Q8_0) rl = 1;   // 68 weight words per row already fill the register budget
    while (rl > 1 && x_bytes + ring(warps, rl) > smem_cap) rl = 1;
    while (nbuf > 2 && x_bytes + ring(warps, rl) > smem_cap) --nbuf;
    while (warps > 1 && x_bytes + ring(warps, rl) > smem_cap) --warps;
    if (x_bytes + ring(warps, rl) > smem_cap) return cudaErrorInvalidConfiguration;   // K too large for shared-memory staging
    const int stage_rows = (32 / L) * rl;
    const int stage_bytes = (int)((stage_rows * row_bytes + 31) / 16 * 16);
    const size_t smem = (size_t)(x_bytes + ring(warps, rl));

    GemvParams p;
    p.w = static_cast<const uint8_t *>(a.w); p.xq = static_cast<const uint8_t *>(a.xq);
    p.grid = a.grid; p.signs = a.signs; p.powers = a.powers; p.y = a.y;
    p.n = a.n; p.nb = nb; p.ldy = a.ldy; p.lanes_per_row = L; p.stage_bytes = stage_bytes; p.nbuf = nbuf; p.status = a.status;
    p.x = a.x;
    // the prologue can quantize X itself when the fp32 rows allow 16-byte loads
    const bool qx = a.x != nullptr;

    const long long stages = (a.n + stage_rows - 1) / stage_rows;
    long long ctas = (stages + warps - 1) / warps;   // never more CTAs than there is work for whole warps
    if (ctas > sm_count) ctas = sm_count;
    if (ctas < 1) ctas = 1;
    dim3 grid((unsigned)ctas, (unsigned)a.m);

#define WEFT_LAUNCH(RLV, BULKV, QXV)                                                                                 \
    do {                                                                                                              \
        cudaError_t e = grant_dynamic_smem(reinterpret_cast<const void *>(gemv_kernel<FMT, RLV, BULKV, QXV>), (int)smem);    \
        if (e != cudaSuccess) return e;                                                                               \
        gemv_kernel<FMT, RLV, BULKV, QXV><<<grid, warps * 32, smem, stream>>>(p);                                     \
    } while (0)
#define WEFT_LAUNCH_Q(RLV, BULKV) do { if (qx) WEFT_LAUNCH(RLV, BULKV, true); else WEFT_LAUNCH(RLV, BULKV, false); } while (0)
    if (rl == 2) { if (bulk) WEFT_LAUNCH_Q(2, true); else WEFT_LAUNCH_Q(2, false); }
    else { if (bulk) WEFT_LAUNCH_Q(1, true); else WEFT_LAUNCH_Q(1, false); }
#undef WEFT_LAUNCH_Q
#undef WEFT_LAUNCH
    return cudaGetLastError();
}

static const bool kGenericOnly = getenv("WEFT_B200_GENERIC_GEMV") != nullptr;

bool gemv_gathers(const GemvArgs &a) {
    // One activation row only: the grid is then at most one CTA per SM, all resident at once.  A warp that waits
    // for a peer's values keeps its SM; with more CTAs than SMs two ranks could each hold back the CTAs whose
    // values the other is waiting for.
    if (a.k % 256 != 0 || a.k == 0 || a.fmt == F_Q4_K_I16 || kGenericOnly || a.m != 1) return false;
    return gemv_q4k_supported(a) || gemv_ring_supported(a);
}

cudaError_t launch_gemv(const GemvArgs &a, int sm_count, cudaStream_t stream) {
    if (a.segments > 1) return gemv_q4k_groups(a) && !kGenericOnly ? launch_gemv_q4k(a, sm_count, stream) : cudaErrorInvalidValue;
    if (a.n == 0 || a.m == 0) return cudaSuccess;
    if (a.m > 65535) return cudaErrorInvalidValue;
    if ((a.fmt == F_Q4_0 || a.fmt == F_Q8_0) && a.k % 256 != 0) {
        const long long blocks = a.k / 32;
        const int warps = 8;
        long long gx = (a.n + warps - 1) / warps;
        if (gx > (long long)sm_count * 8) gx = (long long)sm_count * 8;
        dim3 grid((unsigned)gx, (unsigned)a.m);
        if (a.fmt == F_Q4_0) gemv_block32_kernel<F_Q4_0><<<grid, warps * 32, 0, stream>>>((const uint8_t *)a.w, (const uint8_t *)a.xq, a.y, a.n, blocks, a.ldy);
        else gemv_block32_kernel<F_Q8_0><<<grid, warps * 32, 0, stream>>>((const uint8_t *)a.w, (const uint8_t *)a.xq, a.y, a.n, blocks, a.ldy);
        return cudaGetLastError();
    }
    if (a.k % 256 != 0 || a.k == 0) return cudaErrorInvalidValue;
    if (a.fmt == F_Q4_K_I16) return launch_gemv_q4ki(a, sm_count, stream);
    const bool generic_only = kGenericOnly;
    if (!generic_only && gemv_q4k_supported(a)) return launch_gemv_q4k(a, sm_count, stream);
    if (!generic_only && gemv_ring_supported(a)) return launch_gemv_ring(a, sm_count, stream);
    switch (a.fmt) {
    case F_Q4_0: return launch_fmt<F_Q4_0>(a, sm_count, stream);
    case F_Q8_0: return launch_fmt<F_Q8_0>(a, sm_count, stream);
    case F_Q4_K: return launch_fmt<F_Q4_K>(a, sm_count, stream);
    case F_Q2_K: return launch_fmt<F_Q2_K>(a, sm_count, stream);
    case F_Q3_K: return launch_fmt<F_Q3_K>(a, sm_count, stream);
    case F_Q5_K: return launch_fmt<F_Q5_K>(a, sm_count, stream);
    case F_Q6_K: return launch_fmt<F_Q6_K>(a, sm_count, stream);
    case F_IQ2_XXS: return launch_fmt<F_IQ2_XXS>(a, sm_count, stream);
    case F_IQ2_XS: return launch_fmt<F_IQ2_XS>(a, sm_count, stream);
    case F_IQ3_XXS: return launch_fmt<F_IQ3_XXS>(a, sm_count, stream);
    case F_IQ2_S: return launch_fmt<F_IQ2_S>(a, sm_count, stream);
    case F_IQ3_S: return launch_fmt<F_IQ3_S>(a, sm_count, stream);
    case F_IQ1_S: return launch_fmt<F_IQ1_S>(a, sm_count, stream);
    case F_IQ1_M: return launch_fmt<F_IQ1_M>(a, sm_count, stream);
    case F_TQ1_0: return launch_fmt<F_TQ1_0>(a, sm_count, stream);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace weft
