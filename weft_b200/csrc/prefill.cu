// Prefill path: Y[m, n] = sum over 256-blocks of x.ds * (w.d * isum - w.dmin * msum), the contraction of
// the reference's production_mul_mat_q4_k_staged (examples/kernels/mul_mat/q4_k_staged.py:9-37; per block
// the math of examples/kernels/vec_dot/q4_k_q8_k.py:8-29, GGML ggml-cpu/quants.c:645-718), on the int8
// tensor cores of sm_100a (tcgen05.mma kind::i8, accumulators in tensor memory).
//
// Tensor-core bound: 2*M*N*K useful integer ops (60.1 GOP for 512 x 14336 x 4096).
//
// How Q4_K becomes int8 MMAs without losing exactness.  Inside a 256-block,
//   isum[m,n] = sum_g sc[n,g] * sum_{k in g} q[n,k] * x[m,k]          (q in 0..15, sc in 0..63, x int8)
// The 6-bit scale is folded into the weight operand, which then needs 10 bits, so it is split in two
// int8 limbs:  sc = 8a + c (a, c in 0..7),  q*sc = 8*(q*a) + (q*c),  q*a and q*c <= 105.  One MMA with
// N = 2*BN columns ([q*a | q*c]) accumulates both limbs over the whole block in int32 (exact), and
// isum = 8*D_hi + D_lo.  Useful ops are therefore half of the issued ops.
//   msum[m,n] = sum_g mn[n,g] * (bsum[m,2g] + bsum[m,2g+1])            (mn in 0..63, pair sums in +-8128)
// goes through ONE extra K = 16 MMA of kind::f16 per block: the pair sum is split as 64h + l (l in 0..63),
// the operands are the exact small integers {l, h} and {mn, 64 mn} in f16, products and the 16-term fp32
// sum are exact (< 2^24).  The per-block float combine runs on the CUDA cores in the epilogue with the
// reference's own op order, accumulating in fp32 registers across blocks.
//
// CTA = 128 tokens (TMEM lanes) x BN weights, persistent over tiles.  Warp roles:
//   warps 0-3  epilogue: tcgen05.ld the three accumulator groups, combine, keep 128 x BN fp32 in registers
//   warps 4-7  producers: read Q4_K records and Q8_K records from global memory (in place, no repack in
//              HBM), expand them into the K-major core-matrix layout the MMA reads from shared memory
//   warp 8     allocates TMEM; one lane issues the MMAs and commits them to mbarriers
// Two shared-memory stages let the producers run one 256-block ahead of the tensor core.  Every wait is
// bounded; a wait that runs out sets an abort flag, all roles leave their loops, TMEM is freed, and the
// host sees a status code instead of a hang.
#include "tcgen05.cuh"
#include "kernels.h"

#include <cstdlib>

namespace weft {

namespace {

constexpr int PF_BM = 128;               // tokens per tile = TMEM lanes
constexpr int PF_THREADS = 288;          // 4 epilogue + 4 producer + 1 MMA warp
constexpr int PF_STAGES = 2;
constexpr int PF_SCALE_SLOTS = 4;        // ring of per-block float scales, read by the epilogue after the MMA

template <int BN> struct PfLayout {
    static constexpr int A_Q = PF_BM * 256;          // activations, int8
    static constexpr int B_Q = 2 * BN * 256;         // [q*a | q*c], int8
    static constexpr int A_M = PF_BM * 32;           // {l, h} f16
    static constexpr int B_M = BN * 32;              // {mn, 64 mn} f16
    static constexpr int STAGE = A_Q + B_Q + A_M + B_M;
    static constexpr int WD = BN * 8;                // {d, dmin} per weight row
    static constexpr int XD = PF_BM * 4;             // x.ds per token
    static constexpr int SCALES = WD + XD;
    static constexpr int CONTROL = 1024;
    static constexpr int TOTAL = CONTROL + PF_STAGES * STAGE + PF_SCALE_SLOTS * SCALES;
    static constexpr int TMEM_COLS = 3 * BN <= 32 ? 32 : 3 * BN <= 64 ? 64 : 3 * BN <= 128 ? 128 : 3 * BN <= 256 ? 256 : 512;
};

struct PfParams {
    const uint8_t *w;     // (n, k) Q4_K records, 16-byte aligned rows
    const uint8_t *xq;    // (m, k) Q8_K records
    float *y;             // (m, ldy)
    long long n, m, ldy;
    int nb;               // 256-blocks per row
    int m_tiles, n_tiles;
    int *status;
};

// byte offset of (row, 16-byte K chunk) in a K-major operand without swizzle: 8-row groups of
// `chunks` core matrices (8 rows x 16 bytes each, 128 contiguous bytes)
__device__ __forceinline__ uint32_t core_offset(int row, int chunk, int chunks) {
    return (uint32_t)((row >> 3) * (chunks * 128) + chunk * 128 + (row & 7) * 16);
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    return (uint32_t)__half_as_ushort(__float2half_rn(lo)) | ((uint32_t)__half_as_ushort(__float2half_rn(hi)) << 16);
}

struct Control {
    uint64_t full[PF_STAGES];
    uint64_t empty[PF_STAGES];
    uint64_t tmem_full;
    uint64_t tmem_empty;
    uint32_t tmem_base;
    volatile int abort;
};

// bounded wait that also gives up as soon as another role has aborted
__device__ __forceinline__ bool wait_or_abort(uint64_t *bar, uint32_t parity, Control *ctl, int *status) {
    for (uint32_t i = 0; i < (1u << 20); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (ctl->abort) return false;
    }
    ctl->abort = 1;
    report(status, ST_WAIT_TIMEOUT);
    return false;
}

}  // namespace

namespace {

// ---- producer: one thread expands weight row `p` of the tile and token row `p` of the tile ------------
template <int BN>
__device__ __forceinline__ void produce_block(const PfParams &p, uint8_t *stage, uint8_t *scales, int row, long long n0, long long m0, int b) {
    using L = PfLayout<BN>;
    uint8_t *a_q = stage, *b_q = stage + L::A_Q, *a_m = b_q + L::B_Q, *b_m = a_m + L::A_M;
    float2 *wd = reinterpret_cast<float2 *>(scales);
    float *xd = reinterpret_cast<float *>(scales + L::WD);
    const size_t w_row_bytes = (size_t)p.nb * 144, x_row_bytes = (size_t)p.nb * 292;

    // weights
    if (row < BN) {
        const long long n = n0 + row;
        if (n < p.n) {
            const uint4 *rec = reinterpret_cast<const uint4 *>(p.w + (size_t)n * w_row_bytes + (size_t)b * 144);
            const uint4 hd = __ldg(rec);
            wd[row] = make_float2(half_bits_to_float(hd.x), half_bits_to_float(hd.x >> 16));
            const Q4KScales s = q4k_unpack_scales(hd.y, hd.z, hd.w);
            {   // {mn_g} and {64 mn_g} as f16: chunk 0 and chunk 1 of the min operand
                float mn[8];
#pragma unroll
                for (int g = 0; g < 8; ++g) mn[g] = (float)byte_of(g < 4 ? s.mn_lo : s.mn_hi, g & 3);
                uint4 c0, c1;
                c0.x = pack_half2(mn[0], mn[1]); c0.y = pack_half2(mn[2], mn[3]); c0.z = pack_half2(mn[4], mn[5]); c0.w = pack_half2(mn[6], mn[7]);
                c1.x = pack_half2(64.f * mn[0], 64.f * mn[1]); c1.y = pack_half2(64.f * mn[2], 64.f * mn[3]);
                c1.z = pack_half2(64.f * mn[4], 64.f * mn[5]); c1.w = pack_half2(64.f * mn[6], 64.f * mn[7]);
                *reinterpret_cast<uint4 *>(b_m + core_offset(row, 0, 2)) = c0;
                *reinterpret_cast<uint4 *>(b_m + core_offset(row, 1, 2)) = c1;
            }
#pragma unroll
            for (int c = 0; c < 8; ++c) {   // 16 nibble bytes: low nibbles -> 16 weights, high nibbles -> 16 weights 32 further
                const uint4 qv = __ldg(rec + 1 + c);
                const int j = c >> 1, half = c & 1;
                const uint32_t scv = j < 2 ? s.sc_lo : s.sc_hi;
                const uint32_t sl = byte_of(scv, (2 * j) & 3), sh = byte_of(scv, ((2 * j) & 3) + 1);
                const uint32_t al = sl >> 3, cl = sl & 7u, ah = sh >> 3, ch = sh & 7u;
                const uint32_t M4 = 0x0f0f0f0fu;
                const uint32_t lo[4] = {qv.x & M4, qv.y & M4, qv.z & M4, qv.w & M4};
                const uint32_t hi[4] = {(qv.x >> 4) & M4, (qv.y >> 4) & M4, (qv.z >> 4) & M4, (qv.w >> 4) & M4};
                // every byte product is <= 15 * 7 = 105, so a 32-bit multiply scales four weights at once
                const int kl = 4 * j + half, kh = 4 * j + 2 + half;
                *reinterpret_cast<uint4 *>(b_q + core_offset(row, kl, 16)) = make_uint4(lo[0] * al, lo[1] * al, lo[2] * al, lo[3] * al);
                *reinterpret_cast<uint4 *>(b_q + core_offset(BN + row, kl, 16)) = make_uint4(lo[0] * cl, lo[1] * cl, lo[2] * cl, lo[3] * cl);
                *reinterpret_cast<uint4 *>(b_q + core_offset(row, kh, 16)) = make_uint4(hi[0] * ah, hi[1] * ah, hi[2] * ah, hi[3] * ah);
                *reinterpret_cast<uint4 *>(b_q + core_offset(BN + row, kh, 16)) = make_uint4(hi[0] * ch, hi[1] * ch, hi[2] * ch, hi[3] * ch);
            }
        } else {   // past the last weight row: keep the operand finite, the columns are never stored
            wd[row] = make_float2(0.f, 0.f);
            const uint4 z = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4 *>(b_m + core_offset(row, 0, 2)) = z;
            *reinterpret_cast<uint4 *>(b_m + core_offset(row, 1, 2)) = z;
        }
    }

    // activations
    const long long m = m0 + row;
    if (m < p.m) {
        const uint8_t *rec = p.xq + (size_t)m * x_row_bytes + (size_t)b * 292;
        const uint32_t *words = reinterpret_cast<const uint32_t *>(rec);
        xd[row] = __uint_as_float(__ldg(words));
#pragma unroll
        for (int c = 0; c < 16; ++c)
            *reinterpret_cast<uint4 *>(a_q + core_offset(row, c, 16)) =
                make_uint4(__ldg(words + 1 + 4 * c), __ldg(words + 2 + 4 * c), __ldg(words + 3 + 4 * c), __ldg(words + 4 + 4 * c));
        float lo[8], hi[8];
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            const uint32_t pr = __ldg(words + 65 + g);
            const int s = (int)(int16_t)(pr & 0xffffu) + (int)(int16_t)(pr >> 16);
            const int l = s & 63;
            lo[g] = (float)l;
            hi[g] = (float)((s - l) >> 6);
        }
        *reinterpret_cast<uint4 *>(a_m + core_offset(row, 0, 2)) =
            make_uint4(pack_half2(lo[0], lo[1]), pack_half2(lo[2], lo[3]), pack_half2(lo[4], lo[5]), pack_half2(lo[6], lo[7]));
        *reinterpret_cast<uint4 *>(a_m + core_offset(row, 1, 2)) =
            make_uint4(pack_half2(hi[0], hi[1]), pack_half2(hi[2], hi[3]), pack_half2(hi[4], hi[5]), pack_half2(hi[6], hi[7]));
    } else {
        xd[row] = 0.f;
        const uint4 z = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4 *>(a_m + core_offset(row, 0, 2)) = z;
        *reinterpret_cast<uint4 *>(a_m + core_offset(row, 1, 2)) = z;
    }
}

template <int BN>
__global__ void __launch_bounds__(PF_THREADS) prefill_q4k_kernel(const PfParams p) {
    using L = PfLayout<BN>;
    extern __shared__ __align__(1024) uint8_t smem[];
    Control *ctl = reinterpret_cast<Control *>(smem);
    uint8_t *stages = smem + L::CONTROL;
    uint8_t *scale_ring = stages + PF_STAGES * L::STAGE;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles = p.m_tiles * p.n_tiles;
    const int nb = p.nb;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PF_STAGES; ++s) { mbar_init(&ctl->full[s], 4); mbar_init(&ctl->empty[s], 1); }
        mbar_init(&ctl->tmem_full, 1);
        mbar_init(&ctl->tmem_empty, 4);
        ctl->abort = 0;
        ctl->tmem_base = 0xffffffffu;
        mbar_fence_init();
    }
    __syncthreads();
    if (warp == 8) tc::tmem_alloc(&ctl->tmem_base, L::TMEM_COLS);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = ctl->tmem_base;

    if (warp >= 4 && warp < 8) {
        // ------------------------------------------------------------------ producers
        const int row = threadIdx.x - 128;
        uint32_t it = 0;
        for (int tile = blockIdx.x; tile < tiles && !ctl->abort; tile += gridDim.x) {
            const long long n0 = (long long)(tile / p.m_tiles) * BN, m0 = (long long)(tile % p.m_tiles) * PF_BM;
            for (int b = 0; b < nb; ++b, ++it) {
                const int s = it & 1;
                if (!wait_or_abort(&ctl->empty[s], ((it >> 1) & 1u) ^ 1u, ctl, p.status)) break;
                produce_block<BN>(p, stages + s * L::STAGE, scale_ring + (it & (PF_SCALE_SLOTS - 1)) * L::SCALES, row, n0, m0, b);
                fence_proxy_async();      // generic-proxy stores above must be visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) mbar_arrive(&ctl->full[s]);
            }
        }
    } else if (warp == 8) {
        // ------------------------------------------------------------------ MMA issue
        if (lane == 0) {
            const uint32_t idesc_q = tc::idesc_i8(PF_BM, 2 * BN, true, true);
            const uint32_t idesc_m = tc::idesc_f16_f32acc(PF_BM, BN);
            uint32_t it = 0;
            for (int tile = blockIdx.x; tile < tiles && !ctl->abort; tile += gridDim.x) {
                for (int b = 0; b < nb; ++b, ++it) {
                    const int s = it & 1;
                    if (!wait_or_abort(&ctl->full[s], (it >> 1) & 1u, ctl, p.status)) break;
                    if (!wait_or_abort(&ctl->tmem_empty, (it & 1u) ^ 1u, ctl, p.status)) break;
                    tc::fence_after_sync();
                    const uint32_t a_q = smem_addr(stages + s * L::STAGE), b_q = a_q + L::A_Q, a_m = b_q + L::B_Q, b_m = a_m + L::A_M;
#pragma unroll
                    for (int j = 0; j < 8; ++j)   // K = 32 per instruction = two 16-byte chunks, 256 bytes further per step
                        tc::mma_i8(tmem, tc::smem_desc(a_q + 256 * j, 128, 2048), tc::smem_desc(b_q + 256 * j, 128, 2048), idesc_q, j > 0);
                    tc::mma_f16(tmem + 2 * BN, tc::smem_desc(a_m, 128, 256), tc::smem_desc(b_m, 128, 256), idesc_m, 0);
                    tc::commit(&ctl->empty[s]);     // the stage may be refilled once these MMAs have read it
                    tc::commit(&ctl->tmem_full);    // and the accumulators are complete
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 0-3)
        const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
        float acc[BN];
        uint32_t it = 0;
        for (int tile = blockIdx.x; tile < tiles && !ctl->abort; tile += gridDim.x) {
            const long long n0 = (long long)(tile / p.m_tiles) * BN, m0 = (long long)(tile % p.m_tiles) * PF_BM;
#pragma unroll
            for (int i = 0; i < BN; ++i) acc[i] = 0.f;
            bool ok = true;
            for (int b = 0; b < nb; ++b, ++it) {
                if (!wait_or_abort(&ctl->tmem_full, it & 1u, ctl, p.status)) { ok = false; break; }
                tc::fence_after_sync();
                const uint8_t *scales = scale_ring + (it & (PF_SCALE_SLOTS - 1)) * L::SCALES;
                const float4 *wd = reinterpret_cast<const float4 *>(scales);   // {d, dmin} pairs, two weights per float4
                const float xd = reinterpret_cast<const float *>(scales + L::WD)[threadIdx.x];
#pragma unroll
                for (int c = 0; c < BN / 16; ++c) {
                    uint32_t hi[16], lo[16], mt[16];
                    tc::tmem_ld16(lane_base + 16 * c, hi);
                    tc::tmem_ld16(lane_base + BN + 16 * c, lo);
                    tc::tmem_ld16(lane_base + 2 * BN + 16 * c, mt);
                    tc::tmem_ld_wait();
                    if (c == BN / 16 - 1) {   // last read of this block's accumulators: hand TMEM back to the MMA warp
                        tc::fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&ctl->tmem_empty);
                    }
#pragma unroll
                    for (int i = 0; i < 16; i += 2) {
                        const float4 s2 = wd[(16 * c + i) >> 1];
                        const int v0 = 8 * (int)hi[i] + (int)lo[i], v1 = 8 * (int)hi[i + 1] + (int)lo[i + 1];
                        acc[16 * c + i] += xd * (s2.x * (float)v0 - s2.y * __uint_as_float(mt[i]));
                        acc[16 * c + i + 1] += xd * (s2.z * (float)v1 - s2.w * __uint_as_float(mt[i + 1]));
                    }
                }
            }
            if (!ok) break;
            const long long m = m0 + threadIdx.x;
            if (m < p.m) {
                float *out = p.y + (size_t)m * p.ldy + n0;
                if (n0 + BN <= p.n && ((reinterpret_cast<uintptr_t>(out) & 15u) == 0)) {
#pragma unroll
                    for (int i = 0; i < BN; i += 4) *reinterpret_cast<float4 *>(out + i) = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
                } else {
#pragma unroll
                    for (int i = 0; i < BN; ++i)
                        if (n0 + i < p.n) out[i] = acc[i];
                }
            }
        }
    }

    tc::fence_before_sync();
    __syncthreads();
    if (warp == 8 && tmem != 0xffffffffu) tc::tmem_free(tmem, L::TMEM_COLS);
}

}  // namespace

bool prefill_supported(int fmt, long long n, long long k, long long m, const void *w, const void *xq) {
    static const bool disabled = getenv("WEFT_B200_NO_TENSOR_PREFILL") != nullptr;
    return !disabled && fmt == F_Q4_K && k > 0 && k % 256 == 0 && n > 0 && m >= 32 &&
           (reinterpret_cast<uintptr_t>(w) & 15u) == 0 && (reinterpret_cast<uintptr_t>(xq) & 3u) == 0 &&
           n < (1LL << 31) && m < (1LL << 31);
}

cudaError_t launch_prefill(const PrefillArgs &a, int sm_count, cudaStream_t stream) {
    if (!prefill_supported(a.fmt, a.n, a.k, a.m, a.w, a.xq)) return cudaErrorNotSupported;
    constexpr int BN = 128;
    using L = PfLayout<BN>;
    PfParams p;
    p.w = static_cast<const uint8_t *>(a.w); p.xq = static_cast<const uint8_t *>(a.xq); p.y = a.y;
    p.n = a.n; p.m = a.m; p.ldy = a.ldy; p.nb = (int)(a.k / 256); p.status = a.status;
    p.m_tiles = (int)((a.m + PF_BM - 1) / PF_BM);
    p.n_tiles = (int)((a.n + BN - 1) / BN);
    const long long tiles = (long long)p.m_tiles * p.n_tiles;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(prefill_q4k_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    const int grid = (int)(tiles < sm_count ? tiles : sm_count);
    prefill_q4k_kernel<BN><<<grid, PF_THREADS, L::TOTAL, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace weft
