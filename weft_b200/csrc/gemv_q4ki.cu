// The persistent interleaved weight layout Q4K_I[16] (examples/formats/ggml.py:286-290,
// doc/dsl/encoding-and-artifacts.md:209): the Q4_K records of 16 consecutive rows ("cohort") of one
// 256-block are stored byte-major, byte b of row r at 16 b + r, cohort blocks in (cohort, block) order.
//   * interleave_q4k_kernel: the artifact function <kernel>_W_pack (lib/Target/Emission/Emitter.h:231-272).
//   * gemv_q4ki_kernel: q4_k_q8_k_gemv (examples/kernels/gemv/q4_k.py:8-26) and the per-token loop of
//     production_mul_mat_q4_k_persistent (examples/kernels/mul_mat/q4_k_persistent.py:9-30).
//
// HBM-bound like the plain Q4_K GEMV and streamed the same way: one persistent CTA per SM, a producer lane
// filling a ring of 18 KB stages with bulk copies, three copies outstanding, bounded waits.  A CTA owns
// whole cohorts; a stage is eight 256-blocks of one cohort (8 x 2304 bytes, contiguous in this layout).
// Two teams of eight consumer warps work on alternate stages of a cohort; a warp takes one block of its
// team's stage: it transposes the 2304 bytes back into sixteen ordinary 144-byte records in a private
// scratch (4 x 4 byte transposes with prmt), gives the ring slot back, and then lane (r, h) computes
// half-record h of row r against the staged activations exactly as the plain kernel does.  Every lane
// keeps its row's running sum for the whole cohort and hands it to a last warp, which adds the sixteen
// warps' sums in a fixed order (so results do not depend on timing) and writes the 16 outputs while the
// consumers are already on the next cohort.
#include "gemv_units.cuh"
#include "ring.cuh"

#include <cstdlib>

namespace weft {

namespace {

constexpr int QI_ROWS = 16;                    // rows per cohort
constexpr int QI_BLOCK = QI_ROWS * 144;        // bytes of one cohort block
constexpr int QI_CHUNK = 8;                    // blocks per stage = warps of one consumer team
constexpr int QI_TEAMS = 2;                    // teams work on different stages of a cohort at the same time
constexpr int QI_CONSUMERS = QI_CHUNK * QI_TEAMS;
constexpr int QI_STAGE = QI_CHUNK * QI_BLOCK;  // 18432
constexpr int QI_STAGES = 8;
constexpr int QI_PARTIALS = 4;                 // cohorts whose partial sums may be pending at once
constexpr int QI_THREADS = 32 * (2 + QI_CONSUMERS);   // producer, consumers, one warp that adds the partial sums

struct QiParams {
    const uint8_t *w;
    const uint8_t *xq;
    const float *x;
    float *y;
    long long cohorts;
    long long ldy;
    int nb;
    int inflight;
    int *status;
};

// 4 x 4 byte transpose: in[i] holds byte i of four rows; out[r] holds bytes 0..3 of row r
__device__ __forceinline__ void transpose4(uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t (&out)[4]) {
    const uint32_t ab_lo = __byte_perm(a, b, 0x5140), cd_lo = __byte_perm(c, d, 0x5140);   // rows 0,1
    const uint32_t ab_hi = __byte_perm(a, b, 0x7362), cd_hi = __byte_perm(c, d, 0x7362);   // rows 2,3
    out[0] = __byte_perm(ab_lo, cd_lo, 0x5410);
    out[1] = __byte_perm(ab_lo, cd_lo, 0x7632);
    out[2] = __byte_perm(ab_hi, cd_hi, 0x5410);
    out[3] = __byte_perm(ab_hi, cd_hi, 0x7632);
}

// One interleaved cohort block (2304 bytes at shared address src) -> sixteen plain records at dst.
__device__ __forceinline__ void deinterleave_block(uint32_t src, uint32_t dst, int lane) {
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
        const int t = lane + 32 * pass;   // 36 groups of four byte coordinates
        if (t < 36) {
            const uint4 v0 = lds128(src + 64 * t), v1 = lds128(src + 64 * t + 16), v2 = lds128(src + 64 * t + 32), v3 = lds128(src + 64 * t + 48);
            uint32_t q[4];
            transpose4(v0.x, v1.x, v2.x, v3.x, q);
#pragma unroll
            for (int r = 0; r < 4; ++r) asm volatile("st.shared.u32 [%0], %1;" ::"r"(dst + (r) * 144 + 4 * t), "r"(q[r]) : "memory");
            transpose4(v0.y, v1.y, v2.y, v3.y, q);
#pragma unroll
            for (int r = 0; r < 4; ++r) asm volatile("st.shared.u32 [%0], %1;" ::"r"(dst + (4 + r) * 144 + 4 * t), "r"(q[r]) : "memory");
            transpose4(v0.z, v1.z, v2.z, v3.z, q);
#pragma unroll
            for (int r = 0; r < 4; ++r) asm volatile("st.shared.u32 [%0], %1;" ::"r"(dst + (8 + r) * 144 + 4 * t), "r"(q[r]) : "memory");
            transpose4(v0.w, v1.w, v2.w, v3.w, q);
#pragma unroll
            for (int r = 0; r < 4; ++r) asm volatile("st.shared.u32 [%0], %1;" ::"r"(dst + (12 + r) * 144 + 4 * t), "r"(q[r]) : "memory");
        }
    }
}

// Half-record h (two 64-weight groups) of the plain record at shared address rec against the staged
// activation unit (codes at xq, {d, total, -, -, pair sums[8]} at xaux): d * isum - dmin * msum.
__device__ __forceinline__ float half_record(uint32_t rec, int h, uint32_t xq, uint32_t xaux) {
    const uint4 hd = lds128(rec);
    const Q4KScales s = q4k_unpack_scales(hd.y, hd.z, hd.w);
    const uint32_t sc = h ? s.sc_hi : s.sc_lo, mn = h ? s.mn_hi : s.mn_lo;
    int isum = 0;
#pragma unroll
    for (int jj = 0; jj < 2; ++jj) {
        const uint4 a = lds128(rec + 16 + 64 * h + 32 * jj), b = lds128(rec + 32 + 64 * h + 32 * jj);
        const uint4 x0 = lds128(xq + 128 * h + 64 * jj), x1 = lds128(xq + 128 * h + 64 * jj + 16);
        const uint4 x2 = lds128(xq + 128 * h + 64 * jj + 32), x3 = lds128(xq + 128 * h + 64 * jj + 48);
        const uint32_t L = 0x0f0f0f0fu, H = 0xf0f0f0f0u;
        int lo = dp4a_us(a.x & L, x0.x, 0), hi = dp4a_us(a.x & H, x2.x, 0);
        lo = dp4a_us(a.y & L, x0.y, lo); hi = dp4a_us(a.y & H, x2.y, hi);
        lo = dp4a_us(a.z & L, x0.z, lo); hi = dp4a_us(a.z & H, x2.z, hi);
        lo = dp4a_us(a.w & L, x0.w, lo); hi = dp4a_us(a.w & H, x2.w, hi);
        lo = dp4a_us(b.x & L, x1.x, lo); hi = dp4a_us(b.x & H, x3.x, hi);
        lo = dp4a_us(b.y & L, x1.y, lo); hi = dp4a_us(b.y & H, x3.y, hi);
        lo = dp4a_us(b.z & L, x1.z, lo); hi = dp4a_us(b.z & H, x3.z, hi);
        lo = dp4a_us(b.w & L, x1.w, lo); hi = dp4a_us(b.w & H, x3.w, hi);
        // high nibbles were left in place: their dot product comes out multiplied by 16, exactly
        isum += lo * (int)byte_of(sc, 2 * jj) + (hi >> 4) * (int)byte_of(sc, 2 * jj + 1);
    }
    const uint4 pv = lds128(xaux + 16 + 16 * h);
    const int msum = (int)pv.x * (int)byte_of(mn, 0) + (int)pv.y * (int)byte_of(mn, 1) + (int)pv.z * (int)byte_of(mn, 2) + (int)pv.w * (int)byte_of(mn, 3);
    return half_bits_to_float(hd.x) * (float)isum - half_bits_to_float(hd.x >> 16) * (float)msum;
}

template <bool QX>
__global__ void __launch_bounds__(QI_THREADS) gemv_q4ki_kernel(const QiParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb = p.nb, G = gridDim.x, b = blockIdx.x;
    constexpr int S = QI_STAGES;

    volatile int *s_issued = reinterpret_cast<volatile int *>(smem);
    uint64_t *s_full = reinterpret_cast<uint64_t *>(smem + 16);
    uint64_t *s_empty = s_full + S;
    uint64_t *s_done = s_empty + S, *s_free = s_done + QI_PARTIALS;   // partial sums of a cohort written / consumed
    float *s_partial = reinterpret_cast<float *>(smem + 256);             // [QI_PARTIALS][QI_CONSUMERS][32]
    uint8_t *s_scratch = smem + 256 + QI_PARTIALS * QI_CONSUMERS * 32 * 4;          // [QI_CONSUMERS][16 x 144]
    uint8_t *s_xq = s_scratch + QI_CONSUMERS * QI_BLOCK;
    uint8_t *s_aux = s_xq + (size_t)nb * XQ_PITCH;
    uint8_t *s_ring = smem + ((256 + QI_PARTIALS * QI_CONSUMERS * 32 * 4 + QI_CONSUMERS * QI_BLOCK + (size_t)nb * (XQ_PITCH + XAUX_BYTES) + 127) & ~size_t(127));
    const uint32_t ring_addr = smem_addr(s_ring), full_addr = smem_addr(s_full), empty_addr = smem_addr(s_empty);

    const int chunks = (nb + QI_CHUNK - 1) / QI_CHUNK;                    // stages per cohort
    const long long my_cohorts = p.cohorts > b ? (p.cohorts - b + G - 1) / G : 0;
    const long long total_ll = my_cohorts * chunks;
    const int total_stages = (int)(total_ll < (1LL << 30) ? total_ll : (1LL << 30));
    const size_t xq_row = (size_t)blockIdx.y * nb * 292;
    float *y = p.y + (size_t)blockIdx.y * p.ldy;

    asm volatile("griddepcontrol.launch_dependents;");
    if (threadIdx.x < S) {
        mbar_init(s_full + threadIdx.x, 1);
        mbar_init(s_empty + threadIdx.x, QI_CHUNK);   // every warp of the stage's team arrives once
        if (threadIdx.x < QI_PARTIALS) { mbar_init(s_done + threadIdx.x, QI_CONSUMERS); mbar_init(s_free + threadIdx.x, 1); }
        mbar_fence_init();
    }
    if (threadIdx.x == 0) *s_issued = 0;
    __syncthreads();

    auto issue = [&](int s) {   // one lane: local stage s = (cohort index s / chunks, chunk s % chunks)
        const int slot = s & (S - 1);
        const long long cohort = b + (long long)(s / chunks) * G;
        const int q = s % chunks;
        const int blocks = min(QI_CHUNK, nb - q * QI_CHUNK);
        const uint32_t bytes = (uint32_t)blocks * QI_BLOCK;
        mbar_expect_tx_a(full_addr + 8 * slot, bytes);
        bulk_g2s_a(ring_addr + (uint32_t)slot * QI_STAGE, p.w + ((size_t)cohort * nb + (size_t)q * QI_CHUNK) * QI_BLOCK, bytes, full_addr + 8 * slot);
    };
    const int P = min(S, p.inflight);
    if (warp == 0 && lane == 0) {
        const int first = min(P, total_stages);
        for (int s = 0; s < first; ++s) issue(s);   // weights do not depend on the activations
        *s_issued = first;
    }

    // Activations and outputs may belong to the kernel that precedes this one in the stream.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (QX) quantize_stage_q8_k(p.x + (size_t)blockIdx.y * nb * 256, nb, s_xq, s_aux, b == 0 ? const_cast<uint8_t *>(p.xq) + xq_row : nullptr);
    else stage_q8_k(p.xq + xq_row, nb, s_xq, s_aux);
    __syncthreads();

    if (warp == 0) {   // producer: at most P copies outstanding, a slot refilled once all eight warps have copied out of it
        if (lane == 0) {
            for (int s = min(P, total_stages); s < total_stages; ++s) {
                if (s >= S) {
                    if (!mbar_wait_a(empty_addr + 8 * (s & (S - 1)), (uint32_t)((s / S) - 1) & 1u)) { report(p.status, ST_WAIT_TIMEOUT); return; }
                    fence_proxy_async();
                }
                if (!mbar_wait_a(full_addr + 8 * ((s - P) & (S - 1)), (uint32_t)((s - P) / S) & 1u)) { report(p.status, ST_WAIT_TIMEOUT); return; }
                issue(s);
                *s_issued = s + 1;
            }
        }
        return;
    }

    const uint32_t done_addr = smem_addr(s_done), free_addr = smem_addr(s_free);
    const int r = lane >> 1, h = lane & 1;              // this lane's row of the cohort and half of the record
    if (warp == 1 + QI_CONSUMERS) {
        // the adder: waits for the sixteen partial sums of a cohort, adds them in warp order, writes 16 outputs
        for (long long ci = 0; ci < my_cohorts; ++ci) {
            const int ps = (int)(ci % QI_PARTIALS);
            if (!mbar_wait_a(done_addr + 8 * ps, (uint32_t)(ci / QI_PARTIALS) & 1u, 1u << 24)) { report(p.status, ST_WAIT_TIMEOUT); return; }
            const float *partial = s_partial + ps * (QI_CONSUMERS * 32);
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < QI_CONSUMERS; ++w) v += partial[w * 32 + lane];
            v += __shfl_xor_sync(0xffffffffu, v, 1);    // the two halves of a row
            if (h == 0) y[(b + ci * G) * QI_ROWS + r] = v;
            __syncwarp();                               // every lane has read its partial sums
            if (lane == 0) mbar_arrive_a(free_addr + 8 * ps);
        }
        return;
    }

    const int cw = warp - 1, team = cw / QI_CHUNK, bj = cw % QI_CHUNK;   // consumer index, its team, its block of the team's stage
    const uint32_t scratch = smem_addr(s_scratch) + (uint32_t)cw * QI_BLOCK;
    const uint32_t xq_addr = smem_addr(s_xq), aux_addr = smem_addr(s_aux);
    for (long long ci = 0; ci < my_cohorts; ++ci) {
        float acc = 0.f;
        for (int q = team; q < chunks; q += QI_TEAMS) {
            const int s = (int)(ci * chunks + q);
            // A parity wait cannot tell fill n of a slot from fill n-2: first wait until the stage has been issued.
            if (*s_issued <= s) {
                bool issued = false;
                for (uint32_t spin = 0; spin < (1u << 24) && !issued; ++spin) issued = *s_issued > s;
                if (!issued) { report(p.status, ST_WAIT_TIMEOUT); return; }
            }
            if (!mbar_wait_a(full_addr + 8 * (s & (S - 1)), (uint32_t)(s / S) & 1u)) { report(p.status, ST_WAIT_TIMEOUT); return; }
            const int kb = q * QI_CHUNK + bj;           // this warp's 256-block of the row
            const bool mine = kb < nb;
            if (mine) deinterleave_block(ring_addr + (uint32_t)(s & (S - 1)) * QI_STAGE + (uint32_t)bj * QI_BLOCK, scratch, lane);
            __syncwarp();                               // the scratch is complete, the slot no longer needed by this warp
            if (lane == 0) mbar_arrive_a(empty_addr + 8 * (s & (S - 1)));
            if (mine) {
                const float xd = __uint_as_float(lds32(aux_addr + kb * XAUX_BYTES));
                acc += xd * half_record(scratch + (uint32_t)r * 144u, h, xq_addr + kb * XQ_PITCH, aux_addr + kb * XAUX_BYTES);
            }
            __syncwarp();                               // every lane has read the scratch before the next block overwrites it
        }
        // hand the cohort's partial sums to the adder; a slot is reused QI_PARTIALS cohorts later, once it has been read
        const int ps = (int)(ci % QI_PARTIALS);
        if (ci >= QI_PARTIALS && !mbar_wait_a(free_addr + 8 * ps, (uint32_t)(ci / QI_PARTIALS - 1) & 1u, 1u << 24)) { report(p.status, ST_WAIT_TIMEOUT); return; }
        s_partial[ps * (QI_CONSUMERS * 32) + cw * 32 + lane] = acc;
        __syncwarp();                                   // all 32 sums are written before lane 0 says so
        if (lane == 0) mbar_arrive_a(done_addr + 8 * ps);
    }
}

// byte (cb, byte b, row r) of the packed matrix <- byte b of the record of row 16 cohort + r, block k
__global__ void interleave_q4k_kernel(const uint8_t *__restrict__ source, uint8_t *__restrict__ target, long long cohorts, int nb) {
    const long long total = cohorts * nb * 144;   // one thread per (cohort block, byte coordinate): 16 bytes out
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long cb = i / 144;
        const int byte = (int)(i - cb * 144);
        const long long cohort = cb / nb;
        const int k = (int)(cb - cohort * nb);
        uint32_t out[4] = {0, 0, 0, 0};
#pragma unroll
        for (int r = 0; r < QI_ROWS; ++r) {
            const uint32_t v = source[((size_t)(cohort * QI_ROWS + r) * nb + k) * 144 + byte];
            out[r >> 2] |= v << (8 * (r & 3));
        }
        *reinterpret_cast<uint4 *>(target + (size_t)cb * QI_BLOCK + (size_t)byte * QI_ROWS) = make_uint4(out[0], out[1], out[2], out[3]);
    }
}

constexpr int kQiInflight = 3;

template <bool QX>
cudaError_t launch_variant(const QiParams &p, dim3 grid, size_t smem, cudaStream_t stream) {
    cudaError_t granted = grant_dynamic_smem(reinterpret_cast<const void *>(gemv_q4ki_kernel<QX>), (int)smem);
    if (granted != cudaSuccess) return granted;
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = dim3(QI_THREADS);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, gemv_q4ki_kernel<QX>, p);
}

size_t q4ki_smem(long long nb) {
    return ((256 + QI_PARTIALS * QI_CONSUMERS * 32 * 4 + QI_CONSUMERS * QI_BLOCK + (size_t)nb * (XQ_PITCH + XAUX_BYTES) + 127) & ~size_t(127)) + (size_t)QI_STAGES * QI_STAGE;
}

}  // namespace

bool gemv_q4ki_supported(const GemvArgs &a) {
    return a.fmt == F_Q4_K_I16 && a.k % 256 == 0 && a.k > 0 && a.n % QI_ROWS == 0 && (reinterpret_cast<uintptr_t>(a.w) & 15u) == 0 &&
           a.n < (1LL << 34) && q4ki_smem(a.k / 256) <= 220 * 1024;
}

cudaError_t launch_gemv_q4ki(const GemvArgs &a, int sm_count, cudaStream_t stream) {
    if (!gemv_q4ki_supported(a)) return cudaErrorInvalidValue;
    QiParams p;
    p.w = static_cast<const uint8_t *>(a.w); p.xq = static_cast<const uint8_t *>(a.xq); p.x = a.x; p.y = a.y;
    p.cohorts = a.n / QI_ROWS; p.ldy = a.ldy; p.nb = (int)(a.k / 256); p.status = a.status;
    p.inflight = kQiInflight < 1 ? 1 : kQiInflight;
    long long ctas = p.cohorts < sm_count ? p.cohorts : sm_count;
    if (ctas < 1) ctas = 1;
    dim3 grid((unsigned)ctas, (unsigned)a.m);
    const size_t smem = q4ki_smem(p.nb);
    return a.x ? launch_variant<true>(p, grid, smem, stream) : launch_variant<false>(p, grid, smem, stream);
}

cudaError_t launch_interleave_q4k(const void *source, void *target, long long rows, long long k, int sm_count, cudaStream_t stream) {
    if (rows % QI_ROWS != 0 || k % 256 != 0) return cudaErrorInvalidValue;
    if (rows == 0 || k == 0) return cudaSuccess;
    const long long work = rows / QI_ROWS * (k / 256) * 144;
    long long blocks = (work + 255) / 256;
    if (blocks > (long long)sm_count * 16) blocks = (long long)sm_count * 16;
    interleave_q4k_kernel<<<(unsigned)blocks, 256, 0, stream>>>(static_cast<const uint8_t *>(source), static_cast<uint8_t *>(target), rows / QI_ROWS, (int)(k / 256));
    return cudaGetLastError();
}

}  // namespace weft
