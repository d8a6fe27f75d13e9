// Q4_K x Q8_K decode GEMV, the headline kernel: Y[n] = quantized_vec_dot_q4_k_q8_k(W[n], Xq) for all n
// (examples/kernels/mul_mat/q4_k_decode.py:17-20 around examples/kernels/vec_dot/q4_k_q8_k.py:8-29;
// GGML ggml-cpu/quants.c:645-718).
//
// HBM-bound: 144 bytes per 256 weights, each read once (33.0 MB for 14336 x 4096).
//
// One persistent CTA per SM.  Work is dealt in stages of a few consecutive rows (about 18 KB); in round r
// CTA b owns stage r * gridDim + b, so at any moment the whole grid reads one contiguous window of the
// matrix (measured: ~20 % more HBM throughput than giving each CTA its own contiguous range).  The rows
// left after the last full round are split evenly over the CTAs, so every CTA streams the same number
// of bytes to within one row.
//   * Warp 0 is the producer: one lane streams the CTA's stages into a shared-memory ring with bulk
//     asynchronous copies (cp.async.bulk + mbarrier complete_tx), keeping three copies (54 KB per SM, 8 MB
//     over the GPU) outstanding; the ring of eight slots decouples landing from consumption.
//   * The other warps are consumers.  Consumer w computes the CTA's rows w, w + W, w + 2W, ...: it waits on
//     the stage's "full" barrier, computes the row from shared memory and arrives on the stage's "empty"
//     barrier, which lets the producer refill the slot.
//   * Launched with programmatic stream serialization: the next kernel in the stream may start its
//     prologue and its weight streaming while this one drains; it waits (griddepcontrol.wait) before it
//     touches activations or outputs.
//   * A row of K/256 records is cut into half-records (128 weights: two 64-weight groups, four 6-bit
//     scales): 32 tasks for K = 4096, exactly one per lane.  In that case (tasks <= 32) every lane keeps
//     its 128 activation codes, the block scale and its four bsum pairs in registers for the whole kernel,
//     and a row costs five 16-byte shared loads per lane (header + 64 nibble bytes), 32 dp4a and a
//     shuffle reduction.  Longer rows loop over tasks and read activations from the staged copy.
//   * The prologue optionally quantizes the fp32 activation row itself (same code as q8_K_quantize) while
//     the first stages are in flight; CTA 0 writes the Q8_K records to the caller's Xq workspace.
// A row is never split across warps or GPUs and partial sums are combined in a fixed order, so results do
// not depend on the grid or on which warp claims which row.
//
// Float op tree per half-record h: acc += x.d * (d * f32(isum_h) - dmin * f32(msum_h)); the DSL's
// per-record expression x.ds * (w.d * f32(i32_acc) - w.dmin * f32(minimum)) with the two integer sums
// split in halves (exact in integers; the fp32 sum order differs from the scalar oracle, bound 1e-5 rel L2).
#include "quantize.cuh"
#include "kernels.h"
#include "ring.cuh"

#include <climits>
#include <cstdlib>

namespace weft {

namespace {

constexpr int QK_XQ_PITCH = 272;   // 256 code bytes + 16 so that consecutive records start on different bank groups
constexpr int QK_XAUX = 48;        // {f32 d, 3 x pad, i32 pair_sums[8]}
constexpr int QK_MAX_STAGES = 24;
constexpr int QK_MAX_THREADS = 640;

struct Q4kParams {
    const uint8_t *w;
    const uint8_t *xq;   // Q8_K records: read, or written by CTA column 0 when QX
    const float *x;      // fp32 activations (QX only)
    float *y;
    long long n;
    long long ldy;
    int nb;              // records per row
    int log_stage_rows;  // rows per ring stage = 1 << log_stage_rows
    int log_stages;      // ring depth = 1 << log_stages
    int full_rounds;     // rounds in which every CTA owns one full stage
    int tail_rows;       // rows per CTA in the final, partial round
    int inflight;        // copies the producer keeps outstanding (issued, not yet landed)
    int *status;
    GatherArgs gather;
    // grouped launch: rows [seg_begin[i], seg_begin[i + 1]) of the row sequence belong to matrix i (whole stages each)
    int segments;
    const uint8_t *seg_w[GEMV_MAX_SEGMENTS];
    float *seg_y[GEMV_MAX_SEGMENTS];
    long long seg_begin[GEMV_MAX_SEGMENTS + 1];
};

__device__ __forceinline__ int segment_of(const Q4kParams &p, long long row) {
    int s = 0;
    for (int i = 1; i < p.segments; ++i) s += row >= p.seg_begin[i];
    return s;
}

// One half-record (64 nibble bytes at q0 / q1: two 64-weight groups) of two different rows at once against
// the same activations xr[32] (128 codes), scales/mins of sub-blocks 4h..4h+3 from the record headers h0 / h1,
// bsum pair sums ps[4]; returns d*isum - dmin*msum per row.  Two independent instruction streams per lane
// hide the shared-memory and dp4a latencies of one another.
__device__ __forceinline__ void half_record2(uint32_t q0, uint32_t q1, const uint4 &h0, const uint4 &h1, int h,
                                             const uint32_t (&xr)[32], const int (&ps)[4], float &r0, float &r1) {
    const Q4KScales s0 = q4k_unpack_scales(h0.y, h0.z, h0.w), s1 = q4k_unpack_scales(h1.y, h1.z, h1.w);
    const uint32_t sc0 = h ? s0.sc_hi : s0.sc_lo, mn0 = h ? s0.mn_hi : s0.mn_lo;
    const uint32_t sc1 = h ? s1.sc_hi : s1.sc_lo, mn1 = h ? s1.mn_hi : s1.mn_lo;
    int i0 = 0, i1 = 0;
#pragma unroll
    for (int jj = 0; jj < 2; ++jj) {
        const uint4 a0 = lds128(q0 + 32 * jj), b0 = lds128(q0 + 32 * jj + 16);
        const uint4 a1 = lds128(q1 + 32 * jj), b1 = lds128(q1 + 32 * jj + 16);
        const uint32_t L = 0x0f0f0f0fu, H = 0xf0f0f0f0u;
        const uint32_t *xa = xr + 16 * jj;
        int lo0 = dp4a_us(a0.x & L, xa[0], 0), lo1 = dp4a_us(a1.x & L, xa[0], 0);
        int hi0 = dp4a_us(a0.x & H, xa[8], 0), hi1 = dp4a_us(a1.x & H, xa[8], 0);
        lo0 = dp4a_us(a0.y & L, xa[1], lo0); lo1 = dp4a_us(a1.y & L, xa[1], lo1);
        hi0 = dp4a_us(a0.y & H, xa[9], hi0); hi1 = dp4a_us(a1.y & H, xa[9], hi1);
        lo0 = dp4a_us(a0.z & L, xa[2], lo0); lo1 = dp4a_us(a1.z & L, xa[2], lo1);
        hi0 = dp4a_us(a0.z & H, xa[10], hi0); hi1 = dp4a_us(a1.z & H, xa[10], hi1);
        lo0 = dp4a_us(a0.w & L, xa[3], lo0); lo1 = dp4a_us(a1.w & L, xa[3], lo1);
        hi0 = dp4a_us(a0.w & H, xa[11], hi0); hi1 = dp4a_us(a1.w & H, xa[11], hi1);
        lo0 = dp4a_us(b0.x & L, xa[4], lo0); lo1 = dp4a_us(b1.x & L, xa[4], lo1);
        hi0 = dp4a_us(b0.x & H, xa[12], hi0); hi1 = dp4a_us(b1.x & H, xa[12], hi1);
        lo0 = dp4a_us(b0.y & L, xa[5], lo0); lo1 = dp4a_us(b1.y & L, xa[5], lo1);
        hi0 = dp4a_us(b0.y & H, xa[13], hi0); hi1 = dp4a_us(b1.y & H, xa[13], hi1);
        lo0 = dp4a_us(b0.z & L, xa[6], lo0); lo1 = dp4a_us(b1.z & L, xa[6], lo1);
        hi0 = dp4a_us(b0.z & H, xa[14], hi0); hi1 = dp4a_us(b1.z & H, xa[14], hi1);
        lo0 = dp4a_us(b0.w & L, xa[7], lo0); lo1 = dp4a_us(b1.w & L, xa[7], lo1);
        hi0 = dp4a_us(b0.w & H, xa[15], hi0); hi1 = dp4a_us(b1.w & H, xa[15], hi1);
        // high nibbles were left in place: their dot product comes out multiplied by 16, exactly
        i0 += lo0 * (int)byte_of(sc0, 2 * jj) + (hi0 >> 4) * (int)byte_of(sc0, 2 * jj + 1);
        i1 += lo1 * (int)byte_of(sc1, 2 * jj) + (hi1 >> 4) * (int)byte_of(sc1, 2 * jj + 1);
    }
    const int m0 = ps[0] * (int)byte_of(mn0, 0) + ps[1] * (int)byte_of(mn0, 1) + ps[2] * (int)byte_of(mn0, 2) + ps[3] * (int)byte_of(mn0, 3);
    const int m1 = ps[0] * (int)byte_of(mn1, 0) + ps[1] * (int)byte_of(mn1, 1) + ps[2] * (int)byte_of(mn1, 2) + ps[3] * (int)byte_of(mn1, 3);
    r0 = half_bits_to_float(h0.x) * (float)i0 - half_bits_to_float(h0.x >> 16) * (float)m0;
    r1 = half_bits_to_float(h1.x) * (float)i1 - half_bits_to_float(h1.x >> 16) * (float)m1;
}

// fp32 row -> staged Q8_K records (codes at u*QK_XQ_PITCH, aux {d, pair sums}); optionally also to global.
// A warp's blocks are u = warp, warp + warps, ...; the loads of four of them are issued before the first is worked on
// (a load from L2 takes longer than quantizing a block; 9.54 -> 9.41 us per step for K = 14336).
__device__ void q4k_quantize_stage(const float *__restrict__ x, int nb, uint8_t *s_q, uint8_t *s_aux, uint8_t *out) {
    const int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    constexpr int B = 4;
    for (int u0 = threadIdx.x >> 5; u0 < nb; u0 += B * warps) {
        float v[B][8];
#pragma unroll
        for (int i = 0; i < B; ++i)
            if (u0 + i * warps < nb) load8<true>(x + (u0 + i * warps) * 256 + 8 * lane, v[i]);
#pragma unroll
        for (int i = 0; i < B; ++i) {
            const int u = u0 + i * warps;
            if (u < nb) {
                uint32_t q0, q1;
                int sum16;
                float d;
                q8_k_warp(v[i], q0, q1, sum16, d);
                *reinterpret_cast<uint2 *>(s_q + u * QK_XQ_PITCH + 8 * lane) = make_uint2(q0, q1);
                const int s32 = sum16 + __shfl_xor_sync(0xffffffffu, sum16, 2);
                int *aux = reinterpret_cast<int *>(s_aux + u * QK_XAUX);
                if ((lane & 3) == 0) aux[4 + (lane >> 2)] = s32;
                if (lane == 0) aux[0] = __float_as_int(d);
                if (out) store_q8_k(out + (size_t)u * 292, lane, q0, q1, sum16, d);
            }
        }
    }
}

// Q8_K records -> the same staged form, four loads in flight per thread
__device__ void q4k_stage_records(const uint8_t *__restrict__ xq, int nb, uint8_t *s_q, uint8_t *s_aux) {
    constexpr int B = 4;
    const int threads = blockDim.x;
    for (int i0 = threadIdx.x; i0 < nb * 64; i0 += B * threads) {
        uint32_t w[B];
#pragma unroll
        for (int j = 0; j < B; ++j) {
            const int i = i0 + j * threads;
            if (i < nb * 64) w[j] = *reinterpret_cast<const uint32_t *>(xq + (size_t)(i >> 6) * 292 + 4 + 4 * (i & 63));
        }
#pragma unroll
        for (int j = 0; j < B; ++j) {
            const int i = i0 + j * threads;
            if (i < nb * 64) *reinterpret_cast<uint32_t *>(s_q + (i >> 6) * QK_XQ_PITCH + 4 * (i & 63)) = w[j];
        }
    }
    for (int i = threadIdx.x; i < nb * 9; i += threads) {
        const int u = i / 9, f = i % 9;
        const uint8_t *rec = xq + (size_t)u * 292;
        int *aux = reinterpret_cast<int *>(s_aux + u * QK_XAUX);
        if (f == 8) aux[0] = *reinterpret_cast<const int *>(rec);
        else {
            const uint32_t pr = *reinterpret_cast<const uint32_t *>(rec + 260 + 4 * f);
            aux[4 + f] = (int)(int16_t)(pr & 0xffffu) + (int)(int16_t)(pr >> 16);
        }
    }
}

}  // namespace

namespace {

// MODE 0: one matrix; 1: grouped launch over several matrices; 2: one matrix with the peer all-gather; 3: one matrix
// whose results go to pinned host memory: they are collected in shared memory and one warp stores them when the CTA
// is done, neighbouring rows in one instruction (a store to host memory crosses PCIe by itself; measured 29.3 -> 26.7 us
// per call with host X, Xq and Y against one store per pair of rows as it completes).  Separate instantiations, so that the
// single-matrix kernel carries none of the others' code.
constexpr int QK_HOST_ROWS = 512;   // rows per CTA that MODE 3 can collect
template <bool QX, bool XREG, int MODE>
__global__ void __launch_bounds__(QK_MAX_THREADS) gemv_q4k_kernel(const Q4kParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb = p.nb, LSR = p.log_stage_rows, SR = 1 << LSR, LS = p.log_stages, S = 1 << LS;
    const uint32_t row_bytes = (uint32_t)nb * 144u, stage_bytes = row_bytes << LSR;
    const int G = gridDim.x, b = blockIdx.x;

    volatile int *s_issued = reinterpret_cast<volatile int *>(smem);   // stages the producer has issued so far
    uint64_t *s_full = reinterpret_cast<uint64_t *>(smem + 16);
    uint64_t *s_empty = s_full + QK_MAX_STAGES;
    uint8_t *s_xq = smem + 512;
    uint8_t *s_aux = s_xq + (size_t)nb * QK_XQ_PITCH;
    uint8_t *s_ring = smem + ((512 + (size_t)nb * (QK_XQ_PITCH + QK_XAUX) + 127) & ~size_t(127));
    const uint32_t ring_addr = smem_addr(s_ring), full_addr = smem_addr(s_full), empty_addr = smem_addr(s_empty);

    // this CTA's rows: full_rounds stages of SR rows, then its share of the remainder
    const long long main_rows = (long long)p.full_rounds * G * SR;
    const long long tail_begin = min(p.n, main_rows + (long long)b * p.tail_rows);
    const int tail_here = (int)(min(p.n, tail_begin + p.tail_rows) - tail_begin);
    const int rows_here = p.full_rounds * SR + tail_here;
    const int total_stages = p.full_rounds + (tail_here > 0 ? 1 : 0);
    const size_t xq_row = (size_t)blockIdx.y * nb * 292;
    float *y = p.y + (size_t)blockIdx.y * p.ldy;

    // Let the next kernel in the stream start its own prologue and weight streaming while this one runs
    // (programmatic dependent launch); it waits below, before it touches activations or outputs.
    asm volatile("griddepcontrol.launch_dependents;");
    if (threadIdx.x < S) {
        mbar_init(s_full + threadIdx.x, 1);
        mbar_init(s_empty + threadIdx.x, (uint32_t)SR);
        mbar_fence_init();
    }
    if (threadIdx.x == 0) *s_issued = 0;
    __syncthreads();

    auto issue = [&](int s) {   // one lane: local stage s into slot s % S
        const int slot = s & (S - 1);
        const bool tail = s >= p.full_rounds;
        const long long row0 = tail ? tail_begin : ((long long)s * G + b) << LSR;
        const uint32_t bytes = tail ? (uint32_t)tail_here * row_bytes : stage_bytes;
        const uint8_t *src = p.w + (size_t)row0 * row_bytes;
        if (MODE == 1) {   // a stage never straddles two matrices
            const int sg = segment_of(p, row0);
            src = p.seg_w[sg] + (size_t)(row0 - p.seg_begin[sg]) * row_bytes;
        }
        mbar_expect_tx_a(full_addr + 8 * slot, bytes);
        bulk_g2s_a(ring_addr + (uint32_t)slot * stage_bytes, src, bytes, full_addr + 8 * slot);
    };
    if (warp == 0 && lane == 0) {
        const int first = min(min(S, p.inflight), total_stages);
        for (int s = 0; s < first; ++s) issue(s);   // weights do not depend on the activations
        *s_issued = first;
    }

    // Everything this kernel reads besides the weights (X, Xq) or writes (Xq, Y) may belong to the kernel
    // that precedes it in the stream: wait for that kernel to complete before going on.
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const int epoch = MODE == 2 ? gather_epoch(p.gather) : 0;
    if (QX) q4k_quantize_stage(p.x + (size_t)blockIdx.y * nb * 256, nb, s_xq, s_aux, b == 0 ? const_cast<uint8_t *>(p.xq) + xq_row : nullptr);
    else q4k_stage_records(p.xq + xq_row, nb, s_xq, s_aux);
    __syncthreads();

    if (warp == 0) {
        // Producer.  Stage s goes out when its slot is free (all rows of the slot's previous stage consumed)
        // AND stage s - P has landed, i.e. at most P copies are outstanding.  Issuing the whole ring at once
        // makes every copy of every SM land together, late (measured: first data 3.4 us after the issue, the
        // consumers idle until then, the rest of the matrix requested only afterwards); with P = 3 the stages
        // land in order, the first after 2.2 us, and HBM stays busy until the end (7.6 -> 7.1 us).
        if (lane == 0) {
            const int P = min(S, p.inflight);
            for (int s = min(P, total_stages); s < total_stages; ++s) {
                if (s >= S) {
                    if (!mbar_wait_a(empty_addr + 8 * (s & (S - 1)), (uint32_t)((s >> LS) - 1) & 1u)) { report(p.status, ST_WAIT_TIMEOUT); return; }
                    fence_proxy_async();
                }
                // this thread issued stage s - P itself and has not refilled its slot since: the parity is unambiguous
                if (!mbar_wait_a(full_addr + 8 * ((s - P) & (S - 1)), (uint32_t)((s - P) >> LS) & 1u)) { report(p.status, ST_WAIT_TIMEOUT); return; }
                issue(s);
                *s_issued = s + 1;
            }
        }
        return;
    }

    __shared__ float s_out[MODE == 3 ? QK_HOST_ROWS : 1];
    const int tasks = 2 * nb;
    const int consumers = (blockDim.x >> 5) - 1;
    const uint32_t xq_addr = smem_addr(s_xq), aux_addr = smem_addr(s_aux);
    uint32_t xr[32];
    int ps[4] = {0, 0, 0, 0};
    float xd = 0.f;
    const int my_r = lane >> 1, my_h = lane & 1;
    if (XREG && lane < tasks) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint4 v = lds128(xq_addr + my_r * QK_XQ_PITCH + 128 * my_h + 16 * i);
            xr[4 * i] = v.x; xr[4 * i + 1] = v.y; xr[4 * i + 2] = v.z; xr[4 * i + 3] = v.w;
        }
        const uint4 pv = lds128(aux_addr + my_r * QK_XAUX + 16 + 16 * my_h);
        ps[0] = (int)pv.x; ps[1] = (int)pv.y; ps[2] = (int)pv.z; ps[3] = (int)pv.w;
        xd = __uint_as_float(lds32(aux_addr + my_r * QK_XAUX));
    }
    const uint32_t my_rec = (uint32_t)my_r * 144u;

    // Each consumer iteration takes two consecutive rows of the CTA's row sequence (t, t + 1).
    for (int t = 2 * (warp - 1); t < rows_here; t += 2 * consumers) {
        const bool two = t + 1 < rows_here;
        const int t1 = two ? t + 1 : t;
        const int s0 = t >> LSR, s1 = t1 >> LSR;
        // A parity wait cannot tell fill n of a slot from fill n-2.  The producer issues fill n only after
        // fill n-1 has landed and been consumed, so once it has issued this stage the wait is unambiguous.
        if (*s_issued <= s1) {
            bool issued = false;
            for (uint32_t spin = 0; spin < (1u << 24) && !issued; ++spin) issued = *s_issued > s1;
            if (!issued) { report(p.status, ST_WAIT_TIMEOUT); return; }
        }
        if (!mbar_wait_a(full_addr + 8 * (s0 & (S - 1)), (uint32_t)(s0 >> LS) & 1u)) { report(p.status, ST_WAIT_TIMEOUT); return; }
        if (s1 != s0 && !mbar_wait_a(full_addr + 8 * (s1 & (S - 1)), (uint32_t)(s1 >> LS) & 1u)) { report(p.status, ST_WAIT_TIMEOUT); return; }
        const uint32_t row0 = ring_addr + (uint32_t)(s0 & (S - 1)) * stage_bytes + (uint32_t)(t & (SR - 1)) * row_bytes;
        const uint32_t row1 = ring_addr + (uint32_t)(s1 & (S - 1)) * stage_bytes + (uint32_t)(t1 & (SR - 1)) * row_bytes;
        float acc0 = 0.f, acc1 = 0.f;
        if (XREG) {
            if (lane < tasks) {
                const uint4 h0 = lds128(row0 + my_rec), h1 = lds128(row1 + my_rec);
                float r0, r1;
                half_record2(row0 + my_rec + 16 + 64 * my_h, row1 + my_rec + 16 + 64 * my_h, h0, h1, my_h, xr, ps, r0, r1);
                acc0 = xd * r0;
                acc1 = xd * r1;
            }
        } else {
            for (int task = lane; task < tasks; task += 32) {
                const int r = task >> 1, h = task & 1;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint4 v = lds128(xq_addr + r * QK_XQ_PITCH + 128 * h + 16 * i);
                    xr[4 * i] = v.x; xr[4 * i + 1] = v.y; xr[4 * i + 2] = v.z; xr[4 * i + 3] = v.w;
                }
                const uint4 pv = lds128(aux_addr + r * QK_XAUX + 16 + 16 * h);
                ps[0] = (int)pv.x; ps[1] = (int)pv.y; ps[2] = (int)pv.z; ps[3] = (int)pv.w;
                xd = __uint_as_float(lds32(aux_addr + r * QK_XAUX));
                const uint32_t rec0 = row0 + r * 144, rec1 = row1 + r * 144;
                const uint4 h0 = lds128(rec0), h1 = lds128(rec1);
                float r0, r1;
                half_record2(rec0 + 16 + 64 * h, rec1 + 16 + 64 * h, h0, h1, h, xr, ps, r0, r1);
                acc0 += xd * r0;
                acc1 += xd * r1;
            }
        }
        // two sums, five shuffles: the halves of the warp swap, then each half reduces one row
        const bool upper = lane >= 16;
        float v = (upper ? acc1 : acc0) + __shfl_xor_sync(0xffffffffu, upper ? acc0 : acc1, 16);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if ((lane & 15) == 0 && (!upper || two)) {
            const int tt = upper ? t1 : t, ss = upper ? s1 : s0;
            const long long grow = ss < p.full_rounds ? ((((long long)ss * G + b) << LSR) + (tt & (SR - 1)))
                                                       : tail_begin + (tt - (p.full_rounds << LSR));
            if (MODE == 1) {
                const int sg = segment_of(p, grow);
                p.seg_y[sg][grow - p.seg_begin[sg]] = v;
            } else if (MODE == 3) {
                s_out[tt] = v;
            } else {
                y[grow] = v;
            }
            mbar_arrive_a(empty_addr + 8 * (ss & (S - 1)));   // after the shuffles: every lane's shared loads have completed
        }
        if (MODE == 2 && (!upper || two)) {   // every lane of a half-warp holds its row's sum: lane i stores to peer i
            const int tt = upper ? t1 : t, ss = upper ? s1 : s0;
            const long long grow = ss < p.full_rounds ? ((((long long)ss * G + b) << LSR) + (tt & (SR - 1)))
                                                       : tail_begin + (tt - (p.full_rounds << LSR));
            gather_store_spread(p.gather, epoch, blockIdx.y, grow, p.ldy, v, lane & 15);
        }
    }
    if (MODE == 3) {
        __syncthreads();   // the producer warp and any consumer that gave up have exited: they count as arrived
        if (warp == 1)
            for (int tt = lane; tt < rows_here; tt += 32) {
                const int ss = tt >> LSR;
                const long long grow = ss < p.full_rounds ? ((((long long)ss * G + b) << LSR) + (tt & (SR - 1)))
                                                           : tail_begin + (tt - (p.full_rounds << LSR));
                y[grow] = s_out[tt];
            }
    }
    if (MODE == 2) {
        // a few CTAs receive for the whole grid; the others are done
        const int recv = min((int)gridDim.x, GATHER_RECV_CTAS), warps = (int)(gridDim.x * gridDim.y) * consumers;
        if ((int)blockIdx.x < recv && blockIdx.y == 0)
            gather_receive(p.gather, epoch, gridDim.y, p.n, p.ldy, (int)blockIdx.x * consumers + warp - 1, recv * consumers, p.status);
        gather_finish(p.gather, epoch, p.status, warps);
    }
}

// Measured on B200 for 14336 x 4096: 18 KB stages, 8-deep ring (147 KB in flight per SM), 15 consumer warps.
constexpr int kQ4kConsumers = 15;
constexpr int kQ4kStageBytes = 18432;
constexpr int kQ4kMaxStages = 8;
constexpr int kQ4kOverlap = 1;
constexpr int kQ4kSmemCap = 200;   // per-CTA shared-memory budget tried first
constexpr int kQ4kInflight = 3;   // measured: 2 -> 7.8 us, 3 -> 7.05, 4 -> 7.14, 6 -> 7.6, 8 -> 8.1

template <bool QX, bool XREG, int MODE>
cudaError_t launch_variant(const Q4kParams &p, dim3 grid, int threads, size_t smem, cudaStream_t stream) {
    cudaError_t granted = grant_dynamic_smem(reinterpret_cast<const void *>(gemv_q4k_kernel<QX, XREG, MODE>), (int)smem);
    if (granted != cudaSuccess) return granted;
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = dim3((unsigned)threads);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = kQ4kOverlap ? 1 : 0;
    config.attrs = attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, gemv_q4k_kernel<QX, XREG, MODE>, p);
}

struct Q4kPlan { int log_stage_rows, log_stages; size_t smem; bool ok; };

Q4kPlan plan_q4k(long long nb) {
    Q4kPlan plan{0, 0, 0, false};
    const long long row_bytes = nb * 144;
    const long long fixed = (512 + nb * (QK_XQ_PITCH + QK_XAUX) + 127) & ~127LL;
    int lsr = 0;
    while (lsr < 4 && (row_bytes << (lsr + 1)) <= kQ4kStageBytes) ++lsr;
    for (long long cap : {(long long)kQ4kSmemCap * 1024, 200LL * 1024}) {   // first try to leave room for a second CTA on the SM
        int ls = 0;
        while ((1 << (ls + 1)) <= kQ4kMaxStages && (1 << (ls + 1)) <= QK_MAX_STAGES && fixed + ((row_bytes << lsr) << (ls + 1)) <= cap) ++ls;
        if (ls >= 1) {
            plan.log_stage_rows = lsr; plan.log_stages = ls;
            plan.smem = (size_t)(fixed + ((row_bytes << lsr) << ls));
            plan.ok = true;
            return plan;
        }
    }
    return plan;
}

}  // namespace

bool gemv_q4k_supported(const GemvArgs &a) {
    if (a.segments > 1) return gemv_q4k_groups(a);
    return a.fmt == F_Q4_K && a.k % 256 == 0 && a.k > 0 && (reinterpret_cast<uintptr_t>(a.w) & 15u) == 0 &&
           a.n < (1LL << 30) && plan_q4k(a.k / 256).ok;
}

bool gemv_q4k_groups(const GemvArgs &a) {
    if (a.fmt != F_Q4_K || a.segments < 2 || a.segments > GEMV_MAX_SEGMENTS || a.m != 1 || a.k % 256 != 0 || a.k <= 0 || a.gather.world > 1) return false;
    const Q4kPlan plan = plan_q4k(a.k / 256);
    if (!plan.ok) return false;
    long long total = 0;
    for (int i = 0; i < a.segments; ++i) {
        if (a.seg_rows[i] <= 0 || a.seg_rows[i] % (1LL << plan.log_stage_rows) != 0) return false;   // whole stages per matrix
        if ((reinterpret_cast<uintptr_t>(a.seg_w[i]) & 15u) != 0 || !a.seg_y[i]) return false;
        total += a.seg_rows[i];
    }
    return total < (1LL << 30);
}

cudaError_t launch_gemv_q4k(const GemvArgs &a, int sm_count, cudaStream_t stream) {
    Q4kParams p;
    p.w = static_cast<const uint8_t *>(a.w); p.xq = static_cast<const uint8_t *>(a.xq); p.x = a.x; p.y = a.y; p.gather = a.gather;
    p.n = a.n; p.ldy = a.ldy; p.nb = (int)(a.k / 256); p.status = a.status; p.inflight = kQ4kInflight < 1 ? 1 : kQ4kInflight;
    const Q4kPlan plan = plan_q4k(p.nb);
    if (!plan.ok) return cudaErrorInvalidConfiguration;
    p.log_stage_rows = plan.log_stage_rows; p.log_stages = plan.log_stages;
    const long long stage_rows = 1LL << plan.log_stage_rows;
    p.segments = a.segments > 1 ? a.segments : 0;
    if (p.segments) {
        if (!gemv_q4k_groups(a)) return cudaErrorInvalidConfiguration;
        p.seg_begin[0] = 0;
        for (int i = 0; i < p.segments; ++i) {
            p.seg_w[i] = static_cast<const uint8_t *>(a.seg_w[i]);
            p.seg_y[i] = a.seg_y[i];
            p.seg_begin[i + 1] = p.seg_begin[i] + a.seg_rows[i];
        }
        p.n = p.seg_begin[p.segments];
        p.w = p.seg_w[0]; p.y = p.seg_y[0]; p.ldy = p.n;
    }
    const long long n = p.n;
    long long ctas = (n + stage_rows - 1) / stage_rows;
    if (ctas > sm_count) ctas = sm_count;
    if (ctas < 1) ctas = 1;
    p.full_rounds = (int)(n / (ctas * stage_rows));
    const long long rest = n - (long long)p.full_rounds * ctas * stage_rows;
    p.tail_rows = (int)((rest + ctas - 1) / ctas);
    if (p.segments) {   // a power of two: the tail chunks then never straddle a matrix boundary (a multiple of the stage)
        int pow2 = 1;
        while (pow2 < p.tail_rows) pow2 <<= 1;
        p.tail_rows = p.tail_rows ? pow2 : 0;
    }
    int consumers = kQ4kConsumers < 1 ? 1 : (kQ4kConsumers > QK_MAX_THREADS / 32 - 1 ? QK_MAX_THREADS / 32 - 1 : kQ4kConsumers);
    const int threads = (consumers + 1) * 32;
    dim3 grid((unsigned)ctas, (unsigned)(p.segments ? 1 : a.m));
    const bool xreg = 2 * p.nb <= 32;
    const bool collect = a.y_on_host && !p.segments && p.gather.world <= 1 && (long long)p.full_rounds * stage_rows + p.tail_rows <= QK_HOST_ROWS;
    const int mode = p.segments ? 1 : p.gather.world > 1 ? 2 : collect ? 3 : 0;
#define WEFT_Q4K_LAUNCH(MODE)                                                                                                                  \
    (a.x ? (xreg ? launch_variant<true, true, MODE>(p, grid, threads, plan.smem, stream) : launch_variant<true, false, MODE>(p, grid, threads, plan.smem, stream)) \
         : (xreg ? launch_variant<false, true, MODE>(p, grid, threads, plan.smem, stream) : launch_variant<false, false, MODE>(p, grid, threads, plan.smem, stream)))
    if (mode == 1) return WEFT_Q4K_LAUNCH(1);
    if (mode == 2) return WEFT_Q4K_LAUNCH(2);
    if (mode == 3) return WEFT_Q4K_LAUNCH(3);
    return WEFT_Q4K_LAUNCH(0);
#undef WEFT_Q4K_LAUNCH
}

}  // namespace weft
