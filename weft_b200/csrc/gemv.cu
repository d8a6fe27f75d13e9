// Decode path: Y[m, n] = quantized_vec_dot(W[n], Xq[m]) for every weight row -- the loop the
// reference's production_mul_mat_*_decode kernels spell out (examples/kernels/mul_mat/q4_k_decode.py:17-20)
// around the block dots of examples/kernels/vec_dot/{q4_0_q8_0,q8_0_q8_0,q4_k_q8_k,iq2_xxs_q8_k,tq1_0_q8_k}.py
// (GGML: ggml-cpu/quants.c:174-208, 400-428, 645-718, 855-895, 430-480).
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
#include "quantize.cuh"
#include "kernels.h"

#include <climits>
#include <cstdlib>

namespace weft {

constexpr int XQ_PITCH = 272;   // 256 code bytes + 16: consecutive units start on different bank groups
constexpr int XAUX_BYTES = 64;  // per unit: Q8_K {f32 d, i32 total, -, -, i32 pair_sums[8]}; Q8_0 {f32 d[8], i32 sums[8]}

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

template <int FMT> struct Unit { static constexpr int BYTES = unit_bytes(FMT); };

// ------------------------------------------------------------------ unit dot products
// Each takes RL weight units (same unit index of RL different rows) against one staged activation unit.

template <int RL>
__device__ __forceinline__ void dot_q4_k(const uint8_t *const (&wp)[RL], const uint8_t *xq, const uint8_t *xaux, float (&acc)[RL]) {
    Q4KScales sc[RL];
    float d[RL], dmin[RL];
    int isum[RL];
#pragma unroll
    for (int r = 0; r < RL; ++r) {
        const uint4 h = *reinterpret_cast<const uint4 *>(wp[r]);
        d[r] = half_bits_to_float(h.x);
        dmin[r] = half_bits_to_float(h.x >> 16);
        sc[r] = q4k_unpack_scales(h.y, h.z, h.w);
        isum[r] = 0;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint4 xa = *reinterpret_cast<const uint4 *>(xq + 64 * j);
        const uint4 xb = *reinterpret_cast<const uint4 *>(xq + 64 * j + 16);
        const uint4 xc = *reinterpret_cast<const uint4 *>(xq + 64 * j + 32);
        const uint4 xd = *reinterpret_cast<const uint4 *>(xq + 64 * j + 48);
#pragma unroll
        for (int r = 0; r < RL; ++r) {
            const uint4 qa = *reinterpret_cast<const uint4 *>(wp[r] + 16 + 32 * j);
            const uint4 qb = *reinterpret_cast<const uint4 *>(wp[r] + 32 + 32 * j);
            const uint32_t M = 0x0f0f0f0fu;
            int lo = dp4a_us(qa.x & M, xa.x, 0);
            lo = dp4a_us(qa.y & M, xa.y, lo); lo = dp4a_us(qa.z & M, xa.z, lo); lo = dp4a_us(qa.w & M, xa.w, lo);
            lo = dp4a_us(qb.x & M, xb.x, lo); lo = dp4a_us(qb.y & M, xb.y, lo);
            lo = dp4a_us(qb.z & M, xb.z, lo); lo = dp4a_us(qb.w & M, xb.w, lo);
            int hi = dp4a_us((qa.x >> 4) & M, xc.x, 0);
            hi = dp4a_us((qa.y >> 4) & M, xc.y, hi); hi = dp4a_us((qa.z >> 4) & M, xc.z, hi); hi = dp4a_us((qa.w >> 4) & M, xc.w, hi);
            hi = dp4a_us((qb.x >> 4) & M, xd.x, hi); hi = dp4a_us((qb.y >> 4) & M, xd.y, hi);
            hi = dp4a_us((qb.z >> 4) & M, xd.z, hi); hi = dp4a_us((qb.w >> 4) & M, xd.w, hi);
            const uint32_t scv = j < 2 ? sc[r].sc_lo : sc[r].sc_hi;
            isum[r] += lo * (int)byte_of(scv, (2 * j) & 3) + hi * (int)byte_of(scv, ((2 * j) & 3) + 1);
        }
    }
    const float xd_ = *reinterpret_cast<const float *>(xaux);
    const int4 p0 = *reinterpret_cast<const int4 *>(xaux + 16), p1 = *reinterpret_cast<const int4 *>(xaux + 32);
#pragma unroll
    for (int r = 0; r < RL; ++r) {
        int msum = p0.x * (int)byte_of(sc[r].mn_lo, 0) + p0.y * (int)byte_of(sc[r].mn_lo, 1)
                 + p0.z * (int)byte_of(sc[r].mn_lo, 2) + p0.w * (int)byte_of(sc[r].mn_lo, 3)
                 + p1.x * (int)byte_of(sc[r].mn_hi, 0) + p1.y * (int)byte_of(sc[r].mn_hi, 1)
                 + p1.z * (int)byte_of(sc[r].mn_hi, 2) + p1.w * (int)byte_of(sc[r].mn_hi, 3);
        acc[r] += xd_ * (d[r] * (float)isum[r] - dmin[r] * (float)msum);
    }
}

// 8 consecutive Q4_0 records = 144 bytes. Record r starts at byte 18r: f16 d, then 16 nibble bytes.
template <int RL>
__device__ __forceinline__ void dot_q4_0(const uint8_t *const (&wp)[RL], const uint8_t *xq, const uint8_t *xaux, float (&acc)[RL]) {
    uint32_t wv[RL][36];
#pragma unroll
    for (int r = 0; r < RL; ++r)
#pragma unroll
        for (int i = 0; i < 9; ++i) {
            const uint4 v = *reinterpret_cast<const uint4 *>(wp[r] + 16 * i);
            wv[r][4 * i] = v.x; wv[r][4 * i + 1] = v.y; wv[r][4 * i + 2] = v.z; wv[r][4 * i + 3] = v.w;
        }
#pragma unroll
    for (int b = 0; b < 8; ++b) {
        const uint4 xa = *reinterpret_cast<const uint4 *>(xq + 32 * b);
        const uint4 xb = *reinterpret_cast<const uint4 *>(xq + 32 * b + 16);
        const float xd_ = *reinterpret_cast<const float *>(xaux + 4 * b);
        const int xs = *reinterpret_cast<const int *>(xaux + 32 + 4 * b);
#pragma unroll
        for (int r = 0; r < RL; ++r) {
            const int w0 = (18 * b) / 4;
            uint32_t q[4];
            float d;
            if (b & 1) {   // record starts 2 bytes into word w0: d in its high half, nibbles word-aligned after it
                d = half_bits_to_float(wv[r][w0] >> 16);
#pragma unroll
                for (int i = 0; i < 4; ++i) q[i] = wv[r][w0 + 1 + i];
            } else {       // record word-aligned: d in the low half, nibbles straddle words
                d = half_bits_to_float(wv[r][w0]);
#pragma unroll
                for (int i = 0; i < 4; ++i) q[i] = __funnelshift_r(wv[r][w0 + i], wv[r][w0 + i + 1], 16);
            }
            const uint32_t M = 0x0f0f0f0fu;
            int s = dp4a_us(q[0] & M, xa.x, 0);
            s = dp4a_us(q[1] & M, xa.y, s); s = dp4a_us(q[2] & M, xa.z, s); s = dp4a_us(q[3] & M, xa.w, s);
            s = dp4a_us((q[0] >> 4) & M, xb.x, s); s = dp4a_us((q[1] >> 4) & M, xb.y, s);
            s = dp4a_us((q[2] >> 4) & M, xb.z, s); s = dp4a_us((q[3] >> 4) & M, xb.w, s);
            s -= 8 * xs;   // sum((q-8)*x) = sum(q*x) - 8*sum(x)
            acc[r] += (d * xd_) * (float)s;
        }
    }
}

// 8 consecutive Q8_0 records = 272 bytes. Record r starts at byte 34r: f16 d, then 32 code bytes.
template <int RL>
__device__ __forceinline__ void dot_q8_0(const uint8_t *const (&wp)[RL], const uint8_t *xq, const uint8_t *xaux, float (&acc)[RL]) {
#pragma unroll
    for (int r = 0; r < RL; ++r) {
        uint32_t wv[68];
#pragma unroll
        for (int i = 0; i < 17; ++i) {
            const uint4 v = *reinterpret_cast<const uint4 *>(wp[r] + 16 * i);
            wv[4 * i] = v.x; wv[4 * i + 1] = v.y; wv[4 * i + 2] = v.z; wv[4 * i + 3] = v.w;
        }
#pragma unroll
        for (int b = 0; b < 8; ++b) {
            const uint4 xa = *reinterpret_cast<const uint4 *>(xq + 32 * b);
            const uint4 xb = *reinterpret_cast<const uint4 *>(xq + 32 * b + 16);
            const float xd_ = *reinterpret_cast<const float *>(xaux + 4 * b);
            const int w0 = (34 * b) / 4;
            uint32_t q[8];
            float d;
            if (b & 1) {
                d = half_bits_to_float(wv[w0] >> 16);
#pragma unroll
                for (int i = 0; i < 8; ++i) q[i] = wv[w0 + 1 + i];
            } else {
                d = half_bits_to_float(wv[w0]);
#pragma unroll
                for (int i = 0; i < 8; ++i) q[i] = __funnelshift_r(wv[w0 + i], wv[w0 + i + 1], 16);
            }
            int s = dp4a_ss(q[0], xa.x, 0);
            s = dp4a_ss(q[1], xa.y, s); s = dp4a_ss(q[2], xa.z, s); s = dp4a_ss(q[3], xa.w, s);
            s = dp4a_ss(q[4], xb.x, s); s = dp4a_ss(q[5], xb.y, s); s = dp4a_ss(q[6], xb.z, s); s = dp4a_ss(q[7], xb.w, s);
            acc[r] += (float)s * (d * xd_);
        }
    }
}

// One IQ2_XXS record (66 bytes, 2-byte aligned): f16 d, then 8 x {4 grid indices, u32 sign/scale word}.
// s_grid: int8[256][8]; s_neg: per sign index a byte mask, 0xff where the sign is negative (entries are +1/-1).
template <int RL>
__device__ __forceinline__ void dot_iq2_xxs(const uint8_t *const (&wp)[RL], const uint8_t *xq, const uint8_t *xaux,
                                             const uint8_t *s_grid, const uint8_t *s_neg, float (&acc)[RL]) {
    const float xd_ = *reinterpret_cast<const float *>(xaux);
    uint32_t qw[RL][16];
    int bsum[RL];
#pragma unroll
    for (int r = 0; r < RL; ++r) { ld_words_a2<16>(wp[r] + 2, qw[r]); bsum[r] = 0; }
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        const uint4 xa = *reinterpret_cast<const uint4 *>(xq + 32 * g);
        const uint4 xb = *reinterpret_cast<const uint4 *>(xq + 32 * g + 16);
        const uint32_t xw[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
        for (int r = 0; r < RL; ++r) {
            const uint32_t index = qw[r][2 * g], meta = qw[r][2 * g + 1];
            int pos = 0, neg = 0;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint2 gv = *reinterpret_cast<const uint2 *>(s_grid + 8 * byte_of(index, e));
                const uint2 nm = *reinterpret_cast<const uint2 *>(s_neg + 8 * ((meta >> (7 * e)) & 127u));
                pos = dp4a_ss(gv.x, xw[2 * e], pos);
                pos = dp4a_ss(gv.y, xw[2 * e + 1], pos);
                neg = dp4a_ss(gv.x & nm.x, xw[2 * e], neg);
                neg = dp4a_ss(gv.y & nm.y, xw[2 * e + 1], neg);
            }
            bsum[r] += (pos - 2 * neg) * (int)(2u * (meta >> 28) + 1u);
        }
    }
#pragma unroll
    for (int r = 0; r < RL; ++r) acc[r] += (half_bits_to_float(ld_u16(wp[r])) * xd_) * (float)bsum[r];
}

// digits of four packed bytes at once: ((byte*power) & 255) * 3 >> 8, in 16-bit lanes
__device__ __forceinline__ uint32_t tq1_digits4(uint32_t q4, uint32_t power) {
    const uint32_t M = 0x00ff00ffu;
    uint32_t e = ((q4 & M) * power) & M, o = (((q4 >> 8) & M) * power) & M;
    e = ((e * 3u) >> 8) & M;
    o = ((o * 3u) >> 8) & M;
    return e | (o << 8);
}

// One TQ1_0 record (54 bytes, 2-byte aligned): 32 + 16 bytes of 5 trits, 4 bytes of 4 trits, f16 d.
// sum((digit-1)*x) = sum(digit*x) - sum(x); every element of the unit is covered exactly once.
template <int RL>
__device__ __forceinline__ void dot_tq1_0(const uint8_t *const (&wp)[RL], const uint8_t *xq, const uint8_t *xaux,
                                           const uint32_t (&pw)[5], float (&acc)[RL]) {
    const float xd_ = *reinterpret_cast<const float *>(xaux);
    const int total = *reinterpret_cast<const int *>(xaux + 4);
    uint32_t wv[RL][14];
    int sum[RL];
#pragma unroll
    for (int r = 0; r < RL; ++r) { ld_words_a2<14>(wp[r], wv[r]); sum[r] = -total; }
#pragma unroll
    for (int n = 0; n < 5; ++n) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {   // region 0: x[32n + 16h ..], weight words 4h..4h+3
            const uint4 xv = *reinterpret_cast<const uint4 *>(xq + 32 * n + 16 * h);
            const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int r = 0; r < RL; ++r)
#pragma unroll
                for (int i = 0; i < 4; ++i) sum[r] = dp4a_us(tq1_digits4(wv[r][4 * h + i], pw[n]), xw[i], sum[r]);
        }
        {                                // region 1: x[160 + 16n ..], weight words 8..11
            const uint4 xv = *reinterpret_cast<const uint4 *>(xq + 160 + 16 * n);
            const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int r = 0; r < RL; ++r)
#pragma unroll
                for (int i = 0; i < 4; ++i) sum[r] = dp4a_us(tq1_digits4(wv[r][8 + i], pw[n]), xw[i], sum[r]);
        }
    }
    {                                    // region 2: x[240 + 4n ..], weight word 12
        const uint4 xv = *reinterpret_cast<const uint4 *>(xq + 240);
        const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
        for (int r = 0; r < RL; ++r)
#pragma unroll
            for (int n = 0; n < 4; ++n) sum[r] = dp4a_us(tq1_digits4(wv[r][12], pw[n]), xw[n], sum[r]);
    }
#pragma unroll
    for (int r = 0; r < RL; ++r) acc[r] += (float)sum[r] * (half_bits_to_float(wv[r][13]) * xd_);
}

// ------------------------------------------------------------------ activation staging

// Q8_K records (292 B, 4-byte aligned) -> codes at unit*XQ_PITCH, aux {d, total, pair sums}
__device__ void stage_q8_k(const uint8_t *xq, int nb, uint8_t *s_q, uint8_t *s_aux) {
    for (int i = threadIdx.x; i < nb * 64; i += blockDim.x) {
        const int u = i >> 6, wd = i & 63;
        *reinterpret_cast<uint32_t *>(s_q + u * XQ_PITCH + 4 * wd) = *reinterpret_cast<const uint32_t *>(xq + (size_t)u * 292 + 4 + 4 * wd);
    }
    for (int u = threadIdx.x; u < nb; u += blockDim.x) {
        const uint8_t *rec = xq + (size_t)u * 292;
        int *aux = reinterpret_cast<int *>(s_aux + u * XAUX_BYTES);
        aux[0] = *reinterpret_cast<const int *>(rec);
        int total = 0;
        for (int g = 0; g < 8; ++g) {
            const uint32_t pr = *reinterpret_cast<const uint32_t *>(rec + 260 + 4 * g);
            const int s = (int)(int16_t)(pr & 0xffffu) + (int)(int16_t)(pr >> 16);
            aux[4 + g] = s;
            total += s;
        }
        aux[1] = total;
    }
}

// Q8_0 records (34 B, 2-byte aligned), eight per unit -> codes at unit*XQ_PITCH + 32*b, aux {d[8], sums[8]}
__device__ void stage_q8_0(const uint8_t *xq, int nb, uint8_t *s_q, uint8_t *s_aux) {
    for (int i = threadIdx.x; i < nb * 8; i += blockDim.x) {
        const int u = i >> 3, b = i & 7;
        const uint8_t *rec = xq + (size_t)i * 34;
        reinterpret_cast<float *>(s_aux + u * XAUX_BYTES)[b] = half_bits_to_float(ld_u16(rec));
        int sum = 0;
        for (int wd = 0; wd < 8; ++wd) {
            const uint32_t v = ld_u32_a2(rec + 2 + 4 * wd);
            *reinterpret_cast<uint32_t *>(s_q + u * XQ_PITCH + 32 * b + 4 * wd) = v;
            sum = dp4a_ss(v, 0x01010101u, sum);
        }
        reinterpret_cast<int *>(s_aux + u * XAUX_BYTES + 32)[b] = sum;
    }
}

// fp32 row -> staged Q8_K units (same arithmetic as q8_K_quantize); `out` non-null: also write the records
__device__ void quantize_stage_q8_k(const float *x, int nb, uint8_t *s_q, uint8_t *s_aux, uint8_t *out) {
    const int lane = threadIdx.x & 31;
    for (int u = threadIdx.x >> 5; u < nb; u += blockDim.x >> 5) {
        float v[8];
        load8<true>(x + u * 256 + 8 * lane, v);
        uint32_t q0, q1;
        int sum16;
        float d;
        q8_k_warp(v, q0, q1, sum16, d);
        *reinterpret_cast<uint2 *>(s_q + u * XQ_PITCH + 8 * lane) = make_uint2(q0, q1);
        // pair sum g covers 32 codes = lanes 4g..4g+3; total = all 32 lanes
        int s32 = sum16 + __shfl_xor_sync(0xffffffffu, sum16, 2);
        int total = s32;
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
        int *aux = reinterpret_cast<int *>(s_aux + u * XAUX_BYTES);
        if ((lane & 3) == 0) aux[4 + (lane >> 2)] = s32;
        if (lane == 0) { aux[0] = __float_as_int(d); aux[1] = total; }
        if (out) store_q8_k(out + (size_t)u * 292, lane, q0, q1, sum16, d);
    }
}

// fp32 row -> staged Q8_0 units (same arithmetic as q8_0_quantize); the staged d is the stored f16 value
__device__ void quantize_stage_q8_0(const float *x, int nb, uint8_t *s_q, uint8_t *s_aux, uint8_t *out) {
    const int lane = threadIdx.x & 31, b = lane >> 2, sub = lane & 3;
    for (int u = threadIdx.x >> 5; u < nb; u += blockDim.x >> 5) {
        float v[8];
        load8<true>(x + u * 256 + 8 * lane, v);
        uint32_t q0, q1;
        int sum32;
        float d;
        q8_0_warp(v, q0, q1, sum32, d);
        *reinterpret_cast<uint2 *>(s_q + u * XQ_PITCH + 8 * lane) = make_uint2(q0, q1);
        if (sub == 0) {
            reinterpret_cast<float *>(s_aux + u * XAUX_BYTES)[b] = __half2float(__float2half_rn(d));
            reinterpret_cast<int *>(s_aux + u * XAUX_BYTES + 32)[b] = sum32;
        }
        if (out) store_q8_0(out + ((size_t)u * 8 + b) * 34, sub, q0, q1, d);
    }
}

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
    if (FMT == F_IQ2_XXS) { s_tab1 = cursor + 2048; cursor += 3072; }
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
    if (FMT == F_IQ2_XXS) {
        for (int i = threadIdx.x; i < 2048; i += blockDim.x) s_tab0[i] = (uint8_t)p.grid[i];
        for (int i = threadIdx.x; i < 1024; i += blockDim.x) s_tab1[i] = p.signs[i] < 0 ? 0xffu : 0u;
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
            else if (FMT == F_IQ2_XXS) dot_iq2_xxs<RL>(wp, xu, xa, s_tab0, s_tab1, acc);
            else dot_tq1_0<RL>(wp, xu, xa, pw, acc);
        }
#pragma unroll
        for (int r = 0; r < RL; ++r) {
            float v = acc[r];
            for (int o = L >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (FMT == F_IQ2_XXS) v *= 0.125f;
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

static int env_int(const char *name, int fallback) {
    const char *v = getenv(name);
    return v && *v ? atoi(v) : fallback;
}
// tuning overrides, read once
static const int kEnvWarps = env_int("WEFT_B200_GEMV_WARPS", 12);
static const int kEnvRowsPerLane = env_int("WEFT_B200_GEMV_RL", 1);
static const int kEnvRingDepth = env_int("WEFT_B200_GEMV_NBUF", 3);

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
    const long long x_bytes = (long long)nb * (XQ_PITCH + XAUX_BYTES) + (FMT == F_IQ2_XXS ? 3072 : 0) + 16 + 48 * 16;
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
        static int smem_set = 0;   /* the attribute sticks to the function: raise it only when a launch needs more */ \
        if ((int)smem > smem_set) {                                                                                   \
            cudaError_t e = cudaFuncSetAttribute(gemv_kernel<FMT, RLV, BULKV, QXV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return e;                                                                           \
            smem_set = (int)smem;                                                                                     \
        }                                                                                                             \
        gemv_kernel<FMT, RLV, BULKV, QXV><<<grid, warps * 32, smem, stream>>>(p);                                     \
    } while (0)
#define WEFT_LAUNCH_Q(RLV, BULKV) do { if (qx) WEFT_LAUNCH(RLV, BULKV, true); else WEFT_LAUNCH(RLV, BULKV, false); } while (0)
    if (rl == 2) { if (bulk) WEFT_LAUNCH_Q(2, true); else WEFT_LAUNCH_Q(2, false); }
    else { if (bulk) WEFT_LAUNCH_Q(1, true); else WEFT_LAUNCH_Q(1, false); }
#undef WEFT_LAUNCH_Q
#undef WEFT_LAUNCH
    return cudaGetLastError();
}

cudaError_t launch_gemv(const GemvArgs &a, int sm_count, cudaStream_t stream) {
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
    static const bool generic_only = getenv("WEFT_B200_GENERIC_GEMV") != nullptr;
    if (!generic_only && gemv_q4k_supported(a)) return launch_gemv_q4k(a, sm_count, stream);
    switch (a.fmt) {
    case F_Q4_0: return launch_fmt<F_Q4_0>(a, sm_count, stream);
    case F_Q8_0: return launch_fmt<F_Q8_0>(a, sm_count, stream);
    case F_Q4_K: return launch_fmt<F_Q4_K>(a, sm_count, stream);
    case F_IQ2_XXS: return launch_fmt<F_IQ2_XXS>(a, sm_count, stream);
    case F_TQ1_0: return launch_fmt<F_TQ1_0>(a, sm_count, stream);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace weft
