// Shared pieces of the decode GEMV kernels: the per-format dot product of one 256-element weight unit
// against one staged activation unit, and the staging of activation records (or of fp32 activations,
// quantized on the way) into shared memory.
// (examples/kernels/vec_dot/{q4_0_q8_0,q8_0_q8_0,q2_k_q8_k,q3_k_q8_k,q4_k_q8_k,q5_k_q8_k,q6_k_q8_k,iq2_xxs_q8_k,tq1_0_q8_k}.py;
//  GGML ggml-cpu/quants.c:174-208, 400-428, 514-564, 566-643, 645-718, 720-798, 800-853, 855-895, 430-480.)
#pragma once

#include "quantize.cuh"
#include "kernels.h"

namespace weft {

constexpr int XQ_PITCH = 272;   // 256 code bytes + 16: consecutive units start on different bank groups
// per unit: Q8_K {f32 d, i32 total, -, -, i32 pair_sums[8] (of the record's bsums), i16 sums16[16] (of the codes),
// i16 bsums[16] (as stored)}; Q8_0 {f32 d[8], i32 sums[8]}
constexpr int XAUX_BYTES = 112;

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

// One Q2_K record (84 bytes, 2-byte aligned): scales[16] (low nibble scale, high nibble min), qs[64], f16 d, f16 dmin.
// Weight 128 n + 32 j + l is bits 2j, 2j+1 of qs[32 n + l]; the min term uses the activation record's bsums as stored.
template <int RL>
__device__ __forceinline__ void dot_q2_k(const uint8_t *const (&wp)[RL], const uint8_t *xq, const uint8_t *xaux, float (&acc)[RL]) {
    const float xd_ = *reinterpret_cast<const float *>(xaux);
    const uint4 b0 = *reinterpret_cast<const uint4 *>(xaux + 80), b1 = *reinterpret_cast<const uint4 *>(xaux + 96);
    const uint32_t bs[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
    uint32_t wv[RL][21];
    int isum[RL], msum[RL];
#pragma unroll
    for (int r = 0; r < RL; ++r) {
        ld_words_a2<21>(wp[r], wv[r]);
        isum[r] = 0; msum[r] = 0;
#pragma unroll
        for (int q = 0; q < 4; ++q) {   // four mins as bytes against two pairs of 16-bit sums: two dp2a
            const int mins4 = (int)((wv[r][q] >> 4) & 0x0f0f0f0fu);
            msum[r] = __dp2a_lo((int)bs[2 * q], mins4, msum[r]);
            msum[r] = __dp2a_hi((int)bs[2 * q + 1], mins4, msum[r]);
        }
    }
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const uint4 xv = *reinterpret_cast<const uint4 *>(xq + 128 * n + 32 * j + 16 * c);
                const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
                const int g = 8 * n + 2 * j + c;
#pragma unroll
                for (int r = 0; r < RL; ++r) {
                    // the 2-bit plane is masked where it lies: the sum comes out times 4^j (bytes up to 192, exact)
                    int dp = 0;
#pragma unroll
                    for (int i = 0; i < 4; ++i) dp = dp4a_us(wv[r][4 + 8 * n + 4 * c + i] & (0x03030303u << (2 * j)), xw[i], dp);
                    isum[r] += (int)(byte_of(wv[r][g >> 2], g & 3) & 15u) * (dp >> (2 * j));
                }
            }
#pragma unroll
    for (int r = 0; r < RL; ++r)
        acc[r] += xd_ * (half_bits_to_float(wv[r][20]) * (float)isum[r] - half_bits_to_float(wv[r][20] >> 16) * (float)msum[r]);
}

// One Q3_K record (110 bytes, 2-byte aligned): hmask[32], qs[64] (as Q2_K), scales[12], f16 d.  Weight e is its
// low two bits plus 4 * (bit e / 32 of hmask[e % 32]) minus 4: sum((u - 4) x) = sum(u x) - 4 * (sum of the 16 codes).
template <int RL>
__device__ __forceinline__ void dot_q3_k(const uint8_t *const (&wp)[RL], const uint8_t *xq, const uint8_t *xaux, float (&acc)[RL]) {
    const float xd_ = *reinterpret_cast<const float *>(xaux);
    const uint4 s0 = *reinterpret_cast<const uint4 *>(xaux + 48), s1 = *reinterpret_cast<const uint4 *>(xaux + 64);
    const uint32_t s16[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    uint32_t wv[RL][27], sc4[RL][4];
    int isum[RL];
#pragma unroll
    for (int r = 0; r < RL; ++r) {
        ld_words_a2<27>(wp[r], wv[r]);
        q3k_unpack_scales(wv[r][24], wv[r][25], wv[r][26], sc4[r]);
        isum[r] = 0;
    }
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const uint4 xv = *reinterpret_cast<const uint4 *>(xq + 128 * n + 32 * j + 16 * c);
                const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
                const int g = 8 * n + 2 * j + c, bit = 4 * n + j;
                const int xs = (int)(int16_t)(s16[g >> 1] >> (16 * (g & 1)));
#pragma unroll
                for (int r = 0; r < RL; ++r) {
                    int dp = 0;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t hm = wv[r][4 * c + i];
                        const uint32_t third = bit < 2 ? hm << (2 - bit) : hm >> (bit - 2);   // mask bit -> bit 2 of each byte
                        dp = dp4a_us(((wv[r][8 + 8 * n + 4 * c + i] >> (2 * j)) & 0x03030303u) | (third & 0x04040404u), xw[i], dp);
                    }
                    isum[r] += ((int)byte_of(sc4[r][g >> 2], g & 3) - 32) * (dp - 4 * xs);
                }
            }
#pragma unroll
    for (int r = 0; r < RL; ++r) acc[r] += (half_bits_to_float(ld_u16(wp[r] + 108)) * xd_) * (float)isum[r];
}

// One Q5_K record (176 bytes, 16-byte aligned in a staged row): the Q4_K header, qh[32] at +16, qs[128] at +48.
// Sub-block g of weight byte l is nibble g & 1 of qs[32 (g / 2) + l] plus bit g of qh[l] as the fifth bit.
template <int RL>
__device__ __forceinline__ void dot_q5_k(const uint8_t *const (&wp)[RL], const uint8_t *xq, const uint8_t *xaux, float (&acc)[RL]) {
    Q4KScales sc[RL];
    float d[RL], dmin[RL];
    int isum[RL];
    uint32_t qh[RL][8];
#pragma unroll
    for (int r = 0; r < RL; ++r) {
        const uint4 h = *reinterpret_cast<const uint4 *>(wp[r]);
        d[r] = half_bits_to_float(h.x);
        dmin[r] = half_bits_to_float(h.x >> 16);
        sc[r] = q4k_unpack_scales(h.y, h.z, h.w);
        const uint4 ha = *reinterpret_cast<const uint4 *>(wp[r] + 16), hb = *reinterpret_cast<const uint4 *>(wp[r] + 32);
        qh[r][0] = ha.x; qh[r][1] = ha.y; qh[r][2] = ha.z; qh[r][3] = ha.w;
        qh[r][4] = hb.x; qh[r][5] = hb.y; qh[r][6] = hb.z; qh[r][7] = hb.w;
        isum[r] = 0;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint4 xa = *reinterpret_cast<const uint4 *>(xq + 64 * j);
        const uint4 xb = *reinterpret_cast<const uint4 *>(xq + 64 * j + 16);
        const uint4 xc = *reinterpret_cast<const uint4 *>(xq + 64 * j + 32);
        const uint4 xd = *reinterpret_cast<const uint4 *>(xq + 64 * j + 48);
        const uint32_t xlo[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
        const uint32_t xhi[8] = {xc.x, xc.y, xc.z, xc.w, xd.x, xd.y, xd.z, xd.w};
#pragma unroll
        for (int r = 0; r < RL; ++r) {
            const uint4 qa = *reinterpret_cast<const uint4 *>(wp[r] + 48 + 32 * j);
            const uint4 qb = *reinterpret_cast<const uint4 *>(wp[r] + 64 + 32 * j);
            const uint32_t qs[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
            int lo = 0, hi = 0;
#pragma unroll
            for (int w = 0; w < 8; ++w) {
                const uint32_t hw = qh[r][w];
                // bit 2j -> bit 4 of each byte (low sub-block), bit 2j + 1 -> bit 4 (high sub-block)
                const uint32_t f_lo = j == 0 ? hw << 4 : j == 1 ? hw << 2 : j == 2 ? hw : hw >> 2;
                const uint32_t f_hi = j == 0 ? hw << 3 : j == 1 ? hw << 1 : j == 2 ? hw >> 1 : hw >> 3;
                lo = dp4a_us((qs[w] & 0x0f0f0f0fu) | (f_lo & 0x10101010u), xlo[w], lo);
                hi = dp4a_us(((qs[w] >> 4) & 0x0f0f0f0fu) | (f_hi & 0x10101010u), xhi[w], hi);
            }
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

// One Q6_K record (210 bytes, 2-byte aligned): ql[128] low nibbles, qh[64] high bit pairs, int8 scales[16], f16 d.
// Weight 128 h + 32 p + l = (nibble p / 2 of ql[64 h + 32 (p & 1) + l]) | (bits 2p, 2p + 1 of qh[32 h + l]) << 4, minus 32,
// with scale 8 h + 2 p + l / 16.  sum(sc * (q - 32) * x) = sum_g sc_g * (sum(q * x) - 32 * sum16_g): the activation's
// sums of 16 codes come from the codes themselves, as the reference's loop never reads the record's bsums.
template <int RL>
__device__ __forceinline__ void dot_q6_k(const uint8_t *const (&wp)[RL], const uint8_t *xq, const uint8_t *xaux, float (&acc)[RL]) {
    const float xd_ = *reinterpret_cast<const float *>(xaux);
    const uint4 s0 = *reinterpret_cast<const uint4 *>(xaux + 48), s1 = *reinterpret_cast<const uint4 *>(xaux + 64);
    const uint32_t s16[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    uint32_t scw[RL][4];
    int isum[RL];
#pragma unroll
    for (int r = 0; r < RL; ++r) { ld_words_a2<4>(wp[r] + 192, scw[r]); isum[r] = 0; }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        uint32_t ql[RL][16], qh[RL][8];
#pragma unroll
        for (int r = 0; r < RL; ++r) { ld_words_a2<16>(wp[r] + 64 * h, ql[r]); ld_words_a2<8>(wp[r] + 128 + 32 * h, qh[r]); }
#pragma unroll
        for (int p = 0; p < 4; ++p) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {   // 16 weights = one scale
                const uint4 xv = *reinterpret_cast<const uint4 *>(xq + 128 * h + 32 * p + 16 * c);
                const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
                const int g = 8 * h + 2 * p + c;
                const int xs = (int)(int16_t)(s16[g >> 1] >> (16 * (g & 1)));
#pragma unroll
                for (int r = 0; r < RL; ++r) {
                    int dp = 0;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int w = 4 * c + i;
                        uint32_t lo = ql[r][8 * (p & 1) + w];
                        if (p >= 2) lo >>= 4;
                        const uint32_t hb = qh[r][w];
                        const uint32_t hi = p == 0 ? hb << 4 : p == 1 ? hb << 2 : p == 2 ? hb : hb >> 2;
                        dp = dp4a_us((lo & 0x0f0f0f0fu) | (hi & 0x30303030u), xw[i], dp);
                    }
                    const int sc = (int)(int8_t)(scw[r][g >> 2] >> (8 * (g & 3)));
                    isum[r] += sc * (dp - 32 * xs);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < RL; ++r) acc[r] += (half_bits_to_float(ld_u16(wp[r] + 208)) * xd_) * (float)isum[r];
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
// PITCH: bytes between consecutive table entries (8: plain tables; 128: sixteen bank-striped copies, the caller
// passes the pointers already offset to its lane's copy).
template <int RL, int PITCH = 8>
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
                const uint2 gv = *reinterpret_cast<const uint2 *>(s_grid + PITCH * byte_of(index, e));
                const uint2 nm = *reinterpret_cast<const uint2 *>(s_neg + PITCH * ((meta >> (7 * e)) & 127u));
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

// One IQ2_XS record (74 bytes, 2-byte aligned): f16 d, 32 u16 codes (grid index in bits 0-8, sign index in bits 9-15,
// one code per 8 weights), 8 scale bytes (low nibble: first 16 weights of a 32-group, high nibble: the other 16)
// (examples/kernels/vec_dot/iq2_xs_q8_k.py:9-39, examples/functions/quantization.py:71-83; GGML
// ggml_vec_dot_iq2_xs_q8_K_generic).  s_grid: int8[512][8]; s_neg and PITCH as for IQ2_XXS.
template <int RL, int PITCH = 8>
__device__ __forceinline__ void dot_iq2_xs(const uint8_t *const (&wp)[RL], const uint8_t *xq, const uint8_t *xaux,
                                            const uint8_t *s_grid, const uint8_t *s_neg, float (&acc)[RL]) {
    const float xd_ = *reinterpret_cast<const float *>(xaux);
    uint32_t qw[RL][18];
    int bsum[RL];
#pragma unroll
    for (int r = 0; r < RL; ++r) { ld_words_a2<18>(wp[r] + 2, qw[r]); bsum[r] = 0; }
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        const uint4 xa = *reinterpret_cast<const uint4 *>(xq + 32 * g);
        const uint4 xb = *reinterpret_cast<const uint4 *>(xq + 32 * g + 16);
        const uint32_t xw[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
        for (int r = 0; r < RL; ++r) {
            const uint32_t sc = byte_of(qw[r][16 + (g >> 2)], g & 3);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const uint32_t codes = qw[r][2 * g + half];
                int pos = 0, neg = 0;
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const uint32_t code = e ? codes >> 16 : codes & 0xffffu;
                    const uint2 gv = *reinterpret_cast<const uint2 *>(s_grid + PITCH * (code & 511u));
                    const uint2 nm = *reinterpret_cast<const uint2 *>(s_neg + PITCH * (code >> 9));
                    pos = dp4a_ss(gv.x, xw[4 * half + 2 * e], pos);
                    pos = dp4a_ss(gv.y, xw[4 * half + 2 * e + 1], pos);
                    neg = dp4a_ss(gv.x & nm.x, xw[4 * half + 2 * e], neg);
                    neg = dp4a_ss(gv.y & nm.y, xw[4 * half + 2 * e + 1], neg);
                }
                bsum[r] += (pos - 2 * neg) * (int)(2u * (half ? sc >> 4 : sc & 15u) + 1u);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < RL; ++r) acc[r] += (half_bits_to_float(ld_u16(wp[r])) * xd_) * (float)bsum[r];
}

// One IQ3_XXS record (98 bytes, 2-byte aligned): f16 d, 64 grid-index bytes (one per 4 weights), 8 u32 (four 7-bit sign
// indices, one per 8 weights, and a 4-bit scale in bits 28-31; one word per 32 weights)
// (examples/kernels/vec_dot/iq3_xxs_q8_k.py:8-75; GGML ggml_vec_dot_iq3_xxs_q8_K_generic).  s_grid: int8[256][4] with
// GP bytes between entries (4: plain; 128: thirty-two bank-striped copies); s_neg / SP as for IQ2_XXS.
template <int RL, int GP = 4, int SP = 8>
__device__ __forceinline__ void dot_iq3_xxs(const uint8_t *const (&wp)[RL], const uint8_t *xq, const uint8_t *xaux,
                                             const uint8_t *s_grid, const uint8_t *s_neg, float (&acc)[RL]) {
    const float xd_ = *reinterpret_cast<const float *>(xaux);
    uint32_t qw[RL][24];
    int bsum[RL];
#pragma unroll
    for (int r = 0; r < RL; ++r) { ld_words_a2<24>(wp[r] + 2, qw[r]); bsum[r] = 0; }
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        const uint4 xa = *reinterpret_cast<const uint4 *>(xq + 32 * g);
        const uint4 xb = *reinterpret_cast<const uint4 *>(xq + 32 * g + 16);
        const uint32_t xw[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
        for (int r = 0; r < RL; ++r) {
            const uint32_t meta = qw[r][16 + g];
            int pos = 0, neg = 0;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint32_t pair = qw[r][2 * g + (e >> 1)] >> (16 * (e & 1));   // index bytes 2e and 2e + 1 of the group
                const uint32_t g1 = *reinterpret_cast<const uint32_t *>(s_grid + GP * (pair & 0xffu));
                const uint32_t g2 = *reinterpret_cast<const uint32_t *>(s_grid + GP * ((pair >> 8) & 0xffu));
                const uint2 nm = *reinterpret_cast<const uint2 *>(s_neg + SP * ((meta >> (7 * e)) & 127u));
                pos = dp4a_ss(g1, xw[2 * e], pos);
                pos = dp4a_ss(g2, xw[2 * e + 1], pos);
                neg = dp4a_ss(g1 & nm.x, xw[2 * e], neg);
                neg = dp4a_ss(g2 & nm.y, xw[2 * e + 1], neg);
            }
            bsum[r] += (pos - 2 * neg) * (int)(2u * (meta >> 28) + 1u);
        }
    }
#pragma unroll
    for (int r = 0; r < RL; ++r) acc[r] += (half_bits_to_float(ld_u16(wp[r])) * xd_) * (float)bsum[r];
}

// Eight sign bits (bit j set: weight j negative) as two words of byte masks, 0xff where negative
__device__ __forceinline__ void sign_bits_to_masks(uint32_t bits, uint32_t &m0, uint32_t &m1) {
    // x * 0x00204081 puts bit i of a nibble at bit 8 i; the other product bits are masked away
    m0 = (((bits & 15u) * 0x00204081u) & 0x01010101u) * 0xffu;
    m1 = ((((bits >> 4) & 15u) * 0x00204081u) & 0x01010101u) * 0xffu;
}

// One IQ2_S record (82 bytes, 2-byte aligned): f16 d; 32 bytes: low 8 bits of the grid index of every 8 weights; 32 sign
// bytes; 8 bytes: per 32 weights four 2-bit pairs, index bits 8-9; 8 scale bytes as IQ2_XS
// (examples/kernels/vec_dot/iq2_s_q8_k.py:68-73; GGML ggml_vec_dot_iq2_s_q8_K_generic).  s_grid: int8[1024][8], PITCH bytes
// between entries (the caller passes the pointer already offset to its lane's copy).
template <int RL, int PITCH = 8>
__device__ __forceinline__ void dot_iq2_s(const uint8_t *const (&wp)[RL], const uint8_t *xq, const uint8_t *xaux,
                                           const uint8_t *s_grid, float (&acc)[RL]) {
    const float xd_ = *reinterpret_cast<const float *>(xaux);
    uint32_t qw[RL][20];
    int bsum[RL];
#pragma unroll
    for (int r = 0; r < RL; ++r) { ld_words_a2<20>(wp[r] + 2, qw[r]); bsum[r] = 0; }
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        const uint4 xa = *reinterpret_cast<const uint4 *>(xq + 32 * g);
        const uint4 xb = *reinterpret_cast<const uint4 *>(xq + 32 * g + 16);
        const uint32_t xw[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
        for (int r = 0; r < RL; ++r) {
            const uint32_t low = qw[r][g], sgn = qw[r][8 + g];
            const uint32_t high = byte_of(qw[r][16 + (g >> 2)], g & 3), sc = byte_of(qw[r][18 + (g >> 2)], g & 3);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                int pos = 0, neg = 0;
#pragma unroll
                for (int ee = 0; ee < 2; ++ee) {
                    const int e = 2 * half + ee;
                    const uint32_t index = byte_of(low, e) | ((high << (8 - 2 * e)) & 0x300u);
                    const uint2 gv = *reinterpret_cast<const uint2 *>(s_grid + PITCH * index);
                    uint32_t m0, m1;
                    sign_bits_to_masks(byte_of(sgn, e), m0, m1);
                    pos = dp4a_ss(gv.x, xw[2 * e], pos);
                    pos = dp4a_ss(gv.y, xw[2 * e + 1], pos);
                    neg = dp4a_ss(gv.x & m0, xw[2 * e], neg);
                    neg = dp4a_ss(gv.y & m1, xw[2 * e + 1], neg);
                }
                bsum[r] += (pos - 2 * neg) * (int)(2u * (half ? sc >> 4 : sc & 15u) + 1u);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < RL; ++r) acc[r] += (half_bits_to_float(ld_u16(wp[r])) * xd_) * (float)bsum[r];
}

// One IQ3_S record (110 bytes, 2-byte aligned): f16 d; 64 bytes: low 8 bits of the grid index of every 4 weights; 8 bytes:
// bit e of byte g is index bit 8 of entry e of 32-group g; 32 sign bytes; 4 scale bytes (nibble per 32 weights)
// (examples/kernels/vec_dot/iq3_s_q8_k.py:67-72; GGML ggml_vec_dot_iq3_s_q8_K_generic).  s_grid: int8[512][4], GP bytes
// between entries.  No factor on the result.
template <int RL, int GP = 4>
__device__ __forceinline__ void dot_iq3_s(const uint8_t *const (&wp)[RL], const uint8_t *xq, const uint8_t *xaux,
                                           const uint8_t *s_grid, float (&acc)[RL]) {
    const float xd_ = *reinterpret_cast<const float *>(xaux);
    uint32_t qw[RL][27];
    int bsum[RL];
#pragma unroll
    for (int r = 0; r < RL; ++r) { ld_words_a2<27>(wp[r] + 2, qw[r]); bsum[r] = 0; }
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        const uint4 xa = *reinterpret_cast<const uint4 *>(xq + 32 * g);
        const uint4 xb = *reinterpret_cast<const uint4 *>(xq + 32 * g + 16);
        const uint32_t xw[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
        for (int r = 0; r < RL; ++r) {
            const uint32_t high = byte_of(qw[r][16 + (g >> 2)], g & 3), sgn = qw[r][18 + g];
            const uint32_t sc = byte_of(qw[r][26], g >> 1);
            int pos = 0, neg = 0;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint32_t pair = qw[r][2 * g + (e >> 1)] >> (16 * (e & 1));   // index bytes 2e and 2e + 1 of the group
                const uint32_t i1 = (pair & 0xffu) | (((high >> (2 * e)) & 1u) << 8), i2 = ((pair >> 8) & 0xffu) | (((high >> (2 * e + 1)) & 1u) << 8);
                const uint32_t g1 = *reinterpret_cast<const uint32_t *>(s_grid + GP * i1);
                const uint32_t g2 = *reinterpret_cast<const uint32_t *>(s_grid + GP * i2);
                uint32_t m0, m1;
                sign_bits_to_masks(byte_of(sgn, e), m0, m1);
                pos = dp4a_ss(g1, xw[2 * e], pos);
                pos = dp4a_ss(g2, xw[2 * e + 1], pos);
                neg = dp4a_ss(g1 & m0, xw[2 * e], neg);
                neg = dp4a_ss(g2 & m1, xw[2 * e + 1], neg);
            }
            bsum[r] += (pos - 2 * neg) * (int)(2u * (g & 1 ? sc >> 4 : sc & 15u) + 1u);
        }
    }
#pragma unroll
    for (int r = 0; r < RL; ++r) acc[r] += (half_bits_to_float(ld_u16(wp[r])) * xd_) * (float)bsum[r];
}

// One IQ1_S record (50 bytes, 2-byte aligned): f16 d; 32 bytes: low 8 bits of the grid index of every 8 weights; 8 u16, one per
// 32 weights: four 3-bit index tops, a 3-bit scale, the sign of the shift 0.125
// (examples/kernels/vec_dot/iq1_s_q8_k.py:51-56; GGML ggml_vec_dot_iq1_s_q8_K_generic).  s_grid: int8[2048][8] with values
// -1, 0, +1, PITCH bytes between entries.  The shift term multiplies the activation record's stored sums of 32.
template <int RL, int PITCH = 8>
__device__ __forceinline__ void dot_iq1_s(const uint8_t *const (&wp)[RL], const uint8_t *xq, const uint8_t *xaux,
                                           const uint8_t *s_grid, float (&acc)[RL]) {
    const float xd_ = *reinterpret_cast<const float *>(xaux);
    const int *pair_sums = reinterpret_cast<const int *>(xaux + 16);
    uint32_t qw[RL][12];
    int sumi[RL], sumi1[RL];
#pragma unroll
    for (int r = 0; r < RL; ++r) { ld_words_a2<12>(wp[r] + 2, qw[r]); sumi[r] = 0; sumi1[r] = 0; }
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        const uint4 xa = *reinterpret_cast<const uint4 *>(xq + 32 * g);
        const uint4 xb = *reinterpret_cast<const uint4 *>(xq + 32 * g + 16);
        const uint32_t xw[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
        const int ps = pair_sums[g];
#pragma unroll
        for (int r = 0; r < RL; ++r) {
            const uint32_t low = qw[r][g], qh = (qw[r][8 + (g >> 1)] >> (16 * (g & 1))) & 0xffffu;
            int lsum = 0;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint2 gv = *reinterpret_cast<const uint2 *>(s_grid + PITCH * (byte_of(low, e) | (((qh >> (3 * e)) & 7u) << 8)));
                lsum = dp4a_ss(gv.x, xw[2 * e], lsum);
                lsum = dp4a_ss(gv.y, xw[2 * e + 1], lsum);
            }
            const int ls = (int)(2u * ((qh >> 12) & 7u) + 1u);
            sumi[r] += ls * lsum;
            sumi1[r] += (qh & 0x8000u) ? -ls * ps : ls * ps;
        }
    }
#pragma unroll
    for (int r = 0; r < RL; ++r) acc[r] += (half_bits_to_float(ld_u16(wp[r])) * xd_) * ((float)sumi[r] + 0.125f * (float)sumi1[r]);
}

// One IQ1_M record (56 bytes, no d field, 2-byte aligned here): 32 index bytes; 16 bytes, one per 16 weights: low nibble
// {3 index bits, shift sign} of the first 8 weights, high nibble of the other 8; four u16: bits 0-11 four 3-bit scales (one
// per 16 weights), bits 12-15 a nibble of the record's f16 scale (examples/kernels/vec_dot/iq1_m_q8_k.py:73-79; GGML
// ggml_vec_dot_iq1_m_q8_K_generic).  f16_table: the caller's float[65536] table of f16 bit patterns, as the reference
// kernel takes it.  The shift term needs sums of 8 activation codes: computed with dp4a against ones.
template <int RL, int PITCH = 8>
__device__ __forceinline__ void dot_iq1_m(const uint8_t *const (&wp)[RL], const uint8_t *xq, const uint8_t *xaux,
                                           const uint8_t *s_grid, const float *f16_table, float (&acc)[RL]) {
    const float xd_ = *reinterpret_cast<const float *>(xaux);
    uint32_t qw[RL][14];
    int sumi1[RL], sumi2[RL];
#pragma unroll
    for (int r = 0; r < RL; ++r) { ld_words_a2<14>(wp[r], qw[r]); sumi1[r] = 0; sumi2[r] = 0; }
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        const uint4 xa = *reinterpret_cast<const uint4 *>(xq + 32 * g);
        const uint4 xb = *reinterpret_cast<const uint4 *>(xq + 32 * g + 16);
        const uint32_t xw[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
        int s8[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) s8[e] = dp4a_ss(0x01010101u, xw[2 * e + 1], dp4a_ss(0x01010101u, xw[2 * e], 0));
#pragma unroll
        for (int r = 0; r < RL; ++r) {
            const uint32_t low = qw[r][g], qh = (qw[r][8 + (g >> 1)] >> (16 * (g & 1))) & 0xffffu;     // two qh bytes of the group
            const uint32_t sc = (qw[r][12 + (g >> 2)] >> (16 * ((g >> 1) & 1))) & 0xffffu;           // the u16 that holds the group's scales
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                int sum1 = 0, sum2 = 0;
#pragma unroll
                for (int ee = 0; ee < 2; ++ee) {
                    const int e = 2 * half + ee;
                    const uint32_t nib = (qh >> (4 * e)) & 15u;      // byte e >> 1, nibble e & 1
                    const uint2 gv = *reinterpret_cast<const uint2 *>(s_grid + PITCH * (byte_of(low, e) | ((nib & 7u) << 8)));
                    sum1 = dp4a_ss(gv.x, xw[2 * e], sum1);
                    sum1 = dp4a_ss(gv.y, xw[2 * e + 1], sum1);
                    sum2 += (nib & 8u) ? -s8[e] : s8[e];
                }
                const int ls = (int)(2u * ((sc >> (6 * (g & 1) + 3 * half)) & 7u) + 1u);
                sumi1[r] += sum1 * ls;
                sumi2[r] += sum2 * ls;
            }
        }
    }
#pragma unroll
    for (int r = 0; r < RL; ++r) {
        const uint32_t bits = (qw[r][12] >> 12 & 0xfu) | (qw[r][12] >> 24 & 0xf0u) | (qw[r][13] >> 4 & 0xf00u) | (qw[r][13] >> 16 & 0xf000u);
        acc[r] += (__ldg(f16_table + bits) * xd_) * ((float)sumi1[r] + 0.125f * (float)sumi2[r]);
    }
}

// Bank-striped copies of a codebook: with 8-byte entries, copy c (of sixteen) of entry e sits at e * 128 + c * 8, so copy
// c lives in banks 2c and 2c + 1 only and a half-warp whose lane l reads copy l % 16 never conflicts, whatever the
// entries (an 8-byte shared load is served one half-warp at a time); with 4-byte entries, copy c (of thirty-two) at
// e * 128 + c * 4, one per lane.  `masks`: store 0xff where the entry is negative, 0 elsewhere (the sign tables).
__device__ inline void stage_striped8(const int8_t *table, int entries, uint8_t *dst, bool masks) {
    for (int i = threadIdx.x; i < entries * 2 * 16; i += blockDim.x) {       // (entry word, copy)
        const int word = i >> 4, c = i & 15;
        uint32_t v = __ldg(reinterpret_cast<const uint32_t *>(table) + word);
        if (masks) v = ((v >> 7) & 0x01010101u) * 0xffu;
        reinterpret_cast<uint32_t *>(dst)[(word >> 1) * 32 + c * 2 + (word & 1)] = v;
    }
}
// four copies of 8-byte entries (a table too large for sixteen): copy c of entry e at e * 32 + c * 8; lane l reads copy l % 4
__device__ inline void stage_striped8x4(const int8_t *table, int entries, uint8_t *dst) {
    for (int i = threadIdx.x; i < entries * 2 * 4; i += blockDim.x) {
        const int word = i >> 2, c = i & 3;
        reinterpret_cast<uint32_t *>(dst)[(word >> 1) * 8 + c * 2 + (word & 1)] = __ldg(reinterpret_cast<const uint32_t *>(table) + word);
    }
}
__device__ inline void stage_striped4(const int8_t *table, int entries, uint8_t *dst) {
    for (int i = threadIdx.x; i < entries * 32; i += blockDim.x)
        reinterpret_cast<uint32_t *>(dst)[i] = __ldg(reinterpret_cast<const uint32_t *>(table) + (i >> 5));
}
// IQ2_XXS: s_grid 256 x 128 bytes, s_neg 128 x 128 bytes
__device__ inline void stage_iq2_tables_striped(const int8_t *grid, const int8_t *signs, uint8_t *s_grid, uint8_t *s_neg) {
    stage_striped8(grid, 256, s_grid, false);
    stage_striped8(signs, 128, s_neg, true);
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

// Q8_K records (292 B, 4-byte aligned) -> codes at unit*XQ_PITCH, aux {d, total, pair sums, sums of 16}
__device__ inline void stage_q8_k(const uint8_t *xq, int nb, uint8_t *s_q, uint8_t *s_aux) {
    for (int i = threadIdx.x; i < nb * 64; i += blockDim.x) {
        const int u = i >> 6, wd = i & 63;
        const uint32_t v = *reinterpret_cast<const uint32_t *>(xq + (size_t)u * 292 + 4 + 4 * wd);
        *reinterpret_cast<uint32_t *>(s_q + u * XQ_PITCH + 4 * wd) = v;
        // sums of 16 codes, from the codes (a warp is wholly inside or outside this loop: the bound is a multiple of 64)
        int s = dp4a_ss(v, 0x01010101u, 0);
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        if ((wd & 3) == 0) *reinterpret_cast<int16_t *>(s_aux + u * XAUX_BYTES + 48 + 2 * (wd >> 2)) = (int16_t)s;
    }
    for (int u = threadIdx.x; u < nb; u += blockDim.x) {
        const uint8_t *rec = xq + (size_t)u * 292;
        int *aux = reinterpret_cast<int *>(s_aux + u * XAUX_BYTES);
        aux[0] = *reinterpret_cast<const int *>(rec);
        for (int g = 0; g < 8; ++g) aux[20 + g] = *reinterpret_cast<const int *>(rec + 260 + 4 * g);   // bsums as stored
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
__device__ inline void stage_q8_0(const uint8_t *xq, int nb, uint8_t *s_q, uint8_t *s_aux) {
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
__device__ inline void quantize_stage_q8_k(const float *x, int nb, uint8_t *s_q, uint8_t *s_aux, uint8_t *out) {
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
        if ((lane & 1) == 0) {
            *reinterpret_cast<int16_t *>(s_aux + u * XAUX_BYTES + 48 + lane) = (int16_t)sum16;
            *reinterpret_cast<int16_t *>(s_aux + u * XAUX_BYTES + 80 + lane) = (int16_t)sum16;
        }
        if (lane == 0) { aux[0] = __float_as_int(d); aux[1] = total; }
        if (out) store_q8_k(out + (size_t)u * 292, lane, q0, q1, sum16, d);
    }
}

// fp32 row -> staged Q8_0 units (same arithmetic as q8_0_quantize); the staged d is the stored f16 value
__device__ inline void quantize_stage_q8_0(const float *x, int nb, uint8_t *s_q, uint8_t *s_aux, uint8_t *out) {
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

}  // namespace weft
