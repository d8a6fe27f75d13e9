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
// Activation codes are never touched by a CUDA core.  A Q8_K record is 292 bytes: f32 d, 256 codes, 16
// bsums; with K a multiple of 1024 every token row is a whole number of 16-byte units and record b of a
// row starts 4 * (b & 3) bytes past a 16-byte boundary.  TMA box copies starting at that boundary bring
// the records of 128 tokens straight into the 128-byte-swizzled K-major layout the MMA reads (two boxes
// 128 bytes wide) plus three 16-byte wide boxes for the tail; in that operand the code of weight k sits at
// K position k + S, S = 4 * (b & 3) + 4, and the bytes before and after the codes (d, bsums) are garbage.
// The weight operand is therefore written with the same shift: limb byte k at K position k + S, zeros
// everywhere else, so garbage only ever meets zeros.  The MMA runs over K = 288 (nine K = 32 steps).
//
// CTA = 128 tokens (TMEM lanes) x 128 weights, persistent over tiles.  The 128 weights are two halves of
// 64; each half owns 192 TMEM columns ([q*a | q*c | min term]), so the tensor core works on one half
// while the epilogue drains the other.  Warp roles:
//   warps 0-7   epilogue, warp = (32-token quarter, 32 of the 64 columns of each half): tcgen05.ld the
//               accumulators, combine, keep 32 x 64 fp32 in registers across the blocks of a tile
//   warps 8-11  weight producers, one weight row per thread: the row's Q4_K record is read from global
//               memory in place (no repack in HBM), one block ahead, and expanded into the shifted
//               two-limb operand
//   warps 12-13 read x.ds and the bsums out of the landed activation boxes and build the min-term operand
//   warp 14     one lane issues the activation TMA copies, up to two blocks ahead
//   warp 15     allocates TMEM; one lane issues the MMAs and commits them to mbarriers
// Every wait is bounded; a wait that runs out sets an abort flag, all roles leave their loops, copies in
// flight are waited for, TMEM is freed, and the host sees a status code instead of a hang.
#include "prefill_common.cuh"
#include "kernels.h"

#include <cstdlib>

namespace weft {

namespace {

constexpr int PF_BM = 128;               // tokens per tile = TMEM lanes
constexpr int PF_BN = 128;               // weights per tile, two halves of 64
constexpr int PF_HALF = 64;
constexpr int PF_THREADS = 512;
constexpr int PF_W_WARP0 = 8, PF_S_WARP0 = 12, PF_TMA_WARP = 14, PF_MMA_WARP = 15;
constexpr int PF_S_WARPS = 2;

// Shared memory.  int8 operands: K bytes 0..255 in two 128-byte-swizzled slabs of 128 rows x 128 bytes,
// K bytes 256.. in unswizzled 16-byte columns (128 rows x 16 bytes each = stacked 8 x 16 core matrices).
// The f16 min-term operands are unswizzled core matrices.
constexpr int PF_SLAB = 128 * 128;                     // 16 KB
constexpr int PF_COL = 128 * 16;                       // 2 KB: one 16-byte column of 128 rows
constexpr int PF_A_THIN = 2 * PF_SLAB;                 // three columns: K bytes 256..303
constexpr int PF_A_M = PF_A_THIN + 3 * PF_COL;         // {l, h} f16 per token (128 x 32 bytes)
constexpr int PF_A_SLOT = PF_A_M + PF_BM * 32;         // 42 KB, one 256-block of activations
constexpr int PF_A_TMA_BYTES = 2 * PF_SLAB + 3 * PF_COL;
constexpr int PF_WD_SLOT = PF_HALF * 8;                // per pair of weights of one half {d, d', -dmin, -dmin'}
constexpr int PF_WD_SLOTS = 8;
constexpr int PF_XD_SLOT = PF_BM * 4;                  // x.ds per token
constexpr int PF_XD_SLOTS = 4;
constexpr int PF_CONTROL = 1024;
constexpr int PF_TMEM_COLS = 512;                      // 2 x 192 used
constexpr int PF_HALF_COLS = 192;
constexpr int PF_MAX_A_SLOTS = 3, PF_MAX_B_SLOTS = 4;

// The weight operand of one 64-weight half and the ring depths, per format.
//   Q4_K : rows [q*a 0-63 | q*c 64-127], the f16 {mn, 64 mn} rows; 2 activation slots, 3 weight slots
//   TQ1_0: rows of digits 0-63; 3 activation slots, 4 weight slots
template <int FMT>
struct Cfg {
    static constexpr bool Q4K = FMT == F_Q4_K;
    static constexpr int B_ROWS = Q4K ? 2 * PF_HALF : PF_HALF;
    static constexpr int B_SLAB = B_ROWS * 128;            // K bytes 0..127 / 128..255, swizzled
    static constexpr int B_COL = B_ROWS * 16;              // one 16-byte column
    static constexpr int B_THIN = 2 * B_SLAB;              // two columns: K bytes 256..287
    static constexpr int B_M = B_THIN + 2 * B_COL;         // Q4_K: {mn, 64 mn} f16 per weight (64 x 32 bytes)
    static constexpr int B_SLOT = B_M + (Q4K ? PF_HALF * 32 : 0);   // 38 KB / 18 KB
    static constexpr int A_SLOTS = Q4K ? 2 : 3;
    static constexpr int B_SLOTS = Q4K ? 3 : 4;
    static constexpr int OFF_A = PF_CONTROL;
    static constexpr int OFF_B = OFF_A + A_SLOTS * PF_A_SLOT;
    static constexpr int OFF_WD = OFF_B + B_SLOTS * B_SLOT;
    static constexpr int OFF_XD = OFF_WD + PF_WD_SLOTS * PF_WD_SLOT;
    static constexpr int SMEM = OFF_XD + PF_XD_SLOTS * PF_XD_SLOT;
    static_assert(PF_A_SLOT % 1024 == 0 && B_SLOT % 1024 == 0 && OFF_B % 1024 == 0, "swizzled slabs must stay 1024-byte aligned");
    static_assert(SMEM <= 227 * 1024, "shared memory budget");
    static_assert(A_SLOTS <= PF_MAX_A_SLOTS && B_SLOTS <= PF_MAX_B_SLOTS, "barrier arrays");
};

struct PfParams {
    const uint8_t *w;     // (n, k) weight records (Q4_K: 16-byte aligned rows)
    const uint32_t *powers;   // TQ1_0: {1, 3, 9, 27, 81}
    float *y;             // (m, ldy)
    long long n, m, ldy;
    int nb;               // 256-blocks per row
    int m_tiles, n_tiles;
    int *status;
};

struct Control {
    uint64_t a_landed[PF_MAX_A_SLOTS], a_full[PF_MAX_A_SLOTS], a_empty[PF_MAX_A_SLOTS];
    uint64_t b_full[PF_MAX_B_SLOTS], b_empty[PF_MAX_B_SLOTS];
    uint64_t tmem_full[2], tmem_empty[2];
    uint32_t tmem_base;
    volatile int abort;
};

// Bounded wait by ONE thread that also gives up as soon as another role has aborted.  test_wait does not
// suspend the thread: the hand-offs between the roles are on the critical path of every 256-block
// (measured: try_wait with a suspend hint makes every hand-off, and the whole kernel, 1.6x slower).
__device__ __forceinline__ bool wait_one(uint64_t *bar, uint32_t parity, Control *ctl, int *status) {
    const uint32_t addr = smem_addr(bar);
    for (uint32_t i = 0; i < (1u << 26); ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        if ((i & 63u) == 63u && ctl->abort) return false;
    }
    ctl->abort = 1;
    report(status, ST_WAIT_TIMEOUT);
    return false;
}
// The same for a whole warp: lane 0 polls (32 lanes polling one barrier only slow its arrivals down), the
// result is broadcast, and the barrier's acquire is repeated once by every lane for memory ordering.
__device__ __forceinline__ bool wait_or_abort(uint64_t *bar, uint32_t parity, Control *ctl, int *status) {
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = wait_one(bar, parity, ctl, status) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (ok) mbar_try_wait(bar, parity);   // already complete: returns at once
    return ok != 0;
}


// Coordinates of one 256-block of this CTA's work list (tiles taken round-robin),
// advanced incrementally: no division on the critical path of the producer loops.
struct BlockAt {
    long long n0, m0;
    int b, tile;
    __device__ __forceinline__ void set_tile(const PfParams &p, int t) {
        tile = t;
        n0 = (long long)(t / p.m_tiles) * PF_BN;
        m0 = (long long)(t % p.m_tiles) * PF_BM;
    }
    // Blocks of a tile are taken as 0, 4, 8, ..., 1, 5, 9, ..., 2, ..., 3, ...: blocks with the same operand
    // shift follow each other, so the weight producers stay in one of their four code variants for a
    // quarter of the tile instead of switching (and refetching instructions) every block.
    __device__ __forceinline__ void advance(const PfParams &p) {
        b += 4;
        if (b >= p.nb) {
            b = (b & 3) + 1;
            if (b == 4) { b = 0; set_tile(p, tile + (int)gridDim.x); }
        }
    }
};
__device__ __forceinline__ BlockAt first_block(const PfParams &p) {
    BlockAt at;
    at.b = 0;
    at.set_tile(p, (int)blockIdx.x);
    return at;
}

// ---- producer pieces -----------------------------------------------------------------------------------

// A weight producer thread reads its row's Q4_K record of a block straight from global memory (nine
// 16-byte loads, one block ahead of its use).  Rows past N read as zero.
__device__ __forceinline__ void load_record(const PfParams &p, const BlockAt &at, int row, uint4 (&w)[9]) {
    const long long n = at.n0 + row;
    if (n < p.n) {
        const uint4 *rec = reinterpret_cast<const uint4 *>(p.w + ((size_t)n * p.nb + at.b) * 144);
#pragma unroll
        for (int i = 0; i < 9; ++i) w[i] = __ldg(rec + i);
    } else {
#pragma unroll
        for (int i = 0; i < 9; ++i) w[i] = make_uint4(0, 0, 0, 0);
    }
}

// Expand one Q4_K record (in registers) into this half's B slot: rows rh (q*a) and 64+rh (q*c), limb byte
// k at K position k + 4*W (W = 1..4 words, the shift of this block's activation operand), zeros before
// and after; the f16 {mn | 64 mn} row; {d, dmin} for the epilogue.
// The limb bytes form a stream of 64 words per limb.  Sub-block pair j contributes stream words 16j..16j+15;
// with the W words carried over from pair j-1 in front of them they are exactly the output chunks
// 4j..4j+3, so the shift costs no instructions: it only changes which register goes into which store.
template <int W>
__device__ __forceinline__ void expand_weights(const uint4 (&w)[9], uint8_t *b_slot, uint8_t *wd_slot, int rh) {
    const uint4 hd = w[0];
    // per pair of weights {d, d', -dmin, -dmin'}: the epilogue reads a pair's scales as two packed operands
    reinterpret_cast<float *>(wd_slot)[4 * (rh >> 1) + (rh & 1)] = half_bits_to_float(hd.x);
    reinterpret_cast<float *>(wd_slot)[4 * (rh >> 1) + (rh & 1) + 2] = -half_bits_to_float(hd.x >> 16);
    const Q4KScales s = q4k_unpack_scales(hd.y, hd.z, hd.w);
    float mn[8];
#pragma unroll
    for (int g = 0; g < 8; ++g) mn[g] = (float)byte_of(g < 4 ? s.mn_lo : s.mn_hi, g & 3);
    uint8_t *bm = b_slot + Cfg<F_Q4_K>::B_M;
    *reinterpret_cast<uint4 *>(bm + core_offset(rh, 0, 2)) =
        make_uint4(pack_half2(mn[0], mn[1]), pack_half2(mn[2], mn[3]), pack_half2(mn[4], mn[5]), pack_half2(mn[6], mn[7]));
    *reinterpret_cast<uint4 *>(bm + core_offset(rh, 1, 2)) =
        make_uint4(pack_half2(64.f * mn[0], 64.f * mn[1]), pack_half2(64.f * mn[2], 64.f * mn[3]),
                   pack_half2(64.f * mn[4], 64.f * mn[5]), pack_half2(64.f * mn[6], 64.f * mn[7]));

    // row rh of a swizzled slab; row 64 + rh (the q*c limb) is 8192 bytes further with the same swizzle
    const uint32_t base = smem_addr(b_slot) + (uint32_t)(rh >> 3) * 1024u + (uint32_t)(rh & 7) * 128u;
    const uint32_t x7 = (uint32_t)(rh & 7) << 4;
    uint32_t ca[4] = {0, 0, 0, 0}, cc[4] = {0, 0, 0, 0};   // the last W stream words of the previous pair
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint32_t cur_a[16], cur_c[16];
        const uint32_t scv = j < 2 ? s.sc_lo : s.sc_hi;
        const uint32_t sl = byte_of(scv, (2 * j) & 3), sh = byte_of(scv, ((2 * j) & 3) + 1);
        const uint32_t al = sl >> 3, cl = sl & 7u, ah = sh >> 3, ch = sh & 7u;
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {   // 16 nibble bytes: low nibbles -> 16 weights, high nibbles -> the 16 weights 32 further
            const uint4 qv = w[1 + 2 * j + hf];
            const uint32_t q[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t lo = q[i] & 0x0f0f0f0fu, hi = (q[i] >> 4) & 0x0f0f0f0fu;
                // every byte product is <= 15 * 7 = 105, so one 32-bit multiply scales four weights at once
                cur_a[4 * hf + i] = lo * al;      cur_c[4 * hf + i] = lo * cl;
                cur_a[8 + 4 * hf + i] = hi * ah;  cur_c[8 + 4 * hf + i] = hi * ch;
            }
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint32_t oa[4], oc[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int idx = 4 * q + k;
                oa[k] = idx < W ? ca[idx < W ? idx : 0] : cur_a[idx < W ? 0 : idx - W];
                oc[k] = idx < W ? cc[idx < W ? idx : 0] : cur_c[idx < W ? 0 : idx - W];
            }
            const int chunk = 4 * j + q;   // 16-byte K chunk 0..15
            const uint32_t at = base + (uint32_t)(chunk >> 3) * Cfg<F_Q4_K>::B_SLAB + (((uint32_t)(chunk & 7) << 4) ^ x7);
            sts_u128(at, oa[0], oa[1], oa[2], oa[3]);
            sts_u128(at + 8192u, oc[0], oc[1], oc[2], oc[3]);
        }
#pragma unroll
        for (int i = 0; i < W; ++i) { ca[i] = cur_a[16 - W + i]; cc[i] = cur_c[16 - W + i]; }
    }
    // K chunk 16: the carried words, then zeros; chunk 17: zeros
    const uint32_t thin = smem_addr(b_slot) + Cfg<F_Q4_K>::B_THIN + (uint32_t)rh * 16u;
    sts_u128(thin, ca[0], W > 1 ? ca[1] : 0u, W > 2 ? ca[2] : 0u, W > 3 ? ca[3] : 0u);
    sts_u128(thin + 1024u, cc[0], W > 1 ? cc[1] : 0u, W > 2 ? cc[2] : 0u, W > 3 ? cc[3] : 0u);
    sts_u128(thin + Cfg<F_Q4_K>::B_COL, 0u, 0u, 0u, 0u);
    sts_u128(thin + Cfg<F_Q4_K>::B_COL + 1024u, 0u, 0u, 0u, 0u);
}

// ---- TQ1_0 weights (examples/kernels/vec_dot/tq1_0_q8_k.py; GGML ggml-cpu/quants.c:430-480) ---------------------
// A record is 54 bytes, 2-byte aligned: 32 + 16 bytes of five base-3 digits, 4 bytes of four, f16 d.  The
// digits minus one are the int8 weight operand as they are (one limb, N = 64 per half, no min term), and
// isum = sum (digit - 1) * x comes out of the MMA exactly.

// The record as 14 words {12 x digits, qh, d}: aligned 4-byte loads and a 16-bit funnel shift when the
// record starts in the middle of a word.  Rows past N read as zero (digit - 1 = -1 times d = 0).
__device__ __forceinline__ void load_record_tq1(const PfParams &p, const BlockAt &at, int row, uint32_t (&w)[14]) {
    const long long n = at.n0 + row;
    if (n < p.n) {
        const uintptr_t a = reinterpret_cast<uintptr_t>(p.w + ((size_t)n * p.nb + at.b) * 54);
        const uint32_t *base = reinterpret_cast<const uint32_t *>(a & ~uintptr_t(3));
        uint32_t raw[14];
#pragma unroll
        for (int i = 0; i < 13; ++i) raw[i] = __ldg(base + i);
        if (a & 2u) {
            raw[13] = __ldg(base + 13);
#pragma unroll
            for (int i = 0; i < 13; ++i) w[i] = __funnelshift_r(raw[i], raw[i + 1], 16);
            w[13] = raw[13] >> 16;
        } else {
            raw[13] = (uint32_t)__ldg(reinterpret_cast<const unsigned short *>(base + 13));
#pragma unroll
            for (int i = 0; i < 14; ++i) w[i] = raw[i];
        }
    } else {
#pragma unroll
        for (int i = 0; i < 14; ++i) w[i] = 0;
    }
}

// Element e of the block: digit n of byte j with e = 32 n + j (bytes 0..31), 160 + 16 n + j (bytes 32..47),
// 240 + 4 n + j (qh).  Stream word g (elements 4g..4g+3) is therefore the digits n of one record word.
template <int W>
__device__ __forceinline__ void expand_tq1(const uint32_t (&w)[14], const uint32_t (&pw)[5], uint8_t *b_slot, uint8_t *wd_slot, int rh) {
    reinterpret_cast<float *>(wd_slot)[4 * (rh >> 1) + (rh & 1)] = half_bits_to_float(w[13]);
    const uint32_t base = smem_addr(b_slot) + (uint32_t)(rh >> 3) * 1024u + (uint32_t)(rh & 7) * 128u;
    const uint32_t x7 = (uint32_t)(rh & 7) << 4;
    uint32_t carry[4] = {0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint32_t cur[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int g = 16 * j + i;
            const int n = g < 40 ? g >> 3 : g < 60 ? (g - 40) >> 2 : g - 60;
            const int src = g < 40 ? (g & 7) : g < 60 ? 8 + ((g - 40) & 3) : 12;
            // digits 0..2 -> -1, 0, +1 in every byte
            cur[i] = (tq1_digits4(w[src], pw[n]) + 0x7f7f7f7fu) ^ 0x80808080u;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint32_t o[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int idx = 4 * q + k;
                o[k] = idx < W ? carry[idx < W ? idx : 0] : cur[idx < W ? 0 : idx - W];
            }
            const int chunk = 4 * j + q;
            sts_u128(base + (uint32_t)(chunk >> 3) * Cfg<F_TQ1_0>::B_SLAB + (((uint32_t)(chunk & 7) << 4) ^ x7), o[0], o[1], o[2], o[3]);
        }
#pragma unroll
        for (int i = 0; i < W; ++i) carry[i] = cur[16 - W + i];
    }
    const uint32_t thin = smem_addr(b_slot) + Cfg<F_TQ1_0>::B_THIN + (uint32_t)rh * 16u;
    sts_u128(thin, carry[0], W > 1 ? carry[1] : 0u, W > 2 ? carry[2] : 0u, W > 3 ? carry[3] : 0u);
    sts_u128(thin + Cfg<F_TQ1_0>::B_COL, 0u, 0u, 0u, 0u);
}

// One thread asks for the tile's Q8_K records of a block: word x0 = 73 b - (b & 3) of each token row is the
// 16-byte boundary at or before the record; two swizzled boxes of 128 bytes, three plain columns of 16.
__device__ __forceinline__ void issue_activations(const CUtensorMap *wide, const CUtensorMap *narrow, const BlockAt &at, uint8_t *slot, uint64_t *bar) {
    const int x0 = 73 * at.b - (at.b & 3), m0 = (int)at.m0;
    mbar_expect_tx(bar, PF_A_TMA_BYTES);
    tma_load_2d(slot, wide, x0, m0, bar);
    tma_load_2d(slot + PF_SLAB, wide, x0 + 32, m0, bar);
    tma_load_2d(slot + PF_A_THIN, narrow, x0 + 64, m0, bar);
    tma_load_2d(slot + PF_A_THIN + PF_COL, narrow, x0 + 68, m0, bar);
    tma_load_2d(slot + PF_A_THIN + 2 * PF_COL, narrow, x0 + 72, m0, bar);
}

// Out of the landed boxes: x.ds of every token to the scale ring, and the eight bsum pairs of every token,
// each split as s = 64 h + l (l in 0..63), to the f16 min-term operand {l | h}.  64 threads; thread ts keeps
// pair g = ts & 7 and walks the rows (ts >> 3) + 8 t.  `shift` = 4 * (b & 3): record byte r sits at operand
// byte r + shift.
template <bool MIN_TERM>
__device__ __forceinline__ void build_specials(uint8_t *a_slot, int shift, uint8_t *xd_slot, int ts) {
    const int g = ts & 7, r0 = ts >> 3;
    const uint32_t slot = smem_addr(a_slot);
    if (MIN_TERM) {
    const uint32_t tb = 4u + (uint32_t)shift + 4u * (uint32_t)g;   // byte inside the tail columns (operand byte 256 + tb)
    const uint32_t src = slot + PF_A_THIN + (tb >> 4) * PF_COL + (tb & 15u) + (uint32_t)r0 * 16u;
    const uint32_t dst = slot + PF_A_M + (uint32_t)r0 * 16u + 2u * (uint32_t)g;   // core_offset(r0 + 8 t, 0, 2) = 256 t + 16 r0
    uint32_t v[16];
#pragma unroll
    for (int t = 0; t < 16; ++t) v[t] = lds_u32(src + t * 128);
#pragma unroll
    for (int t = 0; t < 16; ++t) {
        const int s_ = (int)(int16_t)(v[t] & 0xffffu) + (int)(int16_t)(v[t] >> 16);
        const int l = s_ & 63, h = (s_ - l) >> 6;
        sts_u16(dst + t * 256, (uint32_t)__half_as_ushort(__int2half_rn(l)));
        sts_u16(dst + t * 256 + 128, (uint32_t)__half_as_ushort(__int2half_rn(h)));
    }
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int r = ts + 64 * k;
        sts_u32(smem_addr(xd_slot) + 4u * (uint32_t)r, lds_u32(slot + sw128_offset(r, 0) + (uint32_t)shift));
    }
}

template <int FMT>
__global__ void __launch_bounds__(PF_THREADS) prefill_kernel(const PfParams p, const __grid_constant__ CUtensorMap x_wide,
                                                               const __grid_constant__ CUtensorMap x_narrow) {
    using C = Cfg<FMT>;
    constexpr bool Q4K = C::Q4K;
    extern __shared__ __align__(1024) uint8_t smem[];
    Control *ctl = reinterpret_cast<Control *>(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles = p.m_tiles * p.n_tiles;
    const int nb = p.nb;
    const int my_tiles = (tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const int total = my_tiles * nb;   // 256-blocks this CTA works through

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::A_SLOTS; ++s) { mbar_init(&ctl->a_landed[s], 1); mbar_init(&ctl->a_full[s], PF_S_WARPS); mbar_init(&ctl->a_empty[s], 1); }
        for (int s = 0; s < C::B_SLOTS; ++s) { mbar_init(&ctl->b_full[s], 2); mbar_init(&ctl->b_empty[s], 1); }
        for (int h = 0; h < 2; ++h) { mbar_init(&ctl->tmem_full[h], 1); mbar_init(&ctl->tmem_empty[h], 8); }
        ctl->abort = 0;
        ctl->tmem_base = 0xffffffffu;
        mbar_fence_init();
    }
    __syncthreads();
    if (warp == PF_MMA_WARP) tc::tmem_alloc(&ctl->tmem_base, PF_TMEM_COLS);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = ctl->tmem_base;

    if (warp >= PF_W_WARP0 && warp < PF_W_WARP0 + 4) {
        // ------------------------------------------------------------------ weight producers
        const int row = threadIdx.x - 32 * PF_W_WARP0, half = row >> 6, rh = row & 63;
        uint8_t *b_ring = smem + C::OFF_B;
        if constexpr (Q4K) {
            BlockAt next = first_block(p);
            uint4 wn[9];
            if (total > 0) load_record(p, next, row, wn);
            for (int it = 0; it < total && !ctl->abort; ++it) {
                uint4 w[9];
#pragma unroll
                for (int i = 0; i < 9; ++i) w[i] = wn[i];
                const int words = (next.b & 3) + 1;   // this block's operand shift
                next.advance(p);
                if (it + 1 < total) load_record(p, next, row, wn);   // in flight while this block is expanded
                const int u = 2 * it + half;
                const int sb = u % C::B_SLOTS;
                if (!wait_or_abort(&ctl->b_empty[sb], (uint32_t)((u / C::B_SLOTS) & 1) ^ 1u, ctl, p.status)) break;
                uint8_t *slot = b_ring + sb * C::B_SLOT, *wd = smem + C::OFF_WD + (u & (PF_WD_SLOTS - 1)) * PF_WD_SLOT;
                switch (words) {
                case 1: expand_weights<1>(w, slot, wd, rh); break;
                case 2: expand_weights<2>(w, slot, wd, rh); break;
                case 3: expand_weights<3>(w, slot, wd, rh); break;
                default: expand_weights<4>(w, slot, wd, rh); break;
                }
                fence_proxy_async();      // generic-proxy stores must be visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) mbar_arrive(&ctl->b_full[sb]);
            }
        } else {
            BlockAt next = first_block(p);
            uint32_t pw[5];
#pragma unroll
            for (int i = 0; i < 5; ++i) pw[i] = __ldg(p.powers + i) & 0xffu;
            uint32_t wn[14];
            if (total > 0) load_record_tq1(p, next, row, wn);
            for (int it = 0; it < total && !ctl->abort; ++it) {
                uint32_t w[14];
#pragma unroll
                for (int i = 0; i < 14; ++i) w[i] = wn[i];
                const int words = (next.b & 3) + 1;   // this block's operand shift
                next.advance(p);
                if (it + 1 < total) load_record_tq1(p, next, row, wn);   // in flight while this block is expanded
                const int u = 2 * it + half;
                const int sb = u % C::B_SLOTS;
                if (!wait_or_abort(&ctl->b_empty[sb], (uint32_t)((u / C::B_SLOTS) & 1) ^ 1u, ctl, p.status)) break;
                uint8_t *slot = b_ring + sb * C::B_SLOT, *wd = smem + C::OFF_WD + (u & (PF_WD_SLOTS - 1)) * PF_WD_SLOT;
                switch (words) {
                case 1: expand_tq1<1>(w, pw, slot, wd, rh); break;
                case 2: expand_tq1<2>(w, pw, slot, wd, rh); break;
                case 3: expand_tq1<3>(w, pw, slot, wd, rh); break;
                default: expand_tq1<4>(w, pw, slot, wd, rh); break;
                }
                fence_proxy_async();      // generic-proxy stores must be visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) mbar_arrive(&ctl->b_full[sb]);
            }
        }
    } else if (warp >= PF_S_WARP0 && warp < PF_S_WARP0 + PF_S_WARPS) {
        // ------------------------------------------------------------------ scales and bsums of the landed activations
        const int ts = threadIdx.x - 32 * PF_S_WARP0;
        BlockAt at = first_block(p);
        for (int it = 0; it < total && !ctl->abort; ++it) {
            const int sa = it % C::A_SLOTS, shift = 4 * (at.b & 3);
            const uint32_t a_phase = (uint32_t)(it / C::A_SLOTS) & 1u;
            at.advance(p);
            if (!wait_or_abort(&ctl->a_landed[sa], a_phase, ctl, p.status)) break;
            build_specials<Q4K>(smem + C::OFF_A + sa * PF_A_SLOT, shift, smem + C::OFF_XD + (it & (PF_XD_SLOTS - 1)) * PF_XD_SLOT, ts);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->a_full[sa]);
        }
    } else if (warp == PF_TMA_WARP) {
        // ------------------------------------------------------------------ activation copies
        if (lane == 0) {
            BlockAt at = first_block(p);
            int issued = 0;
            for (int it = 0; it < total && !ctl->abort; ++it, at.advance(p)) {
                const int sa = it % C::A_SLOTS;
                const uint32_t a_phase = (uint32_t)(it / C::A_SLOTS) & 1u;
                // the slot was last read by the MMAs of block it - C::A_SLOTS (and, before them, by the warps above)
                if (!wait_one(&ctl->a_empty[sa], a_phase ^ 1u, ctl, p.status)) break;
                fence_proxy_async();
                issue_activations(&x_wide, &x_narrow, at, smem + C::OFF_A + sa * PF_A_SLOT, &ctl->a_landed[sa]);
                issued = it + 1;
            }
            // left early: let the copies in flight land (a phase that has completed already returns at once)
            for (int j = issued > C::A_SLOTS ? issued - C::A_SLOTS : 0; j < issued; ++j) mbar_wait(&ctl->a_landed[j % C::A_SLOTS], (uint32_t)(j / C::A_SLOTS) & 1u);
        }
    } else if (warp == PF_MMA_WARP) {
        // ------------------------------------------------------------------ MMA issue
        if (lane == 0) {
            const uint32_t idesc_q = tc::idesc_i8(PF_BM, Q4K ? 2 * PF_HALF : PF_HALF, true, true);
            const uint32_t idesc_m = tc::idesc_f16_f32acc(PF_BM, PF_HALF);
            bool ok = true;
            for (int it = 0; it < total && ok && !ctl->abort; ++it) {
                const int sa = it % C::A_SLOTS;
                const uint32_t a_phase = (uint32_t)(it / C::A_SLOTS) & 1u;
                if (!wait_one(&ctl->a_landed[sa], a_phase, ctl, p.status)) break;
                if (!wait_one(&ctl->a_full[sa], a_phase, ctl, p.status)) break;
                const uint32_t a_q = smem_addr(smem + C::OFF_A + sa * PF_A_SLOT);
                for (int h = 0; h < 2; ++h) {
                    const int u = 2 * it + h;
                    const int sb = u % C::B_SLOTS;
                    if (!wait_one(&ctl->b_full[sb], (uint32_t)((u / C::B_SLOTS) & 1), ctl, p.status)) { ok = false; break; }
                    if (!wait_one(&ctl->tmem_empty[h], (uint32_t)(it & 1) ^ 1u, ctl, p.status)) { ok = false; break; }
                    tc::fence_after_sync();
                    const uint32_t b_q = smem_addr(smem + C::OFF_B + sb * C::B_SLOT);
                    const uint32_t d = tmem + h * PF_HALF_COLS;
#pragma unroll
                    for (int j = 0; j < 8; ++j)   // K = 32 per instruction: 32 bytes further inside the swizzled row, next slab after 4
                        tc::mma_i8(d, tc::smem_desc_sw128(a_q + (j >> 2) * PF_SLAB + (j & 3) * 32),
                                   tc::smem_desc_sw128(b_q + (j >> 2) * C::B_SLAB + (j & 3) * 32), idesc_q, j > 0);
                    // K bytes 256..287: two 16-byte columns, K-adjacent core matrices one column apart
                    tc::mma_i8(d, tc::smem_desc(a_q + PF_A_THIN, PF_COL, 128), tc::smem_desc(b_q + C::B_THIN, C::B_COL, 128), idesc_q, 1);
                    if (Q4K) tc::mma_f16(d + 2 * PF_HALF, tc::smem_desc(a_q + PF_A_M, 128, 256), tc::smem_desc(b_q + C::B_M, 128, 256), idesc_m, 0);
                    tc::commit(&ctl->tmem_full[h]);   // this half's accumulators are complete
                    tc::commit(&ctl->b_empty[sb]);    // and its weight slot may be refilled
                }
                if (ok) tc::commit(&ctl->a_empty[sa]);
            }
        }
    } else if (warp < 8) {
        // ------------------------------------------------------------------ epilogue: warp = (32-token quarter, column set)
        // Every warp takes 32 of the 64 columns of BOTH halves: while it combines its share of one half the
        // tensor core is already working on the other, so neither waits for a whole half to drain.
        constexpr int EC = PF_HALF / 2;   // columns of one half per warp
        const int quarter = warp & 3, cset = warp >> 2;
        const int row = quarter * 32 + lane;   // token row of the tile = TMEM lane
        const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16) + cset * EC;
        uint64_t acc[2][EC / 2];   // packed pairs of fp32
        int it = 0;
        bool ok = true;
        for (int t = 0; t < my_tiles && ok && !ctl->abort; ++t) {
            const int tile = (int)blockIdx.x + t * (int)gridDim.x;
            const long long n0 = (long long)(tile / p.m_tiles) * PF_BN + cset * EC, m0 = (long long)(tile % p.m_tiles) * PF_BM;
#pragma unroll
            for (int i = 0; i < EC / 2; ++i) { acc[0][i] = 0ull; acc[1][i] = 0ull; }
            for (int b = 0; b < nb && ok; ++b, ++it) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (!wait_or_abort(&ctl->tmem_full[h], (uint32_t)(it & 1), ctl, p.status)) { ok = false; break; }
                    tc::fence_after_sync();
                    // written before the block's MMAs were issued: visible once their accumulators are
                    const float xd = reinterpret_cast<const float *>(smem + C::OFF_XD + (it & (PF_XD_SLOTS - 1)) * PF_XD_SLOT)[row];
                    const ulonglong2 *wd = reinterpret_cast<const ulonglong2 *>(smem + C::OFF_WD + ((2 * it + h) & (PF_WD_SLOTS - 1)) * PF_WD_SLOT) + cset * (EC / 2);
                    const uint64_t xd2 = pack2(xd, xd);
                    const uint32_t half_base = lane_base + h * PF_HALF_COLS;
                    if constexpr (Q4K) {
#pragma unroll
                        for (int c = 0; c < EC / 8; ++c) {
                            uint32_t hi[8], lo[8], mt[8];
                            tc::tmem_ld8(half_base + 8 * c, hi);
                            tc::tmem_ld8(half_base + PF_HALF + 8 * c, lo);
                            tc::tmem_ld8(half_base + 2 * PF_HALF + 8 * c, mt);
                            tc::tmem_ld_wait();
                            if (c == EC / 8 - 1) {   // last read of this half: hand its columns back to the MMA warp
                                tc::fence_before_sync();
                                __syncwarp();
                                if (lane == 0) mbar_arrive(&ctl->tmem_empty[h]);
                            }
#pragma unroll
                            for (int i = 0; i < 8; i += 2) {
                                const ulonglong2 s2 = wd[(8 * c + i) >> 1];   // {d, d'}, {-dmin, -dmin'}
                                // f32(8 hi + lo): both limbs exact as floats, one rounding in the fused multiply-add
                                const uint64_t v = fma2(pack2(8.f, 8.f), ints_to_float2(hi[i], hi[i + 1]), ints_to_float2(lo[i], lo[i + 1]));
                                const uint64_t t = fma2(s2.y, pack2(__uint_as_float(mt[i]), __uint_as_float(mt[i + 1])), mul2(s2.x, v));
                                acc[h][(8 * c + i) >> 1] = fma2(xd2, t, acc[h][(8 * c + i) >> 1]);
                            }
                        }
                    } else {
#pragma unroll
                        for (int c = 0; c < EC / 16; ++c) {
                            uint32_t is[16];
                            tc::tmem_ld16(half_base + 16 * c, is);
                            tc::tmem_ld_wait();
                            if (c == EC / 16 - 1) {
                                tc::fence_before_sync();
                                __syncwarp();
                                if (lane == 0) mbar_arrive(&ctl->tmem_empty[h]);
                            }
#pragma unroll
                            for (int i = 0; i < 16; i += 2) {
                                const ulonglong2 s2 = wd[(16 * c + i) >> 1];   // {d, d'}
                                // |isum| <= 256 * 128: exact as a float
                                acc[h][(16 * c + i) >> 1] = fma2(ints_to_float2(is[i], is[i + 1]), mul2(s2.x, xd2), acc[h][(16 * c + i) >> 1]);
                            }
                        }
                    }
                }
            }
            if (!ok) break;
            const long long m = m0 + row;
            if (m < p.m) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const long long nh = n0 + h * PF_HALF;
                    float *out = p.y + (size_t)m * p.ldy + nh;
                    if (nh + EC <= p.n && ((reinterpret_cast<uintptr_t>(out) & 15u) == 0)) {
#pragma unroll
                        for (int i = 0; i < EC; i += 4) *reinterpret_cast<ulonglong2 *>(out + i) = make_ulonglong2(acc[h][i >> 1], acc[h][(i >> 1) + 1]);
                    } else {
#pragma unroll
                        for (int i = 0; i < EC; i += 2) {
                            float a0, a1;
                            unpack2(acc[h][i >> 1], a0, a1);
                            if (nh + i < p.n) out[i] = a0;
                            if (nh + i + 1 < p.n) out[i + 1] = a1;
                        }
                    }
                }
            }
        }
    }

    tc::fence_before_sync();
    __syncthreads();
    if (warp == PF_MMA_WARP && tmem != 0xffffffffu) tc::tmem_free(tmem, PF_TMEM_COLS);
}

}  // namespace

bool prefill_supported(int fmt, long long n, long long k, long long m, const void *w, const void *xq) {
    static const bool disabled = getenv("WEFT_B200_NO_TENSOR_PREFILL") != nullptr;
    // K a multiple of 1024: Q8_K rows (292 bytes per 256) are then whole 16-byte multiples, which the TMA box loads need
    if (fmt == F_TQ1_0 ? (reinterpret_cast<uintptr_t>(w) & 1u) != 0 : fmt == F_Q4_K ? (reinterpret_cast<uintptr_t>(w) & 15u) != 0 : true) return false;
    return !disabled && k > 0 && k % 1024 == 0 && n > 0 && m >= 32 && (reinterpret_cast<uintptr_t>(xq) & 15u) == 0 &&
           n < (1LL << 31) && m < (1LL << 31);
}

cudaError_t launch_prefill(const PrefillArgs &a, int sm_count, cudaStream_t stream) {
    if (!prefill_supported(a.fmt, a.n, a.k, a.m, a.w, a.xq)) return cudaErrorNotSupported;
    PfParams p;
    p.w = static_cast<const uint8_t *>(a.w); p.powers = a.powers; p.y = a.y;
    if (a.fmt == F_TQ1_0 && !a.powers) return cudaErrorInvalidValue;
    p.n = a.n; p.m = a.m; p.ldy = a.ldy; p.nb = (int)(a.k / 256); p.status = a.status;
    p.m_tiles = (int)((a.m + PF_BM - 1) / PF_BM);
    p.n_tiles = (int)((a.n + PF_BN - 1) / PF_BN);
    const long long tiles = (long long)p.m_tiles * p.n_tiles;
    {
        cudaError_t e = grant_dynamic_smem(reinterpret_cast<const void *>(prefill_kernel<F_Q4_K>), Cfg<F_Q4_K>::SMEM);
        if (e == cudaSuccess) e = grant_dynamic_smem(reinterpret_cast<const void *>(prefill_kernel<F_TQ1_0>), Cfg<F_TQ1_0>::SMEM);
        if (e != cudaSuccess) return e;
    }
    // the Q8_K matrix as (m) rows of 73 * nb 32-bit words
    CUtensorMap x_wide, x_narrow;
    cudaError_t e = encode_tile_map(&x_wide, CU_TENSOR_MAP_DATA_TYPE_UINT32, a.xq, (unsigned long long)p.nb * 73, (unsigned long long)a.m,
                                    (unsigned long long)p.nb * 292, 32, PF_BM, true);
    if (e != cudaSuccess) return e;
    e = encode_tile_map(&x_narrow, CU_TENSOR_MAP_DATA_TYPE_UINT32, a.xq, (unsigned long long)p.nb * 73, (unsigned long long)a.m,
                        (unsigned long long)p.nb * 292, 4, PF_BM, false);
    if (e != cudaSuccess) return e;
    const int grid = (int)(tiles < sm_count ? tiles : sm_count);
    if (a.fmt == F_Q4_K) prefill_kernel<F_Q4_K><<<grid, PF_THREADS, Cfg<F_Q4_K>::SMEM, stream>>>(p, x_wide, x_narrow);
    else prefill_kernel<F_TQ1_0><<<grid, PF_THREADS, Cfg<F_TQ1_0>::SMEM, stream>>>(p, x_wide, x_narrow);
    return cudaGetLastError();
}


}  // namespace weft
