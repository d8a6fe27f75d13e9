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
// CTA = 128 tokens (TMEM lanes) x 128 weights, persistent over tiles.  The 128 weights are two halves of
// 64; each half owns 192 TMEM columns ([q*a | q*c | min term]), so the tensor core works on one half
// while the epilogue drains the other.  Warp roles:
//   warps 0-3  epilogue: tcgen05.ld the accumulators, combine, keep 128 x 128 fp32 in registers
//   warps 4-7  producers: read Q4_K records and Q8_K records from global memory (in place, no repack in
//              HBM; next block prefetched in registers), expand them into the 128-byte-swizzled K-major
//              layout the MMA reads from shared memory
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
constexpr int PF_BN = 128;               // weights per tile, two halves of 64
constexpr int PF_HALF = 64;
constexpr int PF_THREADS = 288;          // 4 epilogue + 4 producer + 1 MMA warp

// Shared memory.  int8 operands live in 128-byte-swizzled slabs of 128 K-bytes (K = 256 -> two slabs);
// the f16 min-term operands are unswizzled core matrices.
constexpr int PF_A_SLAB = PF_BM * 128;                 // 16 KB: 128 tokens x 128 K-bytes
constexpr int PF_A_Q = 2 * PF_A_SLAB;
constexpr int PF_A_M = PF_BM * 32;                     // {l, h} f16 per token
constexpr int PF_A_SLOT = PF_A_Q + PF_A_M;             // 36 KB, one 256-block of activations
constexpr int PF_A_SLOTS = 2;
constexpr int PF_B_SLAB = 2 * PF_HALF * 128;           // 16 KB: [q*a rows 0-63 | q*c rows 64-127] x 128 K-bytes
constexpr int PF_B_Q = 2 * PF_B_SLAB;
constexpr int PF_B_M = PF_HALF * 32;                   // {mn, 64 mn} f16 per weight
constexpr int PF_B_SLOT = PF_B_Q + PF_B_M;             // 34 KB, one 256-block of one 64-weight half
constexpr int PF_B_SLOTS = 3;
constexpr int PF_RAW_SLOT = PF_BN * 144;               // 18 KB of Q4_K records as they are in HBM
constexpr int PF_RAW_SLOTS = 2;
constexpr int PF_WD_SLOT = PF_HALF * 8;                // {d, dmin} per weight of one half
constexpr int PF_WD_SLOTS = 8;
constexpr int PF_XD_SLOT = PF_BM * 4;                  // x.ds per token
constexpr int PF_XD_SLOTS = 4;
constexpr int PF_CONTROL = 1024;
constexpr int PF_OFF_A = PF_CONTROL;
constexpr int PF_OFF_B = PF_OFF_A + PF_A_SLOTS * PF_A_SLOT;
constexpr int PF_OFF_RAW = PF_OFF_B + PF_B_SLOTS * PF_B_SLOT;
constexpr int PF_OFF_WD = PF_OFF_RAW + PF_RAW_SLOTS * PF_RAW_SLOT;
constexpr int PF_OFF_XD = PF_OFF_WD + PF_WD_SLOTS * PF_WD_SLOT;
constexpr int PF_SMEM = PF_OFF_XD + PF_XD_SLOTS * PF_XD_SLOT;
constexpr int PF_TMEM_COLS = 512;                      // 2 x 192 used
constexpr int PF_HALF_COLS = 192;
static_assert(PF_A_SLOT % 1024 == 0 && PF_B_SLOT % 1024 == 0 && PF_OFF_B % 1024 == 0, "swizzled slabs must stay 1024-byte aligned");
static_assert(PF_SMEM <= 227 * 1024, "shared memory budget");

struct PfParams {
    const uint8_t *w;     // (n, k) Q4_K records, 16-byte aligned rows
    const uint8_t *xq;    // (m, k) Q8_K records
    float *y;             // (m, ldy)
    long long n, m, ldy;
    int nb;               // 256-blocks per row
    int m_tiles, n_tiles;
    int debug;            // timing experiments (bit mask of work to skip); 0 in normal use
    int *status;
};

// byte offset of (row, 16-byte chunk 0..7) inside a 128-byte-swizzled slab
__device__ __forceinline__ uint32_t sw128_offset(int row, int chunk) {
    return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4));
}
// byte offset of (row, 16-byte chunk) in an unswizzled K-major operand: 8-row groups of `chunks` core matrices
__device__ __forceinline__ uint32_t core_offset(int row, int chunk, int chunks) {
    return (uint32_t)((row >> 3) * (chunks * 128) + chunk * 128 + (row & 7) * 16);
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    return (uint32_t)__half_as_ushort(__float2half_rn(lo)) | ((uint32_t)__half_as_ushort(__float2half_rn(hi)) << 16);
}

struct Control {
    uint64_t a_full[PF_A_SLOTS], a_empty[PF_A_SLOTS];
    uint64_t b_full[PF_B_SLOTS], b_empty[PF_B_SLOTS];
    uint64_t raw_full[PF_RAW_SLOTS], raw_empty[PF_RAW_SLOTS];
    uint64_t tmem_full[2], tmem_empty[2];
    uint32_t tmem_base;
    volatile int abort;
};

// Bounded wait by ONE thread that also gives up as soon as another role has aborted.  test_wait does not
// suspend the thread: the hand-offs between the roles are on the critical path of every 256-block.
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

// Coordinates of one 256-block of this CTA's work list (tiles taken round-robin, blocks in K order),
// advanced incrementally: no division on the critical path of the producer loop.
struct BlockAt {
    long long n0, m0;
    int b, tile;
    __device__ __forceinline__ void set_tile(const PfParams &p, int t) {
        tile = t;
        n0 = (long long)(t / p.m_tiles) * PF_BN;
        m0 = (long long)(t % p.m_tiles) * PF_BM;
    }
    __device__ __forceinline__ void advance(const PfParams &p) {
        if (++b == p.nb) { b = 0; set_tile(p, tile + (int)gridDim.x); }
    }
};
__device__ __forceinline__ BlockAt first_block(const PfParams &p, int steps) {
    BlockAt at;
    at.b = 0;
    at.set_tile(p, (int)blockIdx.x);
    for (int i = 0; i < steps; ++i) at.advance(p);
    return at;
}

// ---- producer pieces -----------------------------------------------------------------------------------

// Activation codes of one block, coalesced: for each of the warp's 32 token rows, lane l takes code words
// l and 32+l (4-byte loads: Q8_K codes start 4 bytes into a 292-byte record, so nothing wider is
// aligned).  Loaded into registers early, stored into the swizzled A slot after the weight expansion.
__device__ __forceinline__ void load_codes(const PfParams &p, const BlockAt &at, int wg, int lane, uint32_t (&xa)[64]) {
    const size_t x_row_bytes = (size_t)p.nb * 292;
    const uint8_t *src = p.xq + (size_t)(at.m0 + wg * 32) * x_row_bytes + (size_t)at.b * 292 + 4 + 4 * lane;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        if (at.m0 + wg * 32 + i < p.m) {
            xa[2 * i] = __ldg(reinterpret_cast<const uint32_t *>(src));
            xa[2 * i + 1] = __ldg(reinterpret_cast<const uint32_t *>(src + 128));
        } else {
            xa[2 * i] = 0; xa[2 * i + 1] = 0;
        }
        src += x_row_bytes;
    }
}
__device__ __forceinline__ void store_codes(const uint32_t (&xa)[64], uint8_t *a_slot, int wg, int lane) {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        const uint32_t at = sw128_offset(wg * 32 + i, lane >> 2) + (lane & 3) * 4;
        *reinterpret_cast<uint32_t *>(a_slot + at) = xa[2 * i];                  // K bytes 0..127
        *reinterpret_cast<uint32_t *>(a_slot + PF_A_SLAB + at) = xa[2 * i + 1];  // K bytes 128..255
    }
}

// The nine other words of each record (x.ds and eight bsum pairs): 32 rows x 9 words per warp, dealt to
// the lanes as item j = lane + 32 t (row j / 9, word j % 9), so neighbouring lanes read neighbouring words.
__device__ __forceinline__ void load_specials(const PfParams &p, const BlockAt &at, int wg, int lane, uint32_t (&sp)[9]) {
    const size_t x_row_bytes = (size_t)p.nb * 292;
#pragma unroll
    for (int t = 0; t < 9; ++t) {
        const int j = lane + 32 * t, i = j / 9, wd = j - 9 * i;
        const long long m = at.m0 + wg * 32 + i;
        sp[t] = 0;
        if (m < p.m) {
            const uint32_t *words = reinterpret_cast<const uint32_t *>(p.xq + (size_t)m * x_row_bytes + (size_t)at.b * 292);
            sp[t] = __ldg(words + (wd == 0 ? 0 : 64 + wd));
        }
    }
}

// x.ds to the scale ring; each bsum pair s = 64 h + l (l in 0..63) to the f16 min-term operand {l | h}.
__device__ __forceinline__ void store_specials(const uint32_t (&sp)[9], uint8_t *a_slot, uint8_t *xd_slot, int wg, int lane) {
    uint8_t *a_m = a_slot + PF_A_Q;
#pragma unroll
    for (int t = 0; t < 9; ++t) {
        const int j = lane + 32 * t, i = j / 9, wd = j - 9 * i;
        const int r = wg * 32 + i;
        if (wd == 0) {
            reinterpret_cast<uint32_t *>(xd_slot)[r] = sp[t];
        } else {
            const int g = wd - 1;
            const int s = (int)(int16_t)(sp[t] & 0xffffu) + (int)(int16_t)(sp[t] >> 16);
            const int l = s & 63;
            *reinterpret_cast<__half *>(a_m + core_offset(r, 0, 2) + 2 * g) = __float2half_rn((float)l);
            *reinterpret_cast<__half *>(a_m + core_offset(r, 1, 2) + 2 * g) = __float2half_rn((float)((s - l) >> 6));
        }
    }
}

// One thread asks for its weight row's record of the block: a 144-byte bulk copy into the raw slot.
__device__ __forceinline__ void issue_raw(const PfParams &p, const BlockAt &at, uint8_t *raw_slot, int row, uint64_t *bar) {
    const long long n = at.n0 + row;
    if (n < p.n) {
        mbar_expect_tx(bar, 144);
        bulk_g2s(raw_slot + row * 144, p.w + ((size_t)n * p.nb + at.b) * 144, 144, bar);
    } else {
        mbar_arrive(bar);   // past the last weight row: whatever is in the slot is expanded, its columns are never stored
    }
}

// Expand one Q4_K record (in registers) into this half's B slot: rows rh (q*a) and 64+rh (q*c) of both
// K slabs, the f16 {mn | 64 mn} row, and {d, dmin} for the epilogue.
__device__ __forceinline__ void expand_weights(const uint4 (&w)[9], uint8_t *b_slot, uint8_t *wd_slot, int rh) {
    const uint4 hd = w[0];
    reinterpret_cast<float2 *>(wd_slot)[rh] = make_float2(half_bits_to_float(hd.x), half_bits_to_float(hd.x >> 16));
    const Q4KScales s = q4k_unpack_scales(hd.y, hd.z, hd.w);
    float mn[8];
#pragma unroll
    for (int g = 0; g < 8; ++g) mn[g] = (float)byte_of(g < 4 ? s.mn_lo : s.mn_hi, g & 3);
    uint8_t *bm = b_slot + PF_B_Q;
    *reinterpret_cast<uint4 *>(bm + core_offset(rh, 0, 2)) =
        make_uint4(pack_half2(mn[0], mn[1]), pack_half2(mn[2], mn[3]), pack_half2(mn[4], mn[5]), pack_half2(mn[6], mn[7]));
    *reinterpret_cast<uint4 *>(bm + core_offset(rh, 1, 2)) =
        make_uint4(pack_half2(64.f * mn[0], 64.f * mn[1]), pack_half2(64.f * mn[2], 64.f * mn[3]),
                   pack_half2(64.f * mn[4], 64.f * mn[5]), pack_half2(64.f * mn[6], 64.f * mn[7]));
#pragma unroll
    for (int c = 0; c < 8; ++c) {   // 16 nibble bytes: low nibbles -> 16 weights, high nibbles -> the 16 weights 32 further
        const uint4 qv = w[1 + c];
        const int j = c >> 1, hf = c & 1;
        const uint32_t scv = j < 2 ? s.sc_lo : s.sc_hi;
        const uint32_t sl = byte_of(scv, (2 * j) & 3), sh = byte_of(scv, ((2 * j) & 3) + 1);
        const uint32_t al = sl >> 3, cl = sl & 7u, ah = sh >> 3, ch = sh & 7u;
        const uint32_t M4 = 0x0f0f0f0fu;
        const uint32_t lo[4] = {qv.x & M4, qv.y & M4, qv.z & M4, qv.w & M4};
        const uint32_t hi[4] = {(qv.x >> 4) & M4, (qv.y >> 4) & M4, (qv.z >> 4) & M4, (qv.w >> 4) & M4};
        // every byte product is <= 15 * 7 = 105, so one 32-bit multiply scales four weights at once
        const int kl = 4 * j + hf, kh = 4 * j + 2 + hf;          // 16-byte K chunk index 0..15
        uint8_t *slab_l = b_slot + (kl >> 3) * PF_B_SLAB, *slab_h = b_slot + (kh >> 3) * PF_B_SLAB;
        *reinterpret_cast<uint4 *>(slab_l + sw128_offset(rh, kl & 7)) = make_uint4(lo[0] * al, lo[1] * al, lo[2] * al, lo[3] * al);
        *reinterpret_cast<uint4 *>(slab_l + sw128_offset(PF_HALF + rh, kl & 7)) = make_uint4(lo[0] * cl, lo[1] * cl, lo[2] * cl, lo[3] * cl);
        *reinterpret_cast<uint4 *>(slab_h + sw128_offset(rh, kh & 7)) = make_uint4(hi[0] * ah, hi[1] * ah, hi[2] * ah, hi[3] * ah);
        *reinterpret_cast<uint4 *>(slab_h + sw128_offset(PF_HALF + rh, kh & 7)) = make_uint4(hi[0] * ch, hi[1] * ch, hi[2] * ch, hi[3] * ch);
    }
}

__global__ void __launch_bounds__(PF_THREADS) prefill_q4k_kernel(const PfParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    Control *ctl = reinterpret_cast<Control *>(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles = p.m_tiles * p.n_tiles;
    const int nb = p.nb;
    const int my_tiles = (tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const int total = my_tiles * nb;   // 256-blocks this CTA works through

    if (threadIdx.x == 0) {
        for (int s = 0; s < PF_A_SLOTS; ++s) { mbar_init(&ctl->a_full[s], 4); mbar_init(&ctl->a_empty[s], 1); }
        for (int s = 0; s < PF_B_SLOTS; ++s) { mbar_init(&ctl->b_full[s], 2); mbar_init(&ctl->b_empty[s], 1); }
        for (int s = 0; s < PF_RAW_SLOTS; ++s) { mbar_init(&ctl->raw_full[s], 128); mbar_init(&ctl->raw_empty[s], 4); }
        for (int h = 0; h < 2; ++h) { mbar_init(&ctl->tmem_full[h], 1); mbar_init(&ctl->tmem_empty[h], 4); }
        ctl->abort = 0;
        ctl->tmem_base = 0xffffffffu;
        mbar_fence_init();
    }
    __syncthreads();
    if (warp == 8) tc::tmem_alloc(&ctl->tmem_base, PF_TMEM_COLS);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = ctl->tmem_base;

    if (warp >= 4 && warp < 8) {
        // ------------------------------------------------------------------ producers
        const int row = threadIdx.x - 128, wg = warp - 4, half = row >> 6, rh = row & 63;
        uint8_t *a_ring = smem + PF_OFF_A, *b_ring = smem + PF_OFF_B, *raw_ring = smem + PF_OFF_RAW;
        if (total > 0 && !(p.debug & 4)) {
            issue_raw(p, first_block(p, 0), raw_ring, row, &ctl->raw_full[0]);
            if (total > 1) issue_raw(p, first_block(p, 1), raw_ring + PF_RAW_SLOT, row, &ctl->raw_full[1]);
        }
        BlockAt cur = first_block(p, 0), next2 = first_block(p, 2);   // blocks it and it+2
        for (int it = 0; it < total && !ctl->abort; ++it, cur.advance(p), next2.advance(p)) {
            const int sa = it & 1;
            // activations of this block: the slot was last read by the MMAs of block it-2
            if (!wait_or_abort(&ctl->a_empty[sa], (uint32_t)((it >> 1) & 1) ^ 1u, ctl, p.status)) break;
            uint32_t sp[9];
            uint32_t xa[64];
            if (!(p.debug & 1)) load_codes(p, cur, wg, lane, xa);   // in flight while the weights are expanded
            if (!(p.debug & 2)) load_specials(p, cur, wg, lane, sp);

            // weights: this thread's record is in the raw slot
            if (!(p.debug & 4) && !wait_or_abort(&ctl->raw_full[sa], (uint32_t)((it >> 1) & 1), ctl, p.status)) break;
            uint4 w[9];
            {
                const uint4 *rec = reinterpret_cast<const uint4 *>(raw_ring + sa * PF_RAW_SLOT + row * 144);
#pragma unroll
                for (int i = 0; i < 9; ++i) w[i] = rec[i];
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->raw_empty[sa]);
            if (it + 2 < total && !(p.debug & 4)) {   // refill the raw slot two blocks ahead once all four warps have read it
                if (!wait_or_abort(&ctl->raw_empty[sa], (uint32_t)((it >> 1) & 1), ctl, p.status)) break;
                fence_proxy_async();
                issue_raw(p, next2, raw_ring + sa * PF_RAW_SLOT, row, &ctl->raw_full[sa]);
            }
            const int u = 2 * it + half;
            const int sb = u % PF_B_SLOTS;
            if (!wait_or_abort(&ctl->b_empty[sb], (uint32_t)((u / PF_B_SLOTS) & 1) ^ 1u, ctl, p.status)) break;
            if (!(p.debug & 8)) expand_weights(w, b_ring + sb * PF_B_SLOT, smem + PF_OFF_WD + (u & (PF_WD_SLOTS - 1)) * PF_WD_SLOT, rh);
            fence_proxy_async();      // generic-proxy stores must be visible to the tensor core's reads
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->b_full[sb]);

            // finish the activations
            if (!(p.debug & 1)) store_codes(xa, a_ring + sa * PF_A_SLOT, wg, lane);
            if (!(p.debug & 2)) store_specials(sp, a_ring + sa * PF_A_SLOT, smem + PF_OFF_XD + (it & (PF_XD_SLOTS - 1)) * PF_XD_SLOT, wg, lane);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->a_full[sa]);
        }
    } else if (warp == 8) {
        // ------------------------------------------------------------------ MMA issue
        if (lane == 0) {
            const uint32_t idesc_q = tc::idesc_i8(PF_BM, 2 * PF_HALF, true, true);
            const uint32_t idesc_m = tc::idesc_f16_f32acc(PF_BM, PF_HALF);
            bool ok = true;
            for (int it = 0; it < total && ok && !ctl->abort; ++it) {
                const int sa = it & 1;
                if (!wait_one(&ctl->a_full[sa], (uint32_t)((it >> 1) & 1), ctl, p.status)) break;
                const uint32_t a_q = smem_addr(smem + PF_OFF_A + sa * PF_A_SLOT), a_m = a_q + PF_A_Q;
                for (int h = 0; h < 2; ++h) {
                    const int u = 2 * it + h;
                    const int sb = u % PF_B_SLOTS;
                    if (!wait_one(&ctl->b_full[sb], (uint32_t)((u / PF_B_SLOTS) & 1), ctl, p.status)) { ok = false; break; }
                    if (!wait_one(&ctl->tmem_empty[h], (uint32_t)(it & 1) ^ 1u, ctl, p.status)) { ok = false; break; }
                    if (!(p.debug & 256)) tc::fence_after_sync();
                    const uint32_t b_q = smem_addr(smem + PF_OFF_B + sb * PF_B_SLOT), b_m = b_q + PF_B_Q;
                    const uint32_t d = tmem + h * PF_HALF_COLS;
                    if (!(p.debug & 32))
#pragma unroll
                    for (int j = 0; j < 8; ++j)   // K = 32 per instruction: 32 bytes further inside the swizzled row, next slab after 4
                        tc::mma_i8(d, tc::smem_desc_sw128(a_q + (j >> 2) * PF_A_SLAB + (j & 3) * 32),
                                   tc::smem_desc_sw128(b_q + (j >> 2) * PF_B_SLAB + (j & 3) * 32), idesc_q, j > 0);
                    if (!(p.debug & 32)) tc::mma_f16(d + 2 * PF_HALF, tc::smem_desc(a_m, 128, 256), tc::smem_desc(b_m, 128, 256), idesc_m, 0);
                    if (p.debug & 64) mbar_arrive(&ctl->tmem_full[h]); else tc::commit(&ctl->tmem_full[h]);   // this half's accumulators are complete
                    if (p.debug & 64) mbar_arrive(&ctl->b_empty[sb]); else tc::commit(&ctl->b_empty[sb]);    // and its weight slot may be refilled
                }
                if (ok) { if (p.debug & 64) mbar_arrive(&ctl->a_empty[sa]); else tc::commit(&ctl->a_empty[sa]); }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 0-3)
        const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
        float acc[PF_BN];
        int it = 0;
        bool ok = true;
        for (int t = 0; t < my_tiles && ok && !ctl->abort; ++t) {
            const int tile = (int)blockIdx.x + t * (int)gridDim.x;
            const long long n0 = (long long)(tile / p.m_tiles) * PF_BN, m0 = (long long)(tile % p.m_tiles) * PF_BM;
#pragma unroll
            for (int i = 0; i < PF_BN; ++i) acc[i] = 0.f;
            for (int b = 0; b < nb && ok; ++b, ++it) {
                const float *xds = reinterpret_cast<const float *>(smem + PF_OFF_XD + (it & (PF_XD_SLOTS - 1)) * PF_XD_SLOT);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (!wait_or_abort(&ctl->tmem_full[h], (uint32_t)(it & 1), ctl, p.status)) { ok = false; break; }
                    tc::fence_after_sync();
                    const float4 *wd = reinterpret_cast<const float4 *>(smem + PF_OFF_WD + ((2 * it + h) & (PF_WD_SLOTS - 1)) * PF_WD_SLOT);
                    const float xd = xds[threadIdx.x];
                    if (p.debug & 16) {
                        tc::fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&ctl->tmem_empty[h]);
                        continue;
                    }
#pragma unroll
                    for (int c = 0; c < PF_HALF / 16; ++c) {
                        uint32_t hi[16], lo[16], mt[16];
                        tc::tmem_ld16(lane_base + h * PF_HALF_COLS + 16 * c, hi);
                        tc::tmem_ld16(lane_base + h * PF_HALF_COLS + PF_HALF + 16 * c, lo);
                        tc::tmem_ld16(lane_base + h * PF_HALF_COLS + 2 * PF_HALF + 16 * c, mt);
                        tc::tmem_ld_wait();
                        if (c == PF_HALF / 16 - 1) {   // last read of this half: hand its columns back to the MMA warp
                            tc::fence_before_sync();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(&ctl->tmem_empty[h]);
                        }
#pragma unroll
                        for (int i = 0; i < 16; i += 2) {
                            const float4 s2 = wd[(16 * c + i) >> 1];
                            const int v0 = 8 * (int)hi[i] + (int)lo[i], v1 = 8 * (int)hi[i + 1] + (int)lo[i + 1];
                            acc[h * PF_HALF + 16 * c + i] += xd * (s2.x * (float)v0 - s2.y * __uint_as_float(mt[i]));
                            acc[h * PF_HALF + 16 * c + i + 1] += xd * (s2.z * (float)v1 - s2.w * __uint_as_float(mt[i + 1]));
                        }
                    }
                }
            }
            if (!ok) break;
            const long long m = m0 + threadIdx.x;
            if (m < p.m) {
                float *out = p.y + (size_t)m * p.ldy + n0;
                if (n0 + PF_BN <= p.n && ((reinterpret_cast<uintptr_t>(out) & 15u) == 0)) {
#pragma unroll
                    for (int i = 0; i < PF_BN; i += 4) *reinterpret_cast<float4 *>(out + i) = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
                } else {
#pragma unroll
                    for (int i = 0; i < PF_BN; ++i)
                        if (n0 + i < p.n) out[i] = acc[i];
                }
            }
        }
    }

    tc::fence_before_sync();
    __syncthreads();
    if (warp == 8 && tmem != 0xffffffffu) tc::tmem_free(tmem, PF_TMEM_COLS);
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
    PfParams p;
    p.w = static_cast<const uint8_t *>(a.w); p.xq = static_cast<const uint8_t *>(a.xq); p.y = a.y;
    p.n = a.n; p.m = a.m; p.ldy = a.ldy; p.nb = (int)(a.k / 256); p.status = a.status;
    static const int debug = getenv("WEFT_B200_PF_DEBUG") ? atoi(getenv("WEFT_B200_PF_DEBUG")) : 0;
    p.debug = debug;
    p.m_tiles = (int)((a.m + PF_BM - 1) / PF_BM);
    p.n_tiles = (int)((a.n + PF_BN - 1) / PF_BN);
    const long long tiles = (long long)p.m_tiles * p.n_tiles;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(prefill_q4k_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    const int grid = (int)(tiles < sm_count ? tiles : sm_count);
    prefill_q4k_kernel<<<grid, PF_THREADS, PF_SMEM, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace weft
