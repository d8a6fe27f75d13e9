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
//   warps 0-7   epilogue, warp = (half, 32-token quarter): tcgen05.ld the accumulators, combine, keep
//               32 x 64 fp32 in registers across the blocks of a tile
//   warps 8-11  weight producers, one weight row per thread: Q4_K records arrive in a raw ring by
//               144-byte bulk copies (in place, no repack in HBM) and are expanded into the
//               128-byte-swizzled K-major layout the MMA reads from shared memory
//   warps 12-14 activation producers: Q8_K codes, scales and bsums read from global memory one block
//               ahead (in registers) and stored into the swizzled A slot when it is free
//   warp 15     allocates TMEM; one lane issues the MMAs and commits them to mbarriers
// Two activation slots and three weight slots let the producers run ahead of the tensor core.  Every wait is
// bounded; a wait that runs out sets an abort flag, all roles leave their loops, TMEM is freed, and the
// host sees a status code instead of a hang.
#include "tcgen05.cuh"
#include "tensormap.cuh"
#include "kernels.h"

#include <cstdlib>

namespace weft {

namespace {

constexpr int PF_BM = 128;               // tokens per tile = TMEM lanes
constexpr int PF_BN = 128;               // weights per tile, two halves of 64
constexpr int PF_HALF = 64;
constexpr int PF_THREADS = 512;          // 8 epilogue + 4 weight producer + 3 activation producer + 1 MMA warp
constexpr int PF_W_WARP0 = 8, PF_A_WARP0 = 12, PF_MMA_WARP = 15;

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
constexpr int PF_RAWA_WORDS = 76;                      // 304 bytes: a Q8_K record (292) from the 16-byte boundary at or before it
constexpr int PF_RAWA_PITCH = 4 * PF_RAWA_WORDS;
constexpr int PF_RAWA_SLOT = PF_BM * PF_RAWA_PITCH;    // 38 KB: one 256-block of Q8_K records as they are in HBM
constexpr int PF_WD_SLOT = PF_HALF * 8;                // {d, dmin} per weight of one half
constexpr int PF_WD_SLOTS = 8;
constexpr int PF_XD_SLOT = PF_BM * 4;                  // x.ds per token
constexpr int PF_XD_SLOTS = 4;
constexpr int PF_CONTROL = 1024;
constexpr int PF_OFF_A = PF_CONTROL;
constexpr int PF_OFF_B = PF_OFF_A + PF_A_SLOTS * PF_A_SLOT;
constexpr int PF_OFF_RAWA = PF_OFF_B + PF_B_SLOTS * PF_B_SLOT;
constexpr int PF_OFF_WD = PF_OFF_RAWA + PF_RAWA_SLOT;
constexpr int PF_OFF_XD = PF_OFF_WD + PF_WD_SLOTS * PF_WD_SLOT;
constexpr int PF_SMEM = PF_OFF_XD + PF_XD_SLOTS * PF_XD_SLOT;
constexpr int PF_TMEM_COLS = 512;                      // 2 x 192 used
constexpr int PF_HALF_COLS = 192;
static_assert(PF_A_SLOT % 1024 == 0 && PF_B_SLOT % 1024 == 0 && PF_OFF_B % 1024 == 0, "swizzled slabs must stay 1024-byte aligned");
static_assert(PF_OFF_RAWA % 128 == 0, "TMA destinations are 128-byte aligned");
static_assert(PF_SMEM <= 227 * 1024, "shared memory budget");

struct PfParams {
    const uint8_t *w;     // (n, k) Q4_K records, 16-byte aligned rows
    const uint8_t *xq;    // (m, k) Q8_K records
    float *y;             // (m, ldy)
    long long n, m, ldy;
    int nb;               // 256-blocks per row
    int m_tiles, n_tiles;
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

// f32(8 * hi + lo), rounded to nearest like an int-to-float conversion of the sum, on the full-rate fp32 pipe
// (the conversion unit runs at a quarter of it): |hi|, |lo| <= 256 * 105 * 128 < 2^22, so adding the integer
// to the bit pattern of 1.5 * 2^23 and subtracting that constant gives its exact float; 8 * f(hi) + f(lo) is
// exact before the single rounding of the fused multiply-add.
__device__ __forceinline__ float limbs_to_float(uint32_t hi, uint32_t lo) {
    const float fh = __uint_as_float(hi + 0x4b400000u) - 12582912.f;
    const float fl = __uint_as_float(lo + 0x4b400000u) - 12582912.f;
    return fmaf(8.f, fh, fl);
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    return (uint32_t)__half_as_ushort(__float2half_rn(lo)) | ((uint32_t)__half_as_ushort(__float2half_rn(hi)) << 16);
}

struct Control {
    uint64_t a_full[PF_A_SLOTS], a_empty[PF_A_SLOTS];
    uint64_t b_full[PF_B_SLOTS], b_empty[PF_B_SLOTS];
    uint64_t rawa_full, rawa_empty;
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

#ifdef WEFT_PF_PROFILE
__device__ unsigned long long g_pf_prof[16][8];
#define PF_TIMED(slot, call) ([&] { const long long t_ = clock64(); const bool r_ = (call); prof[slot] += clock64() - t_; return r_; }())
#define PF_MARK(slot) do { const long long n_ = clock64(); prof[slot] += n_ - mark; mark = n_; } while (0)
#define PF_MARK0() (mark = clock64())
#else
#define PF_TIMED(slot, call) (call)
#define PF_MARK(slot) do { } while (0)
#define PF_MARK0() do { } while (0)
#endif

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

constexpr int PF_A_WARPS = 3;                                        // activation producer warps
constexpr int PF_A_ROWS = (PF_BM + PF_A_WARPS - 1) / PF_A_WARPS;     // token rows per warp: wa, wa + 3, ...
constexpr int PF_SP_ITEMS = (PF_BM * 9 + 32 * PF_A_WARPS - 1) / (32 * PF_A_WARPS);

// A weight producer thread reads its row's Q4_K record of a block straight from global memory (nine
// 16-byte loads, one block ahead of its use, in place: no repack in HBM).  Rows past N read as zero.
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
// One elected thread asks for the tile's Q8_K records of a block with one TMA box copy.  A record starts 4 * (b & 3) bytes past a 16-byte boundary (rows are
// 16-byte multiples because K is a multiple of 1024), so the box starts at that boundary and is 304 bytes wide.
__device__ __forceinline__ void issue_raw_a(const CUtensorMap *map, const BlockAt &at, uint8_t *raw, uint64_t *bar) {
    mbar_expect_tx(bar, PF_RAWA_SLOT);
    tma_load_2d(raw, map, 73 * at.b - (at.b & 3), (int)at.m0, bar);
}

__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts_u32(uint32_t addr, uint32_t v) { asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory"); }
__device__ __forceinline__ void sts_u16(uint32_t addr, uint32_t v) { asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"((unsigned short)v) : "memory"); }

// Raw Q8_K records -> the MMA's activation operands.
// Codes: warp wa takes the 8-row groups wa, wa + 3, ...; within a group lane l moves code words l and 32 + l
// of each row into the swizzled A slabs: sixteen independent loads, then sixteen stores, all at offsets
// that are compile-time constants from per-lane bases.
// The nine other words of each record: bsum pair g of row r is item j = 8 r + g, dealt to the 96 threads as
// j = thread + 96 t (so a thread keeps its g and walks 12 rows at a time); the pair s = 64 h + l
// (l in 0..63) goes to the f16 min-term operand {l | h}.  x.ds of rows thread, thread + 96 goes to the scale ring.
__device__ __forceinline__ void relayout_activations(const uint8_t *raw, int shift, uint8_t *a_slot, uint8_t *xd_slot, int wa, int ta, int lane) {
    const uint32_t src = smem_addr(raw) + (uint32_t)shift + 4u + 4u * (uint32_t)lane;
    const uint32_t dst = smem_addr(a_slot) + (uint32_t)(lane & 3) * 4u;
    const uint32_t ch = (uint32_t)lane >> 2;
    for (int grp = wa; grp < PF_BM / 8; grp += PF_A_WARPS) {
        uint32_t c[16];
        const uint32_t s0 = src + (uint32_t)grp * (8 * PF_RAWA_PITCH), d0 = dst + (uint32_t)grp * 1024u;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            c[2 * i] = lds_u32(s0 + i * PF_RAWA_PITCH);
            c[2 * i + 1] = lds_u32(s0 + i * PF_RAWA_PITCH + 128);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t at = d0 + i * 128 + ((ch ^ (uint32_t)i) << 4);
            sts_u32(at, c[2 * i]);                  // K bytes 0..127
            sts_u32(at + PF_A_SLAB, c[2 * i + 1]);  // K bytes 128..255
        }
    }
    const uint32_t raw_s = smem_addr(raw) + (uint32_t)shift;
    {
        const int g = ta & 7, r0 = ta >> 3;
        const uint32_t a_m = smem_addr(a_slot) + PF_A_Q + 2u * (uint32_t)g;
        uint32_t v[11];
#pragma unroll
        for (int t = 0; t < 11; ++t) v[t] = (t < 10 || ta < 64) ? lds_u32(raw_s + (uint32_t)(r0 + 12 * t) * PF_RAWA_PITCH + 260u + 4u * (uint32_t)g) : 0u;
#pragma unroll
        for (int t = 0; t < 11; ++t) {
            const int r = r0 + 12 * t;
            if (t == 10 && ta >= 64) break;
            const int s_ = (int)(int16_t)(v[t] & 0xffffu) + (int)(int16_t)(v[t] >> 16);
            const int l = s_ & 63, h = (s_ - l) >> 6;
            const uint32_t at = a_m + (uint32_t)r * 16u + (uint32_t)(r >> 3) * 128u;   // core_offset(r, 0, 2)
            sts_u16(at, (uint32_t)__half_as_ushort(__int2half_rn(l)));
            sts_u16(at + 128u, (uint32_t)__half_as_ushort(__int2half_rn(h)));
        }
    }
    for (int r = ta; r < PF_BM; r += 32 * PF_A_WARPS) reinterpret_cast<uint32_t *>(xd_slot)[r] = lds_u32(raw_s + (uint32_t)r * PF_RAWA_PITCH);
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

__global__ void __launch_bounds__(PF_THREADS) prefill_q4k_kernel(const PfParams p, const __grid_constant__ CUtensorMap x_map) {
    extern __shared__ __align__(1024) uint8_t smem[];
    Control *ctl = reinterpret_cast<Control *>(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles = p.m_tiles * p.n_tiles;
    const int nb = p.nb;
    const int my_tiles = (tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const int total = my_tiles * nb;   // 256-blocks this CTA works through

    if (threadIdx.x == 0) {
        for (int s = 0; s < PF_A_SLOTS; ++s) { mbar_init(&ctl->a_full[s], PF_A_WARPS); mbar_init(&ctl->a_empty[s], 1); }
        for (int s = 0; s < PF_B_SLOTS; ++s) { mbar_init(&ctl->b_full[s], 2); mbar_init(&ctl->b_empty[s], 1); }
        mbar_init(&ctl->rawa_full, 1); mbar_init(&ctl->rawa_empty, PF_A_WARPS);
        for (int h = 0; h < 2; ++h) { mbar_init(&ctl->tmem_full[h], 1); mbar_init(&ctl->tmem_empty[h], 4); }
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
#ifdef WEFT_PF_PROFILE
    long long prof[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const long long prof_begin = clock64();
    long long mark = prof_begin;
#endif

    if (warp >= PF_W_WARP0 && warp < PF_W_WARP0 + 4) {
        // ------------------------------------------------------------------ weight producers
        const int row = threadIdx.x - 32 * PF_W_WARP0, half = row >> 6, rh = row & 63;
        uint8_t *b_ring = smem + PF_OFF_B;
        BlockAt next = first_block(p, 0);
        uint4 wn[9];
        if (total > 0) load_record(p, next, row, wn);
        for (int it = 0; it < total && !ctl->abort; ++it) {
            uint4 w[9];
#pragma unroll
            for (int i = 0; i < 9; ++i) w[i] = wn[i];
            next.advance(p);
            if (it + 1 < total) load_record(p, next, row, wn);   // in flight while this block is expanded
            const int u = 2 * it + half;
            const int sb = u % PF_B_SLOTS;
            if (!PF_TIMED(2, wait_or_abort(&ctl->b_empty[sb], (uint32_t)((u / PF_B_SLOTS) & 1) ^ 1u, ctl, p.status))) break;
            PF_MARK0();
            expand_weights(w, b_ring + sb * PF_B_SLOT, smem + PF_OFF_WD + (u & (PF_WD_SLOTS - 1)) * PF_WD_SLOT, rh);
            PF_MARK(4);
            fence_proxy_async();      // generic-proxy stores must be visible to the tensor core's reads
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->b_full[sb]);
            PF_MARK(5);
        }
    } else if (warp >= PF_A_WARP0 && warp < PF_A_WARP0 + PF_A_WARPS) {
        // ------------------------------------------------------------------ activation producers
        const int wa = warp - PF_A_WARP0, ta = threadIdx.x - 32 * PF_A_WARP0;
        uint8_t *a_ring = smem + PF_OFF_A, *raw = smem + PF_OFF_RAWA;
        BlockAt next = first_block(p, 0);
        int issued = 0, landed = 0;
        if (ta == 0 && total > 0) { issue_raw_a(&x_map, next, raw, &ctl->rawa_full); issued = 1; }
        for (int it = 0; it < total && !ctl->abort; ++it) {
            const int sa = it & 1, shift = 4 * (next.b & 3);
            next.advance(p);
            if (!PF_TIMED(1, wait_or_abort(&ctl->rawa_full, (uint32_t)(it & 1), ctl, p.status))) break;
            landed = it + 1;
            // the A slot was last read by the MMAs of block it - 2
            if (!PF_TIMED(0, wait_or_abort(&ctl->a_empty[sa], (uint32_t)((it >> 1) & 1) ^ 1u, ctl, p.status))) break;
            PF_MARK0();
            relayout_activations(raw, shift, a_ring + sa * PF_A_SLOT, smem + PF_OFF_XD + (it & (PF_XD_SLOTS - 1)) * PF_XD_SLOT, wa, ta, lane);
            PF_MARK(4);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) { mbar_arrive(&ctl->a_full[sa]); mbar_arrive(&ctl->rawa_empty); }
            PF_MARK(5);
            if (ta == 0 && it + 1 < total) {   // refill the raw slot once all three warps have read it
                if (!PF_TIMED(2, wait_one(&ctl->rawa_empty, (uint32_t)(it & 1), ctl, p.status))) break;
                fence_proxy_async();
                issue_raw_a(&x_map, next, raw, &ctl->rawa_full);
                issued = it + 2;
            }
        }
        if (ta == 0 && issued > landed) mbar_wait(&ctl->rawa_full, (uint32_t)(landed & 1));
    } else if (warp == PF_MMA_WARP) {
        // ------------------------------------------------------------------ MMA issue
        if (lane == 0) {
            const uint32_t idesc_q = tc::idesc_i8(PF_BM, 2 * PF_HALF, true, true);
            const uint32_t idesc_m = tc::idesc_f16_f32acc(PF_BM, PF_HALF);
            bool ok = true;
            for (int it = 0; it < total && ok && !ctl->abort; ++it) {
                const int sa = it & 1;
                if (!PF_TIMED(0, wait_one(&ctl->a_full[sa], (uint32_t)((it >> 1) & 1), ctl, p.status))) break;
                const uint32_t a_q = smem_addr(smem + PF_OFF_A + sa * PF_A_SLOT), a_m = a_q + PF_A_Q;
                for (int h = 0; h < 2; ++h) {
                    const int u = 2 * it + h;
                    const int sb = u % PF_B_SLOTS;
                    if (!PF_TIMED(1, wait_one(&ctl->b_full[sb], (uint32_t)((u / PF_B_SLOTS) & 1), ctl, p.status))) { ok = false; break; }
                    if (!PF_TIMED(2, wait_one(&ctl->tmem_empty[h], (uint32_t)(it & 1) ^ 1u, ctl, p.status))) { ok = false; break; }
                    tc::fence_after_sync();
                    PF_MARK0();
                    const uint32_t b_q = smem_addr(smem + PF_OFF_B + sb * PF_B_SLOT), b_m = b_q + PF_B_Q;
                    const uint32_t d = tmem + h * PF_HALF_COLS;
#pragma unroll
                    for (int j = 0; j < 8; ++j)   // K = 32 per instruction: 32 bytes further inside the swizzled row, next slab after 4
                        tc::mma_i8(d, tc::smem_desc_sw128(a_q + (j >> 2) * PF_A_SLAB + (j & 3) * 32),
                                   tc::smem_desc_sw128(b_q + (j >> 2) * PF_B_SLAB + (j & 3) * 32), idesc_q, j > 0);
                    tc::mma_f16(d + 2 * PF_HALF, tc::smem_desc(a_m, 128, 256), tc::smem_desc(b_m, 128, 256), idesc_m, 0);
                    tc::commit(&ctl->tmem_full[h]);   // this half's accumulators are complete
                    tc::commit(&ctl->b_empty[sb]);    // and its weight slot may be refilled
                    PF_MARK(4);
                }
                if (ok) tc::commit(&ctl->a_empty[sa]);
            }
        }
    } else if (warp < 8) {
        // ------------------------------------------------------------------ epilogue: warp = (64-weight half, 32-token quarter)
        const int quarter = warp & 3, h = warp >> 2;
        const int row = quarter * 32 + lane;   // token row of the tile = TMEM lane
        const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16) + h * PF_HALF_COLS;
        float acc[PF_HALF];
        int it = 0;
        bool ok = true;
        for (int t = 0; t < my_tiles && ok && !ctl->abort; ++t) {
            const int tile = (int)blockIdx.x + t * (int)gridDim.x;
            const long long n0 = (long long)(tile / p.m_tiles) * PF_BN + h * PF_HALF, m0 = (long long)(tile % p.m_tiles) * PF_BM;
#pragma unroll
            for (int i = 0; i < PF_HALF; ++i) acc[i] = 0.f;
            for (int b = 0; b < nb; ++b, ++it) {
                if (!PF_TIMED(0, wait_or_abort(&ctl->tmem_full[h], (uint32_t)(it & 1), ctl, p.status))) { ok = false; break; }
                tc::fence_after_sync();
                const float4 *wd = reinterpret_cast<const float4 *>(smem + PF_OFF_WD + ((2 * it + h) & (PF_WD_SLOTS - 1)) * PF_WD_SLOT);
                const float xd = reinterpret_cast<const float *>(smem + PF_OFF_XD + (it & (PF_XD_SLOTS - 1)) * PF_XD_SLOT)[row];
                PF_MARK0();
#pragma unroll
                for (int c = 0; c < PF_HALF / 8; ++c) {
                    uint32_t hi[8], lo[8], mt[8];
                    tc::tmem_ld8(lane_base + 8 * c, hi);
                    tc::tmem_ld8(lane_base + PF_HALF + 8 * c, lo);
                    tc::tmem_ld8(lane_base + 2 * PF_HALF + 8 * c, mt);
                    tc::tmem_ld_wait();
                    if (c == PF_HALF / 8 - 1) {   // last read of this half: hand its columns back to the MMA warp
                        tc::fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&ctl->tmem_empty[h]);
                    }
#pragma unroll
                    for (int i = 0; i < 8; i += 2) {
                        const float4 s2 = wd[(8 * c + i) >> 1];
                        const float v0 = limbs_to_float(hi[i], lo[i]), v1 = limbs_to_float(hi[i + 1], lo[i + 1]);
                        acc[8 * c + i] += xd * (s2.x * v0 - s2.y * __uint_as_float(mt[i]));
                        acc[8 * c + i + 1] += xd * (s2.z * v1 - s2.w * __uint_as_float(mt[i + 1]));
                    }
                }
                PF_MARK(4);
            }
            if (!ok) break;
            const long long m = m0 + row;
            if (m < p.m) {
                float *out = p.y + (size_t)m * p.ldy + n0;
                if (n0 + PF_HALF <= p.n && ((reinterpret_cast<uintptr_t>(out) & 15u) == 0)) {
#pragma unroll
                    for (int i = 0; i < PF_HALF; i += 4) *reinterpret_cast<float4 *>(out + i) = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
                } else {
#pragma unroll
                    for (int i = 0; i < PF_HALF; ++i)
                        if (n0 + i < p.n) out[i] = acc[i];
                }
            }
        }
    }

#ifdef WEFT_PF_PROFILE
    if (blockIdx.x == 0 && lane == 0) {
        prof[7] = clock64() - prof_begin;
        for (int i = 0; i < 8; ++i) g_pf_prof[warp][i] = (unsigned long long)prof[i];
    }
#endif
    tc::fence_before_sync();
    __syncthreads();
    if (warp == PF_MMA_WARP && tmem != 0xffffffffu) tc::tmem_free(tmem, PF_TMEM_COLS);
}

}  // namespace

bool prefill_supported(int fmt, long long n, long long k, long long m, const void *w, const void *xq) {
    static const bool disabled = getenv("WEFT_B200_NO_TENSOR_PREFILL") != nullptr;
    // K a multiple of 1024: Q8_K rows (292 bytes per 256) are then whole 16-byte multiples, which the TMA box loads need
    return !disabled && fmt == F_Q4_K && k > 0 && k % 1024 == 0 && n > 0 && m >= 32 &&
           (reinterpret_cast<uintptr_t>(w) & 15u) == 0 && (reinterpret_cast<uintptr_t>(xq) & 15u) == 0 &&
           n < (1LL << 31) && m < (1LL << 31);
}

cudaError_t launch_prefill(const PrefillArgs &a, int sm_count, cudaStream_t stream) {
    if (!prefill_supported(a.fmt, a.n, a.k, a.m, a.w, a.xq)) return cudaErrorNotSupported;
    PfParams p;
    p.w = static_cast<const uint8_t *>(a.w); p.xq = static_cast<const uint8_t *>(a.xq); p.y = a.y;
    p.n = a.n; p.m = a.m; p.ldy = a.ldy; p.nb = (int)(a.k / 256); p.status = a.status;
    p.m_tiles = (int)((a.m + PF_BM - 1) / PF_BM);
    p.n_tiles = (int)((a.n + PF_BN - 1) / PF_BN);
    const long long tiles = (long long)p.m_tiles * p.n_tiles;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(prefill_q4k_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    CUtensorMap x_map;
    cudaError_t e = encode_tile_map(&x_map, CU_TENSOR_MAP_DATA_TYPE_UINT32, a.xq, (unsigned long long)p.nb * 73, (unsigned long long)a.m,
                        (unsigned long long)p.nb * 292, PF_RAWA_WORDS, PF_BM);
    if (e != cudaSuccess) return e;
    const int grid = (int)(tiles < sm_count ? tiles : sm_count);
    prefill_q4k_kernel<<<grid, PF_THREADS, PF_SMEM, stream>>>(p, x_map);
    return cudaGetLastError();
}

#ifdef WEFT_PF_PROFILE
extern "C" int weft_b200_debug_prefill_profile(unsigned long long *out) {
    return (int)cudaMemcpyFromSymbol(out, g_pf_prof, sizeof(unsigned long long) * 128);
}
#endif

}  // namespace weft
