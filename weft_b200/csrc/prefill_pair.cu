// Prefill contractions for token batches above 128 on the int8 tensor cores with CTA PAIRS (tcgen05.mma
// cta_group::2): Q4_K x Q8_K -- the reference's production_mul_mat_q4_k_staged
// (examples/kernels/mul_mat/q4_k_staged.py:9-37; per block the math of examples/kernels/vec_dot/q4_k_q8_k.py:8-29,
// GGML ggml-cpu/quants.c:645-718) -- and TQ1_0 x Q8_K (production_mul_mat_tq1_0).  Same functions as prefill.cu and
// the same exact-integer formulation (see prefill.cu for the derivation): for Q4_K the 6-bit scale split as 8a + c and
// folded into two int8 weight limbs, the min term as one K = 16 MMA on exact small f16 integers.
//
// Tensor-core bound: 2*M*N*K useful integer ops; Q4_K issues twice that (two limbs).
//
// A pair of CTAs on the two SMs of a TPC owns a tile of 256 tokens x w weights (w picked per launch so that the last
// round of the grid is as full as possible).  Each CTA holds its 128 tokens (TMEM lanes, A operand) and expands HALF of
// the tile's weights: one MMA per K step covers all w weights, so every weight record is expanded once per 256 tokens
// and the activations of a block are read once.
//
// Both kernels read the activations from PLANES that a small kernel makes of the Q8_K records just before: the codes as
// an (M, K) int8 matrix, x.d as a (K/256, M) float matrix (and for Q4_K the min-term operand).  The records themselves
// start every block at a different offset from a 16-byte boundary; the planes make a block's codes 256 aligned bytes
// per token: two 128-byte-swizzled TMA boxes, eight K = 32 MMAs, expanded weights written as whole 16-byte chunks.
//
// Roles (warps): expanders (raw records from a TMA ring -> int8 operand rows), one activation-copy lane, one
// weight-copy lane, two MMA-issuing lanes of the even CTA taking the blocks in turn (the odd CTA's first one forwards
// the landing of its activation boxes), epilogue warps (tensor memory -> scaled fp32 accumulators in registers).  The
// roles trade registers in whole groups of four warps (setmaxnreg); a group can only take what other groups of the same
// CTA have given back, never registers the CTA did not get at launch.
// Every wait is bounded; a wait that runs out raises an abort flag in both CTAs, every role leaves its loop, copies
// in flight are waited for, tensor memory is freed, and the host sees a status code instead of a hang.  No copy,
// store or MMA touches another CTA's shared memory except the barrier arrivals inside the pair; nothing here reads or
// writes another GPU's memory.
#include "prefill_common.cuh"
#include "kernels.h"
#include "ring.cuh"

#include <cstddef>

namespace weft {

namespace {

constexpr int PP_TOKENS = 128;                 // tokens per CTA = TMEM lanes; a pair covers 256
constexpr int PP_RMAX = 80;                    // B rows per CTA at most
constexpr int PP_MMA_WARPS = 2;                // issuer q takes the blocks with it % 2 == q
constexpr int PP_RAW_HEADS = (PP_RMAX / 2) * 144;            // Q4_K raw slot: after the records, the 16-byte headers of the partner's weights
constexpr int PP_RAW_SLOT = PP_RAW_HEADS + (PP_RMAX / 2) * 16;  // 6400 B
constexpr int PP_WD_SLOT = 2 * (PP_RMAX / 2) * 8;            // Q4_K: {d, -dmin} per weight of both halves: 640 B

// ---- tensor memory of the Q4_K kernel: two buffers of 256 columns; limbs [0, 2w), min term [160, 160 + w) ----------
constexpr int PP_TMEM_COLS = 512;
constexpr int PP_BUF_COLS = 256;
constexpr int PP_MIN_COL = 2 * PP_RMAX;
constexpr uint32_t PP_BIAS = 0x4b400000u;      // bit pattern of 1.5 * 2^23 = 12582912.f

struct PairParams {
    float *y;              // (m, ldy)
    long long n, m, ldy;
    int nb;                // 256-blocks per row
    int m_tiles, n_tiles;  // tiles of 256 tokens, of w weights
    int w;                 // weights per tile
    const float *xd;       // (nb, xd_pitch): x.d of every token and block
    long long xd_pitch;
    int *status;
};

// Sleep between failed polls (ns): single lanes that wait for a copy or for tensor memory, and whole warps.  A waiting
// warp that polls without pause issues an instruction every few cycles; with these pauses the Q4_K kernel went from
// 134 to 124 us on 512 x 14336 x 4096 (the TQ1_0 kernel did not change; lengths between 50 and 300 ns measure the same).
constexpr uint32_t PP_LANE_NAP = 300, PP_WARP_NAP = 100;

// Bounded wait by one thread; gives up as soon as another role (of either CTA) has raised the abort flag.  The suspending
// form of the wait: a lane that spins on test_wait issues an instruction every few cycles and takes a third of its
// scheduler's issue slots from the warps that work.
template <class Control>
__device__ __forceinline__ bool pp_wait_one(uint64_t *bar, uint32_t parity, Control *ctl, uint32_t peer_abort, int *status) {
    for (uint32_t i = 0; i < (1u << 22); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 15u) == 15u && ctl->abort) return false;
        __nanosleep(PP_LANE_NAP);
    }
    ctl->abort = 1;
    tc::st_cluster_u32(peer_abort, 1u);
    report(status, ST_WAIT_TIMEOUT);
    return false;
}
// The same for a whole warp: every lane waits on the barrier itself with the suspending form (a waiting warp then
// takes no issue slots from the working ones; measured 214 -> 159 us per launch against one polling lane per warp).
template <class Control>
__device__ __forceinline__ bool pp_wait_warp(uint64_t *bar, uint32_t parity, Control *ctl, uint32_t peer_abort, int *status) {
    for (uint32_t i = 0; i < (1u << 22); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 7u) == 7u && ctl->abort) return false;
        __nanosleep(PP_WARP_NAP);
    }
    if ((threadIdx.x & 31) == 0) { ctl->abort = 1; tc::st_cluster_u32(peer_abort, 1u); report(status, ST_WAIT_TIMEOUT); }
    return false;
}

// For a role with slack: sleep between polls, leaving the issue slots to the roles that the kernel waits for
template <class Control>
__device__ __forceinline__ bool pp_wait_warp_relaxed(uint64_t *bar, uint32_t parity, Control *ctl, uint32_t peer_abort, int *status) {
    for (uint32_t i = 0; i < (1u << 22); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 7u) == 7u && ctl->abort) return false;
        __nanosleep(200);
    }
    if ((threadIdx.x & 31) == 0) { ctl->abort = 1; tc::st_cluster_u32(peer_abort, 1u); report(status, ST_WAIT_TIMEOUT); }
    return false;
}

// Blocks of the pair's work list: tiles round-robin over the pairs; inside a tile the blocks are taken as
// 0, 4, 8, ..., 1, 5, 9, ..., so that blocks with the same operand shift follow each other and the producers stay
// in one of their four code variants for a quarter of the tile.
// ================================================================================================================
// TQ1_0 x Q8_K on CTA pairs (production_mul_mat_tq1_0, examples/kernels/mul_mat/tq1_0.py; per block the math of
// examples/kernels/vec_dot/tq1_0_q8_k.py:9-55, GGML ggml-cpu/quants.c:430-480).  The weight operand is the base-3 digits
// minus one (one limb, no min term): a tile is 256 tokens x w weights with w up to 160 (each CTA expands w/2 weights into
// w/2 operand rows, N = w), an accumulator buffer is w <= 160 columns and THREE of them fit in tensor memory; the epilogue
// is acc += f32(isum) * (d * x.d) on one column per weight.
//
// Activations come from the planes of q8k_planes_kernel: the codes as an (M, K) int8 matrix in the operand order
// described at tq_operand_element(), x.d as an (K/256, M) float matrix.
//
// Per 256-block and CTA:
//   raw weights  two TMA box copies (w/2 records in 80-byte boxes; the 16-byte boxes with the partner's d) into a ring
//   activations  two TMA box copies (128 tokens x 128 bytes) into a ring of their own; the odd CTA's MMA warp forwards
//                the landing of its boxes to the even CTA's barrier
//   expanders    12 warps, four tasks per weight: bytes 0-15, 16-31, 32-47 of the record (16 table lookups, five operand
//                chunks each, in the operand order described at tq_operand_element) and the qh word with the two scales.  A warp is of one task kind; the lanes of a quarter
//                warp store their 16-byte chunks to eight different rows, whose swizzled positions never meet in a bank.
//                The digits come from a table in shared memory (entry v = the five digits of byte value v, built from the
//                caller's powers), sixteen copies so that the lookups of a half warp fall into different banks.
//   MMA          one lane of the even CTA (two issuers taking the blocks in turn): 8 int8 K = 32 steps, N = w
//   epilogue     16 warps = 4 lane quarters x 4 quarters of the tile's weights, up to 40 accumulators per thread; sixteen
//                columns per tensor-memory load, the next load in flight during the arithmetic; x.d by one global load per
//                thread and block, issued a block ahead
// 512 x 28672 x 8192: 214 us per step (321 us on the first pair kernel, which read the records as they lie; 582 us on the
// single-CTA kernel of prefill.cu).  With the expanders and the epilogue arithmetic switched off the kernel still takes
// 146 us: 0.9 us per block of hand-overs between the roles against 0.36 us of tensor work.
// Raw records: 54 bytes, rows of K/256 * 54 bytes (a multiple of 16 when K % 2048 == 0).  Record b of a row starts
// O = (54 b) % 16 bytes past a 16-byte boundary; an 80-byte box from that boundary holds it whole.  Its f16 d (bytes 52, 53)
// lies inside the 16-byte box at (54 b + 52) rounded down to 16: that box is fetched for the PARTNER's weights, so each
// CTA has the scales of all w weights without touching the partner's shared memory.  O takes eight values (b % 8); the
// blocks of a tile are taken as 0, 8, 16, ..., 1, 9, ... so that the expanders stay in one of their eight code variants.
constexpr int PT_E_WARPS = 16, PT_X_WARPS = 12;
constexpr int PT_X_GROUPS = 1;                                 // expander groups taking the blocks in turn (two measured the same as one)
constexpr int PT_X_WARP0 = PT_E_WARPS;
constexpr int PT_ATMA_WARP = PT_X_WARP0 + PT_X_WARPS, PT_WTMA_WARP = PT_ATMA_WARP + 1, PT_MMA_WARP = PT_WTMA_WARP + 1;
constexpr int PT_THREADS = 32 * (PT_MMA_WARP + PP_MMA_WARPS);   // 32 warps
constexpr int PT_A_STAGES = 3, PT_B_STAGES = 3, PT_RAW_SLOTS = 3, PT_RING = 8;
constexpr int PT_BUFS = 3, PT_BUF_COLS = 160;
// Registers: the kernel starts with 64 per thread (1024 threads); the roles then trade them in whole warp groups of four
// warps: the epilogue (warps 0-15) holds 40 accumulators and 16 columns in flight, the copy and MMA lanes need few.
// A group can only take what other groups of the same CTA have given back (registers the CTA never had stay out of reach:
// a kernel whose groups ask for more than the others release waits in setmaxnreg for ever).
constexpr int PT_LAUNCH_REGS = 64, PT_E_REGS = 88, PT_X_REGS = 40, PT_IO_REGS = 24;
static_assert(PT_E_WARPS * (PT_E_REGS - PT_LAUNCH_REGS) <= PT_X_WARPS * (PT_LAUNCH_REGS - PT_X_REGS) + 4 * (PT_LAUNCH_REGS - PT_IO_REGS) &&
              PT_E_WARPS % 4 == 0 && PT_X_WARPS % 4 == 0 && 32 * PT_LAUNCH_REGS * (PT_E_WARPS + PT_X_WARPS + 4) <= 65536,
              "register trade between the warp groups");
constexpr int PT_A_SLAB = 128 * 128, PT_A_SLOT = 2 * PT_A_SLAB;            // 32 KB
constexpr int PT_B_SLAB = PP_RMAX * 128, PT_B_SLOT = 2 * PT_B_SLAB;        // 20 KB
constexpr int PT_RAW_BOX = 80;                                  // bytes per record box
constexpr int PT_RAW_HEADS = PP_RMAX * PT_RAW_BOX;              // after the record boxes: the 16-byte boxes with the partner's d
constexpr int PT_RAW_SLOT = PT_RAW_HEADS + PP_RMAX * 16;        // 7680 B
constexpr int PT_WD_SLOT = 2 * PP_RMAX * 4;                     // d of the pair's 2 x 80 weights as floats
constexpr int PT_LUT_COPIES = 16;
constexpr int PT_OFF_A = 1024;
constexpr int PT_OFF_B = PT_OFF_A + PT_A_STAGES * PT_A_SLOT;
constexpr int PT_OFF_RAW = PT_OFF_B + PT_B_STAGES * PT_B_SLOT;
constexpr int PT_OFF_WD = PT_OFF_RAW + PT_RAW_SLOTS * PT_RAW_SLOT;
constexpr int PT_OFF_LUT = PT_OFF_WD + PT_RING * PT_WD_SLOT;
constexpr int PT_SMEM = PT_OFF_LUT + 256 * 8 * PT_LUT_COPIES;
static_assert(PT_SMEM <= 227 * 1024 && PT_RAW_SLOT % 128 == 0 && PT_B_SLAB % 1024 == 0 && PT_OFF_B % 1024 == 0 && PT_OFF_LUT % 128 == 0,
              "shared memory of the TQ1_0 kernel");
static_assert(PT_RING > PT_B_STAGES + PT_BUFS, "the expanders run at most B slots + accumulator buffers ahead of the epilogue");

struct TqControl {
    uint64_t a_full[PT_A_STAGES];        // this CTA's activation boxes (transaction bytes)
    uint64_t a_peer[PT_A_STAGES];        // EVEN CTA's copy is the live one: the odd CTA's boxes have landed
    uint64_t a_empty[PT_A_STAGES];       // both copies live: the MMAs that read the slot have completed
    uint64_t raw_full[PT_RAW_SLOTS];     // this CTA's raw records (transaction bytes)
    uint64_t raw_empty[PT_RAW_SLOTS];    // expander warps of this CTA are done reading the slot
    uint64_t b_full[PT_B_STAGES];        // EVEN CTA's copy is the live one: expander warps of both CTAs
    uint64_t b_empty[PT_B_STAGES];       // both copies live
    uint64_t tmem_full[PT_BUFS];         // both copies live: the buffer's accumulators are complete
    uint64_t tmem_empty[PT_BUFS];        // EVEN CTA's copy is the live one: epilogue warps of both CTAs
    uint32_t tmem_base;
    volatile int abort;
};
static_assert(sizeof(TqControl) <= PT_OFF_A, "control block");

// Blocks of the pair's work list: tiles round-robin over the pairs; inside a tile the blocks go 0, 8, 16, ..., 1, 9, ...
struct TqAt {
    int n0, m0;          // first weight and first token of the tile (both below 2^31)
    int b, tile, pairs;
    __device__ __forceinline__ void set_tile(const PairParams &p, int t) {
        tile = t;
        n0 = (t / p.m_tiles) * p.w;
        m0 = (t % p.m_tiles) * (2 * PP_TOKENS);
    }
    __device__ __forceinline__ void advance(const PairParams &p) {
        b += 8;
        if (b >= p.nb) {
            b = (b & 7) + 1;
            if (b == 8) { b = 0; set_tile(p, tile + pairs); }
        }
    }
};
__device__ __forceinline__ TqAt tq_first(const PairParams &p, int pair, int pairs) {
    TqAt at;
    at.b = 0;
    at.pairs = pairs;
    at.set_tile(p, pair);
    return at;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
// Table entry of byte i of a record word: {digits 0..3 minus one as int8, digit 4 minus one}.  `lut` already points at the
// lane's copy; the copies of a value's 8-byte entry lie side by side.
__device__ __forceinline__ void tq_lookup(uint32_t lut, uint32_t word, int i, uint32_t &x, uint32_t &y) {
    const uint32_t at = lut + prmt(word, 0u, 0x4440u + (uint32_t)i) * (8u * PT_LUT_COPIES);
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(x), "=r"(y) : "r"(at));
}
// The four record words that start O + 16 PART bytes into the row's box (O even, compile time): two aligned 16-byte loads
// (a quarter warp's rows are 80 bytes apart: eight different bank groups) and 16-bit funnel shifts.
template <int O>
__device__ __forceinline__ void tq_record_words(uint32_t src, uint32_t (&w)[4]) {
    const uint4 lo = lds128(src), hi = lds128(src + 16u);
    const uint32_t r[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
    constexpr int j = O >> 2;
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = (O & 2) ? __funnelshift_r(r[j + i], r[j + i + 1], 16) : r[j + i];
}
// Operand order inside a block.  A dot product does not care in which order its 256 terms are taken, as long as both
// operands use the same one, and the plane kernel writes the activation codes in any order for free.  So the weights
// are laid out the way the table delivers them, without transposing digits: with x(j) = digits 0..3 of record byte j
// (one table word) and y(j) = its digit 4,
//   chunks 5 p + s (p = 0..2, s = 0..3):  x(16 p + 4 s), x(16 p + 4 s + 1), x(16 p + 4 s + 2), x(16 p + 4 s + 3)
//   chunk  5 p + 4:                        y(16 p), y(16 p + 1), ..., y(16 p + 15)
//   chunk  15:                             x(48), x(49), x(50), x(51)      (the qh bytes: four digits each)
// tq_operand_element() gives the block element (the reference's order) that sits at operand position k.
__host__ __device__ constexpr int tq_element_of(int j, int n) {   // digit n of record byte j (qs 0..47, qh 48..51)
    return j < 32 ? 32 * n + j : j < 48 ? 160 + 16 * n + (j - 32) : 240 + 4 * n + (j - 48);
}
__host__ __device__ constexpr int tq_operand_element(int k) {
    if (k >= 240) return tq_element_of(48 + (k - 240) / 4, (k - 240) % 4);
    const int p = k / 80, r = k % 80;
    return r < 64 ? tq_element_of(16 * p + r / 4, r % 4) : tq_element_of(16 * p + (r - 64), 4);
}
constexpr bool tq_operand_order_is_a_permutation() {
    for (int k = 0; k < 256; ++k) {
        const int e = tq_operand_element(k);
        if (e < 0 || e > 255) return false;
        for (int other = 0; other < k; ++other)
            if (tq_operand_element(other) == e) return false;
    }
    return true;
}
static_assert(tq_operand_order_is_a_permutation(), "every element of a block sits at exactly one operand position");
// Heavy task: record bytes 16 PART .. 16 PART + 15 -> operand chunks 5 PART .. 5 PART + 4
template <int PART, int O>
__device__ __forceinline__ void tq_expand_heavy(uint32_t box, uint32_t lut, uint32_t b_slot, int row) {
    uint32_t w[4];
    tq_record_words<O>(box + 16u * (uint32_t)PART, w);
    const uint32_t base = b_slot + (uint32_t)(row >> 3) * 1024u + (uint32_t)(row & 7) * 128u;
    const uint32_t x7 = (uint32_t)(row & 7) << 4;
    uint32_t last[4];
#pragma unroll
    for (int s = 0; s < 4; ++s) {
        uint32_t x[4], y[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) tq_lookup(lut, w[s], i, x[i], y[i]);
        constexpr int first = 5 * PART;
        const int chunk = first + s;
        sts_u128(base + (uint32_t)(chunk >> 3) * PT_B_SLAB + (((uint32_t)(chunk & 7) << 4) ^ x7), x[0], x[1], x[2], x[3]);
        last[s] = prmt(prmt(y[0], y[1], 0x0040u), prmt(y[2], y[3], 0x0040u), 0x5410u);
    }
    constexpr int chunk4 = 5 * PART + 4;
    sts_u128(base + (uint32_t)(chunk4 >> 3) * PT_B_SLAB + (((uint32_t)(chunk4 & 7) << 4) ^ x7), last[0], last[1], last[2], last[3]);
}
// Light task: the qh word (record bytes 48..51, operand chunk 15) and the two scales for the epilogue: this weight's d
// (record bytes 52, 53) and the d of the partner's weight of the same index.
template <int O>
__device__ __forceinline__ void tq_expand_light(uint32_t box, uint32_t head, uint32_t lut, uint32_t b_slot, uint32_t wd_mine, uint32_t wd_partner, int row) {
    constexpr int at_qh = O + 48, at_d = O + 52, at_pd = (O + 52) & 15;
    const uint32_t q0 = lds_u32(box + (uint32_t)(at_qh & ~3)), q1 = lds_u32(box + (uint32_t)(at_qh & ~3) + 4u);
    const uint32_t qh = (at_qh & 2) ? __funnelshift_r(q0, q1, 16) : q0;
    const uint32_t d_mine = (at_d & 2) ? q1 >> 16 : q1;     // bytes O + 52, 53: the half word after qh
    const uint32_t d_partner = lds_u32(head + (uint32_t)(at_pd & ~3)) >> (8 * (at_pd & 2));
    uint32_t x[4], y[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) tq_lookup(lut, qh, i, x[i], y[i]);
    const uint32_t base = b_slot + (uint32_t)(row >> 3) * 1024u + (uint32_t)(row & 7) * 128u;
    const uint32_t x7 = (uint32_t)(row & 7) << 4;
    sts_u128(base + PT_B_SLAB + ((7u << 4) ^ x7), x[0], x[1], x[2], x[3]);
    sts_u32(wd_mine + 4u * (uint32_t)row, __float_as_uint(half_bits_to_float(d_mine & 0xffffu)));
    sts_u32(wd_partner + 4u * (uint32_t)row, __float_as_uint(half_bits_to_float(d_partner & 0xffffu)));
}
// The jobs of one warp for one block: job j = first_job + k * (12 / PT_X_GROUPS) is task kind j / 3 on rows 32 (j % 3) + lane
template <int O>
__device__ __forceinline__ void tq_expand_jobs(int first_job, int lane, int R, uint32_t raw_slot, uint32_t lut, uint32_t b_slot, uint32_t wd_mine, uint32_t wd_partner) {
#pragma unroll 1
    for (int job = first_job; job < PT_X_WARPS; job += PT_X_WARPS / PT_X_GROUPS) {
        const int part = job / 3, row = 32 * (job - 3 * part) + lane;
        if (row < R) {
            const uint32_t box = raw_slot + (uint32_t)row * PT_RAW_BOX, head = raw_slot + PT_RAW_HEADS + (uint32_t)row * 16u;
            if (part == 0) tq_expand_heavy<0, O>(box, lut, b_slot, row);
            else if (part == 1) tq_expand_heavy<1, O>(box, lut, b_slot, row);
            else if (part == 2) tq_expand_heavy<2, O>(box, lut, b_slot, row);
            else tq_expand_light<O>(box, head, lut, b_slot, wd_mine, wd_partner, row);
        }
    }
}

// Epilogue pieces.  Columns [g, g + 16) of the warp's accumulators (eight when the warp has only eight left) into v.
__device__ __forceinline__ void tq_load_columns(uint32_t from, int g, int cols, uint32_t (&v)[16]) {
    if (g + 16 <= cols) tc::tmem_ld16(from + (uint32_t)g, v);
    else {
        uint32_t v8[8];
        tc::tmem_ld8(from + (uint32_t)g, v8);
#pragma unroll
        for (int k = 0; k < 8; ++k) { v[k] = v8[k]; v[8 + k] = 0u; }
    }
}
__device__ __forceinline__ void tq_release(uint32_t empty_bar, int lane) {
    tc::fence_before_sync();
    __syncwarp();
    if (lane == 0) tc::mbar_arrive_cluster(empty_bar);
}
// Two accumulator integers as a packed pair of floats, exactly (|v| < 2^22): v + bits(1.5 * 2^23) is the float
// 1.5 * 2^23 + v; the halves are written straight into the 64-bit register that the packed subtraction reads.
__device__ __forceinline__ uint64_t tq_ints_to_float2(uint32_t a, uint32_t b) {
    uint64_t biased;
    asm("{\n\t.reg .b32 lo, hi;\n\tadd.u32 lo, %1, 0x4b400000;\n\tadd.u32 hi, %2, 0x4b400000;\n\tmov.b64 %0, {lo, hi};\n\t}" : "=l"(biased) : "r"(a), "r"(b));
    return add2(biased, pack2(-12582912.f, -12582912.f));
}
// acc += f32(isum) * (d * x.d) for columns [G, G + 16) (or [G, G + 8)); wd: the weights' d as floats in shared memory,
// read as 64-bit pairs so that no move stands between the load and the packed multiply
template <int G>
__device__ __forceinline__ void tq_scale_add(uint64_t (&acc)[PP_RMAX / 4], const uint32_t (&v)[16], int cols, uint32_t wd, uint64_t xd2) {
    const bool wide = G + 16 <= cols;
#pragma unroll
    for (int k = 0; k < 16; k += 4) {
        if (G + k < PP_RMAX / 2 && (wide || k < 8)) {
            uint64_t s01, s23;
            asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(s01), "=l"(s23) : "r"(wd + 4u * (uint32_t)(G + k)));
            acc[(G + k) >> 1] = fma2(tq_ints_to_float2(v[k], v[k + 1]), mul2(s01, xd2), acc[(G + k) >> 1]);
            acc[((G + k) >> 1) + 1] = fma2(tq_ints_to_float2(v[k + 2], v[k + 3]), mul2(s23, xd2), acc[((G + k) >> 1) + 1]);
        }
    }
}

// Q8_K records -> planes: codes (m, k) int8, every block in the operand order of tq_operand_element(), and x.d
// (k / 256, pitch) float.  A CTA takes sixteen records: their codes go through shared memory, one thread per 16 output bytes.
__global__ void __launch_bounds__(256) q8k_planes_kernel(const uint8_t *__restrict__ xq, int8_t *__restrict__ codes, float *__restrict__ xd, long long m, int nb, long long pitch) {
    __shared__ __align__(16) uint8_t s_codes[16][256 + 16];   // + 16: the records of a CTA start in different banks
    const int r = threadIdx.x >> 4, c = threadIdx.x & 15;
    const long long record = (long long)blockIdx.x * 16 + r;
    const bool live = record < m * nb;
    if (live) {
        const uint32_t *src = reinterpret_cast<const uint32_t *>(xq + record * 292);   // records are 4-byte aligned
        *reinterpret_cast<uint4 *>(&s_codes[r][16 * c]) = make_uint4(src[1 + 4 * c], src[2 + 4 * c], src[3 + 4 * c], src[4 + 4 * c]);
        if (c == 0) {
            const long long t = record / nb;
            xd[(record - t * nb) * pitch + t] = __uint_as_float(src[0]);
        }
    }
    __syncthreads();
    if (!live) return;
    uint32_t out[4];
#pragma unroll
    for (int wd = 0; wd < 4; ++wd) {
        uint32_t v = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            // the element at operand position 16 c + 4 wd + i (tq_operand_element, spelled with run-time c)
            int e;
            if (c == 15) e = 240 + 4 * i + wd;                        // x(48 + wd): digit i -> element 240 + 4 i + wd
            else {
                const int p = c / 5, s = c - 5 * p;
                if (s < 4) { const int j = 16 * p + 4 * s + wd; e = p < 2 ? 32 * i + j : 160 + 16 * i + (j - 32); }
                else { const int j = 16 * p + 4 * wd + i; e = p < 2 ? 128 + j : 224 + (j - 32); }
            }
            v |= (uint32_t)s_codes[r][e] << (8 * i);
        }
        out[wd] = v;
    }
    *reinterpret_cast<uint4 *>(codes + record * 256 + 16 * c) = make_uint4(out[0], out[1], out[2], out[3]);
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PT_THREADS, 1)
prefill_pair_tq1_kernel(const PairParams p, const uint32_t *powers, const __grid_constant__ CUtensorMap x_codes,
                        const __grid_constant__ CUtensorMap w_rows, const __grid_constant__ CUtensorMap w_heads) {
    extern __shared__ __align__(1024) uint8_t smem[];
    TqControl *ctl = reinterpret_cast<TqControl *>(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = tc::cluster_ctarank();
    const int pair = (int)blockIdx.x >> 1, pairs = (int)gridDim.x >> 1;
    const int tiles = p.m_tiles * p.n_tiles;
    const int nb = p.nb;
    const int my_tiles = (tiles - pair + pairs - 1) / pairs;
    const int total = my_tiles * nb;
    const int R = p.w >> 1;                                // weights this CTA expands per block = its B rows

    const uint32_t ctl_addr = smem_addr(ctl);
    const uint32_t ctl_even = tc::map_to_cta(ctl_addr, 0), ctl_peer = tc::map_to_cta(ctl_addr, rank ^ 1u);
    const uint32_t peer_abort = ctl_peer + (uint32_t)offsetof(TqControl, abort);

    if (threadIdx.x == 0) {
        for (int s = 0; s < PT_A_STAGES; ++s) { mbar_init(&ctl->a_full[s], 1); mbar_init(&ctl->a_peer[s], 1); mbar_init(&ctl->a_empty[s], 1); }
        for (int s = 0; s < PT_RAW_SLOTS; ++s) { mbar_init(&ctl->raw_full[s], 1); mbar_init(&ctl->raw_empty[s], PT_X_WARPS / PT_X_GROUPS); }
        for (int s = 0; s < PT_B_STAGES; ++s) { mbar_init(&ctl->b_full[s], 2 * PT_X_WARPS / PT_X_GROUPS); mbar_init(&ctl->b_empty[s], 1); }
        for (int h = 0; h < PT_BUFS; ++h) { mbar_init(&ctl->tmem_full[h], 1); mbar_init(&ctl->tmem_empty[h], 2 * PT_E_WARPS); }
        ctl->abort = 0;
        ctl->tmem_base = 0xffffffffu;
        mbar_fence_init();
    }
    // the digit table, from the caller's powers: entry v = digits 0..4 of byte value v minus one, as int8
    for (int v = threadIdx.x; v < 256; v += PT_THREADS) {
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int n = 0; n < 5; ++n) {
            const uint32_t q = ((uint32_t)v * (__ldg(powers + n) & 0xffu)) & 0xffu;
            const uint32_t digit_minus_one = (((q * 3u) >> 8) + 0xffu) & 0xffu;
            if (n < 4) lo |= digit_minus_one << (8 * n); else hi = digit_minus_one;
        }
#pragma unroll
        for (int c = 0; c < PT_LUT_COPIES; ++c) reinterpret_cast<uint2 *>(smem + PT_OFF_LUT)[v * PT_LUT_COPIES + c] = make_uint2(lo, hi);
    }
    __syncthreads();
    // Each CTA allocates its own tensor memory (cta_group::1: no pair-wide allocation protocol); the pair's MMAs then use
    // the same columns in both.
    if (warp == PT_MMA_WARP) tc::tmem_alloc(&ctl->tmem_base, PP_TMEM_COLS);
    tc::fence_before_sync();
    __syncthreads();
    tc::cluster_sync_all();
    tc::fence_after_sync();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t *>(&ctl->tmem_base);
    const bool tmem_ok = tmem == 0u;
    if (!tmem_ok && threadIdx.x == 0) { ctl->abort = 1; tc::st_cluster_u32(peer_abort, 1u); report(p.status, 0x40000000 | (int)(tmem & 0xffffu) | (int)((tmem >> 16) & 0x3fffu) << 16); }
    if (!tmem_ok) {
        // nothing: fall through to the common exit
    } else if (warp >= PT_X_WARP0 && warp < PT_X_WARP0 + PT_X_WARPS) {
        // ------------------------------------------------------------------ expanders: three warps per task kind
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(PT_X_REGS));
        // The twelve warps form PT_X_GROUPS groups that take the blocks in turn; a warp of a group does PT_X_GROUPS of the
        // twelve jobs (job j: task kind j / 3, rows 32 (j % 3) ..) of its block one after the other.  What a block costs an
        // expander is mostly waiting (the records' way through shared memory, the fence before the hand-over), so two
        // blocks in flight nearly double what the expanders deliver.
        const int xw = warp - PT_X_WARP0;
        const int group = xw % PT_X_GROUPS, first_job = xw / PT_X_GROUPS;
        const uint32_t lut = smem_addr(smem + PT_OFF_LUT) + 8u * (uint32_t)(lane & (PT_LUT_COPIES - 1));
        TqAt at = tq_first(p, pair, pairs);
        for (int k = 0; k < group; ++k) at.advance(p);
        const uint32_t full_even = ctl_even + (uint32_t)offsetof(TqControl, b_full);
        for (int it = group; it < total && !ctl->abort; it += PT_X_GROUPS) {
            const int b = at.b;
#pragma unroll
            for (int k = 0; k < PT_X_GROUPS; ++k) at.advance(p);
            const int s = it % PT_B_STAGES, rs = it % PT_RAW_SLOTS;
            if (!pp_wait_warp(&ctl->raw_full[rs], (uint32_t)(it / PT_RAW_SLOTS) & 1u, ctl, peer_abort, p.status)) break;
            if (!pp_wait_warp(&ctl->b_empty[s], ((uint32_t)(it / PT_B_STAGES) & 1u) ^ 1u, ctl, peer_abort, p.status)) break;
            {
                const uint32_t raw_slot = smem_addr(smem + PT_OFF_RAW + rs * PT_RAW_SLOT);
                const uint32_t b_slot = smem_addr(smem + PT_OFF_B + s * PT_B_SLOT);
                const uint32_t wd_slot = smem_addr(smem + PT_OFF_WD + (it & (PT_RING - 1)) * PT_WD_SLOT);
                const uint32_t wd_mine = wd_slot + rank * (uint32_t)(PT_WD_SLOT / 2), wd_partner = wd_slot + (rank ^ 1u) * (uint32_t)(PT_WD_SLOT / 2);
                switch (b & 7) {   // O = (54 b) % 16
                case 0: tq_expand_jobs<0>(first_job, lane, R, raw_slot, lut, b_slot, wd_mine, wd_partner); break;
                case 1: tq_expand_jobs<6>(first_job, lane, R, raw_slot, lut, b_slot, wd_mine, wd_partner); break;
                case 2: tq_expand_jobs<12>(first_job, lane, R, raw_slot, lut, b_slot, wd_mine, wd_partner); break;
                case 3: tq_expand_jobs<2>(first_job, lane, R, raw_slot, lut, b_slot, wd_mine, wd_partner); break;
                case 4: tq_expand_jobs<8>(first_job, lane, R, raw_slot, lut, b_slot, wd_mine, wd_partner); break;
                case 5: tq_expand_jobs<14>(first_job, lane, R, raw_slot, lut, b_slot, wd_mine, wd_partner); break;
                case 6: tq_expand_jobs<4>(first_job, lane, R, raw_slot, lut, b_slot, wd_mine, wd_partner); break;
                default: tq_expand_jobs<10>(first_job, lane, R, raw_slot, lut, b_slot, wd_mine, wd_partner); break;
                }
            }
            fence_proxy_async();      // generic-proxy stores must be visible to the tensor core's reads
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&ctl->raw_empty[rs]);
                tc::mbar_arrive_cluster(full_even + 8u * (uint32_t)s);
            }
        }
    } else if (warp == PT_ATMA_WARP) {
        // ------------------------------------------------------------------ activation copies (this CTA's 128 tokens)
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(PT_IO_REGS));
        if (lane == 0) {
            TqAt at = tq_first(p, pair, pairs);
            int issued = 0;
            for (int it = 0; it < total && !ctl->abort; ++it, at.advance(p)) {
                const int s = it % PT_A_STAGES;
                if (!pp_wait_one(&ctl->a_empty[s], ((uint32_t)(it / PT_A_STAGES) & 1u) ^ 1u, ctl, peer_abort, p.status)) break;
                uint8_t *slot = smem + PT_OFF_A + s * PT_A_SLOT;
                mbar_expect_tx(&ctl->a_full[s], PT_A_SLOT);
                // tokens past M read as zero
                tma_load_2d(slot, &x_codes, 256 * at.b, at.m0 + (int)rank * PP_TOKENS, &ctl->a_full[s]);
                tma_load_2d(slot + PT_A_SLAB, &x_codes, 256 * at.b + 128, (int)at.m0 + (int)rank * PP_TOKENS, &ctl->a_full[s]);
                issued = it + 1;
            }
            // left early: let the copies in flight land (a phase that has completed already returns at once)
            for (int k = issued > PT_A_STAGES ? issued - PT_A_STAGES : 0; k < issued; ++k) mbar_wait(&ctl->a_full[k % PT_A_STAGES], (uint32_t)(k / PT_A_STAGES) & 1u);
            // The even CTA's commits arrive on this CTA's barriers when the MMAs complete, whoever still waits for them:
            // stay until the last ones have landed, so that none can reach a CTA that has already left the SM.
            for (int k = total > PT_A_STAGES ? total - PT_A_STAGES : 0; k < total && !ctl->abort; ++k)
                if (!pp_wait_one(&ctl->a_empty[k % PT_A_STAGES], (uint32_t)(k / PT_A_STAGES) & 1u, ctl, peer_abort, p.status)) break;
        }
    } else if (warp == PT_WTMA_WARP) {
        // ------------------------------------------------------------------ raw weight records: this CTA's boxes and the partner's d boxes
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(PT_IO_REGS));
        if (lane == 0) {
            TqAt at = tq_first(p, pair, pairs);
            int issued = 0;
            const uint32_t bytes = (uint32_t)R * (PT_RAW_BOX + 16u);
            for (int it = 0; it < total && !ctl->abort; ++it, at.advance(p)) {
                const int rs = it % PT_RAW_SLOTS;
                if (!pp_wait_one(&ctl->raw_empty[rs], ((uint32_t)(it / PT_RAW_SLOTS) & 1u) ^ 1u, ctl, peer_abort, p.status)) break;
                mbar_expect_tx(&ctl->raw_full[rs], bytes);
                // rows past N and bytes past the end of a row read as zero (digits -1 times d = 0: never stored)
                tma_load_2d(smem + PT_OFF_RAW + rs * PT_RAW_SLOT, &w_rows, (54 * at.b) & ~15, (int)at.n0 + (int)rank * R, &ctl->raw_full[rs]);
                tma_load_2d(smem + PT_OFF_RAW + rs * PT_RAW_SLOT + PT_RAW_HEADS, &w_heads, (54 * at.b + 52) & ~15, (int)at.n0 + (int)(rank ^ 1u) * R, &ctl->raw_full[rs]);
                issued = it + 1;
            }
            for (int k = issued > PT_RAW_SLOTS ? issued - PT_RAW_SLOTS : 0; k < issued; ++k) mbar_wait(&ctl->raw_full[k % PT_RAW_SLOTS], (uint32_t)(k / PT_RAW_SLOTS) & 1u);
            // the last commits on this CTA's b_empty barriers (see the activation warp)
            for (int k = total > PT_B_STAGES ? total - PT_B_STAGES : 0; k < total && !ctl->abort; ++k)
                if (!pp_wait_one(&ctl->b_empty[k % PT_B_STAGES], (uint32_t)(k / PT_B_STAGES) & 1u, ctl, peer_abort, p.status)) break;
        }
    } else if (warp >= PT_MMA_WARP) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(PT_IO_REGS));
        const int q = warp - PT_MMA_WARP;
        if (lane == 0 && rank == 0) {
            // -------------------------------------------------------------- MMA issue (even CTA), two issuers taking the blocks in turn
            const uint32_t idesc_q = tc::idesc_i8(2 * PP_TOKENS, 2 * R, true, true);
            for (int it = q; it < total && !ctl->abort; it += PP_MMA_WARPS) {
                const int sa = it % PT_A_STAGES, sb = it % PT_B_STAGES, buf = it % PT_BUFS;
                if (!pp_wait_one(&ctl->a_full[sa], (uint32_t)(it / PT_A_STAGES) & 1u, ctl, peer_abort, p.status)) break;
                if (!pp_wait_one(&ctl->a_peer[sa], (uint32_t)(it / PT_A_STAGES) & 1u, ctl, peer_abort, p.status)) break;
                if (!pp_wait_one(&ctl->b_full[sb], (uint32_t)(it / PT_B_STAGES) & 1u, ctl, peer_abort, p.status)) break;
                if (!pp_wait_one(&ctl->tmem_empty[buf], (uint32_t)(it / PT_BUFS) & 1u, ctl, peer_abort, p.status)) break;
                tc::fence_after_sync();
                const uint32_t d = tmem + (uint32_t)buf * PT_BUF_COLS;
                const uint64_t a0 = tc::smem_desc_sw128(smem_addr(smem + PT_OFF_A + sa * PT_A_SLOT)), b0 = tc::smem_desc_sw128(smem_addr(smem + PT_OFF_B + sb * PT_B_SLOT));
#pragma unroll
                for (int k = 0; k < 8; ++k)   // the first instruction of a block overwrites the accumulators
                    tc::mma_i8_pair(d, a0 + (uint64_t)(((k >> 2) * PT_A_SLAB + (k & 3) * 32) >> 4), b0 + (uint64_t)(((k >> 2) * PT_B_SLAB + (k & 3) * 32) >> 4), idesc_q, k > 0 ? 1u : 0u);
                tc::commit_pair(smem_addr(&ctl->tmem_full[buf]));
                tc::commit_pair(ctl_peer + (uint32_t)offsetof(TqControl, tmem_full) + 8u * (uint32_t)buf);
                tc::commit_pair(smem_addr(&ctl->a_empty[sa]));
                tc::commit_pair(ctl_peer + (uint32_t)offsetof(TqControl, a_empty) + 8u * (uint32_t)sa);
                tc::commit_pair(smem_addr(&ctl->b_empty[sb]));
                tc::commit_pair(ctl_peer + (uint32_t)offsetof(TqControl, b_empty) + 8u * (uint32_t)sb);
            }
            // the epilogues of both CTAs arrive once more after the last use of every buffer: receive those arrivals
            // before this CTA may leave (issuer 0 waits for all three buffers)
            if (q == 0 && !ctl->abort)
                for (int buf = 0; buf < PT_BUFS && buf < total; ++buf) {
                    const int uses = (total - buf + PT_BUFS - 1) / PT_BUFS;
                    if (!pp_wait_one(&ctl->tmem_empty[buf], (uint32_t)uses & 1u, ctl, peer_abort, p.status)) break;
                }
        } else if (lane == 0 && rank == 1 && q == 0) {
            // -------------------------------------------------------------- odd CTA: tell the even CTA that this CTA's activations have landed
            const uint32_t peer_even = ctl_even + (uint32_t)offsetof(TqControl, a_peer);
            for (int it = 0; it < total && !ctl->abort; ++it) {
                const int sa = it % PT_A_STAGES;
                if (!pp_wait_one(&ctl->a_full[sa], (uint32_t)(it / PT_A_STAGES) & 1u, ctl, peer_abort, p.status)) break;
                tc::mbar_arrive_cluster(peer_even + 8u * (uint32_t)sa);
            }
        }
    } else if (warp < PT_E_WARPS) {
        // ------------------------------------------------------------------ epilogue: warp = (32-token quarter, quarter of the tile's weights)
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(PT_E_REGS));
        const int quarter = warp & 3, grp = warp >> 2;       // grp = 2 (CTA whose weights these are) + (half of that CTA's weights)
        const int half = grp >> 1, sub = grp & 1;
        const int row = quarter * 32 + lane;                 // token row of this CTA = TMEM lane
        const int cols = R >> 1;                             // this warp's weights: 8, 16, 24, 32 or 40
        const int col0 = half * R + sub * cols;
        const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)col0;
        const uint32_t empty_even = ctl_even + (uint32_t)offsetof(TqControl, tmem_empty);
        __syncwarp();
        if (lane == 0)
            for (int buf = 0; buf < PT_BUFS; ++buf) tc::mbar_arrive_cluster(empty_even + 8u * (uint32_t)buf);   // all buffers start free
        uint64_t acc[PP_RMAX / 4];   // packed pairs of fp32: up to 40 weights
        TqAt at = tq_first(p, pair, pairs);
        int it = 0;
        bool ok = true;
        int m = at.m0 + (int)rank * PP_TOKENS + row;
        float xd_next = m < p.m ? __ldg(p.xd + (long long)at.b * p.xd_pitch + m) : 0.f;
        for (int t = 0; t < my_tiles && ok && !ctl->abort; ++t) {
            const int n0 = at.n0 + col0;
            m = at.m0 + (int)rank * PP_TOKENS + row;
#pragma unroll
            for (int k = 0; k < PP_RMAX / 4; ++k) acc[k] = 0ull;
            for (int blk = 0; blk < nb && ok; ++blk, ++it) {
                const int buf = it % PT_BUFS;
                const float xd = xd_next;
                at.advance(p);
                if (it + 1 < total) {   // x.d of the next block (of the next tile's tokens after the last block of a tile)
                    const int mn = at.m0 + (int)rank * PP_TOKENS + row;
                    xd_next = mn < p.m ? __ldg(p.xd + (long long)at.b * p.xd_pitch + mn) : 0.f;
                }
                if (!pp_wait_warp(&ctl->tmem_full[buf], (uint32_t)(it / PT_BUFS) & 1u, ctl, peer_abort, p.status)) { ok = false; break; }
                tc::fence_after_sync();
                const uint32_t wd = smem_addr(smem + PT_OFF_WD + (it & (PT_RING - 1)) * PT_WD_SLOT) + (uint32_t)half * (PT_WD_SLOT / 2) + 4u * (uint32_t)(sub * cols);
                const uint64_t xd2 = pack2(xd, xd);
                const uint32_t from = lane_base + (uint32_t)(buf * PT_BUF_COLS);
                // read-out: the first 32 columns by two loads in flight together, the last eight during the arithmetic
                uint32_t va[16], vb[16];
                tq_load_columns(from, 0, cols, va);
                if (cols > 16) tq_load_columns(from, 16, cols, vb);
                tc::tmem_ld_wait();
                if (cols <= 32) tq_release(empty_even + 8u * (uint32_t)buf, lane);   // everything is read: the buffer goes back before the arithmetic
                tq_scale_add<0>(acc, va, cols, wd, xd2);
                if (cols > 32) tq_load_columns(from, 32, cols, va);
                if (cols > 16) tq_scale_add<16>(acc, vb, cols, wd, xd2);
                if (cols > 32) {
                    tc::tmem_ld_wait();
                    tq_release(empty_even + 8u * (uint32_t)buf, lane);
                    tq_scale_add<32>(acc, va, cols, wd, xd2);
                }
            }
            if (!ok) break;
            if (m < p.m) {
                float *out = p.y + (size_t)m * p.ldy + n0;
                const bool vec = (reinterpret_cast<uintptr_t>(out) & 15u) == 0;
#pragma unroll
                for (int k = 0; k < PP_RMAX / 2; k += 4) {
                    if (k < cols) {
                        if (vec && n0 + k + 4 <= p.n) {
                            *reinterpret_cast<ulonglong2 *>(out + k) = make_ulonglong2(acc[k >> 1], acc[(k >> 1) + 1]);
                        } else {
                            float a0, a1, a2, a3;
                            unpack2(acc[k >> 1], a0, a1);
                            unpack2(acc[(k >> 1) + 1], a2, a3);
                            if (n0 + k < p.n) out[k] = a0;
                            if (n0 + k + 1 < p.n) out[k + 1] = a1;
                            if (n0 + k + 2 < p.n) out[k + 2] = a2;
                            if (n0 + k + 3 < p.n) out[k + 3] = a3;
                        }
                    }
                }
            }
        }
    }

    tc::fence_before_sync();
    __syncthreads();
    tc::cluster_sync_all();
    if (warp == PT_MMA_WARP) {
        __syncwarp();
        if (tmem_ok) tc::tmem_free(tmem, PP_TMEM_COLS);
    }
}

// ================================================================================================================
// Q4_K x Q8_K on CTA pairs.  A tile is 256 tokens x w weights, w = 16..80 in steps of 16.  `q8k_planes_q4k_kernel`
// turns the Q8_K records into the codes as an (M, K) int8 matrix, x.d as a (K/256, M) float matrix and, per token and
// block, the min-term operand {l_0..l_7 | h_0..h_7} as sixteen f16 (bsum pair sums split as 64 h + l: those bytes arrive by
// TMA ready for the K = 16 f16 MMA).  Per 256-block and CTA:
//   raw weights  one TMA box copy of w/2 records (144 B each) and one of the partner's 16-byte headers into a 4-slot ring
//   activations  two 128-byte-swizzled boxes of codes and two 16-byte columns of the min-term operand into a 3-slot ring
//   expanders    two groups of 5 warps taking the blocks in turn, four lanes per weight (lane = one pair of sub-blocks):
//                nibbles -> two scaled limbs (8a + c), written as the K-major 128-byte-swizzled operand; lane layout chosen
//                so that the 16-byte stores of a quarter-warp never meet in a bank; the f16 rows {mn | 64 mn} of the min term
//   MMA          8 int8 K steps (N = 2w) + 1 f16 K = 16 step (N = w), into one of two TMEM buffers of 256 columns
//   epilogue     8 warps = 4 lane quarters x the two halves of the tile's weights; per element
//                acc += x.d * (d * f32(8 hi + lo) - dmin * msum) in the reference's op order.  The int32 accumulators start
//                at the bit pattern of 1.5 * 2^23 instead of zero (the epilogue writes it back after every read), so what
//                comes out of TMEM is already the float 1.5 * 2^23 + limb: one packed subtraction converts two limbs.
//                x.d comes by one global load per thread and block, issued a block ahead.
// Measured on 512 x 14336 x 4096: 106 us (the kernel that read the Q8_K records as they lie, with the weight operand shifted
// to meet them, three narrow activation columns and two per-token warps: 117.5 us; a single-CTA kernel: 191 us).
// 24 warps at 80 registers; the epilogue takes 96, the copy and MMA lanes keep 24.
constexpr int PQ_E_WARPS = 8, PQ_X_WARPS = 5, PQ_X_GROUPS = 2;   // two expander groups taking the blocks in turn (one: 121.6 us, three: 113.5 us, two: 108.1 us)
constexpr int PQ_X_WARP0 = PQ_E_WARPS, PQ_PAD_WARP0 = PQ_X_WARP0 + PQ_X_GROUPS * PQ_X_WARPS;   // idle warps up to the next group of four
constexpr int PQ_ATMA_WARP = (PQ_PAD_WARP0 + 3) / 4 * 4, PQ_WTMA_WARP = PQ_ATMA_WARP + 1, PQ_MMA_WARP = PQ_ATMA_WARP + 2;
constexpr int PQ_THREADS = 32 * (PQ_ATMA_WARP + 4);
constexpr int PQ_LAUNCH_REGS = 65536 / PQ_THREADS / 8 * 8, PQ_E_REGS = 96, PQ_IO_REGS = 24;
static_assert(PQ_E_WARPS * (PQ_E_REGS - PQ_LAUNCH_REGS) <= 4 * (PQ_LAUNCH_REGS - PQ_IO_REGS), "warp groups and their register trade");
constexpr int PQ_STAGES = 3, PQ_RAW_SLOTS = 4, PQ_RING = 8;
constexpr int PQ_A_SLAB = 128 * 128, PQ_A_MIN = 2 * PQ_A_SLAB, PQ_A_COL = 128 * 16, PQ_A_SLOT = PQ_A_MIN + 2 * PQ_A_COL;   // 36 KB
constexpr int PQ_B_SLAB = PP_RMAX * 128, PQ_B_M = 2 * PQ_B_SLAB, PQ_B_SLOT = 22 * 1024;
static_assert(PQ_B_M + (PP_RMAX / 2) * 32 <= PQ_B_SLOT && PQ_A_SLOT % 1024 == 0, "operand slots");
constexpr int PQ_OFF_A = 1024;
constexpr int PQ_OFF_B = PQ_OFF_A + PQ_STAGES * PQ_A_SLOT;
constexpr int PQ_OFF_RAW = PQ_OFF_B + PQ_STAGES * PQ_B_SLOT;
constexpr int PQ_OFF_WD = PQ_OFF_RAW + PQ_RAW_SLOTS * PP_RAW_SLOT;
constexpr int PQ_SMEM = PQ_OFF_WD + PQ_RING * PP_WD_SLOT;
static_assert(PQ_SMEM <= 227 * 1024 && PQ_OFF_B % 1024 == 0 && PQ_OFF_RAW % 128 == 0, "shared memory of the Q4_K plane kernel");

struct QpControl {
    uint64_t a_full[PQ_STAGES];          // this CTA's activation boxes (transaction bytes)
    uint64_t a_peer[PQ_STAGES];          // EVEN CTA's copy is the live one: the odd CTA's boxes have landed
    uint64_t raw_full[PQ_RAW_SLOTS];
    uint64_t raw_empty[PQ_RAW_SLOTS];
    uint64_t b_full[PQ_STAGES];          // EVEN CTA's copy is the live one: expander warps of both CTAs
    uint64_t ab_empty[PQ_STAGES];        // both copies live: the MMAs that read the slots have completed
    uint64_t tmem_full[2];               // both copies live
    uint64_t tmem_empty[2];              // EVEN CTA's copy is the live one: epilogue warps of both CTAs
    uint32_t tmem_base;
    volatile int abort;
};
static_assert(sizeof(QpControl) <= PQ_OFF_A, "control block");

struct QpAt {   // blocks in order, tiles round-robin over the pairs
    int n0, m0, b, tile, pairs;
    __device__ __forceinline__ void set_tile(const PairParams &p, int t) {
        tile = t;
        n0 = (t / p.m_tiles) * p.w;
        m0 = (t % p.m_tiles) * (2 * PP_TOKENS);
    }
    __device__ __forceinline__ void advance(const PairParams &p) {
        if (++b == p.nb) { b = 0; set_tile(p, tile + pairs); }
    }
};
__device__ __forceinline__ QpAt qp_first(const PairParams &p, int pair, int pairs) {
    QpAt at;
    at.b = 0;
    at.pairs = pairs;
    at.set_tile(p, pair);
    return at;
}

// Lane (i8, j) as in pp_expand: weight i8 of the warp's eight, part j (sub-blocks 2j and 2j+1, weights 64j..64j+63): two
// scaled limbs into operand chunks 4j..4j+3 of rows i (hi) and half_rows + i (lo); part 0 also writes the min-term rows,
// parts 1 and 2 the {d, -dmin} of this CTA's and of the partner's weight for the epilogue.
__device__ __forceinline__ void pq_expand(uint32_t raw, uint32_t partner_head, uint32_t b_slot, uint32_t wd_mine, uint32_t wd_partner, int i, int j, int half_rows) {
    const uint4 hd = lds128(raw), qa = lds128(raw + 16 + 32 * j), qb = lds128(raw + 32 + 32 * j);
    const Q4KScales s = q4k_unpack_scales(hd.y, hd.z, hd.w);
    const uint32_t scv = j < 2 ? s.sc_lo : s.sc_hi;
    const uint32_t sl = byte_of(scv, (2 * j) & 3), sh = byte_of(scv, ((2 * j) & 3) + 1);
    const uint32_t al = sl >> 3, cl = sl & 7u, ah = sh >> 3, ch = sh & 7u;
    const uint32_t q[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
    const uint32_t base = b_slot + (uint32_t)(i >> 3) * 1024u + (uint32_t)(i & 7) * 128u;
    const uint32_t x7 = (uint32_t)(i & 7) << 4;
    const uint32_t lo_limb = (uint32_t)half_rows * 128u;
#pragma unroll
    for (int g = 0; g < 2; ++g) {   // low nibbles: weights 64j..64j+31 (chunks 4j, 4j+1), high nibbles: 64j+32.. (chunks 4j+2, 4j+3)
        uint32_t va[8], vc[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const uint32_t nib = (g ? q[k] >> 4 : q[k]) & 0x0f0f0f0fu;
            // every byte product is <= 15 * 7 = 105: one 32-bit multiply scales four weights
            va[k] = nib * (g ? ah : al);
            vc[k] = nib * (g ? ch : cl);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int chunk = 4 * j + 2 * g + h;
            const uint32_t at = base + (uint32_t)(chunk >> 3) * PQ_B_SLAB + (((uint32_t)(chunk & 7) << 4) ^ x7);
            sts_u128(at, va[4 * h], va[4 * h + 1], va[4 * h + 2], va[4 * h + 3]);
            sts_u128(at + lo_limb, vc[4 * h], vc[4 * h + 1], vc[4 * h + 2], vc[4 * h + 3]);
        }
    }
    if (j == 0) {   // {mn} and {64 mn} as f16: the min-term rows of this weight
        const uint32_t bm = b_slot + PQ_B_M + core_offset(i, 0, 2);
        float mn[8];
#pragma unroll
        for (int g = 0; g < 8; ++g) mn[g] = (float)byte_of(g < 4 ? s.mn_lo : s.mn_hi, g & 3);
        sts_u128(bm, pack_half2(mn[0], mn[1]), pack_half2(mn[2], mn[3]), pack_half2(mn[4], mn[5]), pack_half2(mn[6], mn[7]));
        sts_u128(bm + 128u, pack_half2(64.f * mn[0], 64.f * mn[1]), pack_half2(64.f * mn[2], 64.f * mn[3]),
                 pack_half2(64.f * mn[4], 64.f * mn[5]), pack_half2(64.f * mn[6], 64.f * mn[7]));
    } else if (j < 3) {   // {d, -dmin} for the epilogue: part 1 takes this CTA's weight i, part 2 weight i of the partner's half
        const uint32_t dd = j == 1 ? hd.x : lds_u32(partner_head);
        const uint32_t d = __float_as_uint(half_bits_to_float(dd)), nm = __float_as_uint(-half_bits_to_float(dd >> 16));
        const uint32_t at = (j == 1 ? wd_mine : wd_partner) + 16u * (uint32_t)(i >> 1) + 4u * (uint32_t)(i & 1);
        sts_u32(at, d);
        sts_u32(at + 8u, nm);
    }
}

// Q8_K records -> planes for the Q4_K kernel: codes (m, k) int8 in the records' own order, x.d (k / 256, pitch) float, and the
// min-term operand (m, k / 256 * 16) f16: per block the eight bsum pair sums s = 64 h + l (l in 0..63) as {l_0..l_7 | h_0..h_7}.
__global__ void __launch_bounds__(256) q8k_planes_q4k_kernel(const uint8_t *__restrict__ xq, int8_t *__restrict__ codes, float *__restrict__ xd, __half *__restrict__ mins,
                                                             long long m, int nb, long long pitch) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long record = idx >> 4;
    const int c = (int)(idx & 15);
    if (record >= m * nb) return;
    const uint32_t *src = reinterpret_cast<const uint32_t *>(xq + record * 292);   // records are 4-byte aligned
    *reinterpret_cast<uint4 *>(codes + record * 256 + 16 * c) = make_uint4(src[1 + 4 * c], src[2 + 4 * c], src[3 + 4 * c], src[4 + 4 * c]);
    if (c < 8) {   // bsums 2c, 2c+1 are the two halves of record word 65 + c
        int sum;
        asm("dp2a.lo.s32.u32 %0, %1, %2, %3;" : "=r"(sum) : "r"(src[65 + c]), "r"(0x0101u), "r"(0));
        const int l = sum & 63;
        mins[record * 16 + c] = __int2half_rn(l);
        mins[record * 16 + 8 + c] = __int2half_rn((sum - l) >> 6);
    } else if (c == 8) {
        const long long t = record / nb;
        xd[(record - t * nb) * pitch + t] = __uint_as_float(src[0]);
    }
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PQ_THREADS, 1)
prefill_pair_q4k_planes_kernel(const PairParams p, const __grid_constant__ CUtensorMap x_codes, const __grid_constant__ CUtensorMap x_mins,
                               const __grid_constant__ CUtensorMap w_rows, const __grid_constant__ CUtensorMap w_heads) {
    extern __shared__ __align__(1024) uint8_t smem[];
    QpControl *ctl = reinterpret_cast<QpControl *>(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = tc::cluster_ctarank();
    const int pair = (int)blockIdx.x >> 1, pairs = (int)gridDim.x >> 1;
    const int tiles = p.m_tiles * p.n_tiles;
    const int nb = p.nb;
    const int my_tiles = (tiles - pair + pairs - 1) / pairs;
    const int total = my_tiles * nb;
    const int half_rows = p.w >> 1;                       // weights this CTA expands per block = rows per limb
    const int R = p.w;                                    // B rows per CTA

    const uint32_t ctl_addr = smem_addr(ctl);
    const uint32_t ctl_even = tc::map_to_cta(ctl_addr, 0), ctl_peer = tc::map_to_cta(ctl_addr, rank ^ 1u);
    const uint32_t peer_abort = ctl_peer + (uint32_t)offsetof(QpControl, abort);

    if (threadIdx.x == 0) {
        for (int s = 0; s < PQ_STAGES; ++s) {
            mbar_init(&ctl->a_full[s], 1);
            mbar_init(&ctl->a_peer[s], 1);
            mbar_init(&ctl->b_full[s], 2 * PQ_X_WARPS);
            mbar_init(&ctl->ab_empty[s], 1);
        }
        for (int s = 0; s < PQ_RAW_SLOTS; ++s) { mbar_init(&ctl->raw_full[s], 1); mbar_init(&ctl->raw_empty[s], PQ_X_WARPS); }
        for (int h = 0; h < 2; ++h) { mbar_init(&ctl->tmem_full[h], 1); mbar_init(&ctl->tmem_empty[h], 2 * PQ_E_WARPS); }
        ctl->abort = 0;
        ctl->tmem_base = 0xffffffffu;
        mbar_fence_init();
    }
    __syncthreads();
    if (warp == PQ_MMA_WARP) tc::tmem_alloc(&ctl->tmem_base, PP_TMEM_COLS);
    tc::fence_before_sync();
    __syncthreads();
    tc::cluster_sync_all();
    tc::fence_after_sync();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t *>(&ctl->tmem_base);
    const bool tmem_ok = tmem == 0u;
    if (!tmem_ok && threadIdx.x == 0) { ctl->abort = 1; tc::st_cluster_u32(peer_abort, 1u); report(p.status, 0x40000000 | (int)(tmem & 0xffffu) | (int)((tmem >> 16) & 0x3fffu) << 16); }
    if (!tmem_ok) {
        // nothing: fall through to the common exit
    } else if (warp >= PQ_X_WARP0 && warp < PQ_PAD_WARP0) {
        // ------------------------------------------------------------------ expanders: two groups taking the blocks in turn
        const int xw = (warp - PQ_X_WARP0) % PQ_X_WARPS, xg = (warp - PQ_X_WARP0) / PQ_X_WARPS;
        const int i8 = (lane >> 1) & 7, j = (lane & 1) | ((lane >> 4) << 1);
        const int i = 8 * xw + i8;
        const bool active = i < half_rows;
        const uint32_t full_even = ctl_even + (uint32_t)offsetof(QpControl, b_full);
        for (int it = xg; it < total && !ctl->abort; it += PQ_X_GROUPS) {
            const int s = it % PQ_STAGES, rs = it % PQ_RAW_SLOTS;
            if (!pp_wait_warp(&ctl->raw_full[rs], (uint32_t)(it / PQ_RAW_SLOTS) & 1u, ctl, peer_abort, p.status)) break;
            if (!pp_wait_warp(&ctl->ab_empty[s], ((uint32_t)(it / PQ_STAGES) & 1u) ^ 1u, ctl, peer_abort, p.status)) break;
            if (active) {
                const uint32_t raw_slot = smem_addr(smem + PQ_OFF_RAW + rs * PP_RAW_SLOT);
                const uint32_t wd_slot = smem_addr(smem + PQ_OFF_WD + (it & (PQ_RING - 1)) * PP_WD_SLOT);
                pq_expand(raw_slot + (uint32_t)i * 144u, raw_slot + PP_RAW_HEADS + (uint32_t)i * 16u, smem_addr(smem + PQ_OFF_B + s * PQ_B_SLOT),
                          wd_slot + rank * (uint32_t)(PP_WD_SLOT / 2), wd_slot + (rank ^ 1u) * (uint32_t)(PP_WD_SLOT / 2), i, j, half_rows);
            }
            fence_proxy_async();      // generic-proxy stores must be visible to the tensor core's reads
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&ctl->raw_empty[rs]);
                tc::mbar_arrive_cluster(full_even + 8u * (uint32_t)s);
            }
        }
    } else if (warp == PQ_ATMA_WARP) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(PQ_IO_REGS));
        // ------------------------------------------------------------------ activation copies (this CTA's 128 tokens)
        if (lane == 0) {
            QpAt at = qp_first(p, pair, pairs);
            int issued = 0;
            for (int it = 0; it < total && !ctl->abort; ++it, at.advance(p)) {
                const int s = it % PQ_STAGES;
                if (!pp_wait_one(&ctl->ab_empty[s], ((uint32_t)(it / PQ_STAGES) & 1u) ^ 1u, ctl, peer_abort, p.status)) break;
                uint8_t *slot = smem + PQ_OFF_A + s * PQ_A_SLOT;
                const int m0 = at.m0 + (int)rank * PP_TOKENS;
                mbar_expect_tx(&ctl->a_full[s], PQ_A_SLOT);
                // tokens past M read as zero
                tma_load_2d(slot, &x_codes, 256 * at.b, m0, &ctl->a_full[s]);
                tma_load_2d(slot + PQ_A_SLAB, &x_codes, 256 * at.b + 128, m0, &ctl->a_full[s]);
                tma_load_2d(slot + PQ_A_MIN, &x_mins, 32 * at.b, m0, &ctl->a_full[s]);                // {l}: 16 bytes per token
                tma_load_2d(slot + PQ_A_MIN + PQ_A_COL, &x_mins, 32 * at.b + 16, m0, &ctl->a_full[s]);  // {h}
                issued = it + 1;
            }
            for (int k = issued > PQ_STAGES ? issued - PQ_STAGES : 0; k < issued; ++k) mbar_wait(&ctl->a_full[k % PQ_STAGES], (uint32_t)(k / PQ_STAGES) & 1u);
            // stay until the even CTA's last commits have arrived on this CTA's barriers
            for (int k = total > PQ_STAGES ? total - PQ_STAGES : 0; k < total && !ctl->abort; ++k)
                if (!pp_wait_one(&ctl->ab_empty[k % PQ_STAGES], (uint32_t)(k / PQ_STAGES) & 1u, ctl, peer_abort, p.status)) break;
        }
    } else if (warp == PQ_WTMA_WARP) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(PQ_IO_REGS));
        // ------------------------------------------------------------------ raw weight records (this CTA's half of the tile's weights)
        if (lane == 0) {
            QpAt at = qp_first(p, pair, pairs);
            int issued = 0;
            const uint32_t bytes = (uint32_t)half_rows * 160u;   // this CTA's records and the 16-byte headers of the partner's
            for (int it = 0; it < total && !ctl->abort; ++it, at.advance(p)) {
                const int rs = it % PQ_RAW_SLOTS;
                if (!pp_wait_one(&ctl->raw_empty[rs], ((uint32_t)(it / PQ_RAW_SLOTS) & 1u) ^ 1u, ctl, peer_abort, p.status)) break;
                mbar_expect_tx(&ctl->raw_full[rs], bytes);
                tma_load_2d(smem + PQ_OFF_RAW + rs * PP_RAW_SLOT, &w_rows, 36 * at.b, at.n0 + (int)rank * half_rows, &ctl->raw_full[rs]);
                tma_load_2d(smem + PQ_OFF_RAW + rs * PP_RAW_SLOT + PP_RAW_HEADS, &w_heads, 36 * at.b, at.n0 + (int)(rank ^ 1u) * half_rows, &ctl->raw_full[rs]);
                issued = it + 1;
            }
            for (int k = issued > PQ_RAW_SLOTS ? issued - PQ_RAW_SLOTS : 0; k < issued; ++k) mbar_wait(&ctl->raw_full[k % PQ_RAW_SLOTS], (uint32_t)(k / PQ_RAW_SLOTS) & 1u);
        }
    } else if (warp >= PQ_MMA_WARP) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(PQ_IO_REGS));
        const int q = warp - PQ_MMA_WARP;
        if (lane == 0 && rank == 0) {
            // -------------------------------------------------------------- MMA issue (even CTA), two issuers, one TMEM buffer each
            const uint32_t idesc_q = tc::idesc_i8(2 * PP_TOKENS, 2 * R, true, true);
            const uint32_t idesc_m = tc::idesc_f16_f32acc(2 * PP_TOKENS, R);
            const uint32_t full_mine = smem_addr(&ctl->tmem_full[q]), full_peer = ctl_peer + (uint32_t)offsetof(QpControl, tmem_full) + 8u * (uint32_t)q;
            const uint32_t empty_peer = ctl_peer + (uint32_t)offsetof(QpControl, ab_empty);
            const uint32_t d = tmem + (uint32_t)q * PP_BUF_COLS;
            int last = -1;
            for (int it = q; it < total && !ctl->abort; it += 2) {
                const int s = it % PQ_STAGES;
                if (!pp_wait_one(&ctl->a_full[s], (uint32_t)(it / PQ_STAGES) & 1u, ctl, peer_abort, p.status)) break;
                if (!pp_wait_one(&ctl->a_peer[s], (uint32_t)(it / PQ_STAGES) & 1u, ctl, peer_abort, p.status)) break;
                if (!pp_wait_one(&ctl->b_full[s], (uint32_t)(it / PQ_STAGES) & 1u, ctl, peer_abort, p.status)) break;
                if (!pp_wait_one(&ctl->tmem_empty[q], (uint32_t)(it >> 1) & 1u, ctl, peer_abort, p.status)) break;
                tc::fence_after_sync();
                const uint32_t a_q = smem_addr(smem + PQ_OFF_A + s * PQ_A_SLOT), b_q = smem_addr(smem + PQ_OFF_B + s * PQ_B_SLOT);
                const uint64_t a0 = tc::smem_desc_sw128(a_q), b0 = tc::smem_desc_sw128(b_q);
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    tc::mma_i8_pair(d, a0 + (uint64_t)(((k >> 2) * PQ_A_SLAB + (k & 3) * 32) >> 4), b0 + (uint64_t)(((k >> 2) * PQ_B_SLAB + (k & 3) * 32) >> 4), idesc_q, 1);
                // min term: A = {l | h} (two 16-byte columns), B = {mn | 64 mn}
                tc::mma_f16_pair(d + PP_MIN_COL, tc::smem_desc(a_q + PQ_A_MIN, PQ_A_COL, 128), tc::smem_desc(b_q + PQ_B_M, 128, 256), idesc_m, 0);
                tc::commit_pair(full_mine);
                tc::commit_pair(full_peer);
                tc::commit_pair(smem_addr(&ctl->ab_empty[s]));
                tc::commit_pair(empty_peer + 8u * (uint32_t)s);
                last = it;
            }
            if (last >= 0 && !ctl->abort) pp_wait_one(&ctl->tmem_empty[q], ((uint32_t)(last >> 1) + 1u) & 1u, ctl, peer_abort, p.status);
        } else if (lane == 0 && rank == 1 && q == 0) {
            // -------------------------------------------------------------- odd CTA: tell the even CTA that this CTA's activations have landed
            const uint32_t peer_even = ctl_even + (uint32_t)offsetof(QpControl, a_peer);
            for (int it = 0; it < total && !ctl->abort; ++it) {
                const int s = it % PQ_STAGES;
                if (!pp_wait_one(&ctl->a_full[s], (uint32_t)(it / PQ_STAGES) & 1u, ctl, peer_abort, p.status)) break;
                tc::mbar_arrive_cluster(peer_even + 8u * (uint32_t)s);
            }
        }
    } else if (warp < PQ_E_WARPS) {
        // ------------------------------------------------------------------ epilogue: warp = (32-token quarter, half of the tile's weights)
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(PQ_E_REGS));
        const int quarter = warp & 3, grp = warp >> 2;
        const int row = quarter * 32 + lane;               // token row of this CTA = TMEM lane
        const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
        const uint32_t empty_even = ctl_even + (uint32_t)offsetof(QpControl, tmem_empty);
        const int chunks = half_rows >> 3;                  // groups of 8 weights
        // accumulators start at the bit pattern of 1.5 * 2^23
        for (int buf = 0; buf < 2; ++buf) {
            for (int c = 0; c < 2 * chunks; ++c) tc::tmem_st8_fill(lane_base + (uint32_t)(buf * PP_BUF_COLS + grp * R + 8 * c), PP_BIAS);
            tc::tmem_st_wait();
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive_cluster(empty_even + 8u * (uint32_t)buf);
        }
        uint64_t acc[PP_RMAX / 4];   // packed pairs of fp32: up to 40 weights
        const uint64_t bias2 = pack2(-12582912.f, -12582912.f), eight2 = pack2(8.f, 8.f);
        QpAt at = qp_first(p, pair, pairs);
        int it = 0;
        bool ok = true;
        int m = at.m0 + (int)rank * PP_TOKENS + row;
        float xd_next = m < p.m ? __ldg(p.xd + (long long)at.b * p.xd_pitch + m) : 0.f;
        for (int t = 0; t < my_tiles && ok && !ctl->abort; ++t) {
            const long long n0 = (long long)at.n0 + grp * half_rows;
            m = at.m0 + (int)rank * PP_TOKENS + row;
#pragma unroll
            for (int k = 0; k < PP_RMAX / 4; ++k) acc[k] = 0ull;
            for (int b = 0; b < nb && ok; ++b, ++it) {
                const int buf = it & 1;
                const float xd = xd_next;
                at.advance(p);
                if (it + 1 < total) {   // x.d of the next block (of the next tile's tokens after the last block of a tile)
                    const int mn = at.m0 + (int)rank * PP_TOKENS + row;
                    xd_next = mn < p.m ? __ldg(p.xd + (long long)at.b * p.xd_pitch + mn) : 0.f;
                }
                if (!pp_wait_warp(&ctl->tmem_full[buf], (uint32_t)(it >> 1) & 1u, ctl, peer_abort, p.status)) { ok = false; break; }
                tc::fence_after_sync();
                const ulonglong2 *wd = reinterpret_cast<const ulonglong2 *>(smem + PQ_OFF_WD + (it & (PQ_RING - 1)) * PP_WD_SLOT + grp * (PP_WD_SLOT / 2));
                const uint64_t xd2 = pack2(xd, xd);
                const uint32_t limb = lane_base + (uint32_t)(buf * PP_BUF_COLS + grp * R);
                const uint32_t mins = lane_base + (uint32_t)(buf * PP_BUF_COLS + PP_MIN_COL + grp * half_rows);
#pragma unroll
                for (int c = 0; c < PP_RMAX / 16; ++c) {
                    if (c < chunks) {
                        uint32_t hi[8], lo[8], mt[8];
                        tc::tmem_ld8(limb + 8 * c, hi);
                        tc::tmem_ld8(limb + half_rows + 8 * c, lo);
                        tc::tmem_ld8(mins + 8 * c, mt);
                        tc::tmem_ld_wait();
                        tc::tmem_st8_fill(limb + 8 * c, PP_BIAS);
                        tc::tmem_st8_fill(limb + half_rows + 8 * c, PP_BIAS);
#pragma unroll
                        for (int k = 0; k < 8; k += 2) {
                            const ulonglong2 s2 = wd[(8 * c + k) >> 1];   // {d, d'}, {-dmin, -dmin'}
                            const uint64_t fh = add2(pack2(__uint_as_float(hi[k]), __uint_as_float(hi[k + 1])), bias2);
                            const uint64_t fl = add2(pack2(__uint_as_float(lo[k]), __uint_as_float(lo[k + 1])), bias2);
                            const uint64_t v = fma2(eight2, fh, fl);
                            const uint64_t u = fma2(s2.y, pack2(__uint_as_float(mt[k]), __uint_as_float(mt[k + 1])), mul2(s2.x, v));
                            acc[(8 * c + k) >> 1] = fma2(xd2, u, acc[(8 * c + k) >> 1]);
                        }
                    }
                }
                tc::tmem_st_wait();
                tc::fence_before_sync();
                __syncwarp();
                if (lane == 0) tc::mbar_arrive_cluster(empty_even + 8u * (uint32_t)buf);
            }
            if (!ok) break;
            if (m < p.m) {
                float *out = p.y + (size_t)m * p.ldy + n0;
                const bool vec = (reinterpret_cast<uintptr_t>(out) & 15u) == 0;
#pragma unroll
                for (int k = 0; k < PP_RMAX / 2; k += 4) {
                    if (k < half_rows) {
                        if (vec && n0 + k + 4 <= p.n) {
                            *reinterpret_cast<ulonglong2 *>(out + k) = make_ulonglong2(acc[k >> 1], acc[(k >> 1) + 1]);
                        } else {
                            float a0, a1, a2, a3;
                            unpack2(acc[k >> 1], a0, a1);
                            unpack2(acc[(k >> 1) + 1], a2, a3);
                            if (n0 + k < p.n) out[k] = a0;
                            if (n0 + k + 1 < p.n) out[k + 1] = a1;
                            if (n0 + k + 2 < p.n) out[k + 2] = a2;
                            if (n0 + k + 3 < p.n) out[k + 3] = a3;
                        }
                    }
                }
            }
        }
    }

    tc::fence_before_sync();
    __syncthreads();
    tc::cluster_sync_all();
    if (warp == PQ_MMA_WARP) {
        __syncwarp();
        if (tmem_ok) tc::tmem_free(tmem, PP_TMEM_COLS);
    }
}

// w in {32, 64, 96, 128, 160} for TQ1_0: minimise (rounds of the grid) x (fixed part + w), ties to the wider tile
int pick_tile_width_tq1(long long n, int m_tiles, int pairs) {
    int best = 32;
    long long best_cost = -1;
    for (int w = 32; w <= 2 * PP_RMAX; w += 32) {
        const long long tiles = (long long)m_tiles * ((n + w - 1) / w);
        const long long cost = ((tiles + pairs - 1) / pairs) * (160 + w);
        if (best_cost < 0 || cost <= best_cost) { best = w; best_cost = cost; }
    }
    return best;
}

// w in {16, 32, 48, 64, 80}.  A block costs a fixed part (hand-offs, activations, the per-token work) plus a part that
// grows with w; measured, the fixed part is about the size of the variable part at w = 80.  Pick the w that minimises
// (rounds of the grid) x (80 + w), ties to the wider tile.
int pick_tile_width(long long n, int m_tiles, int pairs) {
    int best = 16;
    long long best_cost = -1;
    for (int w = 16; w <= PP_RMAX; w += 16) {
        const long long tiles = (long long)m_tiles * ((n + w - 1) / w);
        const long long cost = ((tiles + pairs - 1) / pairs) * (80 + w);
        if (best_cost < 0 || cost <= best_cost) { best = w; best_cost = cost; }
    }
    return best;
}

}  // namespace

bool prefill_pair_supported(int fmt, long long n, long long k, long long m, const void *w, const void *xq) {
    // TQ1_0: K a multiple of 2048 makes the weight rows whole 16-byte multiples (TMA boxes over the raw records)
    if (fmt == F_TQ1_0)
        return m > PP_TOKENS && k > 0 && k % 2048 == 0 && n > 0 && n < (1LL << 31) && m < (1LL << 31) &&
               (reinterpret_cast<uintptr_t>(w) & 15u) == 0 && (reinterpret_cast<uintptr_t>(xq) & 15u) == 0;
    // above 128 tokens a pair's second CTA has work; Q4_K rows are 16-byte multiples for every K, so a 16-byte aligned base
    // lets TMA fetch the raw records; the activations come from planes of the library's own (the records need their 4 bytes)
    return fmt == F_Q4_K && m > PP_TOKENS && k > 0 && k % 256 == 0 && n > 0 && n < (1LL << 31) && m < (1LL << 31) &&
           (reinterpret_cast<uintptr_t>(w) & 15u) == 0 && (reinterpret_cast<uintptr_t>(xq) & 3u) == 0;
}

// The planes of the latest call: one device allocation that only ever grows.  Calls are serialised by the
// library and run on one stream, so the next call's plane kernel starts after this call's contraction has ended.  A
// larger request gets a new allocation; the previous ones stay until the process ends, because work already queued (or a
// captured graph) may still name them.
struct PlaneScratch {
    uint8_t *base = nullptr;
    size_t bytes = 0;
};
static PlaneScratch g_planes;

static cudaError_t reserve_planes(size_t bytes, uint8_t **out) {
    if (bytes > g_planes.bytes) {
        uint8_t *fresh = nullptr;
        const size_t want = (bytes + bytes / 4 + 255) & ~size_t(255);
        const cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&fresh), want);
        if (e != cudaSuccess) return e;
        g_planes.base = fresh;
        g_planes.bytes = want;
    }
    *out = g_planes.base;
    return cudaSuccess;
}

// The register trade assumes the allocation the kernel was compiled with: a build with another one must not run
static cudaError_t check_launch_registers(const void *kernel, int expected) {
    cudaFuncAttributes attr;
    const cudaError_t e = cudaFuncGetAttributes(&attr, kernel);
    if (e != cudaSuccess) return e;
    return attr.numRegs == expected ? cudaSuccess : cudaErrorInvalidConfiguration;
}

static cudaError_t launch_prefill_pair_tq1(const PrefillArgs &a, int sm_count, cudaStream_t stream) {
    if (!a.powers) return cudaErrorInvalidValue;
    cudaError_t e = grant_dynamic_smem(reinterpret_cast<const void *>(prefill_pair_tq1_kernel), PT_SMEM);
    if (e == cudaSuccess) e = check_launch_registers(reinterpret_cast<const void *>(prefill_pair_tq1_kernel), PT_LAUNCH_REGS);
    if (e != cudaSuccess) return e;
    int pairs = 0;
    {
        cudaLaunchConfig_t probe = {};
        probe.gridDim = dim3((unsigned)sm_count & ~1u);
        probe.blockDim = dim3(PT_THREADS);
        probe.dynamicSmemBytes = PT_SMEM;
        if (cudaOccupancyMaxActiveClusters(&pairs, prefill_pair_tq1_kernel, &probe) != cudaSuccess) { cudaGetLastError(); pairs = sm_count / 2; }
        if (pairs < 1) return cudaErrorNotSupported;
        if (pairs > sm_count / 2) pairs = sm_count / 2;
    }
    PairParams p;
    p.y = a.y; p.n = a.n; p.m = a.m; p.ldy = a.ldy; p.nb = (int)(a.k / 256); p.status = a.status;
    p.m_tiles = (int)((a.m + 2 * PP_TOKENS - 1) / (2 * PP_TOKENS));
    p.w = pick_tile_width_tq1(a.n, p.m_tiles, pairs);
    p.n_tiles = (int)((a.n + p.w - 1) / p.w);
    const long long tiles = (long long)p.m_tiles * p.n_tiles;
    if (tiles < pairs) pairs = (int)tiles;
    // planes: codes (m, k) int8, then x.d (nb, pitch) float
    p.xd_pitch = (a.m + 63) & ~63LL;
    const size_t code_bytes = ((size_t)a.m * (size_t)a.k + 255) & ~size_t(255);
    uint8_t *planes = nullptr;
    e = reserve_planes(code_bytes + (size_t)p.nb * (size_t)p.xd_pitch * sizeof(float), &planes);
    if (e != cudaSuccess) return e;
    p.xd = reinterpret_cast<const float *>(planes + code_bytes);
    {
        const long long records = a.m * p.nb;
        q8k_planes_kernel<<<(unsigned)((records + 15) / 16), 256, 0, stream>>>(static_cast<const uint8_t *>(a.xq), reinterpret_cast<int8_t *>(planes),
                                                                                   reinterpret_cast<float *>(planes + code_bytes), a.m, p.nb, p.xd_pitch);
        e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    CUtensorMap x_codes, w_rows, w_heads;
    e = encode_tile_map(&x_codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, planes, (unsigned long long)a.k, (unsigned long long)a.m,
                        (unsigned long long)a.k, 128, PP_TOKENS, true);
    // the weight matrix as (n) rows of 54 * nb bytes
    if (e == cudaSuccess)
        e = encode_tile_map(&w_rows, CU_TENSOR_MAP_DATA_TYPE_UINT8, a.w, (unsigned long long)p.nb * 54, (unsigned long long)a.n,
                            (unsigned long long)p.nb * 54, PT_RAW_BOX, (unsigned)(p.w / 2), false);
    if (e == cudaSuccess)
        e = encode_tile_map(&w_heads, CU_TENSOR_MAP_DATA_TYPE_UINT8, a.w, (unsigned long long)p.nb * 54, (unsigned long long)a.n,
                            (unsigned long long)p.nb * 54, 16, (unsigned)(p.w / 2), false);
    if (e != cudaSuccess) return e;
    prefill_pair_tq1_kernel<<<2 * pairs, PT_THREADS, PT_SMEM, stream>>>(p, a.powers, x_codes, w_rows, w_heads);
    return cudaGetLastError();
}

static cudaError_t launch_prefill_pair_q4k_planes(const PrefillArgs &a, int sm_count, cudaStream_t stream) {
    cudaError_t e = grant_dynamic_smem(reinterpret_cast<const void *>(prefill_pair_q4k_planes_kernel), PQ_SMEM);
    if (e == cudaSuccess) e = check_launch_registers(reinterpret_cast<const void *>(prefill_pair_q4k_planes_kernel), PQ_LAUNCH_REGS);
    if (e != cudaSuccess) return e;
    int pairs = 0;
    {
        cudaLaunchConfig_t probe = {};
        probe.gridDim = dim3((unsigned)sm_count & ~1u);
        probe.blockDim = dim3(PQ_THREADS);
        probe.dynamicSmemBytes = PQ_SMEM;
        if (cudaOccupancyMaxActiveClusters(&pairs, prefill_pair_q4k_planes_kernel, &probe) != cudaSuccess) { cudaGetLastError(); pairs = sm_count / 2; }
        if (pairs < 1) return cudaErrorNotSupported;
        if (pairs > sm_count / 2) pairs = sm_count / 2;
    }
    PairParams p;
    p.y = a.y; p.n = a.n; p.m = a.m; p.ldy = a.ldy; p.nb = (int)(a.k / 256); p.status = a.status;
    p.m_tiles = (int)((a.m + 2 * PP_TOKENS - 1) / (2 * PP_TOKENS));
    p.w = pick_tile_width(a.n, p.m_tiles, pairs);
    p.n_tiles = (int)((a.n + p.w - 1) / p.w);
    const long long tiles = (long long)p.m_tiles * p.n_tiles;
    if (tiles < pairs) pairs = (int)tiles;
    // planes: codes (m, k) int8, x.d (nb, pitch) float, min-term operand (m, nb * 16) f16
    p.xd_pitch = (a.m + 63) & ~63LL;
    const size_t code_bytes = ((size_t)a.m * (size_t)a.k + 255) & ~size_t(255);
    const size_t xd_bytes = ((size_t)p.nb * (size_t)p.xd_pitch * sizeof(float) + 255) & ~size_t(255);
    uint8_t *planes = nullptr;
    e = reserve_planes(code_bytes + xd_bytes + (size_t)a.m * (size_t)p.nb * 32, &planes);
    if (e != cudaSuccess) return e;
    p.xd = reinterpret_cast<const float *>(planes + code_bytes);
    uint8_t *mins = planes + code_bytes + xd_bytes;
    {
        const long long threads = a.m * p.nb * 16;
        q8k_planes_q4k_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(static_cast<const uint8_t *>(a.xq), reinterpret_cast<int8_t *>(planes),
                                                                                       reinterpret_cast<float *>(planes + code_bytes), reinterpret_cast<__half *>(mins), a.m, p.nb, p.xd_pitch);
        e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    CUtensorMap x_codes, x_mins, w_rows, w_heads;
    e = encode_tile_map(&x_codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, planes, (unsigned long long)a.k, (unsigned long long)a.m,
                        (unsigned long long)a.k, 128, PP_TOKENS, true);
    if (e == cudaSuccess)
        e = encode_tile_map(&x_mins, CU_TENSOR_MAP_DATA_TYPE_UINT8, mins, (unsigned long long)p.nb * 32, (unsigned long long)a.m,
                            (unsigned long long)p.nb * 32, 16, PP_TOKENS, false);
    // the weight matrix as (n) rows of 36 * nb words
    if (e == cudaSuccess)
        e = encode_tile_map(&w_rows, CU_TENSOR_MAP_DATA_TYPE_UINT32, a.w, (unsigned long long)p.nb * 36, (unsigned long long)a.n,
                            (unsigned long long)p.nb * 144, 36, (unsigned)(p.w / 2), false);
    if (e == cudaSuccess)
        e = encode_tile_map(&w_heads, CU_TENSOR_MAP_DATA_TYPE_UINT32, a.w, (unsigned long long)p.nb * 36, (unsigned long long)a.n,
                            (unsigned long long)p.nb * 144, 4, (unsigned)(p.w / 2), false);
    if (e != cudaSuccess) return e;
    prefill_pair_q4k_planes_kernel<<<2 * pairs, PQ_THREADS, PQ_SMEM, stream>>>(p, x_codes, x_mins, w_rows, w_heads);
    return cudaGetLastError();
}

int prefill_pair_launches(int) { return 2; }   // plane kernel + contraction

cudaError_t launch_prefill_pair(const PrefillArgs &a, int sm_count, cudaStream_t stream) {
    if (!prefill_pair_supported(a.fmt, a.n, a.k, a.m, a.w, a.xq)) return cudaErrorNotSupported;
    if (a.fmt == F_TQ1_0) return launch_prefill_pair_tq1(a, sm_count, stream);
    return launch_prefill_pair_q4k_planes(a, sm_count, stream);
}

}  // namespace weft
