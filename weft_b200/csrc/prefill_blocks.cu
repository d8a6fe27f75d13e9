// Prefill contraction for the 32-element block formats: production_mul_mat_q4_0 and production_mul_mat_q8_0
// (examples/kernels/mul_mat/q4_0.py:9-30, q8_0.py:9-29; per block the math of examples/kernels/vec_dot/q4_0_q8_0.py:8-23
// and q8_0_q8_0.py:8-22, GGML ggml-cpu/quants.c:174-208, 400-428) on the int8 tensor cores of sm_100a.
//
// Both operands carry an f16 scale per 32 elements, so nothing can be accumulated across blocks in integers: every
// 32-element block is its own K = 32 contraction with its own accumulator, and the fp32 combine
//   Q4_0: acc += (f32(isum) * d_w) * d_x        Q8_0: acc += f32(isum) * (d_w * d_x)
// runs per block in the epilogue (the op order of the two reference kernels differs, and is kept).
// Tensor-core bound by count (2*M*N*K integer ops), CUDA-core bound in practice: M*N*K/32 scale-accumulate steps.
//
// Activations are never repacked by a CUDA core.  Eight Q8_0 records (272 bytes = one unit of 256 elements) start on
// a 16-byte boundary of a token row when K is a multiple of 256, so TMA box copies bring the raw records of 128 tokens
// straight into the K-major operand layout; the f16 scales sit inside that operand as garbage bytes.  Block j of a unit
// has its 32 codes at operand bytes 34 j + 2 .. 34 j + 33, i.e. inside K steps j and j + 1.  Its weight operand is
// therefore a 64-byte row: the block's int8 codes at byte 2 j + 2, zeros everywhere else, so the activation scales and
// the neighbouring blocks' codes only ever meet zeros.  Two K = 32 MMAs per block, N = 32 weights, accumulator j of 8.
// The byte phase of a block inside its record run (2 for even j, 0 for odd j) is the same in the raw records and in
// the 64-byte rows, for Q8_0 and for Q4_0 records alike, so the codes move as whole 32-bit words.
//
// CTA = 128 tokens (TMEM lanes) x 32 weights, persistent over tiles; per unit of 256 elements:
//   TMA lane     raw weight records of the tile (one box) and the activation boxes, three units ahead
//   expanders    4 warps, warp x = blocks 2x and 2x+1, lane = weight: records -> 64-byte rows, d_w to a ring
//   scales       2 warps: the eight d_x of every token out of the landed boxes to a ring (kept as f16)
//   MMA lane     16 MMAs into one of two TMEM buffers (8 accumulators x 32 columns)
//   epilogue     8 warps = 4 lane quarters x 2 halves of the weights.  Accumulators start at the bit pattern of
//                1.5 * 2^23 and are put back there after every read, so the integer sums come out of TMEM as floats.
// Every wait is bounded and ends as a status code.
#include "prefill_common.cuh"
#include "kernels.h"
#include "ring.cuh"

namespace weft {

namespace {

constexpr int PB_TOKENS = 128, PB_NT = 32;
constexpr int PB_STAGES = 3, PB_RING = 8;
constexpr int PB_E_WARPS = 8, PB_X_WARPS = 4, PB_S_WARPS = 2;
constexpr int PB_X_WARP0 = PB_E_WARPS, PB_S_WARP0 = PB_X_WARP0 + PB_X_WARPS, PB_TMA_WARP = PB_S_WARP0 + PB_S_WARPS, PB_MMA_WARP = PB_TMA_WARP + 1;
constexpr int PB_THREADS = 32 * (PB_MMA_WARP + 1);     // 16 warps

// A slot: operand bytes 0..255 in two 128-byte-swizzled slabs of 128 rows, bytes 256..287 in two plain 16-byte columns
constexpr int PB_A_SLAB = 128 * 128, PB_A_COL = 128 * 16;
constexpr int PB_A_THIN = 2 * PB_A_SLAB;
constexpr int PB_A_SLOT = PB_A_THIN + 2 * PB_A_COL;            // 36 KB
// B slot: per block 32 rows x 64 bytes as K-major core matrices (8 rows x 16 bytes): chunk c of row n at
// (n >> 3) * 512 + c * 128 + (n & 7) * 16
constexpr int PB_B_BLOCK = PB_NT * 64;
constexpr int PB_B_SLOT = 8 * PB_B_BLOCK;                      // 16 KB
constexpr int PB_RAW_SLOT = PB_NT * 272;                       // raw records of the tile's weights (Q8_0: 272 B per unit, Q4_0: 144)
constexpr int PB_DW_SLOT = 8 * PB_NT * 4;                      // f32 d_w [block][weight]
constexpr int PB_DX_SLOT = PB_TOKENS * 16;                     // f16 d_x [token][block]
constexpr int PB_CONTROL = 1024;
constexpr int PB_OFF_A = PB_CONTROL;
constexpr int PB_OFF_B = PB_OFF_A + PB_STAGES * PB_A_SLOT;
constexpr int PB_OFF_RAW = PB_OFF_B + PB_STAGES * PB_B_SLOT;
constexpr int PB_OFF_DW = PB_OFF_RAW + PB_STAGES * PB_RAW_SLOT;
constexpr int PB_OFF_DX = PB_OFF_DW + PB_RING * PB_DW_SLOT;
constexpr int PB_SMEM = PB_OFF_DX + PB_RING * PB_DX_SLOT;
static_assert(PB_OFF_A % 1024 == 0 && PB_A_SLOT % 1024 == 0 && PB_OFF_RAW % 128 == 0 && PB_RAW_SLOT % 128 == 0, "operand alignment");
static_assert(PB_SMEM <= 227 * 1024, "shared memory budget");
constexpr int PB_TMEM_COLS = 512, PB_BUF_COLS = 256;
constexpr uint32_t PB_BIAS = 0x4b400000u;                      // 1.5 * 2^23; |isum| <= 32 * 128 * 127 < 2^22

struct BlockParams {
    float *y;
    long long n, m, ldy;
    int units;             // 256-element units per row
    int m_tiles, n_tiles;
    int *status;
};

struct BlockControl {
    uint64_t a_landed[PB_STAGES], raw_landed[PB_STAGES];
    uint64_t ab_full[PB_STAGES], ab_empty[PB_STAGES];
    uint64_t tmem_full[2], tmem_empty[2];
    uint32_t tmem_base;
    volatile int abort;
};
static_assert(sizeof(BlockControl) <= PB_CONTROL, "control block");

__device__ __forceinline__ bool pb_wait(uint64_t *bar, uint32_t parity, BlockControl *ctl, int *status) {
    for (uint32_t i = 0; i < (1u << 22); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (ctl->abort) return false;
    }
    ctl->abort = 1;
    report(status, ST_WAIT_TIMEOUT);
    return false;
}

__device__ __forceinline__ void tmem_st16_fill(uint32_t taddr, uint32_t v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1};" ::"r"(taddr), "r"(v) : "memory");
}

// four 4-bit values per word, already isolated in the low nibble of each byte: q - 8 as int8 in every byte
__device__ __forceinline__ uint32_t nibbles_minus_8(uint32_t v) {
    const uint32_t s = v ^ 0x08080808u;                  // two's complement of q - 8 in 4 bits
    return s | ((s & 0x08080808u) * 30u);                // sign-extend: 8 * 30 = 0xf0 per byte, no carry between bytes
}

// Blocks J = 2X and 2X + 1 of one weight's unit: the raw records -> two 64-byte rows, d_w -> the ring.
// `raw`: this weight's run of eight records in shared memory; b_slot / dw_slot: this unit's slots; n = weight row of the tile.
template <int FMT, int J>
__device__ __forceinline__ void pb_expand_block(uint32_t raw, uint32_t b_slot, uint32_t dw_slot, int n) {
    constexpr int REC = FMT == F_Q8_0 ? 34 : 18;
    constexpr bool EVEN = (J & 1) == 0;                  // even blocks sit at byte phase 2 of a word, odd ones at phase 0
    constexpr int OUT0 = (2 * J + 2) >> 2;               // first word of the 16-word row that receives codes
    uint32_t out[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) out[i] = 0u;
    uint32_t d_bits;
    if (FMT == F_Q8_0) {
        constexpr int IN0 = (REC * J) >> 2;              // EVEN: word holding {d | codes 0, 1}; odd: {previous codes | d}
        if (EVEN) {
            uint32_t w[9];
#pragma unroll
            for (int i = 0; i < 9; ++i) w[i] = lds32(raw + 4u * (IN0 + i));
            d_bits = w[0] & 0xffffu;
            out[OUT0] = w[0] & 0xffff0000u;
#pragma unroll
            for (int i = 1; i < 8; ++i) out[OUT0 + i] = w[i];
            out[OUT0 + 8] = w[8] & 0x0000ffffu;
        } else {
            d_bits = lds32(raw + 4u * IN0) >> 16;
#pragma unroll
            for (int i = 0; i < 8; ++i) out[OUT0 + i] = lds32(raw + 4u * (IN0 + 1 + i));
        }
    } else {
        constexpr int IN0 = (REC * J) >> 2;
        if (EVEN) {                                       // {d | qs0 qs1}, three full words, {qs14 qs15 | next d}
            uint32_t w[5];
#pragma unroll
            for (int i = 0; i < 5; ++i) w[i] = lds32(raw + 4u * (IN0 + i));
            d_bits = w[0] & 0xffffu;
            uint32_t lo[5], hi[5];
#pragma unroll
            for (int i = 0; i < 5; ++i) { lo[i] = nibbles_minus_8(w[i] & 0x0f0f0f0fu); hi[i] = nibbles_minus_8((w[i] >> 4) & 0x0f0f0f0fu); }
            out[OUT0] = lo[0] & 0xffff0000u;
            out[OUT0 + 1] = lo[1]; out[OUT0 + 2] = lo[2]; out[OUT0 + 3] = lo[3];
            out[OUT0 + 4] = (lo[4] & 0x0000ffffu) | (hi[0] & 0xffff0000u);
            out[OUT0 + 5] = hi[1]; out[OUT0 + 6] = hi[2]; out[OUT0 + 7] = hi[3];
            out[OUT0 + 8] = hi[4] & 0x0000ffffu;
        } else {                                          // {.. | d}, then four full words of nibbles
            d_bits = lds32(raw + 4u * IN0) >> 16;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t w = lds32(raw + 4u * (IN0 + 1 + i));
                out[OUT0 + i] = nibbles_minus_8(w & 0x0f0f0f0fu);
                out[OUT0 + 4 + i] = nibbles_minus_8((w >> 4) & 0x0f0f0f0fu);
            }
        }
    }
    const uint32_t row = b_slot + (uint32_t)J * PB_B_BLOCK + (uint32_t)(n >> 3) * 512u + (uint32_t)(n & 7) * 16u;
#pragma unroll
    for (int c = 0; c < 4; ++c) sts_u128(row + 128u * c, out[4 * c], out[4 * c + 1], out[4 * c + 2], out[4 * c + 3]);
    sts_u32(dw_slot + 4u * (uint32_t)(J * PB_NT + n), __float_as_uint(half_bits_to_float(d_bits)));
}

template <int FMT>
__global__ void __launch_bounds__(PB_THREADS, 1) prefill_blocks_kernel(const BlockParams p, const __grid_constant__ CUtensorMap x_wide,
                                                                         const __grid_constant__ CUtensorMap x_narrow,
                                                                         const __grid_constant__ CUtensorMap w_rows) {
    constexpr int RAW_WORDS = FMT == F_Q8_0 ? 68 : 36;   // words of one weight's unit
    extern __shared__ __align__(1024) uint8_t smem[];
    BlockControl *ctl = reinterpret_cast<BlockControl *>(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles = p.m_tiles * p.n_tiles;
    const int my_tiles = (tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const int units = p.units, total = my_tiles * units;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PB_STAGES; ++s) {
            mbar_init(&ctl->a_landed[s], 1); mbar_init(&ctl->raw_landed[s], 1);
            mbar_init(&ctl->ab_full[s], PB_X_WARPS + PB_S_WARPS); mbar_init(&ctl->ab_empty[s], 1);
        }
        for (int h = 0; h < 2; ++h) { mbar_init(&ctl->tmem_full[h], 1); mbar_init(&ctl->tmem_empty[h], PB_E_WARPS); }
        ctl->abort = 0;
        ctl->tmem_base = 0xffffffffu;
        mbar_fence_init();
    }
    __syncthreads();
    if (warp == PB_MMA_WARP) tc::tmem_alloc(&ctl->tmem_base, PB_TMEM_COLS);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = ctl->tmem_base;

    // unit `it` of this CTA's work list: tile (it / units) of its tiles, unit (it % units); tiles that share their weights are neighbours
    auto tile_of = [&](int it) { return (int)blockIdx.x + (it / units) * (int)gridDim.x; };

    if (warp >= PB_X_WARP0 && warp < PB_X_WARP0 + PB_X_WARPS) {
        // ------------------------------------------------------------------ expanders: warp x = blocks 2x, 2x + 1; lane = weight
        const int x = warp - PB_X_WARP0;
        for (int it = 0; it < total && !ctl->abort; ++it) {
            const int s = it % PB_STAGES;
            const uint32_t phase = (uint32_t)(it / PB_STAGES) & 1u;
            if (!pb_wait(&ctl->raw_landed[s], phase, ctl, p.status)) break;
            if (!pb_wait(&ctl->ab_empty[s], phase ^ 1u, ctl, p.status)) break;
            const uint32_t raw = smem_addr(smem + PB_OFF_RAW + s * PB_RAW_SLOT) + (uint32_t)lane * (RAW_WORDS * 4);
            const uint32_t b_slot = smem_addr(smem + PB_OFF_B + s * PB_B_SLOT);
            const uint32_t dw_slot = smem_addr(smem + PB_OFF_DW + (it & (PB_RING - 1)) * PB_DW_SLOT);
            switch (x) {
            case 0: pb_expand_block<FMT, 0>(raw, b_slot, dw_slot, lane); pb_expand_block<FMT, 1>(raw, b_slot, dw_slot, lane); break;
            case 1: pb_expand_block<FMT, 2>(raw, b_slot, dw_slot, lane); pb_expand_block<FMT, 3>(raw, b_slot, dw_slot, lane); break;
            case 2: pb_expand_block<FMT, 4>(raw, b_slot, dw_slot, lane); pb_expand_block<FMT, 5>(raw, b_slot, dw_slot, lane); break;
            default: pb_expand_block<FMT, 6>(raw, b_slot, dw_slot, lane); pb_expand_block<FMT, 7>(raw, b_slot, dw_slot, lane); break;
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->ab_full[s]);
        }
    } else if (warp >= PB_S_WARP0 && warp < PB_S_WARP0 + PB_S_WARPS) {
        // ------------------------------------------------------------------ activation scales: d_x of block j is the f16 at operand byte 34 j
        const int ts = threadIdx.x - 32 * PB_S_WARP0;
        for (int it = 0; it < total && !ctl->abort; ++it) {
            const int s = it % PB_STAGES;
            if (!pb_wait(&ctl->a_landed[s], (uint32_t)(it / PB_STAGES) & 1u, ctl, p.status)) break;
            const uint32_t a_slot = smem_addr(smem + PB_OFF_A + s * PB_A_SLOT);
            const uint32_t dx_slot = smem_addr(smem + PB_OFF_DX + (it & (PB_RING - 1)) * PB_DX_SLOT);
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const int row = ts + 64 * k;
                uint32_t d[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int byte = 34 * j;             // 0, 34, ..., 238: slab byte / 128, chunk (byte % 128) / 16, offset byte % 16
                    const uint32_t word = lds32(a_slot + (uint32_t)(byte >> 7) * PB_A_SLAB + sw128_offset(row, (byte & 127) >> 4) + (uint32_t)(byte & 12));
                    d[j] = (byte & 2) ? word >> 16 : word & 0xffffu;
                }
                sts_u128(dx_slot + 16u * (uint32_t)row, d[0] | (d[1] << 16), d[2] | (d[3] << 16), d[4] | (d[5] << 16), d[6] | (d[7] << 16));
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->ab_full[s]);
        }
    } else if (warp == PB_TMA_WARP) {
        // ------------------------------------------------------------------ raw weight records and activation boxes
        if (lane == 0) {
            int issued = 0;
            for (int it = 0; it < total && !ctl->abort; ++it) {
                const int s = it % PB_STAGES, u = it % units, tile = tile_of(it);
                const int n0 = (tile / p.m_tiles) * PB_NT, m0 = (tile % p.m_tiles) * PB_TOKENS;
                if (!pb_wait(&ctl->ab_empty[s], ((uint32_t)(it / PB_STAGES) & 1u) ^ 1u, ctl, p.status)) break;
                fence_proxy_async();
                mbar_expect_tx(&ctl->raw_landed[s], PB_NT * RAW_WORDS * 4);
                tma_load_2d(smem + PB_OFF_RAW + s * PB_RAW_SLOT, &w_rows, RAW_WORDS * u, n0, &ctl->raw_landed[s]);
                uint8_t *slot = smem + PB_OFF_A + s * PB_A_SLOT;
                mbar_expect_tx(&ctl->a_landed[s], PB_A_SLOT);
                tma_load_2d(slot, &x_wide, 68 * u, m0, &ctl->a_landed[s]);
                tma_load_2d(slot + PB_A_SLAB, &x_wide, 68 * u + 32, m0, &ctl->a_landed[s]);
                tma_load_2d(slot + PB_A_THIN, &x_narrow, 68 * u + 64, m0, &ctl->a_landed[s]);
                tma_load_2d(slot + PB_A_THIN + PB_A_COL, &x_narrow, 68 * u + 68, m0, &ctl->a_landed[s]);
                issued = it + 1;
            }
            for (int k = issued > PB_STAGES ? issued - PB_STAGES : 0; k < issued; ++k) {
                mbar_wait(&ctl->a_landed[k % PB_STAGES], (uint32_t)(k / PB_STAGES) & 1u);
                mbar_wait(&ctl->raw_landed[k % PB_STAGES], (uint32_t)(k / PB_STAGES) & 1u);
            }
        }
    } else if (warp == PB_MMA_WARP) {
        // ------------------------------------------------------------------ MMA issue
        if (lane == 0) {
            const uint32_t idesc = tc::idesc_i8(PB_TOKENS, PB_NT, true, true);
            for (int it = 0; it < total && !ctl->abort; ++it) {
                const int s = it % PB_STAGES, buf = it & 1;
                if (!pb_wait(&ctl->ab_full[s], (uint32_t)(it / PB_STAGES) & 1u, ctl, p.status)) break;
                if (!pb_wait(&ctl->tmem_empty[buf], (uint32_t)(it >> 1) & 1u, ctl, p.status)) break;
                tc::fence_after_sync();
                const uint32_t a_q = smem_addr(smem + PB_OFF_A + s * PB_A_SLOT), b_q = smem_addr(smem + PB_OFF_B + s * PB_B_SLOT);
                const uint64_t a0 = tc::smem_desc_sw128(a_q);
                const uint64_t a_thin = tc::smem_desc(a_q + PB_A_THIN, PB_A_COL, 128);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t d = tmem + (uint32_t)(buf * PB_BUF_COLS + j * PB_NT);
                    const uint32_t bj = b_q + (uint32_t)j * PB_B_BLOCK;
                    // K steps j and j + 1 of the activations against the two halves of block j's rows; accumulate = 1:
                    // the accumulators hold the float bias
                    tc::mma_i8(d, a0 + (uint64_t)(((j >> 2) * PB_A_SLAB + (j & 3) * 32) >> 4), tc::smem_desc(bj, 128, 512), idesc, 1);
                    if (j < 7) tc::mma_i8(d, a0 + (uint64_t)((((j + 1) >> 2) * PB_A_SLAB + ((j + 1) & 3) * 32) >> 4), tc::smem_desc(bj + 256, 128, 512), idesc, 1);
                    else tc::mma_i8(d, a_thin, tc::smem_desc(bj + 256, 128, 512), idesc, 1);
                }
                tc::commit(&ctl->tmem_full[buf]);
                tc::commit(&ctl->ab_empty[s]);
            }
        }
    } else if (warp < PB_E_WARPS) {
        // ------------------------------------------------------------------ epilogue: warp = (32-token quarter, 16 of the 32 weights)
        const int quarter = warp & 3, half = warp >> 2;
        const int row = quarter * 32 + lane;
        const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(half * 16);
        for (int buf = 0; buf < 2; ++buf) {
            for (int j = 0; j < 8; ++j) tmem_st16_fill(lane_base + (uint32_t)(buf * PB_BUF_COLS + j * PB_NT), PB_BIAS);
            tc::tmem_st_wait();
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->tmem_empty[buf]);
        }
        const uint64_t bias2 = pack2(-12582912.f, -12582912.f);
        uint64_t acc[8];
        int it = 0;
        bool ok = true;
        for (int t = 0; t < my_tiles && ok && !ctl->abort; ++t) {
            const int tile = (int)blockIdx.x + t * (int)gridDim.x;
            const long long n0 = (long long)(tile / p.m_tiles) * PB_NT + half * 16, m = (long long)(tile % p.m_tiles) * PB_TOKENS + row;
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = 0ull;
            for (int u = 0; u < units && ok; ++u, ++it) {
                const int buf = it & 1;
                if (!pb_wait(&ctl->tmem_full[buf], (uint32_t)(it >> 1) & 1u, ctl, p.status)) { ok = false; break; }
                tc::fence_after_sync();
                const uint4 dxh = *reinterpret_cast<const uint4 *>(smem + PB_OFF_DX + (it & (PB_RING - 1)) * PB_DX_SLOT + 16 * row);
                const uint32_t dxw[4] = {dxh.x, dxh.y, dxh.z, dxh.w};
                const float *dw = reinterpret_cast<const float *>(smem + PB_OFF_DW + (it & (PB_RING - 1)) * PB_DW_SLOT) + half * 16;
                const uint32_t cols = lane_base + (uint32_t)(buf * PB_BUF_COLS);
                uint32_t cur[16], nxt[16];
                tc::tmem_ld16(cols, cur);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    tc::tmem_ld_wait();
                    tmem_st16_fill(cols + (uint32_t)(j * PB_NT), PB_BIAS);
                    if (j < 7) tc::tmem_ld16(cols + (uint32_t)((j + 1) * PB_NT), nxt);   // in flight while block j is combined
                    const float dx = half_bits_to_float(j & 1 ? dxw[j >> 1] >> 16 : dxw[j >> 1]);
                    const uint64_t dx2 = pack2(dx, dx);
#pragma unroll
                    for (int i = 0; i < 16; i += 2) {
                        const uint64_t dw2 = *reinterpret_cast<const uint64_t *>(dw + j * PB_NT + i);
                        const uint64_t f = add2(pack2(__uint_as_float(cur[i]), __uint_as_float(cur[i + 1])), bias2);   // exact: the integer sum as a float
                        if (FMT == F_Q4_0) acc[i >> 1] = fma2(mul2(f, dw2), dx2, acc[i >> 1]);     // (isum * d_w) * d_x
                        else acc[i >> 1] = fma2(f, mul2(dw2, dx2), acc[i >> 1]);                  // isum * (d_w * d_x)
                    }
                    if (j < 7) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) cur[i] = nxt[i];
                    }
                }
                tc::tmem_st_wait();
                tc::fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&ctl->tmem_empty[buf]);
            }
            if (!ok) break;
            if (m < p.m) {
                float *out = p.y + (size_t)m * p.ldy + n0;
                const bool vec = (reinterpret_cast<uintptr_t>(out) & 15u) == 0;
#pragma unroll
                for (int i = 0; i < 16; i += 4) {
                    if (vec && n0 + i + 4 <= p.n) {
                        *reinterpret_cast<ulonglong2 *>(out + i) = make_ulonglong2(acc[i >> 1], acc[(i >> 1) + 1]);
                    } else {
                        float a0, a1, a2, a3;
                        unpack2(acc[i >> 1], a0, a1);
                        unpack2(acc[(i >> 1) + 1], a2, a3);
                        if (n0 + i < p.n) out[i] = a0;
                        if (n0 + i + 1 < p.n) out[i + 1] = a1;
                        if (n0 + i + 2 < p.n) out[i + 2] = a2;
                        if (n0 + i + 3 < p.n) out[i + 3] = a3;
                    }
                }
            }
        }
    }

    tc::fence_before_sync();
    __syncthreads();
    if (warp == PB_MMA_WARP) {
        __syncwarp();
        if (tmem != 0xffffffffu) tc::tmem_free(tmem, PB_TMEM_COLS);
    }
}


// ---------------------------------------------------------------------------------------------------------------------
// IQ2_XXS x Q8_K (production_mul_mat_iq2_xxs_staged, examples/kernels/mul_mat/iq2_xxs_staged.py:9-97; per block the math
// of examples/kernels/vec_dot/iq2_xxs_q8_k.py:8-54, GGML ggml-cpu/quants.c:855-895).  A 32-element group has its own
// integer scale 2 s + 1 (up to 31) on codebook values of up to 43: the product does not fit int8, so the groups are
// contracted one by one like the blocks above (two K = 32 steps against a 64-byte row, codes at the operand shift of
// the Q8_K record, accumulator g of 8) and combined in integers in the epilogue:
//   isum = sum_g (2 s_g + 1) * D_g;   acc += (d * x.d) * f32(isum);   Y = 0.125 * acc.
// The weight operand holds grid[index] * sign per element, built from the caller's two tables (staged in shared memory,
// the sign table as byte masks).  Records are 66 bytes at 2-byte alignment: the expanders read them from global memory
// with 16-bit loads, one unit ahead.  Activations as in prefill.cu: Q8_K records by TMA, codes at operand byte 4 W.
constexpr int PC_A_SLOT = PB_A_THIN + 3 * PB_A_COL;           // 38 KB: two slabs and three plain columns
constexpr int PC_LS_SLOT = 8 * PB_NT * 4;                      // 2 s + 1 per (group, weight)
constexpr int PC_DW_SLOT = PB_NT * 4;
constexpr int PC_XD_SLOT = PB_TOKENS * 4;
constexpr int PC_OFF_A = PB_CONTROL;
constexpr int PC_OFF_B = PC_OFF_A + PB_STAGES * PC_A_SLOT;
constexpr int PC_OFF_GRID = PC_OFF_B + PB_STAGES * PB_B_SLOT;  // int8[256][8]
constexpr int PC_OFF_NEG = PC_OFF_GRID + 2048;                 // per sign index 8 byte masks (0xff where the sign is -1)
constexpr int PC_OFF_LS = PC_OFF_NEG + 1024;
constexpr int PC_OFF_DW = PC_OFF_LS + PB_RING * PC_LS_SLOT;
constexpr int PC_OFF_XD = PC_OFF_DW + PB_RING * PC_DW_SLOT;
constexpr int PC_SMEM = PC_OFF_XD + PB_RING * PC_XD_SLOT;
static_assert(PC_A_SLOT % 1024 == 0 && PC_OFF_B % 1024 == 0 && PC_SMEM <= 227 * 1024, "codebook kernel shared memory");

struct CodebookParams {
    const uint8_t *w;          // (n, k) IQ2_XXS records
    const int8_t *grid, *signs;
    float *y;
    long long n, m, ldy;
    int units, m_tiles, n_tiles;
    int *status;
};

// the 16 bytes {index, meta} x 2 of groups 2x and 2x + 1 of one record, by 16-bit loads (records are 2-byte aligned)
__device__ __forceinline__ void pc_load_groups(const uint8_t *rec, int x, bool valid, uint32_t (&q)[4], uint32_t &d_bits) {
    if (valid) {
        const unsigned short *h = reinterpret_cast<const unsigned short *>(rec);
        d_bits = __ldg(h);
#pragma unroll
        for (int i = 0; i < 4; ++i) q[i] = (uint32_t)__ldg(h + 1 + 8 * x + 2 * i) | ((uint32_t)__ldg(h + 2 + 8 * x + 2 * i) << 16);
    } else {
        d_bits = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) q[i] = 0;
    }
}

// one group's 64-byte row: the 32 signed codebook values at word W (operand byte 4 W), zeros around them
template <int W>
__device__ __forceinline__ void pc_expand_group(uint32_t index, uint32_t meta, uint32_t grid, uint32_t neg, uint32_t row) {
    uint32_t v[8];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        uint2 gv, nm;
        asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(gv.x), "=r"(gv.y) : "r"(grid + 8u * byte_of(index, e)));
        asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(nm.x), "=r"(nm.y) : "r"(neg + 8u * ((meta >> (7 * e)) & 127u)));
        // negate the bytes under the mask: ~g + 1 per byte; g <= 43, so no carry leaves a byte
        v[2 * e] = (gv.x ^ nm.x) + (nm.x & 0x01010101u);
        v[2 * e + 1] = (gv.y ^ nm.y) + (nm.y & 0x01010101u);
    }
    uint32_t out[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) out[i] = (i >= W && i < W + 8) ? v[(i >= W && i < W + 8) ? i - W : 0] : 0u;
#pragma unroll
    for (int c = 0; c < 4; ++c) sts_u128(row + 128u * c, out[4 * c], out[4 * c + 1], out[4 * c + 2], out[4 * c + 3]);
}

__global__ void __launch_bounds__(PB_THREADS, 1) prefill_codebook_kernel(const CodebookParams p, const __grid_constant__ CUtensorMap x_wide,
                                                                          const __grid_constant__ CUtensorMap x_narrow) {
    extern __shared__ __align__(1024) uint8_t smem[];
    BlockControl *ctl = reinterpret_cast<BlockControl *>(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles = p.m_tiles * p.n_tiles;
    const int my_tiles = (tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const int units = p.units, total = my_tiles * units;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PB_STAGES; ++s) {
            mbar_init(&ctl->a_landed[s], 1);
            mbar_init(&ctl->ab_full[s], PB_X_WARPS + PB_S_WARPS); mbar_init(&ctl->ab_empty[s], 1);
        }
        for (int h = 0; h < 2; ++h) { mbar_init(&ctl->tmem_full[h], 1); mbar_init(&ctl->tmem_empty[h], PB_E_WARPS); }
        ctl->abort = 0;
        ctl->tmem_base = 0xffffffffu;
        mbar_fence_init();
    }
    // the caller's tables: the grid as it is, the signs (+1 / -1 per element) as byte masks
    for (int i = threadIdx.x; i < 512; i += PB_THREADS) reinterpret_cast<uint32_t *>(smem + PC_OFF_GRID)[i] = __ldg(reinterpret_cast<const uint32_t *>(p.grid) + i);
    for (int i = threadIdx.x; i < 256; i += PB_THREADS)
        reinterpret_cast<uint32_t *>(smem + PC_OFF_NEG)[i] = ((__ldg(reinterpret_cast<const uint32_t *>(p.signs) + i) >> 7) & 0x01010101u) * 0xffu;
    __syncthreads();
    if (warp == PB_MMA_WARP) tc::tmem_alloc(&ctl->tmem_base, PB_TMEM_COLS);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = ctl->tmem_base;
    auto tile_of = [&](int it) { return (int)blockIdx.x + (it / units) * (int)gridDim.x; };

    if (warp >= PB_X_WARP0 && warp < PB_X_WARP0 + PB_X_WARPS) {
        // ------------------------------------------------------------------ expanders: warp x = groups 2x, 2x + 1; lane = weight
        const int x = warp - PB_X_WARP0;
        const uint32_t grid = smem_addr(smem + PC_OFF_GRID), neg = smem_addr(smem + PC_OFF_NEG);
        auto record = [&](int it, bool &valid) {
            const int tile = tile_of(it);
            const long long n = (long long)(tile / p.m_tiles) * PB_NT + lane;
            valid = n < p.n;
            return p.w + ((size_t)(valid ? n : 0) * units + (it % units)) * 66;
        };
        uint32_t qn[4], dn;
        bool valid = false;
        if (total > 0) { const uint8_t *rec = record(0, valid); pc_load_groups(rec, x, valid, qn, dn); }
        for (int it = 0; it < total && !ctl->abort; ++it) {
            uint32_t q[4] = {qn[0], qn[1], qn[2], qn[3]};
            const uint32_t d_bits = dn;
            if (it + 1 < total) { const uint8_t *rec = record(it + 1, valid); pc_load_groups(rec, x, valid, qn, dn); }   // in flight while this unit is expanded
            const int s = it % PB_STAGES, words = ((it % units) & 3) + 1;
            if (!pb_wait(&ctl->ab_empty[s], ((uint32_t)(it / PB_STAGES) & 1u) ^ 1u, ctl, p.status)) break;
            const uint32_t b_slot = smem_addr(smem + PC_OFF_B + s * PB_B_SLOT);
            const uint32_t row0 = b_slot + (uint32_t)(2 * x) * PB_B_BLOCK + (uint32_t)(lane >> 3) * 512u + (uint32_t)(lane & 7) * 16u;
            switch (words) {
            case 1: pc_expand_group<1>(q[0], q[1], grid, neg, row0); pc_expand_group<1>(q[2], q[3], grid, neg, row0 + PB_B_BLOCK); break;
            case 2: pc_expand_group<2>(q[0], q[1], grid, neg, row0); pc_expand_group<2>(q[2], q[3], grid, neg, row0 + PB_B_BLOCK); break;
            case 3: pc_expand_group<3>(q[0], q[1], grid, neg, row0); pc_expand_group<3>(q[2], q[3], grid, neg, row0 + PB_B_BLOCK); break;
            default: pc_expand_group<4>(q[0], q[1], grid, neg, row0); pc_expand_group<4>(q[2], q[3], grid, neg, row0 + PB_B_BLOCK); break;
            }
            int *ls = reinterpret_cast<int *>(smem + PC_OFF_LS + (it & (PB_RING - 1)) * PC_LS_SLOT);
            ls[(2 * x) * PB_NT + lane] = (int)(2u * (q[1] >> 28) + 1u);
            ls[(2 * x + 1) * PB_NT + lane] = (int)(2u * (q[3] >> 28) + 1u);
            if (x == 0) reinterpret_cast<float *>(smem + PC_OFF_DW + (it & (PB_RING - 1)) * PC_DW_SLOT)[lane] = half_bits_to_float(d_bits);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->ab_full[s]);
        }
    } else if (warp >= PB_S_WARP0 && warp < PB_S_WARP0 + PB_S_WARPS) {
        // ------------------------------------------------------------------ x.d of every token (record byte 0 = operand byte 4 (W - 1))
        const int ts = threadIdx.x - 32 * PB_S_WARP0;
        for (int it = 0; it < total && !ctl->abort; ++it) {
            const int s = it % PB_STAGES, shift = 4 * ((it % units) & 3);
            if (!pb_wait(&ctl->a_landed[s], (uint32_t)(it / PB_STAGES) & 1u, ctl, p.status)) break;
            const uint32_t a_slot = smem_addr(smem + PC_OFF_A + s * PC_A_SLOT);
            const uint32_t xd_slot = smem_addr(smem + PC_OFF_XD + (it & (PB_RING - 1)) * PC_XD_SLOT);
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const int row = ts + 64 * k;
                sts_u32(xd_slot + 4u * (uint32_t)row, lds32(a_slot + sw128_offset(row, 0) + (uint32_t)shift));
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->ab_full[s]);
        }
    } else if (warp == PB_TMA_WARP) {
        // ------------------------------------------------------------------ activation boxes
        if (lane == 0) {
            int issued = 0;
            for (int it = 0; it < total && !ctl->abort; ++it) {
                const int s = it % PB_STAGES, b = it % units, tile = tile_of(it);
                const int m0 = (tile % p.m_tiles) * PB_TOKENS;
                if (!pb_wait(&ctl->ab_empty[s], ((uint32_t)(it / PB_STAGES) & 1u) ^ 1u, ctl, p.status)) break;
                fence_proxy_async();
                uint8_t *slot = smem + PC_OFF_A + s * PC_A_SLOT;
                const int x0 = 73 * b - (b & 3);       // the 16-byte boundary at or before record b of a token row, in words
                mbar_expect_tx(&ctl->a_landed[s], PC_A_SLOT);
                tma_load_2d(slot, &x_wide, x0, m0, &ctl->a_landed[s]);
                tma_load_2d(slot + PB_A_SLAB, &x_wide, x0 + 32, m0, &ctl->a_landed[s]);
                tma_load_2d(slot + PB_A_THIN, &x_narrow, x0 + 64, m0, &ctl->a_landed[s]);
                tma_load_2d(slot + PB_A_THIN + PB_A_COL, &x_narrow, x0 + 68, m0, &ctl->a_landed[s]);
                tma_load_2d(slot + PB_A_THIN + 2 * PB_A_COL, &x_narrow, x0 + 72, m0, &ctl->a_landed[s]);
                issued = it + 1;
            }
            for (int k = issued > PB_STAGES ? issued - PB_STAGES : 0; k < issued; ++k) mbar_wait(&ctl->a_landed[k % PB_STAGES], (uint32_t)(k / PB_STAGES) & 1u);
        }
    } else if (warp == PB_MMA_WARP) {
        // ------------------------------------------------------------------ MMA issue
        if (lane == 0) {
            const uint32_t idesc = tc::idesc_i8(PB_TOKENS, PB_NT, true, true);
            for (int it = 0; it < total && !ctl->abort; ++it) {
                const int s = it % PB_STAGES, buf = it & 1;
                if (!pb_wait(&ctl->ab_full[s], (uint32_t)(it / PB_STAGES) & 1u, ctl, p.status)) break;
                if (!pb_wait(&ctl->tmem_empty[buf], ((uint32_t)(it >> 1) & 1u) ^ 1u, ctl, p.status)) break;
                tc::fence_after_sync();
                const uint32_t a_q = smem_addr(smem + PC_OFF_A + s * PC_A_SLOT), b_q = smem_addr(smem + PC_OFF_B + s * PB_B_SLOT);
                const uint64_t a0 = tc::smem_desc_sw128(a_q);
                const uint64_t a_thin = tc::smem_desc(a_q + PB_A_THIN, PB_A_COL, 128);
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    const uint32_t d = tmem + (uint32_t)(buf * PB_BUF_COLS + g * PB_NT);
                    const uint32_t bg = b_q + (uint32_t)g * PB_B_BLOCK;
                    tc::mma_i8(d, a0 + (uint64_t)(((g >> 2) * PB_A_SLAB + (g & 3) * 32) >> 4), tc::smem_desc(bg, 128, 512), idesc, 0);
                    if (g < 7) tc::mma_i8(d, a0 + (uint64_t)((((g + 1) >> 2) * PB_A_SLAB + ((g + 1) & 3) * 32) >> 4), tc::smem_desc(bg + 256, 128, 512), idesc, 1);
                    else tc::mma_i8(d, a_thin, tc::smem_desc(bg + 256, 128, 512), idesc, 1);
                }
                tc::commit(&ctl->tmem_full[buf]);
                tc::commit(&ctl->ab_empty[s]);
            }
        }
    } else if (warp < PB_E_WARPS) {
        // ------------------------------------------------------------------ epilogue: warp = (32-token quarter, 16 of the 32 weights)
        const int quarter = warp & 3, half = warp >> 2;
        const int row = quarter * 32 + lane;
        const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(half * 16);
        float acc[16];
        int it = 0;
        bool ok = true;
        for (int t = 0; t < my_tiles && ok && !ctl->abort; ++t) {
            const int tile = (int)blockIdx.x + t * (int)gridDim.x;
            const long long n0 = (long long)(tile / p.m_tiles) * PB_NT + half * 16, m = (long long)(tile % p.m_tiles) * PB_TOKENS + row;
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[i] = 0.f;
            for (int u = 0; u < units && ok; ++u, ++it) {
                const int buf = it & 1;
                if (!pb_wait(&ctl->tmem_full[buf], (uint32_t)(it >> 1) & 1u, ctl, p.status)) { ok = false; break; }
                tc::fence_after_sync();
                const float xd = reinterpret_cast<const float *>(smem + PC_OFF_XD + (it & (PB_RING - 1)) * PC_XD_SLOT)[row];
                const float *dw = reinterpret_cast<const float *>(smem + PC_OFF_DW + (it & (PB_RING - 1)) * PC_DW_SLOT) + half * 16;
                const int4 *ls = reinterpret_cast<const int4 *>(smem + PC_OFF_LS + (it & (PB_RING - 1)) * PC_LS_SLOT) + half * 4;
                const uint32_t cols = lane_base + (uint32_t)(buf * PB_BUF_COLS);
                uint32_t cur[16], nxt[16];
                int isum[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) isum[i] = 0;
                tc::tmem_ld16(cols, cur);
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    tc::tmem_ld_wait();
                    if (g < 7) tc::tmem_ld16(cols + (uint32_t)((g + 1) * PB_NT), nxt);   // in flight while group g is combined
#pragma unroll
                    for (int i = 0; i < 16; i += 4) {
                        const int4 l = ls[g * (PB_NT / 4) + (i >> 2)];
                        isum[i] += (int)cur[i] * l.x; isum[i + 1] += (int)cur[i + 1] * l.y;
                        isum[i + 2] += (int)cur[i + 2] * l.z; isum[i + 3] += (int)cur[i + 3] * l.w;
                    }
                    if (g < 7) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) cur[i] = nxt[i];
                    }
                }
                tc::fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&ctl->tmem_empty[buf]);
#pragma unroll
                for (int i = 0; i < 16; ++i) acc[i] += (dw[i] * xd) * (float)isum[i];
            }
            if (!ok) break;
            if (m < p.m) {
                float *out = p.y + (size_t)m * p.ldy + n0;
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    if (n0 + i < p.n) out[i] = 0.125f * acc[i];
            }
        }
    }

    tc::fence_before_sync();
    __syncthreads();
    if (warp == PB_MMA_WARP) {
        __syncwarp();
        if (tmem != 0xffffffffu) tc::tmem_free(tmem, PB_TMEM_COLS);
    }
}

}  // namespace

bool prefill_blocks_supported(int fmt, long long n, long long k, long long m, const void *w, const void *xq) {
    // K a multiple of 256: a unit of eight records (272 / 144 bytes) then starts on a 16-byte boundary of every row,
    // which the TMA box copies of activations and raw weights need; both bases 16-byte aligned
    return (fmt == F_Q4_0 || fmt == F_Q8_0) && m >= 32 && k > 0 && k % 256 == 0 && n > 0 && n < (1LL << 31) && m < (1LL << 31) &&
           (reinterpret_cast<uintptr_t>(w) & 15u) == 0 && (reinterpret_cast<uintptr_t>(xq) & 15u) == 0;
}

bool prefill_codebook_supported(int fmt, long long n, long long k, long long m, const void *w, const void *xq) {
    // K a multiple of 1024: Q8_K rows (292 bytes per 256) are then whole 16-byte multiples, which the TMA box loads need
    return fmt == F_IQ2_XXS && m >= 32 && k > 0 && k % 1024 == 0 && n > 0 && n < (1LL << 31) && m < (1LL << 31) &&
           (reinterpret_cast<uintptr_t>(w) & 1u) == 0 && (reinterpret_cast<uintptr_t>(xq) & 15u) == 0;
}

cudaError_t launch_prefill_codebook(const PrefillArgs &a, const int8_t *grid, const int8_t *signs, int sm_count, cudaStream_t stream) {
    if (!prefill_codebook_supported(a.fmt, a.n, a.k, a.m, a.w, a.xq) || !grid || !signs) return cudaErrorNotSupported;
    if ((reinterpret_cast<uintptr_t>(grid) & 3u) || (reinterpret_cast<uintptr_t>(signs) & 3u)) return cudaErrorNotSupported;
    CodebookParams p;
    p.w = static_cast<const uint8_t *>(a.w); p.grid = grid; p.signs = signs;
    p.y = a.y; p.n = a.n; p.m = a.m; p.ldy = a.ldy; p.units = (int)(a.k / 256); p.status = a.status;
    p.m_tiles = (int)((a.m + PB_TOKENS - 1) / PB_TOKENS);
    p.n_tiles = (int)((a.n + PB_NT - 1) / PB_NT);
    const long long tiles = (long long)p.m_tiles * p.n_tiles;
    CUtensorMap x_wide, x_narrow;
    cudaError_t e = encode_tile_map(&x_wide, CU_TENSOR_MAP_DATA_TYPE_UINT32, a.xq, (unsigned long long)p.units * 73, (unsigned long long)a.m,
                                    (unsigned long long)p.units * 292, 32, PB_TOKENS, true);
    if (e == cudaSuccess)
        e = encode_tile_map(&x_narrow, CU_TENSOR_MAP_DATA_TYPE_UINT32, a.xq, (unsigned long long)p.units * 73, (unsigned long long)a.m,
                            (unsigned long long)p.units * 292, 4, PB_TOKENS, false);
    if (e == cudaSuccess) e = grant_dynamic_smem(reinterpret_cast<const void *>(prefill_codebook_kernel), PC_SMEM);
    if (e != cudaSuccess) return e;
    const int grid_size = (int)(tiles < sm_count ? tiles : sm_count);
    prefill_codebook_kernel<<<grid_size, PB_THREADS, PC_SMEM, stream>>>(p, x_wide, x_narrow);
    return cudaGetLastError();
}

cudaError_t launch_prefill_blocks(const PrefillArgs &a, int sm_count, cudaStream_t stream) {
    if (!prefill_blocks_supported(a.fmt, a.n, a.k, a.m, a.w, a.xq)) return cudaErrorNotSupported;
    BlockParams p;
    p.y = a.y; p.n = a.n; p.m = a.m; p.ldy = a.ldy; p.units = (int)(a.k / 256); p.status = a.status;
    p.m_tiles = (int)((a.m + PB_TOKENS - 1) / PB_TOKENS);
    p.n_tiles = (int)((a.n + PB_NT - 1) / PB_NT);
    const long long tiles = (long long)p.m_tiles * p.n_tiles;
    const int raw_words = a.fmt == F_Q8_0 ? 68 : 36;
    CUtensorMap x_wide, x_narrow, w_rows;
    // the Q8_0 activations as (m) rows of 68 words per unit; the weights as (n) rows of 68 / 36 words per unit
    cudaError_t e = encode_tile_map(&x_wide, CU_TENSOR_MAP_DATA_TYPE_UINT32, a.xq, (unsigned long long)p.units * 68, (unsigned long long)a.m,
                                    (unsigned long long)p.units * 272, 32, PB_TOKENS, true);
    if (e == cudaSuccess)
        e = encode_tile_map(&x_narrow, CU_TENSOR_MAP_DATA_TYPE_UINT32, a.xq, (unsigned long long)p.units * 68, (unsigned long long)a.m,
                            (unsigned long long)p.units * 272, 4, PB_TOKENS, false);
    if (e == cudaSuccess)
        e = encode_tile_map(&w_rows, CU_TENSOR_MAP_DATA_TYPE_UINT32, a.w, (unsigned long long)p.units * raw_words, (unsigned long long)a.n,
                            (unsigned long long)p.units * raw_words * 4, (unsigned)raw_words, PB_NT, false);
    if (e != cudaSuccess) return e;
    const int grid = (int)(tiles < sm_count ? tiles : sm_count);
    if (a.fmt == F_Q8_0) {
        e = grant_dynamic_smem(reinterpret_cast<const void *>(prefill_blocks_kernel<F_Q8_0>), PB_SMEM);
        if (e != cudaSuccess) return e;
        prefill_blocks_kernel<F_Q8_0><<<grid, PB_THREADS, PB_SMEM, stream>>>(p, x_wide, x_narrow, w_rows);
    } else {
        e = grant_dynamic_smem(reinterpret_cast<const void *>(prefill_blocks_kernel<F_Q4_0>), PB_SMEM);
        if (e != cudaSuccess) return e;
        prefill_blocks_kernel<F_Q4_0><<<grid, PB_THREADS, PB_SMEM, stream>>>(p, x_wide, x_narrow, w_rows);
    }
    return cudaGetLastError();
}

}  // namespace weft
