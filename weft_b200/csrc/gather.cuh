// All-gather of row-sharded mul_mat outputs over NVLink peer memory, without a library collective.
//
// Every rank owns a full (M, N) output buffer, a sync block and (optionally) a staging area, all mapped into
// every other rank (CUDA IPC).  Only peer stores cross NVLink: no peer loads, no multicast.  Two protocols:
//
// * Flagged values, for decode-sized outputs (M * N <= GATHER_LL_MAX_VALUES).  A rank's GEMV stores each result
//   it computes into every peer's staging area as one 8-byte {value, epoch} word; after its own rows a warp
//   turns to the words it expects from the other ranks, polls each (bounded) until its epoch shows up, and
//   writes the value into the local output.  No fence and no barrier: a step costs the GEMV plus one NVLink
//   crossing.  The epoch (one per launch) alternates between two staging halves of GATHER_LL_MAX_VALUES words each,
//   whatever the shape of the call (consecutive calls of different shapes may share one staging area); a rank
//   cannot start storing epoch e + 2 before every peer has finished reading epoch e, because finishing e + 1
//   needs the peers' e + 1.
// * Fence and barrier, for large outputs (prefill).  Results go straight into every rank's output buffer; the
//   last warp of the grid to finish publishes this rank's epoch in every peer's sync block and waits (bounded)
//   until every peer's epoch has arrived in its own.  Writer warps fence at system scope before they count
//   themselves done, the last warp fences again before it publishes, so a rank that sees the epoch sees the
//   data.  Consecutive steps must alternate between two output buffers.
//
// Sync block (int[32], zero-initialised): [p] = last epoch published by rank p (barrier protocol), [16] = done
// counter of the running grid, [17] = this rank's epoch (number of gathers completed).
#pragma once

#include "common.cuh"

namespace weft {

constexpr int GATHER_MAX_RANKS = 8;
constexpr long long GATHER_LL_MAX_VALUES = 1 << 16;   // flagged-value protocol up to this many outputs (M * N)

struct GatherArgs {
    float *y[GATHER_MAX_RANKS];     // per rank: its output buffer, already offset to this rank's first column
    int *sync[GATHER_MAX_RANKS];    // per rank: its sync block
    uint2 *stage[GATHER_MAX_RANKS]; // per rank: its staging area, 2 x GATHER_LL_MAX_VALUES words (flagged-value protocol only)
    long long n0;                   // this rank's first column
    long long values;               // M * N
    int world;                      // 0 or 1: no gather
    int rank;
    int ll;                         // 1: flagged-value protocol
};

// The epoch of this launch; read by every thread after the preceding kernel has completed.
__device__ __forceinline__ int gather_epoch(const GatherArgs &g) {
    return *reinterpret_cast<volatile int *>(g.sync[g.rank] + 17) + 1;
}

// Store one result (output row `row`, column `col` of this rank's block, row pitch ldy = N) for every other rank.
__device__ __forceinline__ void gather_store(const GatherArgs &g, int epoch, long long row, long long col, long long ldy, float v) {
    if (g.ll) {
        const size_t slot = (size_t)(epoch & 1) * GATHER_LL_MAX_VALUES + (size_t)row * ldy + (size_t)(g.n0 + col);
        for (int r = 0; r < g.world; ++r)   // one 8-byte store: value and tag arrive together
            if (r != g.rank)
                asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" :: "l"(g.stage[r] + slot), "r"(__float_as_uint(v)), "r"((uint32_t)epoch) : "memory");
    } else {
        for (int r = 0; r < g.world; ++r)
            if (r != g.rank) g.y[r][(size_t)row * ldy + col] = v;
    }
}

// The same for a group of lanes that all hold the result: lane `sub` of the group stores to ONE peer (the peers' stores
// leave together instead of one after the other from a single lane).  Lanes with sub >= world - 1 do nothing.
__device__ __forceinline__ void gather_store_spread(const GatherArgs &g, int epoch, long long row, long long col, long long ldy, float v, int sub) {
    if (sub >= g.world - 1) return;
    const int r = sub + (sub >= g.rank ? 1 : 0);
    if (g.ll) {
        const size_t slot = (size_t)(epoch & 1) * GATHER_LL_MAX_VALUES + (size_t)row * ldy + (size_t)(g.n0 + col);
        asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" :: "l"(g.stage[r] + slot), "r"(__float_as_uint(v)), "r"((uint32_t)epoch) : "memory");
    } else {
        g.y[r][(size_t)row * ldy + col] = v;
    }
}

// How many CTAs of a fused GEMV take the receiving side.  The others leave as soon as their rows are stored, so the
// next launch in the stream finds free SMs and streams its first weights while the values are still crossing NVLink.
constexpr int GATHER_RECV_CTAS = 12;

// Flagged-value protocol: this warp's share (`warp_index` of `warps`) of the values the other ranks send;
// n_local = columns this rank computes, ldy = N, m = output rows.
__device__ __forceinline__ void gather_receive(const GatherArgs &g, int epoch, long long m, long long n_local, long long ldy,
                                               int warp_index, int warps, int *status) {
    if (!g.ll) return;
    const long long others = ldy - n_local, total = m * others;
    float *out = g.y[g.rank] - g.n0;
    const uint2 *stage = g.stage[g.rank] + (size_t)(epoch & 1) * GATHER_LL_MAX_VALUES;
    for (long long i = (long long)warp_index * 32 + (threadIdx.x & 31); i < total; i += (long long)warps * 32) {
        const long long row = i / others, c = i % others;
        const size_t at = (size_t)row * ldy + (size_t)(c < g.n0 ? c : c + n_local);
        const uint2 *slot = stage + at;
        uint32_t value = 0, tag = 0;
        bool arrived = false;
        for (uint32_t spin = 0; spin < (1u << 22) && !arrived; ++spin) {
            asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(value), "=r"(tag) : "l"(slot));
            arrived = tag == (uint32_t)epoch;
        }
        if (!arrived) { report(status, ST_WAIT_TIMEOUT); return; }
        out[at] = __uint_as_float(value);
    }
}

// Called once by every whole warp that may have stored results, after its last store (and after gather_receive);
// `expected` = how many warps of the grid call it.  Warps that leave early on an error never call it: the epoch
// is then never completed and the peers' bounded waits report the failure.
__device__ __forceinline__ void gather_finish(const GatherArgs &g, int epoch, int *status, int expected) {
    if (!g.ll) __threadfence_system();
    __syncwarp();
    const int lane = threadIdx.x & 31;
    int *local = g.sync[g.rank];
    int last = 0;
    if (lane == 0) last = atomicAdd(local + 16, 1) == expected - 1;
    last = __shfl_sync(0xffffffffu, last, 0);
    if (!last) return;
    __threadfence();
    if (lane == 0) {
        volatile int *state = local;
        state[17] = epoch;
        state[16] = 0;
    }
    if (g.ll) return;
    __threadfence_system();
    if (lane < g.world && lane != g.rank) {
        volatile int *remote = g.sync[lane] + g.rank;
        *remote = epoch;
        volatile int *mine = local + lane;
        bool arrived = false;
        for (uint32_t spin = 0; spin < (1u << 22) && !arrived; ++spin) arrived = (*mine - epoch) >= 0;
        if (!arrived) report(status, ST_WAIT_TIMEOUT);
    }
    __threadfence_system();
}

}  // namespace weft
