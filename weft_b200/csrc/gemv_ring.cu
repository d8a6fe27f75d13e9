// Decode GEMV for Q4_0, Q8_0, Q2_K, Q3_K, Q5_K, Q6_K, IQ1_S, IQ1_M, IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS, IQ3_S and TQ1_0 weights whose rows are whole 16-byte multiples:
// Y[m, n] = quantized_vec_dot(W[n], Xq[m])  (examples/kernels/mul_mat/{q4_0,q8_0,q2_k,q3_k,q5_k,q6_k,iq2_xxs,tq1_0}_decode.py).
//
// Same streaming scheme as the Q4_K kernel: one persistent CTA per SM, a producer warp that fills a
// CTA-wide shared-memory ring with bulk asynchronous copies of about 18 KB (copies of a few KB each
// reach well under half of the HBM rate), stages dealt round-robin over the grid so that the whole grid
// reads one contiguous window of the matrix, consumer warps that wait on a stage's "full" barrier and
// arrive on its "empty" barrier, bounded waits throughout, programmatic dependent launch.
//
// A consumer iteration takes 2 * (32 / L) consecutive rows of one stage, L = lanes per row (the power of
// two >= units per row, at most 32): lane group g computes rows 2g and 2g + 1 of the iteration, each lane
// one 256-element unit of both rows per step (two independent instruction streams), and the group
// reduces with shuffles.  A row is never split across warps, so results do not depend on the grid.
#include "gemv_units.cuh"
#include "ring.cuh"

#include <cstdlib>

namespace weft {

namespace {

constexpr int RG_MAX_STAGES = 24;
constexpr int RG_MAX_THREADS = 512;
// IQ2_XXS waits on table lookups, needs 64 registers, and gains from twice the warps
// (Q5_K and Q3_K were tried with the same bound: capped at 64 registers they spill, 10.7 -> 11.0 us and 8.8 -> 11.4 us)
__host__ __device__ constexpr bool is_codebook(int fmt) { return fmt == F_IQ2_XXS || fmt == F_IQ2_XS || fmt == F_IQ3_XXS || fmt == F_IQ2_S || fmt == F_IQ3_S || fmt == F_IQ1_S || fmt == F_IQ1_M; }
__host__ __device__ constexpr bool has_sign_table(int fmt) { return fmt == F_IQ2_XXS || fmt == F_IQ2_XS || fmt == F_IQ3_XXS; }
// the codebook formats whose two rows of record words fit in 64 registers run twice the warps; the others (20 to 27 words per
// row) spill at that bound and keep 128 registers and fifteen consumer warps (28672 x 8192: IQ2_XS 42.2 -> 31.2 us, IQ2_S
// 49.0 -> 36.8, IQ3_XXS 46.5 -> 33.8, IQ3_S 62.2 -> 46.9; twenty-three warps at 80 registers: 34.1 / 41.1 / 36.6 / 52.4)
__host__ __device__ constexpr bool many_warps(int fmt) { return fmt == F_IQ2_XXS || fmt == F_IQ1_S || fmt == F_IQ1_M; }
constexpr int ring_max_threads(int fmt, int rl = 2) { return (many_warps(fmt) || rl == 1) ? 1024 : RG_MAX_THREADS; }
// bank-striped copies of the grid (IQ2_XXS: 256 entries x 128 bytes; IQ2_XS: 512 x 128; IQ3_XXS: 256 x 128; IQ2_S: 1024
// entries x 32 bytes, four copies; IQ3_S: 512 x 128; IQ1_S / IQ1_M: 2048 entries x 32 bytes, four copies: IQ1_S 31.6 -> 30.6 us against the plain 16 KB table), then, where the format has a sign table, of the sign masks (128 x 128)
__host__ __device__ constexpr int codebook_grid_bytes(int fmt) { return (fmt == F_IQ2_XS || fmt == F_IQ3_S || fmt == F_IQ1_S || fmt == F_IQ1_M) ? 65536 : is_codebook(fmt) ? 32768 : 0; }
__host__ __device__ constexpr int codebook_table_bytes(int fmt) { return is_codebook(fmt) ? codebook_grid_bytes(fmt) + (has_sign_table(fmt) ? 16384 : 0) : 0; }

struct RingParams {
    const uint8_t *w;
    const uint8_t *xq;
    const float *x;
    const int8_t *grid;
    const int8_t *signs;
    const uint32_t *powers;
    float *y;
    long long n;
    long long ldy;
    int nb;              // 256-element units per row
    int log_lanes;       // lanes per row = 1 << log_lanes
    int log_stage_rows;  // rows per ring stage
    int log_stages;      // ring depth
    int full_rounds;
    int tail_rows;
    int inflight;        // copies the producer keeps outstanding (issued, not yet landed)
    int *status;
    GatherArgs gather;
};

// GATHER: the launch also does the peer all-gather (a separate instantiation: the plain kernel carries none of it)
template <int FMT, bool QX, int RL, bool GATHER>
__global__ void __launch_bounds__(ring_max_threads(FMT, RL)) gemv_ring_kernel(const RingParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int UB = Unit<FMT>::BYTES;
    constexpr bool ACT_Q8_0 = (FMT == F_Q4_0 || FMT == F_Q8_0);
    constexpr int TABLE_BYTES = codebook_table_bytes(FMT);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb = p.nb, LSR = p.log_stage_rows, SR = 1 << LSR, LS = p.log_stages, S = 1 << LS;
    const int LL = p.log_lanes, L = 1 << LL, RPI = RL * (32 >> LL);   // rows per consumer iteration
    const uint32_t row_bytes = (uint32_t)nb * UB, stage_bytes = row_bytes << LSR;
    const int G = gridDim.x, b = blockIdx.x;

    volatile int *s_issued = reinterpret_cast<volatile int *>(smem);
    uint64_t *s_full = reinterpret_cast<uint64_t *>(smem + 16);
    uint64_t *s_empty = s_full + RG_MAX_STAGES;
    uint8_t *s_grid = smem + 512, *s_neg = s_grid + codebook_grid_bytes(FMT);
    uint8_t *s_xq = smem + 512 + TABLE_BYTES;
    uint8_t *s_aux = s_xq + (size_t)nb * XQ_PITCH;
    uint8_t *s_ring = smem + ((512 + TABLE_BYTES + (size_t)nb * (XQ_PITCH + XAUX_BYTES) + 127) & ~size_t(127));
    const uint32_t ring_addr = smem_addr(s_ring), full_addr = smem_addr(s_full), empty_addr = smem_addr(s_empty);

    const long long main_rows = (long long)p.full_rounds * G * SR;
    const long long tail_begin = min(p.n, main_rows + (long long)b * p.tail_rows);
    const int tail_here = (int)(min(p.n, tail_begin + p.tail_rows) - tail_begin);
    const int rows_here = p.full_rounds * SR + tail_here;
    const int total_stages = p.full_rounds + (tail_here > 0 ? 1 : 0);
    const size_t xq_row = (size_t)blockIdx.y * nb * (ACT_Q8_0 ? 272 : 292);
    float *y = p.y + (size_t)blockIdx.y * p.ldy;

    asm volatile("griddepcontrol.launch_dependents;");
    if (threadIdx.x < S) {
        mbar_init(s_full + threadIdx.x, 1);
        mbar_init(s_empty + threadIdx.x, (uint32_t)(SR / RPI));   // one arrival per consumer iteration
        mbar_fence_init();
    }
    if (threadIdx.x == 0) *s_issued = 0;
    __syncthreads();

    auto issue = [&](int s) {
        const int slot = s & (S - 1);
        const bool tail = s >= p.full_rounds;
        const long long row0 = tail ? tail_begin : ((long long)s * G + b) << LSR;
        const uint32_t bytes = tail ? (uint32_t)tail_here * row_bytes : stage_bytes;
        mbar_expect_tx_a(full_addr + 8 * slot, bytes);
        bulk_g2s_a(ring_addr + (uint32_t)slot * stage_bytes, p.w + (size_t)row0 * row_bytes, bytes, full_addr + 8 * slot);
    };
    if (warp == 0 && lane == 0) {
        const int first = min(min(S, p.inflight), total_stages);
        for (int s = 0; s < first; ++s) issue(s);
        *s_issued = first;
    }

    // Activations, tables and outputs may belong to the kernel that precedes this one in the stream.
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const int epoch = GATHER ? gather_epoch(p.gather) : 0;
    if (FMT == F_IQ2_XXS) stage_iq2_tables_striped(p.grid, p.signs, s_grid, s_neg);
    if (FMT == F_IQ2_XS) { stage_striped8(p.grid, 512, s_grid, false); stage_striped8(p.signs, 128, s_neg, true); }
    if (FMT == F_IQ3_XXS) { stage_striped4(p.grid, 256, s_grid); stage_striped8(p.signs, 128, s_neg, true); }
    if (FMT == F_IQ2_S) stage_striped8x4(p.grid, 1024, s_grid);
    if (FMT == F_IQ3_S) stage_striped4(p.grid, 512, s_grid);
    if (FMT == F_IQ1_S || FMT == F_IQ1_M) stage_striped8x4(p.grid, 2048, s_grid);
    uint32_t pw[5] = {1, 3, 9, 27, 81};
    if (FMT == F_TQ1_0) {
#pragma unroll
        for (int i = 0; i < 5; ++i) pw[i] = __ldg(p.powers + i) & 0xffu;
    }
    if (QX) {
        uint8_t *out = b == 0 ? const_cast<uint8_t *>(p.xq) + xq_row : nullptr;
        const float *x = p.x + (size_t)blockIdx.y * nb * 256;
        if (ACT_Q8_0) quantize_stage_q8_0(x, nb, s_xq, s_aux, out); else quantize_stage_q8_k(x, nb, s_xq, s_aux, out);
    } else {
        if (ACT_Q8_0) stage_q8_0(p.xq + xq_row, nb, s_xq, s_aux); else stage_q8_k(p.xq + xq_row, nb, s_xq, s_aux);
    }
    __syncthreads();

    if (warp == 0) {
        if (lane == 0) {
            // stage s goes out when its slot is free and stage s - P has landed (at most P copies outstanding:
            // issuing the whole ring at once makes every copy land together, late)
            const int P = min(S, p.inflight);
            for (int s = min(P, total_stages); s < total_stages; ++s) {
                if (s >= S) {
                    if (!mbar_wait_a(empty_addr + 8 * (s & (S - 1)), (uint32_t)((s >> LS) - 1) & 1u)) { report(p.status, ST_WAIT_TIMEOUT); return; }
                    fence_proxy_async();
                }
                if (!mbar_wait_a(full_addr + 8 * ((s - P) & (S - 1)), (uint32_t)((s - P) >> LS) & 1u)) { report(p.status, ST_WAIT_TIMEOUT); return; }
                issue(s);
                *s_issued = s + 1;
            }
        }
        return;
    }

    const int consumers = (blockDim.x >> 5) - 1;
    const int group = lane >> LL, ul = lane & (L - 1);
    for (int t = RPI * (warp - 1); t < rows_here; t += RPI * consumers) {
        const int s = t >> LSR;   // SR is a multiple of RPI: the iteration's rows lie in one stage
        if (*s_issued <= s) {     // a parity wait cannot tell fill n of a slot from fill n-2
            bool issued = false;
            for (uint32_t spin = 0; spin < (1u << 24) && !issued; ++spin) issued = *s_issued > s;
            if (!issued) { report(p.status, ST_WAIT_TIMEOUT); return; }
        }
        if (!mbar_wait_a(full_addr + 8 * (s & (S - 1)), (uint32_t)(s >> LS) & 1u)) { report(p.status, ST_WAIT_TIMEOUT); return; }
        const uint8_t *stage = s_ring + (size_t)(s & (S - 1)) * stage_bytes;
        const int in_stage = (t & (SR - 1)) + RL * group;
        const int ta = t + RL * group;
        bool live[RL];
        const uint8_t *base[RL];
        float acc[RL];
#pragma unroll
        for (int r = 0; r < RL; ++r) {   // rows past the end read row 0 of the stage (always valid) and are dropped
            live[r] = ta + r < rows_here;
            base[r] = stage + (size_t)(live[r] ? in_stage + r : 0) * row_bytes;
            acc[r] = 0.f;
        }
        for (int u = ul; u < nb; u += L) {
            const uint8_t *wp[RL];
#pragma unroll
            for (int r = 0; r < RL; ++r) wp[r] = base[r] + (size_t)u * UB;
            const uint8_t *xu = s_xq + u * XQ_PITCH, *xa = s_aux + u * XAUX_BYTES;
            if (FMT == F_Q4_0) dot_q4_0<RL>(wp, xu, xa, acc);
            else if (FMT == F_Q8_0) dot_q8_0<RL>(wp, xu, xa, acc);
            else if (FMT == F_Q2_K) dot_q2_k<RL>(wp, xu, xa, acc);
            else if (FMT == F_Q3_K) dot_q3_k<RL>(wp, xu, xa, acc);
            else if (FMT == F_Q5_K) dot_q5_k<RL>(wp, xu, xa, acc);
            else if (FMT == F_Q6_K) dot_q6_k<RL>(wp, xu, xa, acc);
            else if (FMT == F_IQ2_XXS) dot_iq2_xxs<RL, 128>(wp, xu, xa, s_grid + 8 * (lane & 15), s_neg + 8 * (lane & 15), acc);
            else if (FMT == F_IQ2_XS) dot_iq2_xs<RL, 128>(wp, xu, xa, s_grid + 8 * (lane & 15), s_neg + 8 * (lane & 15), acc);
            else if (FMT == F_IQ3_XXS) dot_iq3_xxs<RL, 128, 128>(wp, xu, xa, s_grid + 4 * lane, s_neg + 8 * (lane & 15), acc);
            else if (FMT == F_IQ2_S) dot_iq2_s<RL, 32>(wp, xu, xa, s_grid + 8 * (lane & 3), acc);
            else if (FMT == F_IQ3_S) dot_iq3_s<RL, 128>(wp, xu, xa, s_grid + 4 * lane, acc);
            else if (FMT == F_IQ1_S) dot_iq1_s<RL, 32>(wp, xu, xa, s_grid + 8 * (lane & 3), acc);
            else if (FMT == F_IQ1_M) dot_iq1_m<RL, 32>(wp, xu, xa, s_grid + 8 * (lane & 3), reinterpret_cast<const float *>(p.powers), acc);
            else dot_tq1_0<RL>(wp, xu, xa, pw, acc);
        }
#pragma unroll
        for (int r = 0; r < RL; ++r) {
            for (int o = L >> 1; o > 0; o >>= 1) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], o);
            if (FMT == F_IQ2_XXS || FMT == F_IQ2_XS || FMT == F_IQ2_S) acc[r] *= 0.125f;
            if (FMT == F_IQ3_XXS) acc[r] *= 0.25f;
        }
        __syncwarp();   // every lane's shared loads of this stage have completed
        if (ul == 0) {
            const long long grow = s < p.full_rounds ? ((((long long)s * G + b) << LSR) + in_stage) : tail_begin + (ta - (p.full_rounds << LSR));
#pragma unroll
            for (int r = 0; r < RL; ++r) {
                if (!live[r]) continue;
                y[grow + r] = acc[r];
                if (GATHER) gather_store(p.gather, epoch, blockIdx.y, grow + r, p.ldy, acc[r]);
            }
        }
        if (lane == 0) mbar_arrive_a(empty_addr + 8 * (s & (S - 1)));
    }
    if (GATHER) {
        // a few CTAs receive for the whole grid; the others are done
        const int recv = min((int)gridDim.x, GATHER_RECV_CTAS), warps = (int)(gridDim.x * gridDim.y) * consumers;
        if ((int)blockIdx.x < recv && blockIdx.y == 0)
            gather_receive(p.gather, epoch, gridDim.y, p.n, p.ldy, (int)blockIdx.x * consumers + warp - 1, recv * consumers, p.status);
        gather_finish(p.gather, epoch, p.status, warps);
    }
}

constexpr int kRingConsumers = 0;   // 0: 15, or kRingIq2Consumers for IQ2_XXS
constexpr int kRingIq2Consumers = 27;   // measured 28672 x 8192: 15 -> 29.0 us, 19 -> 28.0, 23 -> 27.1, 27 -> 26.5, 31 -> 26.8
constexpr int kRingStageBytes = 18432;
constexpr int kRingMaxStages = 8;
constexpr int kRingOverlap = 1;
constexpr int kRingInflight = 3;
constexpr int kRingSmemKB = 224;
constexpr int kRingTwoIterations = 1;

struct RingPlan { int log_lanes, log_stage_rows, log_stages; size_t smem; bool ok; };

RingPlan plan_ring(int fmt, long long nb) {
    RingPlan plan{0, 0, 0, 0, false};
    const long long row_bytes = nb * unit_bytes(fmt);
    if (row_bytes % 16 != 0 || nb <= 0) return plan;
    const long long fixed = (512 + codebook_table_bytes(fmt) + nb * (XQ_PITCH + XAUX_BYTES) + 127) & ~127LL;
    int ll = 0;
    while ((1 << ll) < 32 && (1 << ll) < nb) ++ll;
    const int log_rpi = 1 + (5 - ll);
    int lsr = log_rpi;   // at least one consumer iteration per stage
    while (lsr < 8 && (row_bytes << (lsr + 1)) <= kRingStageBytes) ++lsr;
    const long long cap = (long long)kRingSmemKB * 1024;
    // A stage that is a single consumer iteration is drained by one warp while the others wait for the next copy:
    // take two iterations per stage when eight such stages still fit (Q5_K 14336 x 4096: 10.7 -> 8.2 us).
    if (lsr == log_rpi && kRingTwoIterations && fixed + ((row_bytes << (lsr + 1)) << 3) <= cap) ++lsr;
    int ls = 0;
    while ((1 << (ls + 1)) <= kRingMaxStages && (1 << (ls + 1)) <= RG_MAX_STAGES && fixed + ((row_bytes << lsr) << (ls + 1)) <= cap) ++ls;
    if (ls < 1) return plan;
    plan.log_lanes = ll; plan.log_stage_rows = lsr; plan.log_stages = ls;
    plan.smem = (size_t)(fixed + ((row_bytes << lsr) << ls)) + 16;   // the 2-byte-aligned record loaders read up to 4 bytes past a record
    plan.ok = true;
    return plan;
}

template <int FMT, bool QX, int RL, bool GATHER>
cudaError_t launch_variant(const RingParams &p, dim3 grid, int threads, size_t smem, cudaStream_t stream) {
    cudaError_t granted = grant_dynamic_smem(reinterpret_cast<const void *>(gemv_ring_kernel<FMT, QX, RL, GATHER>), (int)smem);
    if (granted != cudaSuccess) return granted;
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = dim3((unsigned)threads);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = kRingOverlap ? 1 : 0;
    config.attrs = attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, gemv_ring_kernel<FMT, QX, RL, GATHER>, p);
}

template <int FMT>
cudaError_t launch_fmt(const RingParams &p, bool qx, dim3 grid, int threads, size_t smem, cudaStream_t stream) {
    // two rows per lane group and iteration; one row (half the registers, up to 31 warps) measured no better:
    // Q6_K 14336 x 4096 11.0 vs 10.4 us, Q5_K 8.4 vs 8.5, Q3_K 9.1 vs 9.2, Q2_K 7.7 vs 7.7
    if (p.gather.world > 1)
        return qx ? launch_variant<FMT, true, 2, true>(p, grid, threads, smem, stream) : launch_variant<FMT, false, 2, true>(p, grid, threads, smem, stream);
    return qx ? launch_variant<FMT, true, 2, false>(p, grid, threads, smem, stream) : launch_variant<FMT, false, 2, false>(p, grid, threads, smem, stream);
}

}  // namespace

bool gemv_ring_supported(const GemvArgs &a) {
    if (a.fmt != F_Q4_0 && a.fmt != F_Q8_0 && a.fmt != F_Q2_K && a.fmt != F_Q3_K && a.fmt != F_Q5_K && a.fmt != F_Q6_K && a.fmt != F_IQ2_XXS && a.fmt != F_IQ2_XS && a.fmt != F_IQ3_XXS && a.fmt != F_IQ2_S && a.fmt != F_IQ3_S && a.fmt != F_IQ1_S && a.fmt != F_IQ1_M && a.fmt != F_TQ1_0) return false;
    return a.k % 256 == 0 && a.k > 0 && (reinterpret_cast<uintptr_t>(a.w) & 15u) == 0 && a.n < (1LL << 30) &&
           plan_ring(a.fmt, a.k / 256).ok;
}

cudaError_t launch_gemv_ring(const GemvArgs &a, int sm_count, cudaStream_t stream) {
    RingParams p;
    p.w = static_cast<const uint8_t *>(a.w); p.xq = static_cast<const uint8_t *>(a.xq); p.x = a.x;
    p.grid = a.grid; p.signs = a.signs; p.powers = a.powers; p.y = a.y;
    p.n = a.n; p.ldy = a.ldy; p.nb = (int)(a.k / 256); p.status = a.status; p.gather = a.gather; p.inflight = kRingInflight < 1 ? 1 : kRingInflight;
    const RingPlan plan = plan_ring(a.fmt, p.nb);
    if (!plan.ok) return cudaErrorInvalidConfiguration;
    p.log_lanes = plan.log_lanes; p.log_stage_rows = plan.log_stage_rows; p.log_stages = plan.log_stages;
    const long long stage_rows = 1LL << plan.log_stage_rows;
    long long ctas = (a.n + stage_rows - 1) / stage_rows;
    if (ctas > sm_count) ctas = sm_count;
    if (ctas < 1) ctas = 1;
    p.full_rounds = (int)(a.n / (ctas * stage_rows));
    const long long rest = a.n - (long long)p.full_rounds * ctas * stage_rows;
    p.tail_rows = (int)((rest + ctas - 1) / ctas);
    const int most = ring_max_threads(a.fmt) / 32 - 1;
    int consumers = kRingConsumers < 1 ? (many_warps(a.fmt) ? kRingIq2Consumers : 15) : kRingConsumers;
    if (consumers > most) consumers = most;
    if (consumers < 1) consumers = 1;
    const int threads = (consumers + 1) * 32;
    dim3 grid((unsigned)ctas, (unsigned)a.m);
    const bool qx = a.x != nullptr;
    switch (a.fmt) {
    case F_Q4_0: return launch_fmt<F_Q4_0>(p, qx, grid, threads, plan.smem, stream);
    case F_Q8_0: return launch_fmt<F_Q8_0>(p, qx, grid, threads, plan.smem, stream);
    case F_Q2_K: return launch_fmt<F_Q2_K>(p, qx, grid, threads, plan.smem, stream);
    case F_Q3_K: return launch_fmt<F_Q3_K>(p, qx, grid, threads, plan.smem, stream);
    case F_Q5_K: return launch_fmt<F_Q5_K>(p, qx, grid, threads, plan.smem, stream);
    case F_Q6_K: return launch_fmt<F_Q6_K>(p, qx, grid, threads, plan.smem, stream);
    case F_IQ2_XXS: return launch_fmt<F_IQ2_XXS>(p, qx, grid, threads, plan.smem, stream);
    case F_IQ2_XS: return launch_fmt<F_IQ2_XS>(p, qx, grid, threads, plan.smem, stream);
    case F_IQ3_XXS: return launch_fmt<F_IQ3_XXS>(p, qx, grid, threads, plan.smem, stream);
    case F_IQ2_S: return launch_fmt<F_IQ2_S>(p, qx, grid, threads, plan.smem, stream);
    case F_IQ3_S: return launch_fmt<F_IQ3_S>(p, qx, grid, threads, plan.smem, stream);
    case F_IQ1_S: return launch_fmt<F_IQ1_S>(p, qx, grid, threads, plan.smem, stream);
    case F_IQ1_M: return launch_fmt<F_IQ1_M>(p, qx, grid, threads, plan.smem, stream);
    default: return launch_fmt<F_TQ1_0>(p, qx, grid, threads, plan.smem, stream);
    }
}

}  // namespace weft
