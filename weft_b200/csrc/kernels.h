// Host-side launchers of the sm_100a kernels (internal; the public surface is include/weft_b200.h).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "gather.cuh"

namespace weft {

// Raises a kernel's dynamic shared-memory limit to at least `bytes` on the CURRENT device.  The attribute belongs
// to the (function, device) pair, so what was already granted is remembered per device; defined in gemv.cu.
cudaError_t grant_dynamic_smem(const void *kernel, int bytes);

// W: `elements` logical values as contiguous records of `fmt`; Y: `elements` floats.
cudaError_t launch_dequantize(int fmt, const void *w, const int8_t *grid, const int8_t *signs, const uint32_t *powers,
                              float *y, long long elements, int sm_count, cudaStream_t stream);

// dst[0..bytes) = src[0..bytes) by a kernel (either side may be mapped pinned host memory): for the small host
// arguments of a call this is a few microseconds quicker than a copy-engine transfer between two kernels.
cudaError_t launch_copy_bytes(void *dst, const void *src, size_t bytes, cudaStream_t stream);

// X (rows, k) fp32 -> Q8_0 / Q8_K records, Weft rounding and tie rules.
cudaError_t launch_quantize(int act_fmt, const float *x, void *y, long long rows, long long k, int sm_count, cudaStream_t stream);

constexpr int GEMV_MAX_SEGMENTS = 4;

struct GemvArgs {
    int fmt;                 // weight format
    const void *w;           // (n, k) records
    const void *xq;          // (m, k) activation records (Q8_0 or Q8_K); written when x is given
    const float *x;          // (m, k) fp32 activations, 16-byte aligned rows: the kernel quantizes them itself; else NULL
    const int8_t *grid;      // IQ2_XXS only
    const int8_t *signs;     // IQ2_XXS only
    const uint32_t *powers;  // TQ1_0 only
    float *y;                // (m, ldy) fp32; column n of row r at y[r * ldy + n]
    long long n, k, m, ldy;
    int *status;             // mapped status word
    bool y_on_host;          // y is pinned host memory seen through its device mapping: store it in few, wide pieces
    GatherArgs gather;       // world > 1: results also go to every peer's buffer and the launch ends with the ranks' barrier
    // Several weight matrices against the same activations in one launch (m = 1): matrix i has seg_rows[i] rows at
    // seg_w[i] and writes seg_y[i]; w / y / n are then unused.  0 or 1: the single matrix w.
    int segments;
    const void *seg_w[GEMV_MAX_SEGMENTS];
    float *seg_y[GEMV_MAX_SEGMENTS];
    long long seg_rows[GEMV_MAX_SEGMENTS];
};
// true when launch_gemv_q4k takes these matrices as one grouped launch
bool gemv_q4k_groups(const GemvArgs &a);
// true when the kernel launch_gemv() picks for `a` does the peer stores and the barrier itself
bool gemv_gathers(const GemvArgs &a);
cudaError_t launch_gemv(const GemvArgs &a, int sm_count, cudaStream_t stream);
// Q4_K x Q8_K specialisation (producer/consumer ring, activations in registers)
bool gemv_q4k_supported(const GemvArgs &a);
cudaError_t launch_gemv_q4k(const GemvArgs &a, int sm_count, cudaStream_t stream);
// Q4_0 / Q8_0 / IQ2_XXS / TQ1_0 with 16-byte-multiple rows: the same CTA-wide producer/consumer ring
bool gemv_ring_supported(const GemvArgs &a);
cudaError_t launch_gemv_ring(const GemvArgs &a, int sm_count, cudaStream_t stream);

// Q4K_I[16]: the same GEMV over 16-row byte-interleaved Q4_K records (n a multiple of 16), and the
// artifact function that produces that layout from plain records
bool gemv_q4ki_supported(const GemvArgs &a);
cudaError_t launch_gemv_q4ki(const GemvArgs &a, int sm_count, cudaStream_t stream);
cudaError_t launch_interleave_q4k(const void *source, void *target, long long rows, long long k, int sm_count, cudaStream_t stream);

struct PrefillArgs {
    int fmt;
    const void *w;           // (n, k) records
    const void *xq;          // (m, k) Q8_K records (already quantized)
    const uint32_t *powers;  // TQ1_0 only
    float *y;                // (m, ldy)
    long long n, k, m, ldy;
    int *status;
};
// tcgen05 int8 tensor-core path; returns cudaErrorNotSupported for shapes it does not take.
cudaError_t launch_prefill(const PrefillArgs &a, int sm_count, cudaStream_t stream);
bool prefill_supported(int fmt, long long n, long long k, long long m, const void *w, const void *xq);
// The same contraction on CTA pairs (256 tokens per tile, tcgen05 cta_group::2): Q4_K with more than 128 tokens.
cudaError_t launch_prefill_pair(const PrefillArgs &a, int sm_count, cudaStream_t stream);
bool prefill_pair_supported(int fmt, long long n, long long k, long long m, const void *w, const void *xq);
int prefill_pair_launches(int fmt);   // kernels one launch_prefill_pair call puts on the stream (the plane kernel counts)

// Q4_0 / Q8_0 x Q8_0 with more than a few tokens: one K = 32 contraction per 32-element block (both operands carry a
// scale per block), accumulators rotating through tensor memory, scales applied in the epilogue.
cudaError_t launch_prefill_blocks(const PrefillArgs &a, int sm_count, cudaStream_t stream);
bool prefill_blocks_supported(int fmt, long long n, long long k, long long m, const void *w, const void *xq);

// IQ2_XXS x Q8_K with more than a few tokens: one contraction per 32-element group (integer scale 2 s + 1 per group),
// combined in integers in the epilogue; grid int8[256][8] and signs int8[128][8] (+1 / -1) in device memory.
cudaError_t launch_prefill_codebook(const PrefillArgs &a, const int8_t *grid, const int8_t *signs, int sm_count, cudaStream_t stream);
bool prefill_codebook_supported(int fmt, long long n, long long k, long long m, const void *w, const void *xq);

// Bare tcgen05.mma issue loop on every SM (mode 0: kind::i8, one CTA per SM; 1: kind::i8 on CTA pairs; 2: kind::f16):
// spans_dev receives the nanoseconds each issuing CTA took; *ops_per_launch the operations the whole launch performs.
cudaError_t measure_mma_peak(int mode, int iterations, int sm_count, unsigned long long *spans_dev, int *status, cudaStream_t stream, double *ops_per_launch);

// Push an (m, n_local) column block that this rank has already written into its own buffer (g.y[g.rank], row
// pitch ldy) to every peer, then run the ranks' barrier: the two-launch form for kernels without fused stores.
cudaError_t launch_gather_push(const GatherArgs &g, long long m, long long n_local, long long ldy, int *status, int sm_count, cudaStream_t stream);

}  // namespace weft
