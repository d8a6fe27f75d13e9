/* weft_b200 -- C ABI of the B200 (sm_100a) quantized matrix path.
 *
 * Every kernel symbol below carries the name, pointer order and trailing size_t dimension order of
 * the C function the reference compiler emits for the same @weft.kernel definition (one function per
 * kernel: pointers in signature order, then every unbound shape symbol as size_t in first-appearance
 * order -- lib/Target/Emission/Emitter.h:205-229,491-512), so the reference's FFI
 * (python/weft/runtime/compiler.py:91-97,154: argtypes = void* x nargs + size_t x ndims) binds them
 * unchanged.  Two differences, both additive:
 *   - the reference functions return void; these return int (0 = ok, non-zero = error, message from
 *     weft_b200_last_error()).  A caller that ignores the return value sees the reference behaviour.
 *   - every pointer may be a device pointer or a host pointer.  Device pointers are used in place.
 *     Host pointers are staged through a device-side arena the library keeps and grows on demand
 *     (inputs copied in, written arguments copied back inside the call) -- the literal drop-in for
 *     the reference's host-memory callers.  Host weights registered with weft_b200_weights_resident() are uploaded once and
 *     found again by address, so only activations and outputs move per call.
 *
 * Records are the GGML block formats, never repacked: Q4_0 18 B/32, Q8_0 34 B/32, Q4_K 144 B/256,
 * Q2_K 84 B/256, Q3_K 110 B/256, Q5_K 176 B/256, Q6_K 210 B/256, Q8_K 292 B/256, IQ2_XXS 66 B/256, IQ1_S 50 B/256, IQ1_M 56 B/256, IQ2_XS 74 B/256, IQ2_S 82 B/256, IQ3_XXS 98 B/256, IQ3_S 110 B/256, TQ1_0 54 B/256.  No entry point allocates a hidden workspace for
 * device-pointer arguments: Xq is the caller's written workspace, as in the reference.
 * Codebook tables arrive as arguments: grid int8[256][8] (IQ2_XXS), int8[512][8] (IQ2_XS), int8[256][4] (IQ3_XXS, values
 * 4..62), int8[1024][8] (IQ2_S), int8[512][4] (IQ3_S), int8[2048][8] with values -1 / 0 / +1 (IQ1_S, IQ1_M); signs int8[128][8] with entries +1 / -1 (IQ2_S and IQ3_S carry
 * their sign bits in the record and take no sign table).
 * TQ1_0 takes powers uint32[5] = {1, 3, 9, 27, 81}.
 *
 * Calls are synchronous by default (they return after the work has finished, like the reference's
 * blocking C call).  weft_b200_set_stream / weft_b200_set_async let a caller that owns a CUDA stream
 * enqueue without waiting.
 */
#ifndef WEFT_B200_H
#define WEFT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ library control (no reference counterpart) */

const char *weft_b200_last_error(void);              /* message of the calling thread's last failure */
int weft_b200_init(int device);                      /* select the device (default: current); idempotent */
int weft_b200_device_info(int *cc_major, int *cc_minor, int *sm_count, size_t *total_bytes, char *name, size_t name_len);
int weft_b200_set_stream(void *cuda_stream);         /* NULL = the library's own stream */
int weft_b200_set_async(int enabled);                /* 1: device-pointer calls return after enqueue */
int weft_b200_synchronize(void);                     /* wait for the stream and report device-side status */
unsigned long long weft_b200_launch_count(void);     /* kernels launched by this library so far */
int weft_b200_peek_status(void);                     /* the raw device status word (0 = none); makes no CUDA call, so it
                                                        can still be read after the context has reported an error */
/* Tensor-core issue rate of the bound device, measured: a bare loop of tcgen05.mma instructions (M 128 per SM, N 256)
 * on every SM, slowest SM's time.  mode 0: kind::i8, K = 32; 1: the same on CTA pairs (cta_group::2); 2: kind::f16,
 * K = 16.  *tera_ops = 1e12 operations per second.  The roofline denominator of the prefill kernels. */
int weft_b200_mma_peak(int mode, double *tera_ops);
/* Keep a device copy of a host weight buffer; later calls that receive an address inside
 * [host, host+bytes) use the copy.  The host bytes must not change while registered. */
int weft_b200_weights_resident(const void *host, size_t bytes);
int weft_b200_weights_release(const void *host);

/* ------------------------------------------------------------------ quantized_vec_dot: one row x one activation row -> Y[1]
 * examples/kernels/vec_dot/q4_0_q8_0.py:18-23      harness binding examples/repro/weft/vec_dot_runtime.cpp:191 */
int quantized_vec_dot_q4_0_q8_0(const uint8_t *W, const uint8_t *X, float *Y, size_t K);
/* examples/kernels/vec_dot/q8_0_q8_0.py:17-22      vec_dot_runtime.cpp:223 */
int quantized_vec_dot_q8_0_q8_0(const uint8_t *W, const uint8_t *X, float *Y, size_t K);
/* examples/kernels/vec_dot/q4_k_q8_k.py:31-36      vec_dot_runtime.cpp:247 */
int quantized_vec_dot_q4_k_q8_k(const uint8_t *W, const uint8_t *X, float *Y, size_t K);
/* examples/kernels/vec_dot/iq2_xxs_q8_k.py:45-54   vec_dot_runtime.cpp:303 */
int quantized_vec_dot_iq2_xxs_q8_k(const uint8_t *W, const uint8_t *X, const int8_t *grid, const int8_t *signs, float *Y, size_t K);
/* examples/kernels/vec_dot/iq2_xs_q8_k.py:9-39     vec_dot_runtime.cpp:289-296 */
int quantized_vec_dot_iq2_xs_q8_k(const uint8_t *W, const uint8_t *X, const int8_t *grid, const int8_t *signs, float *Y, size_t K);
/* examples/kernels/vec_dot/iq3_xxs_q8_k.py:70-76   vec_dot_runtime.cpp:313-320 */
int quantized_vec_dot_iq3_xxs_q8_k(const uint8_t *W, const uint8_t *X, const int8_t *grid, const int8_t *signs, float *Y, size_t K);
/* examples/kernels/vec_dot/iq2_s_q8_k.py:68-73     vec_dot_runtime.cpp:281-288 */
int quantized_vec_dot_iq2_s_q8_k(const uint8_t *W, const uint8_t *X, const int8_t *grid, float *Y, size_t K);
/* examples/kernels/vec_dot/iq3_s_q8_k.py:67-72     vec_dot_runtime.cpp:305-312 */
int quantized_vec_dot_iq3_s_q8_k(const uint8_t *W, const uint8_t *X, const int8_t *grid, float *Y, size_t K);
/* examples/kernels/vec_dot/iq1_s_q8_k.py:51-56     vec_dot_runtime.cpp:265-272 */
int quantized_vec_dot_iq1_s_q8_k(const uint8_t *W, const uint8_t *X, const int8_t *grid, float *Y, size_t K);
/* examples/kernels/vec_dot/iq1_m_q8_k.py:73-79, iq1_m_q8_k_lane16.py:85-91   vec_dot_runtime.cpp:273-280
 * (f16_bits: float[65536], entry b the value of the f16 bit pattern b, as the reference's harness builds it) */
int quantized_vec_dot_iq1_m_q8_k(const uint8_t *W, const uint8_t *X, const int8_t *grid, const float *f16_bits, float *Y, size_t K);
int quantized_vec_dot_iq1_m_q8_k_lane16(const uint8_t *W, const uint8_t *X, const int8_t *grid, const float *f16_bits, float *Y, size_t K);
/* examples/kernels/vec_dot/tq1_0_q8_k.py:47-55     vec_dot_runtime.cpp:343 */
int quantized_vec_dot_tq1_0_q8_k(const uint8_t *W, const uint8_t *X, const uint32_t *powers, float *Y, size_t K);
/* examples/kernels/vec_dot/tq1_0_q8_k_lane16.py:9-54 (the same dot product written with sixteen-wide partial sums
 * for the reference's vector target; identical integer sums, so the same kernel serves both names) */
int quantized_vec_dot_tq1_0_q8_k_lane16(const uint8_t *W, const uint8_t *X, const uint32_t *powers, float *Y, size_t K);

/* ------------------------------------------------------------------ row_dequantize: one row of K elements -> fp32
 * examples/kernels/dequantize/q4_0.py:9-13, q8_0.py:9-13, q4_k.py:9-20   examples/repro/weft/row_dequantize_runtime.cpp:177,197,212 */
int row_dequantize_q4_0(const uint8_t *W, float *Y, size_t K);
int row_dequantize_q8_0(const uint8_t *W, float *Y, size_t K);
int row_dequantize_q4_k(const uint8_t *W, float *Y, size_t K);
/* examples/kernels/dequantize/iq2_xxs.py:9-53; grid int8[2048], signs int8[1024]   row_dequantize_runtime.cpp:247 */
int row_dequantize_iq2_xxs(const uint8_t *W, const int8_t *grid, const int8_t *signs, float *Y, size_t K);
/* examples/kernels/dequantize/iq2_xs.py:9-68; grid int8[4096], signs int8[1024]    row_dequantize_runtime.cpp:239-242 */
int row_dequantize_iq2_xs(const uint8_t *W, const int8_t *grid, const int8_t *signs, float *Y, size_t K);
/* examples/kernels/dequantize/iq3_xxs.py:9-14; grid int8[1024], signs int8[1024]   row_dequantize_runtime.cpp:254-257 */
int row_dequantize_iq3_xxs(const uint8_t *W, const int8_t *grid, const int8_t *signs, float *Y, size_t K);
/* examples/kernels/dequantize/iq2_s.py:9-13; grid int8[8192]    row_dequantize_runtime.cpp:234-237 */
int row_dequantize_iq2_s(const uint8_t *W, const int8_t *grid, float *Y, size_t K);
/* examples/kernels/dequantize/iq3_s.py:9-13; grid int8[2048]    row_dequantize_runtime.cpp:249-252 */
int row_dequantize_iq3_s(const uint8_t *W, const int8_t *grid, float *Y, size_t K);
/* examples/kernels/dequantize/iq1_s.py:9-13, iq1_m.py:18-23; grid int8[16384] */
int row_dequantize_iq1_s(const uint8_t *W, const int8_t *grid, float *Y, size_t K);
int row_dequantize_iq1_m(const uint8_t *W, const int8_t *grid, const float *f16_bits, float *Y, size_t K);
/* examples/kernels/dequantize/tq1_0.py:9-46        row_dequantize_runtime.cpp:272 */
int row_dequantize_tq1_0(const uint8_t *W, const uint32_t *powers, float *Y, size_t K);

/* ------------------------------------------------------------------ activation quantizers, one row
 * examples/kernels/quantize/q8_0.py:20-23, q8_1.py:28-30, q8_k.py:32-35   examples/repro/weft/q8_quantize_runtime.cpp:13-26
 * Q8_1 (36 B/32: f16 d, f16 s = f16(sum of codes * d), 32 codes) is the activation format of the *_1 weight
 * formats; only its quantizer is exported. */
int q8_0_quantize(const float *X, uint8_t *Y, size_t K);
int q8_1_quantize(const float *X, uint8_t *Y, size_t K);
int q8_K_quantize(const float *X, uint8_t *Y, size_t K);

/* ------------------------------------------------------------------ production_mul_mat, decode form (GEMV per activation row)
 * W (N,K) records, X (M,K) fp32, Xq (M,K) activation records (written), Y (M,N) fp32 (written).
 * examples/kernels/mul_mat/q4_0_decode.py:10-20, q8_0_decode.py, q4_k_decode.py:10-20
 * examples/repro/weft/mul_mat_runtime.cpp:217-221,277-281,332-336 */
int production_mul_mat_q4_0_decode(const uint8_t *W, const float *X, uint8_t *Xq, float *Y, size_t N, size_t K, size_t M);
int production_mul_mat_q8_0_decode(const uint8_t *W, const float *X, uint8_t *Xq, float *Y, size_t N, size_t K, size_t M);
int production_mul_mat_q4_k_decode(const uint8_t *W, const float *X, uint8_t *Xq, float *Y, size_t N, size_t K, size_t M);
/* examples/kernels/mul_mat/iq2_xxs_decode.py:10-23   mul_mat_runtime.cpp:458-473 */
int production_mul_mat_iq2_xxs_decode(const uint8_t *W, const float *X, uint8_t *Xq, const int8_t *grid, const int8_t *signs,
                                      float *Y, size_t N, size_t K, size_t M);
/* examples/kernels/mul_mat/tq1_0_decode.py:10-21     mul_mat_runtime.cpp:534-538 */
int production_mul_mat_tq1_0_decode(const uint8_t *W, const float *X, uint8_t *Xq, const uint32_t *powers,
                                    float *Y, size_t N, size_t K, size_t M);
/* examples/kernels/mul_mat/tq1_0_lane16_decode.py:10-23 (decode GEMV over the lane16 dot product: same function) */
int production_mul_mat_tq1_0_lane16_decode(const uint8_t *W, const float *X, uint8_t *Xq, const uint32_t *powers,
                                           float *Y, size_t N, size_t K, size_t M);

/* ------------------------------------------------------------------ production_mul_mat, prefill form (tiled contraction)
 * Same arguments.  The reference binds its tile sizes (NC/MC/MR/NR/KC) at compile time
 * (Emitter.h:505-510), so they are not C parameters here either.
 * examples/kernels/mul_mat/q4_0.py:9-30, q8_0.py:9-29, q4_k_staged.py:9-37   mul_mat_runtime.cpp:217-221,277-281,350-357
 * From 32 tokens on these run on the int8 tensor cores (Q4_K: two scaled limbs per 256-block, CTA pairs above 128
 * tokens; Q4_0 / Q8_0: one contraction per 32-element block); smaller batches run the decode GEMV per token row. */
int production_mul_mat_q4_0(const uint8_t *W, const float *X, uint8_t *Xq, float *Y, size_t N, size_t K, size_t M);
int production_mul_mat_q8_0(const uint8_t *W, const float *X, uint8_t *Xq, float *Y, size_t N, size_t K, size_t M);
int production_mul_mat_q4_k_staged(const uint8_t *W, const float *X, uint8_t *Xq, float *Y, size_t N, size_t K, size_t M);
/* examples/kernels/mul_mat/tq1_0.py:10-64            mul_mat_runtime.cpp:534-538
 * (tensor cores from 32 tokens on when K is a multiple of 1024; CTA pairs above 128 tokens when K is a multiple of 2048) */
int production_mul_mat_tq1_0(const uint8_t *W, const float *X, uint8_t *Xq, const uint32_t *powers,
                             float *Y, size_t N, size_t K, size_t M);
/* examples/kernels/mul_mat/iq2_xxs_staged.py:9-97    mul_mat_runtime.cpp:458-473
 * (from 32 tokens on, K a multiple of 1024: one tensor-core contraction per 32-element group, integer group scales
 * combined in the epilogue) */
int production_mul_mat_iq2_xxs_staged(const uint8_t *W, const float *X, uint8_t *Xq, const int8_t *grid, const int8_t *signs,
                                      float *Y, size_t N, size_t K, size_t M);
/* examples/kernels/mul_mat/iq2_xxs.py:10-17: the function of the staged form under the reference's other name */
int production_mul_mat_iq2_xxs(const uint8_t *W, const float *X, uint8_t *Xq, const int8_t *grid, const int8_t *signs,
                               float *Y, size_t N, size_t K, size_t M);
/* examples/kernels/mul_mat/iq2_xs.py:26-33, iq2_xs_staged.py:29-36   mul_mat_runtime.cpp:434-447;
 * examples/kernels/mul_mat/iq3_xxs.py:10-17                          mul_mat_runtime.cpp:485-494
 * (the decode GEMV once per token row at any token count) */
int production_mul_mat_iq2_xs(const uint8_t *W, const float *X, uint8_t *Xq, const int8_t *grid, const int8_t *signs,
                              float *Y, size_t N, size_t K, size_t M);
int production_mul_mat_iq2_xs_staged(const uint8_t *W, const float *X, uint8_t *Xq, const int8_t *grid, const int8_t *signs,
                                     float *Y, size_t N, size_t K, size_t M);
int production_mul_mat_iq3_xxs(const uint8_t *W, const float *X, uint8_t *Xq, const int8_t *grid, const int8_t *signs,
                               float *Y, size_t N, size_t K, size_t M);
/* examples/kernels/mul_mat/iq2_s.py:10-16, iq2_s_staged.py:29-35   mul_mat_runtime.cpp:419-431;
 * examples/kernels/mul_mat/iq3_s.py:10-16                         mul_mat_runtime.cpp:475-483 */
int production_mul_mat_iq2_s(const uint8_t *W, const float *X, uint8_t *Xq, const int8_t *grid, float *Y, size_t N, size_t K, size_t M);
int production_mul_mat_iq2_s_staged(const uint8_t *W, const float *X, uint8_t *Xq, const int8_t *grid, float *Y, size_t N, size_t K, size_t M);
int production_mul_mat_iq3_s(const uint8_t *W, const float *X, uint8_t *Xq, const int8_t *grid, float *Y, size_t N, size_t K, size_t M);
/* examples/kernels/mul_mat/iq1_s.py:9-15, iq1_s_decode.py:10-16           mul_mat_runtime.cpp:389-401;
 * examples/kernels/mul_mat/iq1_m.py:10-17, iq1_m_decode.py:10-17, iq1_m_lane16_decode.py:10-17   mul_mat_runtime.cpp:404-416 */
int production_mul_mat_iq1_s(const uint8_t *W, const float *X, uint8_t *Xq, const int8_t *grid, float *Y, size_t N, size_t K, size_t M);
int production_mul_mat_iq1_s_decode(const uint8_t *W, const float *X, uint8_t *Xq, const int8_t *grid, float *Y, size_t N, size_t K, size_t M);
int production_mul_mat_iq1_m(const uint8_t *W, const float *X, uint8_t *Xq, const int8_t *grid, const float *f16_bits, float *Y, size_t N, size_t K, size_t M);
int production_mul_mat_iq1_m_decode(const uint8_t *W, const float *X, uint8_t *Xq, const int8_t *grid, const float *f16_bits, float *Y, size_t N, size_t K, size_t M);
int production_mul_mat_iq1_m_lane16_decode(const uint8_t *W, const float *X, uint8_t *Xq, const int8_t *grid, const float *f16_bits, float *Y, size_t N, size_t K, size_t M);

/* ------------------------------------------------------------------ whole-matrix forms (no reference counterpart)
 * The reference's standalone symbols above take one row and its harness loops rows on the host
 * (vec_dot_runtime.cpp:468-475, row_dequantize_runtime.cpp:433-438).  One launch per row is
 * meaningless on a GPU, so the same kernels are also exported over (N,K) views. */
int row_dequantize_q4_0_rows(const uint8_t *W, float *Y, size_t N, size_t K);
int row_dequantize_q8_0_rows(const uint8_t *W, float *Y, size_t N, size_t K);
int row_dequantize_q4_k_rows(const uint8_t *W, float *Y, size_t N, size_t K);
int row_dequantize_iq2_xxs_rows(const uint8_t *W, const int8_t *grid, const int8_t *signs, float *Y, size_t N, size_t K);
int row_dequantize_iq2_xs_rows(const uint8_t *W, const int8_t *grid, const int8_t *signs, float *Y, size_t N, size_t K);
int row_dequantize_iq3_xxs_rows(const uint8_t *W, const int8_t *grid, const int8_t *signs, float *Y, size_t N, size_t K);
int row_dequantize_iq2_s_rows(const uint8_t *W, const int8_t *grid, float *Y, size_t N, size_t K);
int row_dequantize_iq3_s_rows(const uint8_t *W, const int8_t *grid, float *Y, size_t N, size_t K);
int row_dequantize_iq1_s_rows(const uint8_t *W, const int8_t *grid, float *Y, size_t N, size_t K);
int row_dequantize_iq1_m_rows(const uint8_t *W, const int8_t *grid, const float *f16_bits, float *Y, size_t N, size_t K);
int row_dequantize_tq1_0_rows(const uint8_t *W, const uint32_t *powers, float *Y, size_t N, size_t K);
/* Y[n] = vec_dot(W[n], X) for n < N; X one row of activation records */
int quantized_vec_dot_q4_0_q8_0_rows(const uint8_t *W, const uint8_t *X, float *Y, size_t N, size_t K);
int quantized_vec_dot_q8_0_q8_0_rows(const uint8_t *W, const uint8_t *X, float *Y, size_t N, size_t K);
int quantized_vec_dot_q4_k_q8_k_rows(const uint8_t *W, const uint8_t *X, float *Y, size_t N, size_t K);
int quantized_vec_dot_iq2_xxs_q8_k_rows(const uint8_t *W, const uint8_t *X, const int8_t *grid, const int8_t *signs, float *Y, size_t N, size_t K);
int quantized_vec_dot_iq2_xs_q8_k_rows(const uint8_t *W, const uint8_t *X, const int8_t *grid, const int8_t *signs, float *Y, size_t N, size_t K);
int quantized_vec_dot_iq3_xxs_q8_k_rows(const uint8_t *W, const uint8_t *X, const int8_t *grid, const int8_t *signs, float *Y, size_t N, size_t K);
int quantized_vec_dot_iq2_s_q8_k_rows(const uint8_t *W, const uint8_t *X, const int8_t *grid, float *Y, size_t N, size_t K);
int quantized_vec_dot_iq3_s_q8_k_rows(const uint8_t *W, const uint8_t *X, const int8_t *grid, float *Y, size_t N, size_t K);
int quantized_vec_dot_iq1_s_q8_k_rows(const uint8_t *W, const uint8_t *X, const int8_t *grid, float *Y, size_t N, size_t K);
int quantized_vec_dot_iq1_m_q8_k_rows(const uint8_t *W, const uint8_t *X, const int8_t *grid, const float *f16_bits, float *Y, size_t N, size_t K);
int quantized_vec_dot_iq1_m_q8_k_lane16_rows(const uint8_t *W, const uint8_t *X, const int8_t *grid, const float *f16_bits, float *Y, size_t N, size_t K);
int quantized_vec_dot_tq1_0_q8_k_rows(const uint8_t *W, const uint8_t *X, const uint32_t *powers, float *Y, size_t N, size_t K);
int q8_0_quantize_rows(const float *X, uint8_t *Y, size_t M, size_t K);
int q8_1_quantize_rows(const float *X, uint8_t *Y, size_t M, size_t K);
int q8_K_quantize_rows(const float *X, uint8_t *Y, size_t M, size_t K);

/* ------------------------------------------------------------------ Q2_K x Q8_K (ggml-common.h:288-298 block_q2_K: scales[16],
 * qs[64], f16 d, f16 dmin; ggml-quants.c:903-933, ggml-cpu/quants.c:514-564; Encoding examples/formats/ggml.py:64-72).
 * examples/kernels/vec_dot/q2_k_q8_k.py:28-32          vec_dot_runtime.cpp:231-232 */
int quantized_vec_dot_q2_k_q8_k(const uint8_t *W, const uint8_t *X, float *Y, size_t K);
int quantized_vec_dot_q2_k_q8_k_rows(const uint8_t *W, const uint8_t *X, float *Y, size_t N, size_t K);
/* examples/kernels/dequantize/q2_k.py:8-17             row_dequantize_runtime.cpp:202,358 */
int row_dequantize_q2_k(const uint8_t *W, float *Y, size_t K);
int row_dequantize_q2_k_rows(const uint8_t *W, float *Y, size_t N, size_t K);
/* examples/kernels/mul_mat/q2_k_decode.py:10-20, q2_k.py:9-41     mul_mat_runtime.cpp:292-296
 * (both run the decode GEMV once per activation row) */
int production_mul_mat_q2_k_decode(const uint8_t *W, const float *X, uint8_t *Xq, float *Y, size_t N, size_t K, size_t M);
int production_mul_mat_q2_k(const uint8_t *W, const float *X, uint8_t *Xq, float *Y, size_t N, size_t K, size_t M);

/* ------------------------------------------------------------------ Q3_K x Q8_K (ggml-common.h:305-311 block_q3_K: hmask[32],
 * qs[64], scales[12], f16 d; ggml-quants.c:1247-1294, ggml-cpu/quants.c:566-643; Encoding examples/formats/ggml.py:75-84).
 * examples/kernels/vec_dot/q3_k_q8_k.py:46-50          vec_dot_runtime.cpp:239-240 */
int quantized_vec_dot_q3_k_q8_k(const uint8_t *W, const uint8_t *X, float *Y, size_t K);
int quantized_vec_dot_q3_k_q8_k_rows(const uint8_t *W, const uint8_t *X, float *Y, size_t N, size_t K);
/* examples/kernels/dequantize/q3_k.py:8-17             row_dequantize_runtime.cpp:207,362 */
int row_dequantize_q3_k(const uint8_t *W, float *Y, size_t K);
int row_dequantize_q3_k_rows(const uint8_t *W, float *Y, size_t N, size_t K);
/* examples/kernels/mul_mat/q3_k_decode.py:10-20, q3_k.py:9-61     mul_mat_runtime.cpp:311-312,319-320 */
int production_mul_mat_q3_k_decode(const uint8_t *W, const float *X, uint8_t *Xq, float *Y, size_t N, size_t K, size_t M);
int production_mul_mat_q3_k(const uint8_t *W, const float *X, uint8_t *Xq, float *Y, size_t N, size_t K, size_t M);
/* examples/kernels/mul_mat/q3_k_predecoded_scales_decode.py:10-21, q3_k_predecoded_scales.py:10-61: the same
 * arguments and results; the reference decodes the sixteen 6-bit scales of a record ahead of its inner loop there,
 * which these kernels always do. */
int production_mul_mat_q3_k_predecoded_scales_decode(const uint8_t *W, const float *X, uint8_t *Xq, float *Y, size_t N, size_t K, size_t M);
int production_mul_mat_q3_k_predecoded_scales(const uint8_t *W, const float *X, uint8_t *Xq, float *Y, size_t N, size_t K, size_t M);

/* ------------------------------------------------------------------ Q5_K x Q8_K (ggml-common.h block_q5_K: f16 d, f16 dmin,
 * scales[12] as in Q4_K, qh[32], qs[128]; ggml-quants.c:1673-1698, ggml-cpu/quants.c:720-798; Encoding
 * examples/formats/ggml.py:100-110, 2-byte aligned).
 * examples/kernels/vec_dot/q5_k_q8_k.py:34-38          vec_dot_runtime.cpp:255-256 */
int quantized_vec_dot_q5_k_q8_k(const uint8_t *W, const uint8_t *X, float *Y, size_t K);
int quantized_vec_dot_q5_k_q8_k_rows(const uint8_t *W, const uint8_t *X, float *Y, size_t N, size_t K);
/* examples/kernels/dequantize/q5_k.py:9-15             row_dequantize_runtime.cpp:217,370 */
int row_dequantize_q5_k(const uint8_t *W, float *Y, size_t K);
int row_dequantize_q5_k_rows(const uint8_t *W, float *Y, size_t N, size_t K);
/* examples/kernels/mul_mat/q5_k_decode.py:10-20        mul_mat_runtime.cpp:368-369 */
int production_mul_mat_q5_k_decode(const uint8_t *W, const float *X, uint8_t *Xq, float *Y, size_t N, size_t K, size_t M);
/* examples/kernels/mul_mat/q5_k.py                     mul_mat_runtime.cpp:371-372
 * (runs the decode GEMV once per activation row: no tensor-core path for this format yet) */
int production_mul_mat_q5_k(const uint8_t *W, const float *X, uint8_t *Xq, float *Y, size_t N, size_t K, size_t M);

/* ------------------------------------------------------------------ Q6_K x Q8_K (ggml-common.h block_q6_K: ql[128], qh[64],
 * int8 scales[16], f16 d; ggml-quants.c:1881-1910, ggml-cpu/quants.c:800-853).  The reference's Q6_K Encoding
 * (examples/formats/ggml.py:113-120) states no alignment, so W may start at any byte: a device W at an odd
 * address is first moved to an aligned slice of the library's arena (one device-to-device copy inside the call).
 * examples/kernels/vec_dot/q6_k_q8_k.py:39-43          vec_dot_runtime.cpp:263-264 */
int quantized_vec_dot_q6_k_q8_k(const uint8_t *W, const uint8_t *X, float *Y, size_t K);
int quantized_vec_dot_q6_k_q8_k_rows(const uint8_t *W, const uint8_t *X, float *Y, size_t N, size_t K);
/* examples/kernels/dequantize/q6_k.py:8-15             row_dequantize_runtime.cpp:222,374 */
int row_dequantize_q6_k(const uint8_t *W, float *Y, size_t K);
int row_dequantize_q6_k_rows(const uint8_t *W, float *Y, size_t N, size_t K);
/* examples/kernels/mul_mat/q6_k_decode.py:10-20        mul_mat_runtime.cpp:383-384 */
int production_mul_mat_q6_k_decode(const uint8_t *W, const float *X, uint8_t *Xq, float *Y, size_t N, size_t K, size_t M);
/* examples/kernels/mul_mat/q6_k.py:9-37                mul_mat_runtime.cpp:386-387
 * (runs the decode GEMV once per activation row: no tensor-core path for this format yet) */
int production_mul_mat_q6_k(const uint8_t *W, const float *X, uint8_t *Xq, float *Y, size_t N, size_t K, size_t M);

/* Persistent interleaved weight layout Q4K_I[16] (examples/formats/ggml.py:286-290): the Q4_K records of each
 * cohort of 16 rows stored byte-major, byte b of row r of a 256-block at 16 b + r, blocks in (cohort, block)
 * order (doc/dsl/encoding-and-artifacts.md:209).  Artifact functions as the reference emits them next to every
 * kernel with a derived-Encoding parameter (lib/Target/Emission/Emitter.h:231-272); rows must be a multiple
 * of 16 and K of 256 (packed_size returns 0 otherwise, pack fails); the packed object must be 16-byte aligned.
 * examples/kernels/gemv/q4_k.py:8-26                   q4_k_gemv_runtime.cpp:28-32,243-247 */
size_t q4_k_q8_k_gemv_W_packed_size(size_t M, size_t K);
int q4_k_q8_k_gemv_W_pack(const uint8_t *source, uint8_t *target, size_t M, size_t K);
int q4_k_q8_k_gemv(const uint8_t *W, const uint8_t *X, float *Y, size_t M, size_t K);
/* examples/kernels/gemv/q4_k_groups4.py:8-27, q4_k_contract.py:8-27   q4_k_gemv_runtime.cpp:12-25
 * (two more statements of the same GEMV for the reference's vector and matrix units: same layout and results) */
size_t q4_k_q8_k_gemv_groups4_W_packed_size(size_t M, size_t K);
int q4_k_q8_k_gemv_groups4_W_pack(const uint8_t *source, uint8_t *target, size_t M, size_t K);
int q4_k_q8_k_gemv_groups4(const uint8_t *W, const uint8_t *X, float *Y, size_t M, size_t K);
size_t q4_k_q8_k_gemv_contract_W_packed_size(size_t M, size_t K);
int q4_k_q8_k_gemv_contract_W_pack(const uint8_t *source, uint8_t *target, size_t M, size_t K);
int q4_k_q8_k_gemv_contract(const uint8_t *W, const uint8_t *X, float *Y, size_t M, size_t K);
/* examples/kernels/mul_mat/q4_k_persistent.py:9-30     mul_mat_runtime.cpp:337-348,805-810
 * Extents in the order (M, K, N): the derived Encoding's builder declares M and K first. */
size_t production_mul_mat_q4_k_persistent_W_packed_size(size_t N, size_t K);
int production_mul_mat_q4_k_persistent_W_pack(const uint8_t *source, uint8_t *target, size_t N, size_t K);
int production_mul_mat_q4_k_persistent(const uint8_t *W, const float *X, uint8_t *Xq, float *Y, size_t M, size_t K, size_t N);

/* Row-sharded mul_mat: this process holds weight rows [n0, n0+N_local) of an (N,K) matrix and writes
 * columns n0.. of Y, whose rows are ldy floats apart.  format: 1 Q4_0, 5 Q8_0, 6 Q2_K, 7 Q3_K, 8 Q4_K, 9 Q5_K, 10 Q6_K, 11 IQ1_S, 12 IQ1_M, 13 IQ2_S, 14 IQ2_XS, 15 IQ2_XXS, 16 IQ3_S, 17 IQ3_XXS,
 * 20 TQ1_0 (the reference harness numbering).  mode: 0 decode (GEMV), 1 prefill (tensor cores).
 * flags bit 0: Xq already holds the quantized activations (X may be NULL). */
int weft_b200_mul_mat_shard(int format, int mode, const uint8_t *W_local, const float *X, uint8_t *Xq,
                            const int8_t *grid, const int8_t *signs, const uint32_t *powers,
                            float *Y_columns, size_t N_local, size_t K, size_t M, size_t ldy, unsigned flags);

/* Several decode mul_mats issued back to back in one call, in order, on the library's stream: the projections of
 * a transformer layer at batch 1 (Q, K, V, O, gate, up, down), as the reference's model-level entry runs them through
 * llama.cpp (examples/run/ggml.sh:35-43).  Each step is one production_mul_mat_<format>_decode; consecutive kernels
 * overlap (the next one streams its first weights while the previous one drains).  flags bit 0: Xq of this step
 * already holds the quantized activations (steps that share an input quantize it once).  Up to four consecutive
 * Q4_K steps with one activation row that name the same Xq, the later ones with flags bit 0 set (Q/K/V, gate/up),
 * run as ONE launch over the concatenated rows when every N is a whole number of the kernel's stages; results are
 * the same either way.  grid / signs / powers as
 * for the single calls, NULL where the format takes none.  Stops at the first failing step. */
typedef struct weft_b200_mul_mat_step {
    int format;                  /* harness numbering, as for weft_b200_mul_mat_shard */
    unsigned flags;
    const uint8_t *W;            /* (N, K) records */
    const float *X;              /* (M, K) fp32 */
    uint8_t *Xq;                 /* (M, K) activation records, written unless flags bit 0 */
    float *Y;                    /* (M, N) fp32, written */
    const int8_t *grid, *signs;
    const uint32_t *powers;
    size_t N, K, M;
} weft_b200_mul_mat_step;
int weft_b200_mul_mat_chain(const weft_b200_mul_mat_step *steps, size_t count);

/* The same shard with the all-gather done by the library's own kernels over NVLink peer memory instead of a
 * collective library (the north star's "row-sharded along N ... all-gather of outputs"): every rank owns a full
 * (M, N) fp32 output and a sync block of 32 ints, both allocated with weft_b200_peer_alloc (zero-filled, exported
 * as a 64-byte CUDA IPC handle) and opened by every other rank with weft_b200_peer_open.  Y_ranks[r] / sync_ranks[r]
 * are rank r's buffers as mapped in this process (own buffers at index `rank`).  The call computes columns
 * [n0, n0 + N_local) and stores them into every rank's output; it returns (or, in async mode, its last kernel
 * ends) after all ranks' columns have arrived in this rank's output.  All ranks must make the same sequence of
 * calls; alternate two output buffers between consecutive calls.  stage_ranks (may be NULL) are staging areas of
 * WEFT_B200_GATHER_STAGE_BYTES (2 halves x 65536 words of 8 bytes, whatever the call's shape, so that calls of
 * different shapes can share one area) made and opened the same way: with them, outputs of up to 65536 values (decode)
 * travel as 8-byte {value, epoch} words that the receiving kernel polls for, with no fence and no barrier (one
 * launch and one NVLink crossing per step); larger outputs go directly into the peers' output buffers and end with
 * a flag barrier between the ranks.  Waits on a peer are bounded and surface as a device-side failure.  One
 * process per GPU. */
#define WEFT_B200_GATHER_STAGE_BYTES (2 * 8 * 65536)
int weft_b200_peer_alloc(size_t bytes, void **ptr, unsigned char *handle64);
int weft_b200_peer_open(const unsigned char *handle64, void **ptr);
int weft_b200_peer_close(void *ptr);
int weft_b200_peer_free(void *ptr);
/* waits for the library's stream, then copies `bytes` of a buffer made by peer_alloc to host memory */
int weft_b200_peer_read(void *host, const void *device, size_t bytes);
int weft_b200_mul_mat_shard_gather(int format, int mode, const uint8_t *W_local, const float *X, uint8_t *Xq,
                                   const int8_t *grid, const int8_t *signs, const uint32_t *powers,
                                   float *const *Y_ranks, int *const *sync_ranks, void *const *stage_ranks, int world, int rank,
                                   size_t n0, size_t N_local, size_t N, size_t K, size_t M, unsigned flags);

/* ------------------------------------------------------------------ no-allocation variant (no counterpart in the reference)
 * production_mul_mat_q4_k_decode for hosts that cannot allocate device memory once running (all device
 * memory owned by the host's own pool, a frozen memory budget, or a loop that cannot afford the device-wide
 * synchronisation of cudaMalloc).  Host-side X / Xq / Y are staged through a fixed WEFT_B200_NOALLOC_BYTES
 * array inside the library image instead of an arena grown on demand; nothing is allocated.  W must be
 * device memory.  Calls needing more staging than the array holds are refused.  Calls are serialised (the
 * array is shared and keeps the last call's contents); the first call on a device resolves the array's
 * address and should happen outside stream capture.  Runs on the legacy default stream, returns when done.
 * Message of the last refusal: weft_b200_noalloc_last_error(). */
#define WEFT_B200_NOALLOC_BYTES (1 << 20)
int production_mul_mat_q4_k_decode_noalloc(const uint8_t *W, const float *X, uint8_t *Xq, float *Y, size_t N, size_t K, size_t M);
const char *weft_b200_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* WEFT_B200_H */
