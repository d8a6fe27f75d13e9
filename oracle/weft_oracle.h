/* CPU oracle for the quantized matrix path -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the GGML-semantics algorithms that the reference
 * (zzyu5/Weft) uses as its own correctness oracle.  Only tests/, the smoke
 * check and the cpu_baseline leg of bench.py may load this library; the
 * product (libweft_b200.so) never links or calls it.
 *
 * Parity status: PINNED.  Every function here is checked bit-for-bit against
 * the reference's own GGML C compiled from its sources (oracle/_ref) on the
 * reference harnesses' closed-form inputs and on seeded random inputs; the
 * resulting golden vectors are committed under tests/golden/.
 *
 * Paths cited as "ggml/..." are under source/c/ggml/llama.cpp/ggml/ of the
 * reference; "examples/..." are under the reference root.
 */
#ifndef WEFT_ORACLE_H
#define WEFT_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Format ids: the numbering of the reference harnesses
 * (examples/repro/weft/vec_dot_runtime.cpp:185-344); 100 is local (Q8_K). */
enum wo_format {
    WO_Q4_0 = 1,
    WO_Q8_0 = 5,
    WO_Q4_K = 8,
    WO_Q2_K = 6,
    WO_Q3_K = 7,
    WO_Q5_K = 9,
    WO_Q6_K = 10,
    WO_IQ1_S = 11,
    WO_IQ1_M = 12,
    WO_IQ2_S = 13,
    WO_IQ2_XS = 14,
    WO_IQ2_XXS = 15,
    WO_IQ3_S = 16,
    WO_IQ3_XXS = 17,
    WO_TQ1_0 = 20,
    WO_Q8_K = 100,
    WO_Q8_1 = 101   /* activation-only format: local id */
};

/* record geometry (ggml/src/ggml-common.h:184-189,241-246,266-271,317-328,361-366,371-375) */
size_t wo_record_bytes(int fmt);
size_t wo_record_elements(int fmt);
size_t wo_row_bytes(int fmt, int64_t k);

float wo_f16_to_f32(uint16_t h);
uint16_t wo_f32_to_f16(float f);

/* weight quantizers (inputs for the tests; IQ2_XXS has none here, see weft_oracle.c) */
void wo_quantize_row_q4_0(const float *x, uint8_t *y, int64_t k);
void wo_quantize_row_q4_K(const float *x, uint8_t *y, int64_t k);
void wo_quantize_row_tq1_0(const float *x, uint8_t *y, int64_t k);
/* activation quantizers, GGML rule */
void wo_quantize_row_q8_0(const float *x, uint8_t *y, int64_t k);
void wo_quantize_row_q8_K(const float *x, uint8_t *y, int64_t k);
/* activation quantizers, Weft DSL rule (differs from GGML only on exact ties) */
void wo_quantize_row_q8_0_weft(const float *x, uint8_t *y, int64_t k);
void wo_quantize_row_q8_1(const float *x, uint8_t *y, int64_t k);
void wo_quantize_row_q8_1_weft(const float *x, uint8_t *y, int64_t k);
void wo_quantize_row_q8_K_weft(const float *x, uint8_t *y, int64_t k);
/* rows [0,nrows) of a row-major matrix, one thread per contiguous row range; rule: 0 = GGML, 1 = Weft (activations only) */
int wo_quantize_rows(int fmt, int rule, const float *x, uint8_t *y, int64_t nrows, int64_t k);

/* dequantizers; grid = int8[256*8], signs = int8[128*8] (+1/-1), the tables in kernel-argument form */
void wo_dequantize_row_q4_0(const uint8_t *w, float *y, int64_t k);
void wo_dequantize_row_q8_0(const uint8_t *w, float *y, int64_t k);
void wo_dequantize_row_q4_K(const uint8_t *w, float *y, int64_t k);
void wo_dequantize_row_q2_K(const uint8_t *w, float *y, int64_t k);
void wo_dequantize_row_q3_K(const uint8_t *w, float *y, int64_t k);
void wo_dequantize_row_q5_K(const uint8_t *w, float *y, int64_t k);
void wo_dequantize_row_q6_K(const uint8_t *w, float *y, int64_t k);
void wo_dequantize_row_iq2_xxs(const uint8_t *w, const int8_t *grid, const int8_t *signs, float *y, int64_t k);
void wo_dequantize_row_iq2_xs(const uint8_t *w, const int8_t *grid /* [512*8] */, const int8_t *signs, float *y, int64_t k);
void wo_dequantize_row_iq1_s(const uint8_t *w, const int8_t *grid /* [2048*8] */, float *y, int64_t k);
void wo_dequantize_row_iq1_m(const uint8_t *w, const int8_t *grid /* [2048*8] */, float *y, int64_t k);
void wo_dequantize_row_iq2_s(const uint8_t *w, const int8_t *grid /* [1024*8] */, float *y, int64_t k);
void wo_dequantize_row_iq3_s(const uint8_t *w, const int8_t *grid /* [512*4] */, float *y, int64_t k);
void wo_dequantize_row_iq3_xxs(const uint8_t *w, const int8_t *grid /* [256*4] */, const int8_t *signs, float *y, int64_t k);
void wo_dequantize_row_tq1_0(const uint8_t *w, float *y, int64_t k);
int wo_dequantize_rows(int fmt, const uint8_t *w, const int8_t *grid, const int8_t *signs,
                       float *y, int64_t nrows, int64_t k);

/* block dot products, one output */
float wo_vec_dot_q4_0_q8_0(const uint8_t *w, const uint8_t *x, int64_t k);
float wo_vec_dot_q8_0_q8_0(const uint8_t *w, const uint8_t *x, int64_t k);
float wo_vec_dot_q4_K_q8_K(const uint8_t *w, const uint8_t *x, int64_t k);
float wo_vec_dot_iq2_xxs_q8_K(const uint8_t *w, const uint8_t *x, const int8_t *grid, const int8_t *signs, int64_t k);
float wo_vec_dot_iq2_xs_q8_K(const uint8_t *w, const uint8_t *x, const int8_t *grid, const int8_t *signs, int64_t k);
float wo_vec_dot_iq1_s_q8_K(const uint8_t *w, const uint8_t *x, const int8_t *grid, int64_t k);
float wo_vec_dot_iq1_m_q8_K(const uint8_t *w, const uint8_t *x, const int8_t *grid, int64_t k);
float wo_vec_dot_iq2_s_q8_K(const uint8_t *w, const uint8_t *x, const int8_t *grid, int64_t k);
float wo_vec_dot_iq3_s_q8_K(const uint8_t *w, const uint8_t *x, const int8_t *grid, int64_t k);
float wo_vec_dot_iq3_xxs_q8_K(const uint8_t *w, const uint8_t *x, const int8_t *grid, const int8_t *signs, int64_t k);
float wo_vec_dot_tq1_0_q8_K(const uint8_t *w, const uint8_t *x, int64_t k);
float wo_vec_dot_q2_K_q8_K(const uint8_t *w, const uint8_t *x, int64_t k);
float wo_vec_dot_q3_K_q8_K(const uint8_t *w, const uint8_t *x, int64_t k);
float wo_vec_dot_q5_K_q8_K(const uint8_t *w, const uint8_t *x, int64_t k);
float wo_vec_dot_q6_K_q8_K(const uint8_t *w, const uint8_t *x, int64_t k);
int wo_vec_dot(int fmt, const uint8_t *w, const uint8_t *x, const int8_t *grid, const int8_t *signs,
               int64_t k, float *out);

/* Y[m, n] for n in [n0, n1): optional activation quantize into xq (rule as above),
 * then the double loop over vec_dot, threads over weight rows. */
int wo_mul_mat(int fmt, int rule, const uint8_t *w, const float *x, uint8_t *xq,
               const int8_t *grid, const int8_t *signs, float *y,
               int64_t n, int64_t k, int64_t m, int64_t n0, int64_t n1, int quantize_x);

/* sign table in kernel-argument form, derived (7 index bits + even-parity bit) */
void wo_iq2_sign_table(int8_t *signs /* [128*8] */);

/* Persistent interleaved layout Family[R] of a record format (R rows of one cohort, byte-major): byte b of
 * the record of row r, block k sits at ((r / R) * blocks + k) * R * record_bytes + b * R + (r % R)
 * (doc/dsl/encoding-and-artifacts.md:209; record stride record_bytes * R and cohort stride
 * blocks * record_bytes per row in lib/Target/Emission/Memory.cpp:1344-1348; ABI of the artifact functions
 * <kernel>_W_packed_size / <kernel>_W_pack in lib/Target/Emission/Emitter.h:231-272).  rows % R must be 0:
 * returns -1 otherwise (the builder declares no tail cohort). */
size_t wo_interleave_packed_size(size_t record_bytes, int64_t rows, int64_t blocks);
int wo_interleave_pack(const uint8_t *source, uint8_t *target, size_t record_bytes, int64_t R, int64_t rows, int64_t blocks);
int wo_interleave_unpack(const uint8_t *source, uint8_t *target, size_t record_bytes, int64_t R, int64_t rows, int64_t blocks);

int wo_max_threads(void);
void wo_set_threads(int n);

#ifdef __cplusplus
}
#endif
#endif
