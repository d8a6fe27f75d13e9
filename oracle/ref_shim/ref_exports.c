/* Glue for building the reference's own GGML C sources into a shared library
 * (oracle/_ref/libweft_ref.so).  TEST INFRASTRUCTURE ONLY: the product path
 * never loads this library.
 *
 * Nothing here restates reference code: the file supplies (1) the two lookup
 * tables that ggml-cpu.c normally defines (source/c/ggml/llama.cpp/ggml/src/
 * ggml-cpu/ggml-cpu.c:80-83, filled at :3784-3799) because ggml-cpu.c itself
 * needs files that are not vendored, (2) aborting stubs for two backend calls
 * that ggml.c references but the quantization path never reaches, and (3) a
 * flat C surface with stable names over the reference's functions so the test
 * suite can reach them through ctypes.
 */
#define GGML_COMMON_IMPL_C   /* static tables (iq2xxs_grid, ksigns_iq2xs, kmask_iq2xs) */
#define GGML_COMMON_DECL_C
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "ggml.h"
#include "ggml-common.h"   /* via -I: block layouts, iq2xxs_grid, ksigns_iq2xs */
#include "ggml-quants.h"
#include "ggml-cpu/quants.h"

float ggml_table_f32_f16[1 << 16];
float ggml_table_f32_e8m0_half[1 << 8];

void ggml_backend_tensor_set(struct ggml_tensor *t, const void *d, size_t o, size_t s) {
    (void)t; (void)d; (void)o; (void)s;
    fprintf(stderr, "weft_ref: ggml_backend_tensor_set is not available\n");
    abort();
}
void ggml_backend_tensor_memset(struct ggml_tensor *t, uint8_t v, size_t o, size_t s) {
    (void)t; (void)v; (void)o; (void)s;
    fprintf(stderr, "weft_ref: ggml_backend_tensor_memset is not available\n");
    abort();
}

__attribute__((constructor)) static void weft_ref_init(void) {
    for (int i = 0; i < (1 << 16); ++i) {
        ggml_table_f32_f16[i] = ggml_fp16_to_fp32((ggml_fp16_t)i);
    }
    for (int i = 0; i < (1 << 8); ++i) {
        /* 2^(e-127) / 2; unused by the formats under test, filled for completeness */
        uint32_t bits = i < 2 ? (0x00200000u << i) : ((uint32_t)(i - 1) << 23);
        float f; memcpy(&f, &bits, 4);
        ggml_table_f32_e8m0_half[i] = f;
    }
}

/* format ids follow the reference harnesses (vec_dot_runtime.cpp:185-344) */
enum { WEFT_Q4_0 = 1, WEFT_Q8_0 = 5, WEFT_Q2_K = 6, WEFT_Q3_K = 7, WEFT_Q4_K = 8, WEFT_Q5_K = 9, WEFT_Q6_K = 10, WEFT_IQ1_S = 11, WEFT_IQ1_M = 12, WEFT_IQ2_S = 13, WEFT_IQ2_XS = 14, WEFT_IQ2_XXS = 15, WEFT_IQ3_S = 16, WEFT_IQ3_XXS = 17, WEFT_TQ1_0 = 20,
       WEFT_Q8_K = 100 };

static enum ggml_type to_type(int fmt) {
    switch (fmt) {
    case WEFT_Q4_0: return GGML_TYPE_Q4_0;
    case WEFT_Q8_0: return GGML_TYPE_Q8_0;
    case WEFT_Q4_K: return GGML_TYPE_Q4_K;
    case WEFT_Q2_K: return GGML_TYPE_Q2_K;
    case WEFT_Q3_K: return GGML_TYPE_Q3_K;
    case WEFT_Q5_K: return GGML_TYPE_Q5_K;
    case WEFT_Q6_K: return GGML_TYPE_Q6_K;
    case WEFT_IQ2_XXS: return GGML_TYPE_IQ2_XXS;
    case WEFT_IQ2_XS: return GGML_TYPE_IQ2_XS;
    case WEFT_IQ3_XXS: return GGML_TYPE_IQ3_XXS;
    case WEFT_IQ2_S: return GGML_TYPE_IQ2_S;
    case WEFT_IQ1_S: return GGML_TYPE_IQ1_S;
    case WEFT_IQ1_M: return GGML_TYPE_IQ1_M;
    case WEFT_IQ3_S: return GGML_TYPE_IQ3_S;
    case WEFT_TQ1_0: return GGML_TYPE_TQ1_0;
    case WEFT_Q8_K: return GGML_TYPE_Q8_K;
    default: return GGML_TYPE_COUNT;
    }
}

size_t weft_ref_row_bytes(int fmt, int64_t k) { return ggml_row_size(to_type(fmt), k); }

/* weights: ggml_quantize_chunk(type, src, dst, 0, nrows, k, imatrix) */
int weft_ref_quantize_weights(int fmt, const float *src, void *dst, int64_t nrows, int64_t k) {
    enum ggml_type type = to_type(fmt);
    if (type == GGML_TYPE_COUNT || fmt == WEFT_Q8_K) return -1;
    float *imatrix = NULL;
    if (ggml_quantize_requires_imatrix(type)) {
        imatrix = (float *)malloc(sizeof(float) * (size_t)k);
        for (int64_t i = 0; i < k; ++i) imatrix[i] = 1.0f;
    }
    ggml_quantize_init(type);
    ggml_quantize_chunk(type, src, dst, 0, nrows, k, imatrix);
    free(imatrix);
    return 0;
}

/* activations */
void weft_ref_quantize_q8_0(const float *x, void *y, int64_t k) { quantize_row_q8_0_ref(x, (block_q8_0 *)y, k); }
void weft_ref_quantize_q8_K(const float *x, void *y, int64_t k) { quantize_row_q8_K_ref(x, (block_q8_K *)y, k); }
void weft_ref_quantize_q8_1(const float *x, void *y, int64_t k) { quantize_row_q8_1_ref(x, (block_q8_1 *)y, k); }

int weft_ref_dequantize(int fmt, const void *w, float *y, int64_t k) {
    switch (fmt) {
    case WEFT_Q4_0: dequantize_row_q4_0((const block_q4_0 *)w, y, k); return 0;
    case WEFT_Q8_0: dequantize_row_q8_0((const block_q8_0 *)w, y, k); return 0;
    case WEFT_Q4_K: dequantize_row_q4_K((const block_q4_K *)w, y, k); return 0;
    case WEFT_Q2_K: dequantize_row_q2_K((const block_q2_K *)w, y, k); return 0;
    case WEFT_Q3_K: dequantize_row_q3_K((const block_q3_K *)w, y, k); return 0;
    case WEFT_Q5_K: dequantize_row_q5_K((const block_q5_K *)w, y, k); return 0;
    case WEFT_Q6_K: dequantize_row_q6_K((const block_q6_K *)w, y, k); return 0;
    case WEFT_IQ2_XXS: dequantize_row_iq2_xxs((const block_iq2_xxs *)w, y, k); return 0;
    case WEFT_IQ2_XS: dequantize_row_iq2_xs((const block_iq2_xs *)w, y, k); return 0;
    case WEFT_IQ3_XXS: dequantize_row_iq3_xxs((const block_iq3_xxs *)w, y, k); return 0;
    case WEFT_IQ2_S: dequantize_row_iq2_s((const block_iq2_s *)w, y, k); return 0;
    case WEFT_IQ1_S: dequantize_row_iq1_s((const block_iq1_s *)w, y, k); return 0;
    case WEFT_IQ1_M: dequantize_row_iq1_m((const block_iq1_m *)w, y, k); return 0;
    case WEFT_IQ3_S: dequantize_row_iq3_s((const block_iq3_s *)w, y, k); return 0;
    case WEFT_TQ1_0: dequantize_row_tq1_0((const block_tq1_0 *)w, y, k); return 0;
    default: return -1;
    }
}

/* GGML_CPU_GENERIC is defined for this build, so the *_generic bodies carry the plain names */
int weft_ref_vec_dot(int fmt, int64_t k, float *s, const void *w, const void *x) {
    switch (fmt) {
    case WEFT_Q4_0: ggml_vec_dot_q4_0_q8_0((int)k, s, 0, w, 0, x, 0, 1); return 0;
    case WEFT_Q8_0: ggml_vec_dot_q8_0_q8_0((int)k, s, 0, w, 0, x, 0, 1); return 0;
    case WEFT_Q4_K: ggml_vec_dot_q4_K_q8_K((int)k, s, 0, w, 0, x, 0, 1); return 0;
    case WEFT_Q2_K: ggml_vec_dot_q2_K_q8_K((int)k, s, 0, w, 0, x, 0, 1); return 0;
    case WEFT_Q3_K: ggml_vec_dot_q3_K_q8_K((int)k, s, 0, w, 0, x, 0, 1); return 0;
    case WEFT_Q5_K: ggml_vec_dot_q5_K_q8_K((int)k, s, 0, w, 0, x, 0, 1); return 0;
    case WEFT_Q6_K: ggml_vec_dot_q6_K_q8_K((int)k, s, 0, w, 0, x, 0, 1); return 0;
    case WEFT_IQ2_XXS: ggml_vec_dot_iq2_xxs_q8_K((int)k, s, 0, w, 0, x, 0, 1); return 0;
    case WEFT_IQ2_XS: ggml_vec_dot_iq2_xs_q8_K((int)k, s, 0, w, 0, x, 0, 1); return 0;
    case WEFT_IQ3_XXS: ggml_vec_dot_iq3_xxs_q8_K((int)k, s, 0, w, 0, x, 0, 1); return 0;
    case WEFT_IQ2_S: ggml_vec_dot_iq2_s_q8_K((int)k, s, 0, w, 0, x, 0, 1); return 0;
    case WEFT_IQ1_S: ggml_vec_dot_iq1_s_q8_K((int)k, s, 0, w, 0, x, 0, 1); return 0;
    case WEFT_IQ1_M: ggml_vec_dot_iq1_m_q8_K((int)k, s, 0, w, 0, x, 0, 1); return 0;
    case WEFT_IQ3_S: ggml_vec_dot_iq3_s_q8_K((int)k, s, 0, w, 0, x, 0, 1); return 0;
    case WEFT_TQ1_0: ggml_vec_dot_tq1_0_q8_K((int)k, s, 0, w, 0, x, 0, 1); return 0;
    default: return -1;
    }
}

/* mul_mat as ggml-cpu.c:1202-1242 performs it: from_float on each X row, then
 * the double loop over vec_dot.  xq is the caller's workspace. rows [n0,n1). */
int weft_ref_mul_mat(int fmt, const void *w, const float *x, void *xq, float *y,
                     int64_t n, int64_t k, int64_t m, int64_t n0, int64_t n1, int quantize_x) {
    const int act = (fmt == WEFT_Q4_0 || fmt == WEFT_Q8_0) ? WEFT_Q8_0 : WEFT_Q8_K;
    const size_t wrow = weft_ref_row_bytes(fmt, k), xrow = weft_ref_row_bytes(act, k);
    if (quantize_x) {
        for (int64_t r = 0; r < m; ++r) {
            if (act == WEFT_Q8_0) weft_ref_quantize_q8_0(x + r * k, (char *)xq + r * xrow, k);
            else weft_ref_quantize_q8_K(x + r * k, (char *)xq + r * xrow, k);
        }
    }
    for (int64_t r = 0; r < m; ++r)
        for (int64_t c = n0; c < n1; ++c)
            if (weft_ref_vec_dot(fmt, k, y + r * n + c, (const char *)w + c * wrow, (const char *)xq + r * xrow)) return -1;
    return 0;
}

/* codebook tables as the reference kernels receive them (vec_dot_runtime.cpp:101-134):
 * grid int8[256][8], signs int8[128][8] with entries +1/-1 */
void weft_ref_iq2xxs_tables(int8_t *grid, int8_t *signs) {
    for (int i = 0; i < 256; ++i) {
        const uint8_t *g = (const uint8_t *)(iq2xxs_grid + i);
        for (int j = 0; j < 8; ++j) grid[i * 8 + j] = (int8_t)g[j];
    }
    for (int i = 0; i < 128; ++i)
        for (int j = 0; j < 8; ++j) signs[i * 8 + j] = (ksigns_iq2xs[i] & kmask_iq2xs[j]) ? -1 : 1;
}

/* the other two codebooks in kernel-argument form (vec_dot_runtime.cpp:101-134,438-440): iq2xs_grid as int8[512][8],
 * iq3xxs_grid as int8[256][4] (bytes of the table entries in memory order) */
void weft_ref_iq2xs_grid(int8_t *grid) {
    for (int i = 0; i < 512; ++i) {
        const uint8_t *g = (const uint8_t *)(iq2xs_grid + i);
        for (int j = 0; j < 8; ++j) grid[i * 8 + j] = (int8_t)g[j];
    }
}
void weft_ref_iq3xxs_grid(int8_t *grid) {
    for (int i = 0; i < 256; ++i) {
        const uint8_t *g = (const uint8_t *)(iq3xxs_grid + i);
        for (int j = 0; j < 4; ++j) grid[i * 4 + j] = (int8_t)g[j];
    }
}
/* iq2s_grid as int8[1024][8], iq3s_grid as int8[512][4] (vec_dot_runtime.cpp:439,441) */
void weft_ref_iq2s_grid(int8_t *grid) {
    for (int i = 0; i < 1024; ++i) {
        const uint8_t *g = (const uint8_t *)(iq2s_grid + i);
        for (int j = 0; j < 8; ++j) grid[i * 8 + j] = (int8_t)g[j];
    }
}
void weft_ref_iq3s_grid(int8_t *grid) {
    for (int i = 0; i < 512; ++i) {
        const uint8_t *g = (const uint8_t *)(iq3s_grid + i);
        for (int j = 0; j < 4; ++j) grid[i * 4 + j] = (int8_t)g[j];
    }
}
/* iq1s_grid as int8[2048][8] (vec_dot_runtime.cpp:436) */
void weft_ref_iq1s_grid(int8_t *grid) {
    for (int i = 0; i < 2048; ++i) {
        const int8_t *g = (const int8_t *)(iq1s_grid + i);
        for (int j = 0; j < 8; ++j) grid[i * 8 + j] = g[j];
    }
}
