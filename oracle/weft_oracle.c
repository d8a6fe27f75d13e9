/* CPU oracle for the quantized matrix path -- TEST INFRASTRUCTURE ONLY.
 * See weft_oracle.h for the role of this file and its parity status (pinned).
 *
 * Each function names the reference source it restates.  "ggml/" stands for
 * source/c/ggml/llama.cpp/ggml/ inside the reference tree.  Float operation
 * order is kept exactly as the reference writes it, and the file is compiled
 * with -ffp-contract=off, so results are bit-identical to the reference's C.
 *
 * Not restated: the IQ2_XXS weight quantizer (ggml/src/ggml-quants.c:3222-3398
 * plus the neighbour-grid builder at :2781-3186).  It only produces test
 * inputs; IQ2_XXS inputs come from the compiled reference (oracle/_ref), from
 * the committed fixture made with it, or from random valid records.
 */
#include "weft_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

/* ------------------------------------------------------------ row parallelism */

static int g_threads = 0; /* 0 = all online cores */

int wo_max_threads(void) {
    if (g_threads > 0) return g_threads;
    const long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}

void wo_set_threads(int n) { g_threads = n > 0 ? n : 0; }

typedef void (*wo_range_fn)(int64_t begin, int64_t end, void *ctx);
typedef struct { wo_range_fn fn; void *ctx; int64_t begin, end; } wo_task;

static void *wo_task_main(void *p) {
    wo_task *t = (wo_task *)p;
    t->fn(t->begin, t->end, t->ctx);
    return NULL;
}

/* static split of [0, n) into contiguous ranges, one per thread */
static void wo_parallel_for(int64_t n, wo_range_fn fn, void *ctx) {
    int threads = wo_max_threads();
    if (threads > n) threads = (int)(n > 0 ? n : 1);
    if (threads <= 1) { fn(0, n, ctx); return; }
    pthread_t *ids = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)threads);
    char *started = (char *)calloc((size_t)threads, 1);
    wo_task *tasks = (wo_task *)malloc(sizeof(wo_task) * (size_t)threads);
    for (int t = 0; t < threads; ++t) {
        tasks[t].fn = fn; tasks[t].ctx = ctx;
        tasks[t].begin = n * t / threads; tasks[t].end = n * (t + 1) / threads;
        if (pthread_create(&ids[t], NULL, wo_task_main, &tasks[t]) == 0) started[t] = 1;
        else wo_task_main(&tasks[t]);
    }
    for (int t = 0; t < threads; ++t) if (started[t]) pthread_join(ids[t], NULL);
    free(ids); free(started); free(tasks);
}

/* ---------------------------------------------------------------- geometry */

size_t wo_record_bytes(int fmt) {
    switch (fmt) {
    case WO_Q4_0: return 18;
    case WO_Q8_0: return 34;
    case WO_Q8_1: return 36;
    case WO_Q4_K: return 144;
    case WO_Q2_K: return 84;
    case WO_Q3_K: return 110;
    case WO_Q5_K: return 176;
    case WO_Q6_K: return 210;
    case WO_IQ2_XXS: return 66;
    case WO_IQ2_XS: return 74;
    case WO_IQ2_S: return 82;
    case WO_IQ1_S: return 50;
    case WO_IQ1_M: return 56;
    case WO_IQ3_S: return 110;
    case WO_IQ3_XXS: return 98;
    case WO_TQ1_0: return 54;
    case WO_Q8_K: return 292;
    default: return 0;
    }
}

size_t wo_record_elements(int fmt) {
    switch (fmt) {
    case WO_Q4_0: case WO_Q8_0: case WO_Q8_1: return 32;
    case WO_Q2_K: case WO_Q3_K: case WO_Q4_K: case WO_Q5_K: case WO_Q6_K: case WO_IQ2_XXS: case WO_IQ2_XS: case WO_IQ3_XXS: case WO_IQ2_S: case WO_IQ3_S: case WO_IQ1_S: case WO_IQ1_M: case WO_TQ1_0: case WO_Q8_K: return 256;
    default: return 0;
    }
}

size_t wo_row_bytes(int fmt, int64_t k) {
    const size_t e = wo_record_elements(fmt);
    return e ? (size_t)k / e * wo_record_bytes(fmt) : 0;
}

/* ------------------------------------------------------------- half floats */

/* IEEE binary16 -> binary32, exact (the value set of ggml_fp16_to_fp32) */
float wo_f16_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: renormalise */
            int e = -1;
            do { man <<= 1; ++e; } while (!(man & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* binary32 -> binary16, round to nearest even (the rounding of GGML_FP32_TO_FP16) */
uint16_t wo_f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    const uint32_t ax = x & 0x7fffffffu;
    if (ax >= 0x7f800000u) return (uint16_t)(sign | (ax > 0x7f800000u ? 0x7e00u : 0x7c00u));
    if (ax >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);   /* rounds to >= 65520 -> inf */
    if (ax < 0x33000001u) return sign;                          /* <= 2^-25 -> 0 (ties to even) */
    int e = (int)(ax >> 23) - 127;
    uint32_t man = (ax & 0x7fffffu) | 0x800000u;
    int shift;
    uint32_t base;
    if (e < -14) { shift = 13 + (-14 - e); base = 0; }          /* subnormal half */
    else { shift = 13; base = (uint32_t)(e + 15) << 10; man &= 0x7fffffu; }
    uint32_t q = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1u);
    const uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) ++q;           /* carry may bump the exponent: intended */
    return (uint16_t)(sign | (base + q));
}

static inline uint16_t ld_u16(const uint8_t *p) { uint16_t v; memcpy(&v, p, 2); return v; }
static inline void st_u16(uint8_t *p, uint16_t v) { memcpy(p, &v, 2); }
static inline float ld_f32(const uint8_t *p) { float v; memcpy(&v, p, 4); return v; }
static inline int16_t ld_i16(const uint8_t *p) { int16_t v; memcpy(&v, p, 2); return v; }

/* round half to even for |v| <= 2^22: the value of nearest_int, ggml/src/ggml-quants.c:563-568 */
static inline int rne_int(float v) { return (int)rintf(v); }

/* ------------------------------------------------------------- quantizers */

/* ggml/src/ggml-quants.c:75-110 (quantize_row_q4_0_ref).  Record: f16 d @0, 16 nibble bytes @2. */
void wo_quantize_row_q4_0(const float *x, uint8_t *y, int64_t k) {
    for (int64_t b = 0; b < k / 32; ++b, x += 32, y += 18) {
        float amax = 0.0f, signed_max = 0.0f;
        for (int j = 0; j < 32; ++j) {
            if (amax < fabsf(x[j])) { amax = fabsf(x[j]); signed_max = x[j]; }
        }
        const float d = signed_max / -8;
        const float id = d ? 1.0f / d : 0.0f;
        st_u16(y, wo_f32_to_f16(d));
        for (int j = 0; j < 16; ++j) {
            const float lo = x[j] * id, hi = x[16 + j] * id;
            int a = (int8_t)(lo + 8.5f), c = (int8_t)(hi + 8.5f);
            if (a > 15) a = 15;
            if (c > 15) c = 15;
            y[2 + j] = (uint8_t)((uint8_t)a | ((uint8_t)c << 4));
        }
    }
}

/* ggml/src/ggml-quants.c:238-261 (quantize_row_q8_0_ref): roundf = half away from zero */
void wo_quantize_row_q8_0(const float *x, uint8_t *y, int64_t k) {
    for (int64_t b = 0; b < k / 32; ++b, x += 32, y += 34) {
        float amax = 0.0f;
        for (int j = 0; j < 32; ++j) amax = amax > fabsf(x[j]) ? amax : fabsf(x[j]);
        const float d = amax / 127;
        const float id = d ? 1.0f / d : 0.0f;
        st_u16(y, wo_f32_to_f16(d));
        for (int j = 0; j < 32; ++j) y[2 + j] = (uint8_t)(int8_t)roundf(x[j] * id);
    }
}

/* examples/kernels/quantize/q8_0.py:8-23 and its scalar restatement
 * examples/repro/weft/q8_quantize_runtime.cpp:117-127: same scale, but the
 * code is rounded to nearest even ("dynamic" rounding) and clamped to int8. */
void wo_quantize_row_q8_0_weft(const float *x, uint8_t *y, int64_t k) {
    for (int64_t b = 0; b < k / 32; ++b, x += 32, y += 34) {
        float amax = 0.0f;
        for (int j = 0; j < 32; ++j) amax = amax > fabsf(x[j]) ? amax : fabsf(x[j]);
        const float d = amax / 127.0f;
        const float id = amax == 0.0f ? 0.0f : 1.0f / d;
        st_u16(y, wo_f32_to_f16(d));
        for (int j = 0; j < 32; ++j) {
            float r = rintf(x[j] * id);
            r = r < -128.0f ? -128.0f : (r > 127.0f ? 127.0f : r);
            y[2 + j] = (uint8_t)(int8_t)r;
        }
    }
}

/* ggml/src/ggml-quants.c quantize_row_q8_1_ref: Q8_0 plus s = f16(sum(q) * d), d the fp32 scale */
void wo_quantize_row_q8_1(const float *x, uint8_t *y, int64_t k) {
    for (int64_t b = 0; b < k / 32; ++b, x += 32, y += 36) {
        float amax = 0.0f;
        for (int j = 0; j < 32; ++j) amax = amax > fabsf(x[j]) ? amax : fabsf(x[j]);
        const float d = amax / 127;
        const float id = d ? 1.0f / d : 0.0f;
        st_u16(y, wo_f32_to_f16(d));
        int sum = 0;
        for (int j = 0; j < 32; ++j) {
            const int8_t q = (int8_t)roundf(x[j] * id);
            y[4 + j] = (uint8_t)q;
            sum += q;
        }
        st_u16(y + 2, wo_f32_to_f16(sum * d));
    }
}

/* examples/kernels/quantize/q8_1.py:8-20; examples/repro/weft/q8_quantize_runtime.cpp:117-139 (kind 1):
 * codes rounded to nearest even and clamped, s = f16(f32(sum) * d) */
void wo_quantize_row_q8_1_weft(const float *x, uint8_t *y, int64_t k) {
    for (int64_t b = 0; b < k / 32; ++b, x += 32, y += 36) {
        float amax = 0.0f;
        for (int j = 0; j < 32; ++j) amax = amax > fabsf(x[j]) ? amax : fabsf(x[j]);
        const float d = amax / 127.0f;
        const float id = amax == 0.0f ? 0.0f : 1.0f / d;
        st_u16(y, wo_f32_to_f16(d));
        int sum = 0;
        for (int j = 0; j < 32; ++j) {
            float r = rintf(x[j] * id);
            r = r < -128.0f ? -128.0f : (r > 127.0f ? 127.0f : r);
            y[4 + j] = (uint8_t)(int8_t)r;
            sum += (int8_t)r;
        }
        st_u16(y + 2, wo_f32_to_f16((float)sum * d));
    }
}

static void q8_K_fill(const float *x, uint8_t *y, float iscale, float d) {
    memcpy(y, &d, 4);
    int8_t *q = (int8_t *)(y + 4);
    for (int j = 0; j < 256; ++j) {
        int v = rne_int(iscale * x[j]);
        if (v > 127) v = 127;
        if (v < -128) v = -128;
        q[j] = (int8_t)v;
    }
    for (int g = 0; g < 16; ++g) {
        int sum = 0;
        for (int j = 0; j < 16; ++j) sum += q[16 * g + j];
        const int16_t s = (int16_t)sum;
        memcpy(y + 260 + 2 * g, &s, 2);
    }
}

/* ggml/src/ggml-quants.c:2696-2733 (quantize_row_q8_K_ref): the scale comes from the FIRST
 * element of largest magnitude.  An all-zero block gets d = 0 and zero codes; the reference
 * leaves its bsums untouched there, the oracle zeroes them (callers compare on zeroed output). */
void wo_quantize_row_q8_K(const float *x, uint8_t *y, int64_t k) {
    for (int64_t b = 0; b < k / 256; ++b, x += 256, y += 292) {
        float amax = 0.0f, signed_max = 0.0f;
        for (int j = 0; j < 256; ++j) {
            const float ax = fabsf(x[j]);
            if (ax > amax) { amax = ax; signed_max = x[j]; }
        }
        if (!amax) { memset(y, 0, 292); continue; }
        const float iscale = -127.f / signed_max;
        q8_K_fill(x, y, iscale, 1 / iscale);
    }
}

/* examples/kernels/quantize/q8_k.py:8-30 and examples/repro/weft/q8_quantize_runtime.cpp:94-116:
 * extreme = max if |max| > |min| else min (so an exact +a/-a tie picks the negative one). */
void wo_quantize_row_q8_K_weft(const float *x, uint8_t *y, int64_t k) {
    for (int64_t b = 0; b < k / 256; ++b, x += 256, y += 292) {
        float hi = -INFINITY, lo = INFINITY;
        for (int j = 0; j < 256; ++j) {
            hi = hi > x[j] ? hi : x[j];
            lo = lo < x[j] ? lo : x[j];
        }
        const float extreme = fabsf(hi) > fabsf(lo) ? hi : lo;
        const float inverse = extreme == 0.0f ? 0.0f : -127.0f / extreme;
        const float d = inverse == 0.0f ? 0.0f : 1.0f / inverse;
        q8_K_fill(x, y, inverse, d);
    }
}

/* ggml/src/ggml-quants.c:741-820 (make_qkx2_quants) for n = 32, nmax = 15, rmin = -1,
 * rdelta = 0.1, nstep = 20, squared error: weighted least-squares (scale, min) search. */
static float fit_scale_min_32(const float *x, const float *wt, uint8_t *L, float *the_min) {
    uint8_t Laux[32];
    float lo = x[0], hi = x[0];
    float sum_w = wt[0];
    float sum_x = sum_w * x[0];
    for (int i = 1; i < 32; ++i) {
        if (x[i] < lo) lo = x[i];
        if (x[i] > hi) hi = x[i];
        sum_w += wt[i];
        sum_x += wt[i] * x[i];
    }
    if (lo > 0) lo = 0;
    if (hi == lo) {
        memset(L, 0, 32);
        *the_min = -lo;
        return 0.f;
    }
    float iscale = 15 / (hi - lo);
    float scale = 1 / iscale;
    float best = 0;
    for (int i = 0; i < 32; ++i) {
        int l = rne_int(iscale * (x[i] - lo));
        l = l < 0 ? 0 : (l > 15 ? 15 : l);
        L[i] = (uint8_t)l;
        float diff = scale * L[i] + lo - x[i];
        diff = diff * diff;
        best += wt[i] * diff;
    }
    for (int step = 0; step <= 20; ++step) {
        iscale = (-1.f + 0.1f * step + 15) / (hi - lo);
        float sum_l = 0, sum_l2 = 0, sum_xl = 0;
        for (int i = 0; i < 32; ++i) {
            int l = rne_int(iscale * (x[i] - lo));
            l = l < 0 ? 0 : (l > 15 ? 15 : l);
            Laux[i] = (uint8_t)l;
            const float w = wt[i];
            sum_l += w * l;
            sum_l2 += w * l * l;
            sum_xl += w * l * x[i];
        }
        const float D = sum_w * sum_l2 - sum_l * sum_l;
        if (D > 0) {
            float this_scale = (sum_w * sum_xl - sum_x * sum_l) / D;
            float this_min = (sum_l2 * sum_x - sum_l * sum_xl) / D;
            if (this_min > 0) {
                this_min = 0;
                this_scale = sum_xl / sum_l2;
            }
            float err = 0;
            for (int i = 0; i < 32; ++i) {
                float diff = this_scale * Laux[i] + this_min - x[i];
                diff = diff * diff;
                err += wt[i] * diff;
            }
            if (err < best) {
                memcpy(L, Laux, 32);
                best = err;
                scale = this_scale;
                lo = this_min;
            }
        }
    }
    *the_min = -lo;
    return scale;
}

/* 6-bit (scale, min) pair g of a Q4_K record: ggml/src/ggml-quants.c:822-829 (get_scale_min_k4) */
static inline void q4k_scale_min(const uint8_t *s12, int g, int *sc, int *mn) {
    if (g < 4) {
        *sc = s12[g] & 63;
        *mn = s12[g + 4] & 63;
    } else {
        *sc = (s12[g + 4] & 0x0f) | ((s12[g - 4] >> 6) << 4);
        *mn = (s12[g + 4] >> 4) | ((s12[g] >> 6) << 4);
    }
}

/* ggml/src/ggml-quants.c:1399-1469 (quantize_row_q4_K_ref).
 * Record: f16 d @0, f16 dmin @2, 12 scale bytes @4, 128 nibble bytes @16. */
void wo_quantize_row_q4_K(const float *x, uint8_t *y, int64_t k) {
    uint8_t L[256];
    float wt[32], mins[8], scales[8];
    for (int64_t b = 0; b < k / 256; ++b, x += 256, y += 144) {
        float max_scale = 0, max_min = 0;
        for (int g = 0; g < 8; ++g) {
            const float *xs = x + 32 * g;
            float sum_x2 = 0;
            for (int l = 0; l < 32; ++l) sum_x2 += xs[l] * xs[l];
            const float av_x = sqrtf(sum_x2 / 32);
            for (int l = 0; l < 32; ++l) wt[l] = av_x + fabsf(xs[l]);
            scales[g] = fit_scale_min_32(xs, wt, L + 32 * g, &mins[g]);
            if (scales[g] > max_scale) max_scale = scales[g];
            if (mins[g] > max_min) max_min = mins[g];
        }
        const float inv_scale = max_scale > 0 ? 63.f / max_scale : 0.f;
        const float inv_min = max_min > 0 ? 63.f / max_min : 0.f;
        uint8_t *s12 = y + 4;
        memset(s12, 0, 12);
        for (int g = 0; g < 8; ++g) {
            uint8_t ls = (uint8_t)rne_int(inv_scale * scales[g]);
            uint8_t lm = (uint8_t)rne_int(inv_min * mins[g]);
            if (ls > 63) ls = 63;
            if (lm > 63) lm = 63;
            if (g < 4) {
                s12[g] |= ls;          /* bits 6-7 of these bytes are filled by groups 4..7 below */
                s12[g + 4] |= lm;
            } else {
                s12[g + 4] = (uint8_t)((ls & 0x0f) | ((lm & 0x0f) << 4));
                s12[g - 4] |= (uint8_t)((ls >> 4) << 6);
                s12[g] |= (uint8_t)((lm >> 4) << 6);
            }
        }
        st_u16(y, wo_f32_to_f16(max_scale / 63.f));
        st_u16(y + 2, wo_f32_to_f16(max_min / 63.f));
        const float fd = wo_f16_to_f32(ld_u16(y)), fmin = wo_f16_to_f32(ld_u16(y + 2));
        for (int g = 0; g < 8; ++g) {
            int sc, mn;
            q4k_scale_min(s12, g, &sc, &mn);
            const float d = fd * sc;
            if (!d) continue;
            const float dm = fmin * mn;
            for (int l = 0; l < 32; ++l) {
                int q = rne_int((x[32 * g + l] + dm) / d);
                L[32 * g + l] = (uint8_t)(q < 0 ? 0 : (q > 15 ? 15 : q));
            }
        }
        uint8_t *qs = y + 16;
        for (int j = 0; j < 4; ++j)
            for (int l = 0; l < 32; ++l) qs[32 * j + l] = (uint8_t)(L[64 * j + l] | (L[64 * j + 32 + l] << 4));
    }
}

/* one packed byte from `count` trits taken at stride `stride` (most significant first),
 * then the ceil(q*256/243) fixed-point scaling of ggml/src/ggml-quants.c:2271-2272 */
static uint8_t tq1_pack(const float *x, float id, int count, int stride) {
    uint8_t q = 0;
    for (int n = 0; n < count; ++n) {
        const int t = (int)lroundf(x[n * stride] * id) + 1;
        q = (uint8_t)(q * 3 + t);
    }
    if (count == 4) q = (uint8_t)(q * 3);
    return (uint8_t)(((uint16_t)q * 256 + 242) / 243);
}

/* ggml/src/ggml-quants.c:2244-2308 (quantize_row_tq1_0_ref).
 * Record: 48 bytes of 5 trits @0 (32 bytes over 160 elements, 16 over 80), 4 bytes of 4 trits @48, f16 d @52. */
void wo_quantize_row_tq1_0(const float *x, uint8_t *y, int64_t k) {
    for (int64_t b = 0; b < k / 256; ++b, x += 256, y += 54) {
        float amax = 0.0f;
        for (int j = 0; j < 256; ++j) amax = amax > fabsf(x[j]) ? amax : fabsf(x[j]);
        const float id = amax ? 1.0f / amax : 0.0f;
        st_u16(y + 52, wo_f32_to_f16(amax));
        for (int m = 0; m < 32; ++m) y[m] = tq1_pack(x + m, id, 5, 32);
        for (int m = 0; m < 16; ++m) y[32 + m] = tq1_pack(x + 160 + m, id, 5, 16);
        for (int j = 0; j < 4; ++j) y[48 + j] = tq1_pack(x + 240 + j, id, 4, 4);
    }
}

typedef struct { int fmt, rule; const float *x; uint8_t *y; int64_t k; size_t rb; } wo_quant_ctx;

static void wo_quantize_range(int64_t begin, int64_t end, void *p) {
    const wo_quant_ctx *c = (const wo_quant_ctx *)p;
    const int fmt = c->fmt, rule = c->rule;
    const int64_t k = c->k;
    for (int64_t r = begin; r < end; ++r) {
        const float *xr = c->x + r * k;
        uint8_t *yr = c->y + r * c->rb;
        switch (fmt) {
        case WO_Q4_0: wo_quantize_row_q4_0(xr, yr, k); break;
        case WO_Q4_K: wo_quantize_row_q4_K(xr, yr, k); break;
        case WO_TQ1_0: wo_quantize_row_tq1_0(xr, yr, k); break;
        case WO_Q8_0: if (rule) wo_quantize_row_q8_0_weft(xr, yr, k); else wo_quantize_row_q8_0(xr, yr, k); break;
        case WO_Q8_1: if (rule) wo_quantize_row_q8_1_weft(xr, yr, k); else wo_quantize_row_q8_1(xr, yr, k); break;
        case WO_Q8_K: if (rule) wo_quantize_row_q8_K_weft(xr, yr, k); else wo_quantize_row_q8_K(xr, yr, k); break;
        default: break;
        }
    }
}

int wo_quantize_rows(int fmt, int rule, const float *x, uint8_t *y, int64_t nrows, int64_t k) {
    wo_quant_ctx c = {fmt, rule, x, y, k, wo_row_bytes(fmt, k)};
    if (!c.rb || fmt == WO_IQ2_XXS || fmt == WO_IQ2_XS || fmt == WO_IQ3_XXS || fmt == WO_IQ2_S || fmt == WO_IQ3_S || fmt == WO_IQ1_S || fmt == WO_IQ1_M) return -1;
    wo_parallel_for(nrows, wo_quantize_range, &c);
    return 0;
}

/* ----------------------------------------------------------- dequantizers */

/* ggml/src/ggml-quants.c:401-419; examples/kernels/dequantize/q4_0.py:9-13 */
void wo_dequantize_row_q4_0(const uint8_t *w, float *y, int64_t k) {
    for (int64_t b = 0; b < k / 32; ++b, w += 18, y += 32) {
        const float d = wo_f16_to_f32(ld_u16(w));
        for (int j = 0; j < 16; ++j) {
            y[j] = (float)((w[2 + j] & 0x0f) - 8) * d;
            y[j + 16] = (float)((w[2 + j] >> 4) - 8) * d;
        }
    }
}

/* ggml/src/ggml-quants.c:495-509; examples/kernels/dequantize/q8_0.py:9-13 */
void wo_dequantize_row_q8_0(const uint8_t *w, float *y, int64_t k) {
    for (int64_t b = 0; b < k / 32; ++b, w += 34, y += 32) {
        const float d = wo_f16_to_f32(ld_u16(w));
        for (int j = 0; j < 32; ++j) y[j] = (float)(int8_t)w[2 + j] * d;
    }
}

/* ggml/src/ggml-quants.c:1471-1493; examples/functions/quantization.py:14-17:
 * (d*sc)*q - (dmin*m) with three separately rounded multiplies and one subtract. */
void wo_dequantize_row_q4_K(const uint8_t *w, float *y, int64_t k) {
    for (int64_t b = 0; b < k / 256; ++b, w += 144) {
        const float d = wo_f16_to_f32(ld_u16(w)), dmin = wo_f16_to_f32(ld_u16(w + 2));
        const uint8_t *qs = w + 16;
        for (int j = 0; j < 4; ++j, qs += 32) {
            int sc, mn;
            q4k_scale_min(w + 4, 2 * j, &sc, &mn);
            const float d1 = d * sc, m1 = dmin * mn;
            q4k_scale_min(w + 4, 2 * j + 1, &sc, &mn);
            const float d2 = d * sc, m2 = dmin * mn;
            for (int l = 0; l < 32; ++l) *y++ = d1 * (qs[l] & 0x0f) - m1;
            for (int l = 0; l < 32; ++l) *y++ = d2 * (qs[l] >> 4) - m2;
        }
    }
}

/* ggml/src/ggml-quants.c:2416-2440; examples/kernels/dequantize/iq2_xxs.py:9-53.
 * Record: f16 d @0, then 8 groups of {4 grid-index bytes, u32: 4 x 7-bit sign index | 4-bit scale << 28}. */
void wo_dequantize_row_iq2_xxs(const uint8_t *w, const int8_t *grid, const int8_t *signs, float *y, int64_t k) {
    for (int64_t b = 0; b < k / 256; ++b, w += 66) {
        const float d = wo_f16_to_f32(ld_u16(w));
        for (int g = 0; g < 8; ++g) {
            const uint8_t *idx = w + 2 + 8 * g;
            uint32_t meta;
            memcpy(&meta, idx + 4, 4);
            const float db = d * (0.5f + (float)(meta >> 28)) * 0.25f;
            for (int e = 0; e < 4; ++e) {
                const int8_t *gv = grid + 8 * idx[e];
                const int8_t *sv = signs + 8 * ((meta >> (7 * e)) & 127);
                for (int j = 0; j < 8; ++j) *y++ = db * (float)gv[j] * (float)sv[j];
            }
        }
    }
}

/* ggml/src/ggml-quants.c:2444-2468; examples/kernels/dequantize/iq2_xs.py:9-68.
 * Record (74 bytes): f16 d @0, 32 u16 codes @2 (grid index in bits 0-8, sign index in bits 9-15, one code per 8
 * weights), 8 scale bytes @66 (low nibble: first 16 weights of a 32-group, high nibble: the other 16). */
void wo_dequantize_row_iq2_xs(const uint8_t *w, const int8_t *grid, const int8_t *signs, float *y, int64_t k) {
    for (int64_t b = 0; b < k / 256; ++b, w += 74) {
        const float d = wo_f16_to_f32(ld_u16(w));
        for (int g = 0; g < 8; ++g) {
            const uint8_t sc = w[66 + g];
            const float db[2] = {d * (0.5f + (float)(sc & 15)) * 0.25f, d * (0.5f + (float)(sc >> 4)) * 0.25f};
            for (int e = 0; e < 4; ++e) {
                const uint16_t code = ld_u16(w + 2 + 2 * (4 * g + e));
                const int8_t *gv = grid + 8 * (code & 511);
                const int8_t *sv = signs + 8 * (code >> 9);
                for (int j = 0; j < 8; ++j) *y++ = db[e >> 1] * (float)(uint8_t)gv[j] * (float)sv[j];
            }
        }
    }
}

/* ggml/src/ggml-quants.c:2506-2536; examples/kernels/dequantize/iq3_xxs.py.
 * Record (98 bytes): f16 d @0, 64 grid-index bytes @2 (one per 4 weights), 8 u32 @66: four 7-bit sign indices (one per
 * 8 weights) and a 4-bit scale in bits 28-31, one word per 32 weights. */
void wo_dequantize_row_iq3_xxs(const uint8_t *w, const int8_t *grid, const int8_t *signs, float *y, int64_t k) {
    for (int64_t b = 0; b < k / 256; ++b, w += 98) {
        const float d = wo_f16_to_f32(ld_u16(w));
        for (int g = 0; g < 8; ++g) {
            uint32_t meta;
            memcpy(&meta, w + 66 + 4 * g, 4);
            const float db = d * (0.5f + (float)(meta >> 28)) * 0.5f;
            for (int e = 0; e < 4; ++e) {
                const int8_t *sv = signs + 8 * ((meta >> (7 * e)) & 127);
                const int8_t *g1 = grid + 4 * w[2 + 8 * g + 2 * e], *g2 = grid + 4 * w[2 + 8 * g + 2 * e + 1];
                for (int j = 0; j < 4; ++j) y[j] = db * (float)(uint8_t)g1[j] * (float)sv[j];
                for (int j = 0; j < 4; ++j) y[4 + j] = db * (float)(uint8_t)g2[j] * (float)sv[4 + j];
                y += 8;
            }
        }
    }
}

/* ggml/src/ggml-quants.c (dequantize_row_iq2_s); examples/kernels/dequantize/iq2_s.py.
 * Record (82 bytes): f16 d @0; 32 bytes @2: the low 8 bits of the grid index of every 8 weights; 32 bytes @34: their
 * sign bits (bit j set: weight j negative); 8 bytes @66: per 32 weights four 2-bit pairs, index bits 8-9; 8 scale
 * bytes @74 (low nibble: first 16 weights of the 32, high nibble: the other 16). */
static inline int iq2s_index(const uint8_t *w, int g, int e) { return w[2 + 4 * g + e] | ((w[66 + g] << (8 - 2 * e)) & 0x300); }

void wo_dequantize_row_iq2_s(const uint8_t *w, const int8_t *grid, float *y, int64_t k) {
    for (int64_t b = 0; b < k / 256; ++b, w += 82) {
        const float d = wo_f16_to_f32(ld_u16(w));
        for (int g = 0; g < 8; ++g) {
            const uint8_t sc = w[74 + g];
            const float db[2] = {d * (0.5f + (float)(sc & 15)) * 0.25f, d * (0.5f + (float)(sc >> 4)) * 0.25f};
            for (int e = 0; e < 4; ++e) {
                const int8_t *gv = grid + 8 * iq2s_index(w, g, e);
                const uint8_t sb = w[34 + 4 * g + e];
                for (int j = 0; j < 8; ++j) *y++ = db[e >> 1] * (float)(uint8_t)gv[j] * ((sb >> j) & 1 ? -1.f : 1.f);
            }
        }
    }
}

/* ggml/src/ggml-quants.c (dequantize_row_iq3_s); examples/kernels/dequantize/iq3_s.py.
 * Record (110 bytes): f16 d @0; 64 bytes @2: the low 8 bits of the grid index of every 4 weights; 8 bytes @66: bit e of
 * byte g is bit 8 of index e of 32-group g; 32 sign bytes @74 (one per 8 weights); 4 scale bytes @106 (nibble per 32
 * weights, low nibble first).  Scale d * (1 + 2 s). */
static inline int iq3s_index(const uint8_t *w, int g, int e) { return w[2 + 8 * g + e] | (((w[66 + g] >> e) & 1) << 8); }

void wo_dequantize_row_iq3_s(const uint8_t *w, const int8_t *grid, float *y, int64_t k) {
    for (int64_t b = 0; b < k / 256; ++b, w += 110) {
        const float d = wo_f16_to_f32(ld_u16(w));
        for (int g = 0; g < 8; ++g) {
            const uint8_t sc = w[106 + (g >> 1)];
            const float db = d * (float)(1 + 2 * (g & 1 ? sc >> 4 : sc & 15));
            for (int e = 0; e < 4; ++e) {
                const int8_t *g1 = grid + 4 * iq3s_index(w, g, 2 * e), *g2 = grid + 4 * iq3s_index(w, g, 2 * e + 1);
                const uint8_t sb = w[74 + 4 * g + e];
                for (int j = 0; j < 4; ++j) y[j] = db * (float)(uint8_t)g1[j] * ((sb >> j) & 1 ? -1.f : 1.f);
                for (int j = 0; j < 4; ++j) y[4 + j] = db * (float)(uint8_t)g2[j] * ((sb >> (4 + j)) & 1 ? -1.f : 1.f);
                y += 8;
            }
        }
    }
}

/* ggml/src/ggml-quants.c (dequantize_row_iq1_s); examples/kernels/dequantize/iq1_s.py.
 * Record (50 bytes): f16 d @0; 32 bytes @2: low 8 bits of the grid index of every 8 weights; 8 u16 @34, one per 32 weights:
 * bits 0-11 four 3-bit index tops, bits 12-14 scale, bit 15 the sign of the shift 0.125.  Grid values are -1, 0, +1. */
void wo_dequantize_row_iq1_s(const uint8_t *w, const int8_t *grid, float *y, int64_t k) {
    for (int64_t b = 0; b < k / 256; ++b, w += 50) {
        const float d = wo_f16_to_f32(ld_u16(w));
        for (int g = 0; g < 8; ++g) {
            const uint16_t qh = ld_u16(w + 34 + 2 * g);
            const float dl = d * (float)(2 * ((qh >> 12) & 7) + 1);
            const float delta = qh & 0x8000 ? -0.125f : 0.125f;
            for (int e = 0; e < 4; ++e) {
                const int8_t *gv = grid + 8 * (w[2 + 4 * g + e] | (((qh >> (3 * e)) & 7) << 8));
                for (int j = 0; j < 8; ++j) *y++ = dl * ((float)gv[j] + delta);
            }
        }
    }
}

/* IQ1_M (56 bytes, no d field): 32 index bytes @0; 16 bytes @32, one per 16 weights: low nibble {3 index bits, shift
 * sign} of the first 8 weights, high nibble of the other 8; 8 bytes @48 read as four u16: bits 0-11 four 3-bit scales
 * (one per 16 weights), bits 12-15 a nibble of the record's f16 scale.  ggml/src/ggml-quants.c (dequantize_row_iq1_m). */
static inline float iq1m_scale(const uint8_t *w) {
    const uint16_t s0 = ld_u16(w + 48), s1 = ld_u16(w + 50), s2 = ld_u16(w + 52), s3 = ld_u16(w + 54);
    return wo_f16_to_f32((uint16_t)((s0 >> 12) | ((s1 >> 8) & 0x00f0) | ((s2 >> 4) & 0x0f00) | (s3 & 0xf000)));
}
static inline int iq1m_index(const uint8_t *w, int g, int e) {
    const uint8_t qh = w[32 + 2 * g + (e >> 1)];
    return w[4 * g + e] | (((e & 1 ? qh >> 4 : qh) & 7) << 8);
}
static inline int iq1m_negative(const uint8_t *w, int g, int e) { return (w[32 + 2 * g + (e >> 1)] >> (e & 1 ? 7 : 3)) & 1; }
static inline int iq1m_sub_scale(const uint8_t *w, int g, int half) { return (ld_u16(w + 48 + 2 * (g >> 1)) >> (6 * (g & 1) + 3 * half)) & 7; }

void wo_dequantize_row_iq1_m(const uint8_t *w, const int8_t *grid, float *y, int64_t k) {
    for (int64_t b = 0; b < k / 256; ++b, w += 56) {
        const float d = iq1m_scale(w);
        for (int g = 0; g < 8; ++g)
            for (int e = 0; e < 4; ++e) {
                const float dl = d * (float)(2 * iq1m_sub_scale(w, g, e >> 1) + 1);
                const float delta = iq1m_negative(w, g, e) ? -0.125f : 0.125f;
                const int8_t *gv = grid + 8 * iq1m_index(w, g, e);
                for (int j = 0; j < 8; ++j) *y++ = dl * ((float)gv[j] + delta);
            }
    }
}

/* one base-3 digit of a packed byte, digit 0 = most significant:
 * ggml/src/ggml-quants.c:2369-2371; examples/functions/quantization.py:49-64 */
static inline int tq1_digit(uint8_t packed, int n) {
    static const uint8_t pow3[5] = {1, 3, 9, 27, 81};
    const uint8_t q = (uint8_t)(packed * pow3[n]);
    return (int)(((uint16_t)q * 3) >> 8) - 1;
}

/* ggml/src/ggml-quants.c:2356-2393; examples/kernels/dequantize/tq1_0.py:9-46 */
void wo_dequantize_row_tq1_0(const uint8_t *w, float *y, int64_t k) {
    for (int64_t b = 0; b < k / 256; ++b, w += 54) {
        const float d = wo_f16_to_f32(ld_u16(w + 52));
        for (int n = 0; n < 5; ++n)
            for (int m = 0; m < 32; ++m) *y++ = (float)tq1_digit(w[m], n) * d;
        for (int n = 0; n < 5; ++n)
            for (int m = 0; m < 16; ++m) *y++ = (float)tq1_digit(w[32 + m], n) * d;
        for (int n = 0; n < 4; ++n)
            for (int j = 0; j < 4; ++j) *y++ = (float)tq1_digit(w[48 + j], n) * d;
    }
}

typedef struct { int fmt; const uint8_t *w; const int8_t *grid, *signs; float *y; int64_t k; size_t rb; } wo_deq_ctx;

static void wo_dequantize_range(int64_t begin, int64_t end, void *p) {
    const wo_deq_ctx *c = (const wo_deq_ctx *)p;
    for (int64_t r = begin; r < end; ++r) {
        const uint8_t *wr = c->w + r * c->rb;
        float *yr = c->y + r * c->k;
        switch (c->fmt) {
        case WO_Q4_0: wo_dequantize_row_q4_0(wr, yr, c->k); break;
        case WO_Q8_0: wo_dequantize_row_q8_0(wr, yr, c->k); break;
        case WO_Q4_K: wo_dequantize_row_q4_K(wr, yr, c->k); break;
        case WO_Q2_K: wo_dequantize_row_q2_K(wr, yr, c->k); break;
        case WO_Q3_K: wo_dequantize_row_q3_K(wr, yr, c->k); break;
        case WO_Q5_K: wo_dequantize_row_q5_K(wr, yr, c->k); break;
        case WO_Q6_K: wo_dequantize_row_q6_K(wr, yr, c->k); break;
        case WO_IQ2_XXS: wo_dequantize_row_iq2_xxs(wr, c->grid, c->signs, yr, c->k); break;
        case WO_IQ2_XS: wo_dequantize_row_iq2_xs(wr, c->grid, c->signs, yr, c->k); break;
        case WO_IQ3_XXS: wo_dequantize_row_iq3_xxs(wr, c->grid, c->signs, yr, c->k); break;
        case WO_IQ2_S: wo_dequantize_row_iq2_s(wr, c->grid, yr, c->k); break;
        case WO_IQ1_S: wo_dequantize_row_iq1_s(wr, c->grid, yr, c->k); break;
        case WO_IQ1_M: wo_dequantize_row_iq1_m(wr, c->grid, yr, c->k); break;
        case WO_IQ3_S: wo_dequantize_row_iq3_s(wr, c->grid, yr, c->k); break;
        case WO_TQ1_0: wo_dequantize_row_tq1_0(wr, yr, c->k); break;
        default: break;
        }
    }
}

int wo_dequantize_rows(int fmt, const uint8_t *w, const int8_t *grid, const int8_t *signs,
                       float *y, int64_t nrows, int64_t k) {
    wo_deq_ctx c = {fmt, w, grid, signs, y, k, wo_row_bytes(fmt, k)};
    if (!c.rb || fmt == WO_Q8_K) return -1;
    wo_parallel_for(nrows, wo_dequantize_range, &c);
    return 0;
}

/* ------------------------------------------------------------ dot products */

/* ggml/src/ggml-cpu/quants.c:174-208: sumf += sumi * d_w * d_x (left to right) */
float wo_vec_dot_q4_0_q8_0(const uint8_t *w, const uint8_t *x, int64_t k) {
    float sumf = 0;
    for (int64_t b = 0; b < k / 32; ++b, w += 18, x += 34) {
        const int8_t *xq = (const int8_t *)(x + 2);
        int lo = 0, hi = 0;
        for (int j = 0; j < 16; ++j) {
            lo += ((w[2 + j] & 0x0f) - 8) * xq[j];
            hi += ((w[2 + j] >> 4) - 8) * xq[j + 16];
        }
        const int sumi = lo + hi;
        sumf += sumi * wo_f16_to_f32(ld_u16(w)) * wo_f16_to_f32(ld_u16(x));
    }
    return sumf;
}

/* ggml/src/ggml-cpu/quants.c:400-428: sumf += sumi * (d_w * d_x) */
float wo_vec_dot_q8_0_q8_0(const uint8_t *w, const uint8_t *x, int64_t k) {
    float sumf = 0;
    for (int64_t b = 0; b < k / 32; ++b, w += 34, x += 34) {
        const int8_t *wq = (const int8_t *)(w + 2), *xq = (const int8_t *)(x + 2);
        int sumi = 0;
        for (int j = 0; j < 32; ++j) sumi += wq[j] * xq[j];
        sumf += sumi * (wo_f16_to_f32(ld_u16(w)) * wo_f16_to_f32(ld_u16(x)));
    }
    return sumf;
}

/* ggml/src/ggml-cpu/quants.c:645-718: eight float lane sums (element index mod 8), the
 * min correction subtracted from a ninth running sum, lanes added at the end. */
float wo_vec_dot_q4_K_q8_K(const uint8_t *w, const uint8_t *x, int64_t k) {
    float lanes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    float sumf = 0;
    int8_t a[256];
    for (int64_t b = 0; b < k / 256; ++b, w += 144, x += 292) {
        const uint8_t *qs = w + 16;
        const int8_t *xq = (const int8_t *)(x + 4);
        for (int j = 0; j < 4; ++j)
            for (int l = 0; l < 32; ++l) {
                a[64 * j + l] = (int8_t)(qs[32 * j + l] & 0x0f);
                a[64 * j + 32 + l] = (int8_t)(qs[32 * j + l] >> 4);
            }
        int32_t lane_i[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        int sum_min = 0;
        for (int g = 0; g < 8; ++g) {
            int sc, mn;
            q4k_scale_min(w + 4, g, &sc, &mn);
            sum_min += (ld_i16(x + 260 + 4 * g) + ld_i16(x + 260 + 4 * g + 2)) * mn;
            for (int l = 0; l < 32; ++l) lane_i[l & 7] += sc * (int16_t)(xq[32 * g + l] * a[32 * g + l]);
        }
        const float xd = ld_f32(x);
        const float d = wo_f16_to_f32(ld_u16(w)) * xd;
        for (int l = 0; l < 8; ++l) lanes[l] += d * lane_i[l];
        const float dmin = wo_f16_to_f32(ld_u16(w + 2)) * xd;
        sumf -= dmin * sum_min;
    }
    for (int l = 0; l < 8; ++l) sumf += lanes[l];
    return sumf;
}

/* ---- Q2_K: 84 bytes per 256 weights = scales[16] (low nibble scale, high nibble min, one per 16 weights),
 * qs[64] (2-bit weights), f16 d, f16 dmin  (ggml/src/ggml-common.h:288-298; examples/formats/ggml.py class Q2_K).
 * Weight 128 n + 32 j + l is bits 2j, 2j+1 of qs[32 n + l]; its scale byte is scales[e / 16]. */
static int q2k_value(const uint8_t *rec, int e) {
    return (rec[16 + 32 * (e >> 7) + (e & 31)] >> (2 * ((e >> 5) & 3))) & 3;
}

/* ggml/src/ggml-quants.c:903-933; examples/kernels/dequantize/q2_k.py:8-17: (d*sc)*q - (dmin*m) */
void wo_dequantize_row_q2_K(const uint8_t *w, float *y, int64_t k) {
    for (int64_t b = 0; b < k / 256; ++b, w += 84, y += 256) {
        const float d = wo_f16_to_f32(ld_u16(w + 80)), dmin = wo_f16_to_f32(ld_u16(w + 82));
        for (int g = 0; g < 16; ++g) {
            const float dl = d * (w[g] & 0x0f), ml = dmin * (w[g] >> 4);
            for (int l = 0; l < 16; ++l) y[16 * g + l] = dl * (int8_t)q2k_value(w, 16 * g + l) - ml;
        }
    }
}

/* ggml/src/ggml-cpu/quants.c:514-564; examples/kernels/vec_dot/q2_k_q8_k.py:8-25:
 * sumf += (x.d * d) * isum - (x.d * dmin) * sum_g bsums[g] * min_g */
float wo_vec_dot_q2_K_q8_K(const uint8_t *w, const uint8_t *x, int64_t k) {
    float sumf = 0;
    for (int64_t b = 0; b < k / 256; ++b, w += 84, x += 292) {
        const int8_t *xq = (const int8_t *)(x + 4);
        int summs = 0, isum = 0;
        for (int g = 0; g < 16; ++g) summs += ld_i16(x + 260 + 2 * g) * (w[g] >> 4);
        const float xd = ld_f32(x);
        const float dall = xd * wo_f16_to_f32(ld_u16(w + 80)), dmin = xd * wo_f16_to_f32(ld_u16(w + 82));
        for (int g = 0; g < 16; ++g) {
            int part = 0;
            for (int l = 0; l < 16; ++l) part += xq[16 * g + l] * q2k_value(w, 16 * g + l);
            isum += (w[g] & 0x0f) * part;
        }
        sumf += dall * isum - dmin * summs;
    }
    return sumf;
}

/* ---- Q3_K: 110 bytes per 256 weights = hmask[32] (third bits), qs[64] (low two bits, laid out as Q2_K),
 * scales[12] (sixteen 6-bit scales), f16 d  (ggml/src/ggml-common.h:305-311; examples/formats/ggml.py class Q3_K).
 * Weight e = low two bits minus 4 unless bit e / 32 of hmask[e % 32] is set; scale e / 16, stored plus 32:
 * low nibble from byte g % 8 (high nibble for g >= 8), bits 4-5 from bits 2 (g / 4) of byte 8 + g % 4. */
static int q3k_value(const uint8_t *rec, int e) {
    const int low = (rec[32 + 32 * (e >> 7) + (e & 31)] >> (2 * ((e >> 5) & 3))) & 3;
    return low - (((rec[e & 31] >> (e >> 5)) & 1) ? 0 : 4);
}
static int q3k_scale(const uint8_t *s12, int g) {
    const int low = g < 8 ? (s12[g] & 0x0f) : (s12[g - 8] >> 4);
    const int high = (s12[8 + (g & 3)] >> (2 * (g >> 2))) & 3;
    return (int8_t)(low | (high << 4)) - 32;
}

/* ggml/src/ggml-quants.c:1247-1294; examples/kernels/dequantize/q3_k.py:8-17: (d * scale) * q */
void wo_dequantize_row_q3_K(const uint8_t *w, float *y, int64_t k) {
    for (int64_t b = 0; b < k / 256; ++b, w += 110, y += 256) {
        const float d = wo_f16_to_f32(ld_u16(w + 108));
        for (int g = 0; g < 16; ++g) {
            const float dl = d * q3k_scale(w + 96, g);
            for (int l = 0; l < 16; ++l) y[16 * g + l] = dl * q3k_value(w, 16 * g + l);
        }
    }
}

/* ggml/src/ggml-cpu/quants.c:566-643; examples/kernels/vec_dot/q3_k_q8_k.py:8-43: eight int32 lane sums per
 * block, float lanes, lanes added at the end */
float wo_vec_dot_q3_K_q8_K(const uint8_t *w, const uint8_t *x, int64_t k) {
    float lanes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int64_t b = 0; b < k / 256; ++b, w += 110, x += 292) {
        const int8_t *xq = (const int8_t *)(x + 4);
        int32_t lane_i[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int e = 0; e < 256; ++e) lane_i[e & 7] += q3k_scale(w + 96, e >> 4) * (int16_t)(xq[e] * (int8_t)q3k_value(w, e));
        const float d = wo_f16_to_f32(ld_u16(w + 108)) * ld_f32(x);
        for (int l = 0; l < 8; ++l) lanes[l] += d * lane_i[l];
    }
    float sumf = 0;
    for (int l = 0; l < 8; ++l) sumf += lanes[l];
    return sumf;
}

/* ---- Q5_K: 176 bytes per 256 weights = f16 d, f16 dmin, the Q4_K 12-byte (scale, min) field, qh[32] (fifth
 * bits), qs[128] (nibbles, laid out as in Q4_K)  (ggml/src/ggml-common.h block_q5_K; examples/formats/ggml.py
 * class Q5_K).  Weight 32 g + l (g = 0..7): nibble g & 1 of qs[32 (g / 2) + l], plus 16 when bit g of qh[l] is set. */
static int q5k_value(const uint8_t *rec, int e) {
    const int g = e >> 5, l = e & 31;
    const uint8_t lo = rec[48 + 32 * (g >> 1) + l];
    return ((g & 1) ? (lo >> 4) : (lo & 0x0f)) + (((rec[16 + l] >> g) & 1) ? 16 : 0);
}

/* ggml/src/ggml-quants.c:1673-1698; examples/kernels/dequantize/q5_k.py:9-15: (d*sc)*q - (dmin*m) */
void wo_dequantize_row_q5_K(const uint8_t *w, float *y, int64_t k) {
    for (int64_t b = 0; b < k / 256; ++b, w += 176, y += 256) {
        const float d = wo_f16_to_f32(ld_u16(w)), dmin = wo_f16_to_f32(ld_u16(w + 2));
        for (int g = 0; g < 8; ++g) {
            int sc, mn;
            q4k_scale_min(w + 4, g, &sc, &mn);
            const float d1 = d * sc, m1 = dmin * mn;
            for (int l = 0; l < 32; ++l) y[32 * g + l] = d1 * q5k_value(w, 32 * g + l) - m1;
        }
    }
}

/* ggml/src/ggml-cpu/quants.c:720-798; examples/kernels/vec_dot/q5_k_q8_k.py:8-31: as Q4_K with 5-bit weights */
float wo_vec_dot_q5_K_q8_K(const uint8_t *w, const uint8_t *x, int64_t k) {
    float lanes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    float sumf = 0;
    for (int64_t b = 0; b < k / 256; ++b, w += 176, x += 292) {
        const int8_t *xq = (const int8_t *)(x + 4);
        int32_t lane_i[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        int sum_min = 0;
        for (int g = 0; g < 8; ++g) {
            int sc, mn;
            q4k_scale_min(w + 4, g, &sc, &mn);
            sum_min += (ld_i16(x + 260 + 4 * g) + ld_i16(x + 260 + 4 * g + 2)) * mn;
            for (int l = 0; l < 32; ++l) lane_i[l & 7] += sc * (int16_t)(xq[32 * g + l] * q5k_value(w, 32 * g + l));
        }
        const float xd = ld_f32(x);
        const float d = wo_f16_to_f32(ld_u16(w)) * xd;
        for (int l = 0; l < 8; ++l) lanes[l] += d * lane_i[l];
        const float dmin = wo_f16_to_f32(ld_u16(w + 2)) * xd;
        sumf -= dmin * sum_min;
    }
    for (int l = 0; l < 8; ++l) sumf += lanes[l];
    return sumf;
}

/* ---- Q6_K: 210 bytes per 256 weights = ql[128] (low nibbles), qh[64] (high 2 bits), int8 scales[16], f16 d
 * (ggml/src/ggml-common.h:349-358; examples/formats/ggml.py class Q6_K).  In each half of 128 weights,
 * weight 32 p + l (p = 0..3, l = 0..31) takes its low nibble from ql[l + 32 (p & 1)] (low half for p < 2, high
 * half otherwise) and its two high bits from bits 2p, 2p+1 of qh[l]; value = that 6-bit number - 32; its
 * scale is scales[8 half + 2 p + l / 16]. */
static int q6k_value(const uint8_t *rec, int e) {
    const int half = e >> 7, p = (e >> 5) & 3, l = e & 31;
    const uint8_t lo = rec[64 * half + l + 32 * (p & 1)];
    const int nib = p < 2 ? (lo & 0x0f) : (lo >> 4);
    const int hi = (rec[128 + 32 * half + l] >> (2 * p)) & 3;
    return (int8_t)(nib | (hi << 4)) - 32;
}

/* ggml/src/ggml-quants.c:1881-1910; examples/kernels/dequantize/q6_k.py:8-14: y = (d * scale) * q */
void wo_dequantize_row_q6_K(const uint8_t *w, float *y, int64_t k) {
    for (int64_t b = 0; b < k / 256; ++b, w += 210, y += 256) {
        const float d = wo_f16_to_f32(ld_u16(w + 208));
        const int8_t *sc = (const int8_t *)(w + 192);
        for (int e = 0; e < 256; ++e) y[e] = d * sc[e >> 4] * q6k_value(w, e);
    }
}

/* ggml/src/ggml-cpu/quants.c:800-853; examples/kernels/vec_dot/q6_k_q8_k.py:8-36: per block eight int32 lane
 * sums (element index mod 8) of scale * (x * q), each added to its float lane as (d_w * d_x) * sum; the
 * eight float lanes are added at the end, lane 0 first. */
float wo_vec_dot_q6_K_q8_K(const uint8_t *w, const uint8_t *x, int64_t k) {
    float lanes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int64_t b = 0; b < k / 256; ++b, w += 210, x += 292) {
        const int8_t *xq = (const int8_t *)(x + 4);
        const int8_t *sc = (const int8_t *)(w + 192);
        int32_t lane_i[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int e = 0; e < 256; ++e) lane_i[e & 7] += sc[e >> 4] * (int16_t)(xq[e] * q6k_value(w, e));
        const float d = wo_f16_to_f32(ld_u16(w + 208)) * ld_f32(x);
        for (int l = 0; l < 8; ++l) lanes[l] += d * lane_i[l];
    }
    float sumf = 0;
    for (int l = 0; l < 8; ++l) sumf += lanes[l];
    return sumf;
}

/* ggml/src/ggml-cpu/quants.c:855-895; examples/kernels/vec_dot/iq2_xxs_q8_k.py:8-54 */
float wo_vec_dot_iq2_xxs_q8_K(const uint8_t *w, const uint8_t *x, const int8_t *grid, const int8_t *signs, int64_t k) {
    float sumf = 0.f;
    for (int64_t b = 0; b < k / 256; ++b, w += 66, x += 292) {
        const float d = wo_f16_to_f32(ld_u16(w)) * ld_f32(x);
        const int8_t *xq = (const int8_t *)(x + 4);
        int32_t bsum = 0;
        for (int g = 0; g < 8; ++g) {
            const uint8_t *idx = w + 2 + 8 * g;
            uint32_t meta;
            memcpy(&meta, idx + 4, 4);
            const int32_t ls = (int32_t)(2 * (meta >> 28) + 1);
            int32_t sumi = 0;
            for (int e = 0; e < 4; ++e) {
                const int8_t *gv = grid + 8 * idx[e];
                const int8_t *sv = signs + 8 * ((meta >> (7 * e)) & 127);
                for (int j = 0; j < 8; ++j) sumi += gv[j] * xq[32 * g + 8 * e + j] * sv[j];
            }
            bsum += sumi * ls;
        }
        sumf += d * bsum;
    }
    return 0.125f * sumf;
}

/* ggml/src/ggml-cpu/quants.c (ggml_vec_dot_iq2_xs_q8_K_generic); examples/kernels/vec_dot/iq2_xs_q8_k.py:9-39,
 * examples/functions/quantization.py:71-83: per 16 weights an odd integer scale 2 s + 1, result times 0.125 */
float wo_vec_dot_iq2_xs_q8_K(const uint8_t *w, const uint8_t *x, const int8_t *grid, const int8_t *signs, int64_t k) {
    float sumf = 0.f;
    for (int64_t b = 0; b < k / 256; ++b, w += 74, x += 292) {
        const float d = wo_f16_to_f32(ld_u16(w)) * ld_f32(x);
        const int8_t *xq = (const int8_t *)(x + 4);
        int32_t bsum = 0;
        for (int g = 0; g < 8; ++g) {
            const uint8_t sc = w[66 + g];
            for (int half = 0; half < 2; ++half) {
                const int32_t ls = 2 * (half ? sc >> 4 : sc & 15) + 1;
                int32_t sumi = 0;
                for (int e = 2 * half; e < 2 * half + 2; ++e) {
                    const uint16_t code = ld_u16(w + 2 + 2 * (4 * g + e));
                    const int8_t *gv = grid + 8 * (code & 511);
                    const int8_t *sv = signs + 8 * (code >> 9);
                    for (int j = 0; j < 8; ++j) sumi += (int)(uint8_t)gv[j] * xq[32 * g + 8 * e + j] * sv[j];
                }
                bsum += sumi * ls;
            }
        }
        sumf += d * bsum;
    }
    return 0.125f * sumf;
}

/* ggml/src/ggml-cpu/quants.c (ggml_vec_dot_iq3_xxs_q8_K_generic); examples/kernels/vec_dot/iq3_xxs_q8_k.py:8-75:
 * per 32 weights an odd integer scale, result times 0.25 */
float wo_vec_dot_iq3_xxs_q8_K(const uint8_t *w, const uint8_t *x, const int8_t *grid, const int8_t *signs, int64_t k) {
    float sumf = 0.f;
    for (int64_t b = 0; b < k / 256; ++b, w += 98, x += 292) {
        const float d = wo_f16_to_f32(ld_u16(w)) * ld_f32(x);
        const int8_t *xq = (const int8_t *)(x + 4);
        int32_t bsum = 0;
        for (int g = 0; g < 8; ++g) {
            uint32_t meta;
            memcpy(&meta, w + 66 + 4 * g, 4);
            const int32_t ls = (int32_t)(2 * (meta >> 28) + 1);
            int32_t sumi = 0;
            for (int e = 0; e < 4; ++e) {
                const int8_t *sv = signs + 8 * ((meta >> (7 * e)) & 127);
                const int8_t *g1 = grid + 4 * w[2 + 8 * g + 2 * e], *g2 = grid + 4 * w[2 + 8 * g + 2 * e + 1];
                for (int j = 0; j < 4; ++j) {
                    sumi += (int)(uint8_t)g1[j] * xq[32 * g + 8 * e + j] * sv[j];
                    sumi += (int)(uint8_t)g2[j] * xq[32 * g + 8 * e + 4 + j] * sv[4 + j];
                }
            }
            bsum += sumi * ls;
        }
        sumf += d * bsum;
    }
    return 0.25f * sumf;
}

/* ggml/src/ggml-cpu/quants.c (ggml_vec_dot_iq2_s_q8_K_generic); examples/kernels/vec_dot/iq2_s_q8_k.py:68-73 */
float wo_vec_dot_iq2_s_q8_K(const uint8_t *w, const uint8_t *x, const int8_t *grid, int64_t k) {
    float sumf = 0.f;
    for (int64_t b = 0; b < k / 256; ++b, w += 82, x += 292) {
        const float d = wo_f16_to_f32(ld_u16(w)) * ld_f32(x);
        const int8_t *xq = (const int8_t *)(x + 4);
        int32_t bsum = 0;
        for (int g = 0; g < 8; ++g) {
            const uint8_t sc = w[74 + g];
            for (int half = 0; half < 2; ++half) {
                const int32_t ls = 1 + 2 * (half ? sc >> 4 : sc & 15);
                int32_t sumi = 0;
                for (int e = 2 * half; e < 2 * half + 2; ++e) {
                    const int8_t *gv = grid + 8 * iq2s_index(w, g, e);
                    const uint8_t sb = w[34 + 4 * g + e];
                    for (int j = 0; j < 8; ++j) sumi += xq[32 * g + 8 * e + j] * (int)(uint8_t)gv[j] * ((sb >> j) & 1 ? -1 : 1);
                }
                bsum += ls * sumi;
            }
        }
        sumf += d * bsum;
    }
    return 0.125f * sumf;
}

/* ggml/src/ggml-cpu/quants.c (ggml_vec_dot_iq3_s_q8_K_generic); examples/kernels/vec_dot/iq3_s_q8_k.py:67-72 */
float wo_vec_dot_iq3_s_q8_K(const uint8_t *w, const uint8_t *x, const int8_t *grid, int64_t k) {
    float sumf = 0.f;
    for (int64_t b = 0; b < k / 256; ++b, w += 110, x += 292) {
        const float d = wo_f16_to_f32(ld_u16(w)) * ld_f32(x);
        const int8_t *xq = (const int8_t *)(x + 4);
        int32_t bsum = 0;
        for (int g = 0; g < 8; ++g) {
            const uint8_t sc = w[106 + (g >> 1)];
            const int32_t ls = 2 * (g & 1 ? sc >> 4 : sc & 15) + 1;
            int32_t sumi = 0;
            for (int e = 0; e < 4; ++e) {
                const int8_t *g1 = grid + 4 * iq3s_index(w, g, 2 * e), *g2 = grid + 4 * iq3s_index(w, g, 2 * e + 1);
                const uint8_t sb = w[74 + 4 * g + e];
                for (int j = 0; j < 4; ++j) {
                    sumi += (int)(uint8_t)g1[j] * xq[32 * g + 8 * e + j] * ((sb >> j) & 1 ? -1 : 1);
                    sumi += (int)(uint8_t)g2[j] * xq[32 * g + 8 * e + 4 + j] * ((sb >> (4 + j)) & 1 ? -1 : 1);
                }
            }
            bsum += sumi * ls;
        }
        sumf += d * bsum;
    }
    return sumf;
}

/* ggml/src/ggml-cpu/quants.c (ggml_vec_dot_iq1_s_q8_K_generic); examples/kernels/vec_dot/iq1_s_q8_k.py:51-56: the shift
 * term uses the activation record's stored sums of 16 */
float wo_vec_dot_iq1_s_q8_K(const uint8_t *w, const uint8_t *x, const int8_t *grid, int64_t k) {
    float sumf = 0.f;
    for (int64_t b = 0; b < k / 256; ++b, w += 50, x += 292) {
        const int8_t *xq = (const int8_t *)(x + 4);
        int sumi = 0, sumi1 = 0;
        for (int g = 0; g < 8; ++g) {
            const uint16_t qh = ld_u16(w + 34 + 2 * g);
            const int ls = 2 * ((qh >> 12) & 7) + 1, delta = qh & 0x8000 ? -1 : 1;
            int lsum = 0;
            for (int e = 0; e < 4; ++e) {
                const int8_t *gv = grid + 8 * (w[2 + 4 * g + e] | (((qh >> (3 * e)) & 7) << 8));
                for (int j = 0; j < 8; ++j) lsum += xq[32 * g + 8 * e + j] * gv[j];
            }
            sumi += ls * lsum;
            sumi1 += ls * delta * (ld_i16(x + 260 + 4 * g) + ld_i16(x + 260 + 4 * g + 2));
        }
        sumf += wo_f16_to_f32(ld_u16(w)) * ld_f32(x) * ((float)sumi + 0.125f * (float)sumi1);
    }
    return sumf;
}

/* ggml/src/ggml-cpu/quants.c (ggml_vec_dot_iq1_m_q8_K_generic); examples/kernels/vec_dot/iq1_m_q8_k.py:73-79: the shift term
 * uses sums of 8 codes, computed here */
float wo_vec_dot_iq1_m_q8_K(const uint8_t *w, const uint8_t *x, const int8_t *grid, int64_t k) {
    float sumf = 0.f;
    for (int64_t b = 0; b < k / 256; ++b, w += 56, x += 292) {
        const int8_t *xq = (const int8_t *)(x + 4);
        int sumi1 = 0, sumi2 = 0;
        for (int g = 0; g < 8; ++g) {
            int sum1[2] = {0, 0}, sum2[2] = {0, 0};
            for (int e = 0; e < 4; ++e) {
                const int8_t *gv = grid + 8 * iq1m_index(w, g, e);
                int lsum1 = 0, lsum2 = 0;
                for (int j = 0; j < 8; ++j) { lsum1 += xq[32 * g + 8 * e + j] * gv[j]; lsum2 += xq[32 * g + 8 * e + j]; }
                sum1[e >> 1] += lsum1;
                sum2[e >> 1] += lsum2 * (iq1m_negative(w, g, e) ? -1 : 1);
            }
            const int ls1 = 2 * iq1m_sub_scale(w, g, 0) + 1, ls2 = 2 * iq1m_sub_scale(w, g, 1) + 1;
            sumi1 += sum1[0] * ls1 + sum1[1] * ls2;
            sumi2 += sum2[0] * ls1 + sum2[1] * ls2;
        }
        sumf += iq1m_scale(w) * ld_f32(x) * ((float)sumi1 + 0.125f * (float)sumi2);
    }
    return sumf;
}

/* ggml/src/ggml-cpu/quants.c:430-480; examples/kernels/vec_dot/tq1_0_q8_k.py:9-55 */
float wo_vec_dot_tq1_0_q8_K(const uint8_t *w, const uint8_t *x, int64_t k) {
    float sumf = 0.0f;
    for (int64_t b = 0; b < k / 256; ++b, w += 54, x += 292) {
        const int8_t *xq = (const int8_t *)(x + 4);
        int sum = 0;
        for (int n = 0; n < 5; ++n)
            for (int m = 0; m < 32; ++m) sum += tq1_digit(w[m], n) * xq[32 * n + m];
        for (int n = 0; n < 5; ++n)
            for (int m = 0; m < 16; ++m) sum += tq1_digit(w[32 + m], n) * xq[160 + 16 * n + m];
        for (int n = 0; n < 4; ++n)
            for (int j = 0; j < 4; ++j) sum += tq1_digit(w[48 + j], n) * xq[240 + 4 * n + j];
        sumf += (float)sum * (wo_f16_to_f32(ld_u16(w + 52)) * ld_f32(x));
    }
    return sumf;
}

int wo_vec_dot(int fmt, const uint8_t *w, const uint8_t *x, const int8_t *grid, const int8_t *signs,
               int64_t k, float *out) {
    switch (fmt) {
    case WO_Q4_0: *out = wo_vec_dot_q4_0_q8_0(w, x, k); return 0;
    case WO_Q8_0: *out = wo_vec_dot_q8_0_q8_0(w, x, k); return 0;
    case WO_Q4_K: *out = wo_vec_dot_q4_K_q8_K(w, x, k); return 0;
    case WO_Q2_K: *out = wo_vec_dot_q2_K_q8_K(w, x, k); return 0;
    case WO_Q3_K: *out = wo_vec_dot_q3_K_q8_K(w, x, k); return 0;
    case WO_Q5_K: *out = wo_vec_dot_q5_K_q8_K(w, x, k); return 0;
    case WO_Q6_K: *out = wo_vec_dot_q6_K_q8_K(w, x, k); return 0;
    case WO_IQ2_XXS: *out = wo_vec_dot_iq2_xxs_q8_K(w, x, grid, signs, k); return 0;
    case WO_IQ2_XS: *out = wo_vec_dot_iq2_xs_q8_K(w, x, grid, signs, k); return 0;
    case WO_IQ3_XXS: *out = wo_vec_dot_iq3_xxs_q8_K(w, x, grid, signs, k); return 0;
    case WO_IQ2_S: *out = wo_vec_dot_iq2_s_q8_K(w, x, grid, k); return 0;
    case WO_IQ1_S: *out = wo_vec_dot_iq1_s_q8_K(w, x, grid, k); return 0;
    case WO_IQ1_M: *out = wo_vec_dot_iq1_m_q8_K(w, x, grid, k); return 0;
    case WO_IQ3_S: *out = wo_vec_dot_iq3_s_q8_K(w, x, grid, k); return 0;
    case WO_TQ1_0: *out = wo_vec_dot_tq1_0_q8_K(w, x, k); return 0;
    default: return -1;
    }
}

/* ------------------------------------------------------------------ mul_mat */

/* The CPU graph path of the reference: quantize each activation row, then the double loop
 * over vec_dot (ggml/src/ggml-cpu/ggml-cpu.c:1202-1242; examples/kernels/mul_mat/q4_k_decode.py:17-20). */
typedef struct {
    int fmt; const uint8_t *w, *xq; const int8_t *grid, *signs; float *y;
    int64_t n, k, m, n0; size_t wrow, xrow;
} wo_mm_ctx;

static void wo_mul_mat_range(int64_t begin, int64_t end, void *p) {
    const wo_mm_ctx *c = (const wo_mm_ctx *)p;
    for (int64_t col = c->n0 + begin; col < c->n0 + end; ++col)
        for (int64_t r = 0; r < c->m; ++r)
            wo_vec_dot(c->fmt, c->w + col * c->wrow, c->xq + r * c->xrow, c->grid, c->signs, c->k,
                       c->y + r * c->n + col);
}

int wo_mul_mat(int fmt, int rule, const uint8_t *w, const float *x, uint8_t *xq,
               const int8_t *grid, const int8_t *signs, float *y,
               int64_t n, int64_t k, int64_t m, int64_t n0, int64_t n1, int quantize_x) {
    const int act = (fmt == WO_Q4_0 || fmt == WO_Q8_0) ? WO_Q8_0 : WO_Q8_K;
    wo_mm_ctx c = {fmt, w, xq, grid, signs, y, n, k, m, n0, wo_row_bytes(fmt, k), wo_row_bytes(act, k)};
    if (!c.wrow || fmt == WO_Q8_K) return -1;
    if (quantize_x && wo_quantize_rows(act, rule, x, xq, m, k)) return -1;
    wo_parallel_for(n1 - n0, wo_mul_mat_range, &c);
    return 0;
}

/* ksigns_iq2xs in kernel-argument form (examples/repro/weft/vec_dot_runtime.cpp:101-134):
 * sign index i carries 7 explicit sign bits; the 8th makes the number of minus signs even. */
void wo_iq2_sign_table(int8_t *signs) {
    for (int i = 0; i < 128; ++i) {
        const int full = i | ((__builtin_popcount((unsigned)i) & 1) << 7);
        for (int j = 0; j < 8; ++j) signs[8 * i + j] = (full >> j) & 1 ? -1 : 1;
    }
}

/* ---- persistent interleaved layout (doc/dsl/encoding-and-artifacts.md:209) ---------------------------------- */

size_t wo_interleave_packed_size(size_t record_bytes, int64_t rows, int64_t blocks) {
    return (size_t)rows * (size_t)blocks * record_bytes;
}

static int wo_interleave_move(const uint8_t *source, uint8_t *target, size_t record_bytes, int64_t R, int64_t rows,
                              int64_t blocks, int pack) {
    if (R <= 0 || rows < 0 || blocks < 0 || rows % R != 0) return -1;
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t k = 0; k < blocks; ++k) {
            const size_t plain = ((size_t)r * (size_t)blocks + (size_t)k) * record_bytes;
            const size_t cohort = (((size_t)(r / R) * (size_t)blocks + (size_t)k) * (size_t)R) * record_bytes + (size_t)(r % R);
            for (size_t b = 0; b < record_bytes; ++b) {
                if (pack) target[cohort + b * (size_t)R] = source[plain + b];
                else target[plain + b] = source[cohort + b * (size_t)R];
            }
        }
    return 0;
}

int wo_interleave_pack(const uint8_t *source, uint8_t *target, size_t record_bytes, int64_t R, int64_t rows, int64_t blocks) {
    return wo_interleave_move(source, target, record_bytes, R, rows, blocks, 1);
}

int wo_interleave_unpack(const uint8_t *source, uint8_t *target, size_t record_bytes, int64_t R, int64_t rows, int64_t blocks) {
    return wo_interleave_move(source, target, record_bytes, R, rows, blocks, 0);
}
