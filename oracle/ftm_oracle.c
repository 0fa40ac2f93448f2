/*
 * TEST INFRASTRUCTURE ONLY -- see ftm_oracle.h.  CPU restatement of the
 * reference's host NVFP4 MoE path, compiled with
 *   gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC
 * (no -ffast-math: every f32 operation must round exactly once, in the order
 * written, as the reference's Rust does).
 */
#include "ftm_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "../include/ftm_exact_math.h"

#ifdef _OPENMP
#include <omp.h>
#endif

/* ---- the steps either side of the block ------------------------------------------------------- */

/* src/models/qwen3_6/forward.rs:48-61 */
void ftmo_rms_norm(const float* x, const float* w, float eps, size_t rows, size_t row_len, float* out) {
    float inv_rowlen = 1.0f / (float)row_len;
    for (size_t r = 0; r < rows; r++) {
        const float* row = x + r * row_len;
        float sum = 0.0f;
        for (size_t j = 0; j < row_len; j++) sum = sum + row[j] * row[j];
        float mean = sum * inv_rowlen;
        float inv = 1.0f / sqrtf(mean + eps);
        for (size_t j = 0; j < row_len; j++) out[r * row_len + j] = row[j] * inv * w[j];
    }
}

/* python/ferrum_kernel/norm.py:35-110: the bf16 stream's rounding points, the tower's reduction order */
void ftmo_add_rmsnorm(const uint16_t* x, const uint16_t* r, const uint16_t* w, float eps, size_t rows,
                      size_t hidden, uint16_t* sum_out, uint16_t* out) {
    float inv_rowlen = 1.0f / (float)hidden;
    for (size_t t = 0; t < rows; t++) {
        float sum = 0.0f;
        for (size_t j = 0; j < hidden; j++) {
            float s = ftmo_bf16_to_f32(x[t * hidden + j]) + ftmo_bf16_to_f32(r[t * hidden + j]);
            uint16_t sb = ftmo_f32_to_bf16(s);
            sum_out[t * hidden + j] = sb;
            float sf = ftmo_bf16_to_f32(sb);
            sum = sum + sf * sf;
        }
        float var = sum * inv_rowlen;
        float recip = 1.0f / sqrtf(var + eps);
        for (size_t j = 0; j < hidden; j++) {
            float sf = ftmo_bf16_to_f32(sum_out[t * hidden + j]);
            out[t * hidden + j] = ftmo_f32_to_bf16((sf * recip) * ftmo_bf16_to_f32(w[j]));
        }
    }
}

/* python/ferrum_kernel/linear.py:152-168 on the K-major bank of src/infrastructure/cuda_linear.rs:103-111 */
void ftmo_nvfp4_dense_gemv(const float* a, const uint32_t* packed_kmajor, const uint8_t* scale_kmajor,
                           const uint16_t* global, size_t m, size_t n, size_t k, float* c, int threads) {
    if (threads < 1) threads = 1;
#pragma omp parallel for num_threads(threads) schedule(static)
    for (long long row = 0; row < (long long)n; row++) {
        float g = ftmo_f16_to_f32(global[row]);
        /* w[row, kk] = (lut[code] * scale) * global, as the oracle widens it before the matmul */
        float* wrow = (float*)malloc(sizeof(float) * k);
        for (size_t kk = 0; kk < k; kk++) {
            uint32_t word = packed_kmajor[(kk / 8) * n + (size_t)row];
            uint8_t code = (uint8_t)((word >> (4 * (kk % 8))) & 0xF);
            float v = ftmo_fp4_nibble(code, 0);
            float sc = ftmo_e4m3fn_to_f32(scale_kmajor[(kk / 16) * n + (size_t)row]);
            wrow[kk] = (v * sc) * g;
        }
        for (size_t t = 0; t < m; t++) {
            float acc = 0.0f;
            for (size_t kk = 0; kk < k; kk++) acc = acc + a[t * k + kk] * wrow[kk];
            c[t * n + (size_t)row] = acc;
        }
        free(wrow);
    }
}

int ftmo_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------ decoders */

/* src/domain/numerics.rs:6-8 */
float ftmo_bf16_to_f32(uint16_t bits) { return ftm_bf16_bits_to_f32(bits); }

uint16_t ftmo_f32_to_bf16(float v) { return ftm_f32_to_bf16_bits(v); }

float ftmo_expf(float x) { return ftm_expf(x); }

/* src/domain/numerics.rs:13-29.  The reference's subnormal branch returns
 * man * 2^-24 without the sign; that behaviour is kept. */
float ftmo_f16_to_f32(uint16_t bits) {
    uint32_t sign = ((uint32_t)(bits & 0x8000u)) << 16;
    uint32_t exp = (bits >> 10) & 0x1fu;
    uint32_t man = bits & 0x3ffu;
    if (exp == 0) {
        if (man == 0) return ftm_bits_to_f32(sign);
        return (float)man * 0x1p-24f;
    }
    if (exp == 0x1f) return ftm_bits_to_f32(sign | 0x7f800000u | (man << 13));
    return ftm_bits_to_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

/* src/domain/numerics.rs:34-52 */
float ftmo_e4m3fn_to_f32(uint8_t bits) {
    float sign = (bits & 0x80u) ? -1.0f : 1.0f;
    int exp = (bits >> 3) & 0x0f;
    int man = bits & 0x07;
    float mag;
    if (exp == 0) {
        mag = (float)man * 0x1p-9f;
    } else if (exp == 0x0f) {
        if (man == 0x07) return NAN;
        mag = (1.0f + (float)man / 8.0f) * 256.0f;
    } else {
        mag = (1.0f + (float)man / 8.0f) * ldexpf(1.0f, exp - 7);
    }
    return sign * mag;
}

/* src/domain/numerics.rs:58-68 */
static const float FP4_VALUES[16] = {0.0f,  0.5f,  1.0f,  1.5f,  2.0f,  3.0f,  4.0f,  6.0f,
                                     -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

float ftmo_fp4_nibble(uint8_t byte, int high) {
    return FP4_VALUES[high ? (byte >> 4) : (byte & 0x0f)];
}

/* src/domain/dequant.rs:74-85 */
void ftmo_nvfp4_block(const uint8_t* packed, size_t rows, size_t cols, const uint8_t* scale,
                      float* out) {
    for (size_t r = 0; r < rows; r++) {
        size_t pbase = r * (cols / 2), sbase = r * (cols / 16);
        for (size_t k = 0; k < cols; k++)
            out[r * cols + k] = ftmo_fp4_nibble(packed[pbase + k / 2], (k % 2) == 1) *
                                ftmo_e4m3fn_to_f32(scale[sbase + k / 16]);
    }
}

/* ------------------------------------------------------------- routed half */

/* src/domain/expert_kernel.rs:591-618: one accumulator per row, blocks in
 * order, sixteen k per block, x * fp4 * scale evaluated left to right, the f16
 * row global applied once after the K loop. */
void ftmo_gemv_rows(const float* x, const uint8_t* packed, const uint8_t* scale,
                    const uint8_t* global, size_t global_len, size_t rows, size_t cols, float* y) {
    size_t cols2 = cols / 2, cols16 = cols / 16;
    for (size_t r = 0; r < rows; r++) {
        float g = 1.0f;
        if (global_len >= 2 * rows)
            g = ftmo_f16_to_f32((uint16_t)(global[2 * r] | ((uint16_t)global[2 * r + 1] << 8)));
        float acc = 0.0f;
        for (size_t b = 0; b < cols16; b++) {
            float s = ftmo_e4m3fn_to_f32(scale[r * cols16 + b]);
            for (size_t j = 0; j < 16; j++) {
                size_t k = b * 16 + j;
                float term = x[k] * ftmo_fp4_nibble(packed[r * cols2 + k / 2], (k % 2) == 1);
                term = term * s;
                acc = acc + term;
            }
        }
        y[r] = acc * g;
    }
}

/* src/models/qwen3_6/forward.rs:184-218 */
void ftmo_tower_nvfp4_gemv(const float* x, const uint8_t* packed, const uint8_t* scale,
                           const uint8_t* global, size_t global_len, size_t rows, size_t cols,
                           float* y) {
    size_t cols2 = cols / 2, cols16 = cols / 16;
    for (size_t r = 0; r < rows; r++) {
        float g = 1.0f;
        if (global_len >= 2 * rows)
            g = ftmo_f16_to_f32((uint16_t)(global[2 * r] | ((uint16_t)global[2 * r + 1] << 8)));
        float acc = 0.0f;
        for (size_t b = 0; b < cols16; b++) {
            float s = ftmo_e4m3fn_to_f32(scale[r * cols16 + b]) * g;
            if (s == 0.0f) continue;
            for (size_t j = 0; j < 16; j++) {
                size_t k = b * 16 + j;
                float v = ftmo_fp4_nibble(packed[r * cols2 + k / 2], (k % 2) == 1) * s;
                if (v != 0.0f) acc = acc + x[k] * v;
            }
        }
        y[r] = acc;
    }
}

static int banks_ok(const ftmo_banks* b, size_t h, size_t i) {
    if (b->gu_rows != 2 * i || b->gu_cols != h || b->dn_rows != h || b->dn_cols != i) return 0;
    if (h == 0 || i == 0 || (h % 16) != 0 || (i % 16) != 0) return 0;
    size_t s = b->slots;
    if (b->gu_packed_len != s * (b->gu_rows * h / 2)) return 0;
    if (b->gu_scale_len != s * (b->gu_rows * h / 16)) return 0;
    if (b->gu_global_len != s * (b->gu_rows * 2)) return 0;
    if (b->dn_packed_len != s * (h * i / 2)) return 0;
    if (b->dn_scale_len != s * (h * i / 16)) return 0;
    if (b->dn_global_len != s * (h * 2)) return 0;
    return 1;
}

/* one (token, route) pair: gate_up gemv, silu(gate) * up, down gemv
 * (src/domain/expert_kernel.rs:547-577) */
static void one_route(const ftmo_banks* b, size_t h, size_t i, const float* xrow, size_t slot,
                      float* ic1, float* ic2, float* ic3) {
    size_t gu_pb = b->gu_rows * h / 2, gu_sb = b->gu_rows * h / 16, gu_gb = b->gu_rows * 2;
    size_t dn_pb = h * i / 2, dn_sb = h * i / 16, dn_gb = h * 2;
    ftmo_gemv_rows(xrow, b->gu_packed + slot * gu_pb, b->gu_scale + slot * gu_sb,
                   b->gu_global + slot * gu_gb, gu_gb, 2 * i, h, ic1);
    for (size_t k = 0; k < i; k++) {
        float g = ic1[k] / (1.0f + expf(-ic1[k]));
        ic2[k] = g * ic1[i + k];
    }
    ftmo_gemv_rows(ic2, b->dn_packed + slot * dn_pb, b->dn_scale + slot * dn_sb,
                   b->dn_global + slot * dn_gb, dn_gb, h, i, ic3);
}

/* src/domain/expert_kernel.rs:465-587 */
int ftmo_grouped_moe_reference(const ftmo_banks* banks, size_t hidden, size_t inter,
                               const float* x, size_t x_len, size_t top_k, const int32_t* routes,
                               size_t routes_len, const float* weights, size_t weights_len,
                               float* out, size_t out_len, float* abs_sum, size_t abs_len,
                               size_t* bad_slot) {
    size_t h = hidden, i = inter;
    if (!banks_ok(banks, h, i)) return FTMO_BAD;
    size_t tokens = x_len / h;
    size_t nroutes = tokens * top_k;
    if (x_len != tokens * h || routes_len < nroutes || weights_len < nroutes ||
        out_len < tokens * h)
        return FTMO_BAD;
    memset(out, 0, tokens * h * sizeof(float));
    if (abs_sum) {
        if (abs_len < tokens * h) return FTMO_BAD;
        memset(abs_sum, 0, tokens * h * sizeof(float));
    }
    float* ic1 = (float*)malloc(sizeof(float) * 2 * i);
    float* ic2 = (float*)malloc(sizeof(float) * i);
    float* ic3 = (float*)malloc(sizeof(float) * h);
    int rc = FTMO_OK;
    for (size_t t = 0; t < tokens && rc == FTMO_OK; t++) {
        const float* xrow = x + t * h;
        for (size_t j = 0; j < top_k; j++) {
            int32_t slot = routes[t * top_k + j];
            if (slot < 0) continue;
            if ((size_t)slot >= banks->slots) {
                if (bad_slot) *bad_slot = (size_t)slot;
                rc = FTMO_SLOT_OUT_OF_RANGE;
                break;
            }
            float w = weights[t * top_k + j];
            one_route(banks, h, i, xrow, (size_t)slot, ic1, ic2, ic3);
            for (size_t d = 0; d < h; d++) {
                float term = w * ic3[d];
                out[t * h + d] = out[t * h + d] + term;
                if (abs_sum) abs_sum[t * h + d] = abs_sum[t * h + d] + fabsf(term);
            }
        }
    }
    free(ic1);
    free(ic2);
    free(ic3);
    return rc;
}

int ftmo_grouped_moe_reference_mt(const ftmo_banks* banks, size_t hidden, size_t inter,
                                  const float* x, size_t tokens, size_t top_k,
                                  const int32_t* routes, const float* weights, float* out,
                                  int threads) {
    size_t h = hidden, i = inter;
    if (!banks_ok(banks, h, i)) return FTMO_BAD;
    size_t nroutes = tokens * top_k;
    for (size_t r = 0; r < nroutes; r++)
        if (routes[r] >= 0 && (size_t)routes[r] >= banks->slots) return FTMO_SLOT_OUT_OF_RANGE;
    float* ic3_all = (float*)malloc(sizeof(float) * nroutes * h);
    if (!ic3_all) return FTMO_BAD;
    if (threads < 1) threads = 1;
#pragma omp parallel num_threads(threads)
    {
        float* ic1 = (float*)malloc(sizeof(float) * 2 * i);
        float* ic2 = (float*)malloc(sizeof(float) * i);
#pragma omp for schedule(dynamic, 1)
        for (long r = 0; r < (long)nroutes; r++) {
            int32_t slot = routes[r];
            if (slot < 0) continue;
            one_route(banks, h, i, x + ((size_t)r / top_k) * h, (size_t)slot, ic1, ic2,
                      ic3_all + (size_t)r * h);
        }
        free(ic1);
        free(ic2);
#pragma omp for schedule(static)
        for (long t = 0; t < (long)tokens; t++) {
            float* o = out + (size_t)t * h;
            memset(o, 0, h * sizeof(float));
            for (size_t j = 0; j < top_k; j++) {
                size_t r = (size_t)t * top_k + j;
                if (routes[r] < 0) continue;
                float w = weights[r];
                const float* ic3 = ic3_all + r * h;
                for (size_t d = 0; d < h; d++) o[d] = o[d] + w * ic3[d];
            }
        }
    }
    free(ic3_all);
    return FTMO_OK;
}

/* src/domain/expert_kernel.rs:223-243 */
int ftmo_route_lists(const int32_t* routes, size_t routes_len, size_t tokens, size_t top_k,
                     int32_t* route_token, int32_t* route_slot) {
    if (tokens == 0 || top_k == 0 || routes_len != tokens * top_k) return FTMO_BAD;
    for (size_t t = 0; t < tokens; t++)
        for (size_t j = 0; j < top_k; j++) {
            route_token[t * top_k + j] = (int32_t)t;
            route_slot[t * top_k + j] = routes[t * top_k + j];
        }
    return FTMO_OK;
}

/* src/infrastructure/cuda_moe.rs:2328-2362 */
int ftmo_build_grouped_csr(const int32_t* route_slot, size_t routes, size_t slots, int32_t* seg,
                           int32_t* route_idx, int* why) {
    int32_t* counts = (int32_t*)calloc(slots ? slots : 1, sizeof(int32_t));
    for (size_t r = 0; r < routes; r++) {
        int32_t s = route_slot[r];
        if (s < 0) {
            if (why) *why = 1;
            free(counts);
            return FTMO_BAD;
        }
        if ((size_t)s >= slots) {
            if (why) *why = 2;
            free(counts);
            return FTMO_BAD;
        }
        counts[s]++;
    }
    seg[0] = 0;
    for (size_t s = 0; s < slots; s++) seg[s + 1] = seg[s] + counts[s];
    for (size_t s = 0; s < slots; s++) counts[s] = seg[s]; /* cursors */
    for (size_t r = 0; r < routes; r++) route_idx[counts[route_slot[r]]++] = (int32_t)r;
    free(counts);
    return FTMO_OK;
}

/* ------------------------------------------------ router and shared expert */

/* src/models/qwen3_6/forward.rs:162-179 */
void ftmo_bf16_gemm(const float* x, const uint16_t* w, size_t t, size_t rows, size_t cols,
                    float* y) {
    for (size_t tt = 0; tt < t; tt++) {
        const float* xr = x + tt * cols;
        for (size_t r = 0; r < rows; r++) {
            const uint16_t* wr = w + r * cols;
            float acc = 0.0f;
            for (size_t k = 0; k < cols; k++) acc = acc + xr[k] * ftm_bf16_bits_to_f32(wr[k]);
            y[tt * rows + r] = acc;
        }
    }
}

static void bf16_gemm_mt(const float* x, const uint16_t* w, size_t t, size_t rows, size_t cols,
                         float* y, int threads) {
#pragma omp parallel for schedule(static) num_threads(threads)
    for (long idx = 0; idx < (long)(t * rows); idx++) {
        size_t tt = (size_t)idx / rows, r = (size_t)idx % rows;
        const float* xr = x + tt * cols;
        const uint16_t* wr = w + r * cols;
        float acc = 0.0f;
        for (size_t k = 0; k < cols; k++) acc = acc + xr[k] * ftm_bf16_bits_to_f32(wr[k]);
        y[idx] = acc;
    }
}

/* src/models/qwen3_6/forward.rs:793-806 */
void ftmo_softmax_rows(float* logits, size_t n, size_t e) {
    for (size_t r = 0; r < n; r++) {
        float* row = logits + r * e;
        float max = -INFINITY;
        for (size_t c = 0; c < e; c++) max = row[c] > max ? row[c] : max;
        float sum = 0.0f;
        for (size_t c = 0; c < e; c++) {
            row[c] = ftm_expf(row[c] - max);
            sum = sum + row[c];
        }
        float inv = 1.0f / sum;
        for (size_t c = 0; c < e; c++) row[c] = row[c] * inv;
    }
}

/* src/models/qwen3_6/forward.rs:808-830: descending top-k, weights divided by
 * the top-k sum through its reciprocal.  The reference sorts with an unstable
 * sort whose order among equal probabilities is unspecified; the rule the
 * device kernel and the gating test state is "lowest index first"
 * (python/ferrum_kernel/elementwise.py:372-373, tests/cudarc_forward.rs:89-97),
 * implemented here as k passes of a strict-greater argmax. */
void ftmo_topk_renorm(const float* p, size_t n, size_t e, size_t k, int32_t* ids, float* w) {
    unsigned char* used = (unsigned char*)malloc(e);
    for (size_t r = 0; r < n; r++) {
        memset(used, 0, e);
        float sum = 0.0f;
        for (size_t j = 0; j < k; j++) {
            size_t best = e;
            for (size_t c = 0; c < e; c++) {
                if (used[c]) continue;
                if (best == e || p[r * e + c] > p[r * e + best]) best = c;
            }
            used[best] = 1;
            ids[r * k + j] = (int32_t)best;
            w[r * k + j] = p[r * e + best];
            sum = sum + p[r * e + best];
        }
        float inv = 1.0f / sum;
        for (size_t j = 0; j < k; j++) w[r * k + j] = w[r * k + j] * inv;
    }
    free(used);
}

float ftmo_silu(float x) { return x / (1.0f + expf(-x)); }
float ftmo_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }

void ftmo_router(const ftmo_layer* L, const float* x, size_t t, int32_t* ids, float* w,
                 float* probs_or_null) {
    float* probs = probs_or_null ? probs_or_null : (float*)malloc(sizeof(float) * t * L->experts);
    bf16_gemm_mt(x, L->gate_w, t, L->experts, L->hidden, probs, ftmo_max_threads());
    ftmo_softmax_rows(probs, t, L->experts);
    ftmo_topk_renorm(probs, t, L->experts, L->top_k, ids, w);
    if (!probs_or_null) free(probs);
}

static void shared_expert_mt(const ftmo_layer* L, const float* x, size_t t, float* out,
                             int threads) {
    size_t si = L->shared_inter, h = L->hidden;
    float* ic1 = (float*)malloc(sizeof(float) * t * 2 * si);
    float* ic2 = (float*)malloc(sizeof(float) * t * si);
    bf16_gemm_mt(x, L->sh_gate_up, t, 2 * si, h, ic1, threads);
    for (size_t tt = 0; tt < t; tt++)
        for (size_t k = 0; k < si; k++)
            ic2[tt * si + k] = ftmo_silu(ic1[tt * 2 * si + k]) * ic1[tt * 2 * si + si + k];
    bf16_gemm_mt(ic2, L->sh_down, t, h, si, out, threads);
    free(ic1);
    free(ic2);
}

/* src/models/qwen3_6/forward.rs:684-714, weights in bf16 (:162-179) */
void ftmo_shared_expert(const ftmo_layer* L, const float* x, size_t t, float* out) {
    shared_expert_mt(L, x, t, out, 1);
}

/* src/models/qwen3_6/forward.rs:716-791 */
static int moe_block_impl(const ftmo_layer* L, const float* x, size_t t, float* out,
                          int32_t* ids_out, float* w_out, int threads, int dequant_once) {
    size_t h = L->hidden, i = L->inter, k = L->top_k, e = L->experts;
    if (!banks_ok(&L->banks, h, i) || L->banks.slots < e) return FTMO_BAD;
    int32_t* ids = (int32_t*)malloc(sizeof(int32_t) * t * k);
    float* w = (float*)malloc(sizeof(float) * t * k);
    float* probs = (float*)malloc(sizeof(float) * t * e);
    bf16_gemm_mt(x, L->gate_w, t, e, h, probs, threads);
    ftmo_softmax_rows(probs, t, e);
    ftmo_topk_renorm(probs, t, e, k, ids, w);
    free(probs);

    float* gate_out = (float*)malloc(sizeof(float) * t);
    bf16_gemm_mt(x, L->sh_gate, t, 1, h, gate_out, threads);
    float* se = (float*)malloc(sizeof(float) * t * h);
    shared_expert_mt(L, x, t, se, threads);
    for (size_t tt = 0; tt < t; tt++) {
        float sg = ftmo_sigmoid(gate_out[tt]);
        for (size_t d = 0; d < h; d++) out[tt * h + d] = se[tt * h + d] * sg;
    }
    free(se);
    free(gate_out);

    size_t nroutes = t * k;
    float* ic3_all = (float*)malloc(sizeof(float) * nroutes * h);
    if (!dequant_once) {
#pragma omp parallel num_threads(threads)
        {
            float* ic1 = (float*)malloc(sizeof(float) * 2 * i);
            float* ic2 = (float*)malloc(sizeof(float) * i);
#pragma omp for schedule(dynamic, 1)
            for (long r = 0; r < (long)nroutes; r++)
                one_route(&L->banks, h, i, x + ((size_t)r / k) * h, (size_t)ids[r], ic1, ic2,
                          ic3_all + (size_t)r * h);
            free(ic1);
            free(ic2);
        }
    } else {
        /* per expert: widen both slabs once (block scale folded in, row global
         * kept separate and applied after the dot), then a dense dot per token */
        int32_t* seg = (int32_t*)malloc(sizeof(int32_t) * (e + 1));
        int32_t* ridx = (int32_t*)malloc(sizeof(int32_t) * nroutes);
        int why = 0;
        if (ftmo_build_grouped_csr(ids, nroutes, e, seg, ridx, &why) != FTMO_OK) return FTMO_BAD;
        const ftmo_banks* b = &L->banks;
        size_t gu_pb = b->gu_rows * h / 2, gu_sb = b->gu_rows * h / 16, gu_gb = b->gu_rows * 2;
        size_t dn_pb = h * i / 2, dn_sb = h * i / 16, dn_gb = h * 2;
#pragma omp parallel num_threads(threads)
        {
            float* wgu = (float*)malloc(sizeof(float) * 2 * i * h);
            float* wdn = (float*)malloc(sizeof(float) * h * i);
            float* ic1 = (float*)malloc(sizeof(float) * 2 * i);
            float* ic2 = (float*)malloc(sizeof(float) * i);
#pragma omp for schedule(dynamic, 1)
            for (long ex = 0; ex < (long)e; ex++) {
                if (seg[ex + 1] == seg[ex]) continue;
                ftmo_nvfp4_block(b->gu_packed + ex * gu_pb, 2 * i, h, b->gu_scale + ex * gu_sb, wgu);
                ftmo_nvfp4_block(b->dn_packed + ex * dn_pb, h, i, b->dn_scale + ex * dn_sb, wdn);
                const uint8_t* gug = b->gu_global + ex * gu_gb;
                const uint8_t* dng = b->dn_global + ex * dn_gb;
                for (int32_t q = seg[ex]; q < seg[ex + 1]; q++) {
                    size_t r = (size_t)ridx[q];
                    const float* xr = x + (r / k) * h;
                    for (size_t n = 0; n < 2 * i; n++) {
                        float acc = 0.0f;
                        const float* wr = wgu + n * h;
                        for (size_t kk = 0; kk < h; kk++) acc = acc + xr[kk] * wr[kk];
                        ic1[n] = acc * ftmo_f16_to_f32((uint16_t)(gug[2 * n] | (gug[2 * n + 1] << 8)));
                    }
                    for (size_t n = 0; n < i; n++) ic2[n] = ftmo_silu(ic1[n]) * ic1[i + n];
                    float* ic3 = ic3_all + r * h;
                    for (size_t n = 0; n < h; n++) {
                        float acc = 0.0f;
                        const float* wr = wdn + n * i;
                        for (size_t kk = 0; kk < i; kk++) acc = acc + ic2[kk] * wr[kk];
                        ic3[n] = acc * ftmo_f16_to_f32((uint16_t)(dng[2 * n] | (dng[2 * n + 1] << 8)));
                    }
                }
            }
            free(wgu);
            free(wdn);
            free(ic1);
            free(ic2);
        }
        free(seg);
        free(ridx);
    }
#pragma omp parallel for schedule(static) num_threads(threads)
    for (long tt = 0; tt < (long)t; tt++) {
        float* o = out + (size_t)tt * h;
        for (size_t j = 0; j < k; j++) {
            size_t r = (size_t)tt * k + j;
            float wj = w[r];
            const float* ic3 = ic3_all + r * h;
            for (size_t d = 0; d < h; d++) o[d] = o[d] + wj * ic3[d];
        }
    }
    free(ic3_all);
    if (ids_out) memcpy(ids_out, ids, sizeof(int32_t) * t * k);
    if (w_out) memcpy(w_out, w, sizeof(float) * t * k);
    free(ids);
    free(w);
    return FTMO_OK;
}

int ftmo_moe_block(const ftmo_layer* L, const float* x, size_t t, float* out, int32_t* ids_out,
                   float* w_out) {
    return moe_block_impl(L, x, t, out, ids_out, w_out, 1, 0);
}

int ftmo_moe_block_mt(const ftmo_layer* L, const float* x, size_t t, float* out, int32_t* ids_out,
                      float* w_out, int threads) {
    return moe_block_impl(L, x, t, out, ids_out, w_out, threads < 1 ? 1 : threads, 0);
}

int ftmo_moe_block_dequant_once_mt(const ftmo_layer* L, const float* x, size_t t, float* out,
                                   int threads) {
    return moe_block_impl(L, x, t, out, NULL, NULL, threads < 1 ? 1 : threads, 1);
}

/* ------------------------------------------------------- expert-slot LRU */

/* src/domain/expert_cache.rs:8-16 */
struct ftmo_cache {
    size_t layers, experts, cache_size;
    int32_t* slot_for_id;
    int32_t* id_of_slot;
    uint64_t* usage;
    uint64_t step;
};

ftmo_cache* ftmo_cache_new(size_t layers, size_t experts, size_t cache_size) {
    if (layers * experts == 0 || cache_size == 0) return NULL;
    ftmo_cache* c = (ftmo_cache*)calloc(1, sizeof(*c));
    c->layers = layers;
    c->experts = experts;
    c->cache_size = cache_size;
    c->slot_for_id = (int32_t*)malloc(sizeof(int32_t) * layers * experts);
    c->id_of_slot = (int32_t*)malloc(sizeof(int32_t) * cache_size);
    c->usage = (uint64_t*)calloc(cache_size, sizeof(uint64_t));
    for (size_t n = 0; n < layers * experts; n++) c->slot_for_id[n] = -1;
    for (size_t n = 0; n < cache_size; n++) c->id_of_slot[n] = -1;
    return c;
}

void ftmo_cache_free(ftmo_cache* c) {
    if (!c) return;
    free(c->slot_for_id);
    free(c->id_of_slot);
    free(c->usage);
    free(c);
}

int32_t ftmo_cache_slot_of(const ftmo_cache* c, size_t layer, uint32_t expert) {
    return c->slot_for_id[layer * c->experts + expert];
}

int32_t ftmo_cache_id_of_slot(const ftmo_cache* c, size_t slot) { return c->id_of_slot[slot]; }

/* src/domain/expert_cache.rs:122-134: least recently used slot, lower slot on a tie */
static size_t cache_victim(const ftmo_cache* c) {
    size_t victim = 0;
    for (size_t s = 1; s < c->cache_size; s++)
        if (c->usage[s] < c->usage[victim]) victim = s;
    return victim;
}

static int cmp_u32(const void* a, const void* b) {
    uint32_t x = *(const uint32_t*)a, y = *(const uint32_t*)b;
    return (x > y) - (x < y);
}

/* src/domain/expert_cache.rs:66-120 */
size_t ftmo_cache_ensure(ftmo_cache* c, size_t layer, const uint32_t* routed, size_t n,
                         uint32_t* misses, uint32_t* write_slots, int32_t* rewrites) {
    size_t id_base = layer * c->experts;
    uint32_t* seen = (uint32_t*)malloc(sizeof(uint32_t) * (n ? n : 1));
    size_t nseen = 0;
    for (size_t q = 0; q < n; q++) {
        int dup = 0;
        for (size_t s = 0; s < nseen; s++)
            if (seen[s] == routed[q]) dup = 1;
        if (!dup) seen[nseen++] = routed[q];
    }
    c->step += 1;
    uint64_t step = c->step;
    for (size_t s = 0; s < nseen; s++) {
        int32_t slot = c->slot_for_id[id_base + seen[s]];
        if (slot >= 0) c->usage[slot] = step;
    }
    size_t nmiss = 0;
    for (size_t s = 0; s < nseen; s++)
        if (c->slot_for_id[id_base + seen[s]] == -1) misses[nmiss++] = seen[s];
    qsort(misses, nmiss, sizeof(uint32_t), cmp_u32);
    for (size_t m = 0; m < nmiss; m++) {
        size_t victim = cache_victim(c);
        int32_t old = c->id_of_slot[victim];
        if (old >= 0) c->slot_for_id[old] = -1;
        c->id_of_slot[victim] = (int32_t)(id_base + misses[m]);
        c->slot_for_id[id_base + misses[m]] = (int32_t)victim;
        c->usage[victim] = step;
        write_slots[m] = (uint32_t)victim;
    }
    for (size_t q = 0; q < n; q++) rewrites[q] = c->slot_for_id[id_base + routed[q]];
    free(seen);
    return nmiss;
}
