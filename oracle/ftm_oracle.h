/*
 * TEST INFRASTRUCTURE ONLY.  CPU restatement of the reference's host
 * (dequantise-and-matmul) NVFP4 mixture-of-experts path.  Nothing in the
 * product library may include, link or call this; only the test-suite, the
 * smoke check and the benchmark's CPU-baseline leg do.
 *
 * Each function names the reference source it follows (path:line inside the
 * reference project).  Loop orders are kept, so f32 sums round the same way.
 *
 * Parity pin: the known-answer cases of the reference's own unit tests
 * (src/domain/expert_kernel.rs:744-1258, src/domain/numerics.rs:75-136,
 * src/domain/expert_cache.rs:141-283, src/models/qwen3_6/forward.rs:1219-1236,
 * src/infrastructure/cuda_moe.rs:2718-2720) and outputs of the reference's
 * importable torch oracle (python/ferrum_kernel/selftest.py:48-115) stored as
 * fixtures; see tests/test_oracle_*.py.
 */
#ifndef FTM_ORACLE_H
#define FTM_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes mirror MoEError (src/domain/expert_kernel.rs:21-39) */
#define FTMO_OK 0
#define FTMO_BAD 1
#define FTMO_SLOT_OUT_OF_RANGE 2

/* ---- decoders: src/domain/numerics.rs:6-68 ---- */
float ftmo_bf16_to_f32(uint16_t bits);
float ftmo_f16_to_f32(uint16_t bits);
float ftmo_e4m3fn_to_f32(uint8_t bits);
float ftmo_fp4_nibble(uint8_t byte, int high);
uint16_t ftmo_f32_to_bf16(float v);
float ftmo_expf(float x); /* the shared reproducible exponential */

/* ---- dequant: src/domain/dequant.rs:74-97 ---- */
void ftmo_nvfp4_block(const uint8_t* packed, size_t rows, size_t cols, const uint8_t* scale,
                      float* out);

/* slot-major banks, src/domain/expert_kernel.rs:429-441 */
typedef struct ftmo_banks {
    const uint8_t* gu_packed;
    const uint8_t* gu_scale;
    const uint8_t* gu_global;
    const uint8_t* dn_packed;
    const uint8_t* dn_scale;
    const uint8_t* dn_global;
    size_t gu_packed_len, gu_scale_len, gu_global_len;
    size_t dn_packed_len, dn_scale_len, dn_global_len;
    size_t slots, gu_rows, gu_cols, dn_rows, dn_cols;
} ftmo_banks;

/* src/domain/expert_kernel.rs:591-618 */
void ftmo_gemv_rows(const float* x, const uint8_t* packed, const uint8_t* scale,
                    const uint8_t* global, size_t global_len, size_t rows, size_t cols, float* y);

/* the scalar tower's variant, global folded into the block scale and zero
 * terms skipped: src/models/qwen3_6/forward.rs:184-218 */
void ftmo_tower_nvfp4_gemv(const float* x, const uint8_t* packed, const uint8_t* scale,
                           const uint8_t* global, size_t global_len, size_t rows, size_t cols,
                           float* y);

/* src/domain/expert_kernel.rs:445-587; abs_sum may be NULL.  On
 * FTMO_SLOT_OUT_OF_RANGE, *bad_slot receives the offending slot. */
int ftmo_grouped_moe_reference(const ftmo_banks* banks, size_t hidden, size_t inter,
                               const float* x, size_t x_len, size_t top_k, const int32_t* routes,
                               size_t routes_len, const float* weights, size_t weights_len,
                               float* out, size_t out_len, float* abs_sum, size_t abs_len,
                               size_t* bad_slot);

/* same arithmetic, (token, route) pairs spread over OpenMP threads; the sum
 * over a token's routes is still taken in route order */
int ftmo_grouped_moe_reference_mt(const ftmo_banks* banks, size_t hidden, size_t inter,
                                  const float* x, size_t tokens, size_t top_k,
                                  const int32_t* routes, const float* weights, float* out,
                                  int threads);

/* src/domain/expert_kernel.rs:223-243 */
int ftmo_route_lists(const int32_t* routes, size_t routes_len, size_t tokens, size_t top_k,
                     int32_t* route_token, int32_t* route_slot);

/* src/infrastructure/cuda_moe.rs:2328-2362; returns FTMO_BAD with *why = 1 for
 * a non-resident route, 2 for a slot past the bank */
int ftmo_build_grouped_csr(const int32_t* route_slot, size_t routes, size_t slots, int32_t* seg,
                           int32_t* route_idx, int* why);

/* ---- router and shared expert: src/models/qwen3_6/forward.rs ---- */
/* :162-179  y[t,r] = sum_k x[t,k] * bf16(w[r,k]) left to right */
void ftmo_bf16_gemm(const float* x, const uint16_t* w, size_t t, size_t rows, size_t cols, float* y);
/* :793-806 (exp = ftmo_expf) */
void ftmo_softmax_rows(float* logits, size_t n, size_t e);
/* :808-830 with the tie rule of python/ferrum_kernel/elementwise.py:372-373 and
 * tests/cudarc_forward.rs:89-97: equal probabilities go to the lowest index */
void ftmo_topk_renorm(const float* p, size_t n, size_t e, size_t k, int32_t* ids, float* w);
float ftmo_silu(float x);    /* :30-33 */
float ftmo_sigmoid(float x); /* :35-39 */

typedef struct ftmo_layer {
    size_t hidden, inter, experts, top_k, shared_inter;
    const uint16_t* gate_w;        /* [experts, hidden] bf16 */
    const uint16_t* sh_gate_up;    /* [2*shared_inter, hidden] bf16 */
    const uint16_t* sh_down;       /* [hidden, shared_inter] bf16 */
    const uint16_t* sh_gate;       /* [1, hidden] bf16 */
    ftmo_banks banks;              /* slots == experts (slot id = expert id) */
} ftmo_layer;

/* router only: :721-723 */
void ftmo_router(const ftmo_layer* L, const float* x, size_t t, int32_t* ids, float* w,
                 float* probs_or_null);
/* bf16 shared expert with `bf16_gemm` semantics: :684-714 with :162-179 */
void ftmo_shared_expert(const ftmo_layer* L, const float* x, size_t t, float* out);
/* the whole block: :716-791.  ids_out / w_out may be NULL. */
int ftmo_moe_block(const ftmo_layer* L, const float* x, size_t t, float* out, int32_t* ids_out,
                   float* w_out);
/* same arithmetic per (token, route) and per output row, spread over threads */
int ftmo_moe_block_mt(const ftmo_layer* L, const float* x, size_t t, float* out, int32_t* ids_out,
                      float* w_out, int threads);
/* prefill form the reference's inline fallback uses: dequantise an expert once,
 * then a dense matmul over its tokens (src/models/qwen3_6/forward_cudarc.rs:1629-1659,
 * src/domain/dequant.rs:99-103).  Same sums in a different association. */
int ftmo_moe_block_dequant_once_mt(const ftmo_layer* L, const float* x, size_t t, float* out,
                                   int threads);

/* ---- expert-slot LRU: src/domain/expert_cache.rs:8-134 ---- */
typedef struct ftmo_cache ftmo_cache;
ftmo_cache* ftmo_cache_new(size_t layers, size_t experts, size_t cache_size);
void ftmo_cache_free(ftmo_cache* c);
int32_t ftmo_cache_slot_of(const ftmo_cache* c, size_t layer, uint32_t expert);
int32_t ftmo_cache_id_of_slot(const ftmo_cache* c, size_t slot);
/* returns the number of misses; misses / write_slots hold at most n entries */
size_t ftmo_cache_ensure(ftmo_cache* c, size_t layer, const uint32_t* routed, size_t n,
                         uint32_t* misses, uint32_t* write_slots, int32_t* rewrites);

/* ---- the steps either side of the block ---- */
/* Fused residual add + RMSNorm on the bf16 stream: python/ferrum_kernel/norm.py:35-110
 * (`_add_rmsnorm_kernel`, `add_rmsnorm_reference`) with the row reduction in the order of the host tower's
 * rms_norm (src/models/qwen3_6/forward.rs:48-61: squares summed left to right, times 1 / row_len, then
 * 1 / sqrt(mean + eps)).  x, r, w are bf16 bit patterns; sum_out and out receive bf16 bit patterns. */
void ftmo_add_rmsnorm(const uint16_t* x, const uint16_t* r, const uint16_t* w, float eps, size_t rows,
                      size_t hidden, uint16_t* sum_out, uint16_t* out);
/* the host tower's f32 rms_norm itself: src/models/qwen3_6/forward.rs:48-61 */
void ftmo_rms_norm(const float* x, const float* w, float eps, size_t rows, size_t row_len, float* out);

/* Dense NVFP4 GEMV of the decode tail: python/ferrum_kernel/linear.py:152-168
 * (`nvfp4_dense_gemv_reference`: widen the whole weight, global included, then one f32 matmul), on the
 * K-major bank the launcher takes (src/infrastructure/cuda_linear.rs:103-111): packed [K/8, N] int32 with
 * nibble j of word (w, n) = code k = 8w + j of row n, scale [K/16, N] e4m3, global [N] f16.
 * a [M, K] f32, c [M, N] f32; sums over k left to right. */
void ftmo_nvfp4_dense_gemv(const float* a, const uint32_t* packed_kmajor, const uint8_t* scale_kmajor,
                           const uint16_t* global, size_t m, size_t n, size_t k, float* c, int threads);

int ftmo_max_threads(void);

#ifdef __cplusplus
}
#endif
#endif
