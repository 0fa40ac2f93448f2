/*
 * libftmoe -- C ABI of the B200 (sm_100a) NVFP4 mixture-of-experts layer.
 *
 * This is the seam a host engine binds through FFI.  Every entry point takes
 * plain pointers, sizes and integer codes; no C++ or framework types cross it.
 * Each declaration names the interface of the reference engine it stands in
 * for (path:line inside the reference project, butzist/ferrum-torrens).
 *
 * Conventions
 *  - "dev" pointers are device addresses valid in the PRIMARY context of the
 *    ordinal given at creation (the context the engine's tensor runtime uses,
 *    src/infrastructure/cuda_driver.rs:389-399).  "host" pointers are ordinary
 *    host memory.
 *  - `stream` is a CUstream / cudaStream_t passed as void*.  NULL selects the
 *    stream given to ftm_create.  Calls documented as asynchronous only enqueue
 *    work: no allocation, no host read-back, no synchronisation
 *    (src/infrastructure/cuda_moe.rs:1283-1286).
 *  - Every shape, dtype and length is validated before anything is launched
 *    (src/infrastructure/cuda_moe.rs:959-1003); a rejected call has no effect.
 *  - Return value: FTM_OK or one of the codes below, which map one to one onto
 *    the reference's MoEError variants (src/domain/expert_kernel.rs:21-39).
 *    ftm_last_error(h) returns the message of the last failed call on h.
 *    Nothing aborts or throws across this boundary.
 *  - One handle serialises its calls internally (the reference wraps its
 *    adapter in one Mutex, src/infrastructure/cuda_moe.rs:197-203).
 */
#ifndef FTMOE_H
#define FTMOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FTM_ABI_VERSION 1

#if defined(__GNUC__)
#define FTM_API __attribute__((visibility("default")))
#else
#define FTM_API
#endif

typedef struct ftm_handle ftm_handle;

/* MoEError (src/domain/expert_kernel.rs:21-39) */
enum {
    FTM_OK = 0,
    FTM_ERR_BAD = 1,               /* MoEError::Bad */
    FTM_ERR_SLOT_OUT_OF_RANGE = 2, /* MoEError::SlotOutOfRange */
    FTM_ERR_MISSING = 3,           /* MoEError::Missing */
    FTM_ERR_OUT_OF_MEMORY = 4,     /* MoEError::OutOfMemory (retryable) */
    FTM_ERR_READ = 5,              /* MoEError::Read */
    FTM_ERR_NOT_SUPPORTED = 6,     /* the `Ok(None)` answers of begin_staged */
    FTM_ERR_CUDA = 7               /* a CUDA runtime error; reported as MoEError::Bad("driver: ..") */
};

/* element types accepted at the boundary (src/infrastructure/cuda_moe.rs:67-86, :1101-1107) */
enum { FTM_BF16 = 0, FTM_F32 = 1, FTM_I32 = 2, FTM_I64 = 3 };

/* bank order, a cross-adapter contract (src/domain/expert_kernel.rs:62-80) */
enum {
    FTM_BANK_GATE_UP_PACKED = 0,
    FTM_BANK_GATE_UP_SCALE = 1,
    FTM_BANK_GATE_UP_GLOBAL = 2,
    FTM_BANK_DOWN_PACKED = 3,
    FTM_BANK_DOWN_SCALE = 4,
    FTM_BANK_DOWN_GLOBAL = 5,
    FTM_NUM_BANKS = 6
};

/* which routed-expert kernels a call may use */
enum {
    FTM_PATH_AUTO = 0,   /* decode GEMV for small batches, grouped GEMM for large */
    FTM_PATH_GEMV = 1,   /* bandwidth-bound decode path */
    FTM_PATH_GROUPED = 2, /* tcgen05 grouped GEMM (prefill) */
    FTM_PATH_SCALAR = 3   /* one CTA column per route, CUDA-core dot products; any multiple-of-16 shape */
};

/* CudaMoE::new_with_stream(device, source, shapes, slots, stream)
 * (src/infrastructure/cuda_moe.rs:406-480) */
typedef struct ftm_config {
    int32_t ordinal;      /* CUDA device ordinal; its primary context is used */
    int32_t hidden;       /* 2048; nonzero multiple of 16 (ExpertShapes::new, expert_kernel.rs:186-193) */
    int32_t inter;        /* 512;  nonzero multiple of 16 */
    int32_t top_k;        /* 8 */
    int32_t experts;      /* experts per layer (256) */
    int32_t layers;       /* layers sharing the banks (flat id = layer * experts + expert) */
    int32_t slots;        /* expert slots in the device banks, >= 1.  layers * experts keeps
                             every expert resident, which is the B200 configuration. */
    int32_t shared_inter; /* shared-expert intermediate size (512); 0 = no shared expert calls */
    int32_t max_tokens;   /* largest token count of one call; scratch is allocated for it here */
    int32_t ep_rank;      /* expert-parallel rank and size; 0 / 1 on one GPU */
    int32_t ep_size;
} ftm_config;

FTM_API int ftm_abi_version(void);

/* Creates the adapter, allocates banks and scratch.  `stream` is the engine's
 * stream; all work is ordered on it unless a call passes another one. */
FTM_API int ftm_create(const ftm_config* cfg, void* stream, ftm_handle** out);
FTM_API void ftm_destroy(ftm_handle* h);
/* Message of the last failed call; valid until the next call on h.  ftm_last_error(NULL)
 * returns the message of the last failed ftm_create on this thread. */
FTM_API const char* ftm_last_error(const ftm_handle* h);

/* ---- ExpertSlotStore (src/domain/expert_kernel.rs:140-161) ------------------------------ */

/* `load(layer, expert, slot)`: copies one expert's six byte fields (bank order) from host
 * memory into row `slot` of each bank and records the expert as resident in that slot,
 * displacing the slot's previous occupant (src/infrastructure/cuda_moe.rs:552-576).
 * lens[b] must equal bank_row_bytes(b) (expert_kernel.rs:211-218).  Synchronous. */
FTM_API int ftm_load_expert(ftm_handle* h, int32_t layer, int32_t expert, int32_t slot,
                    const uint8_t* const host_fields[FTM_NUM_BANKS], const size_t lens[FTM_NUM_BANKS]);
/* same, the six fields already in device memory (asynchronous on the handle's stream) */
FTM_API int ftm_load_expert_dev(ftm_handle* h, int32_t layer, int32_t expert, int32_t slot,
                        const void* const dev_fields[FTM_NUM_BANKS], const size_t lens[FTM_NUM_BANKS]);
FTM_API int ftm_slots(const ftm_handle* h);
FTM_API int ftm_release_banks(ftm_handle* h);   /* :596-611 frees the banks, keeps the slot count */
FTM_API int ftm_rehydrate_banks(ftm_handle* h); /* :613-625 reallocates them, every slot empty */
FTM_API int ftm_banks_resident(const ftm_handle* h);
/* device base address of each bank, bank order (src/infrastructure/cuda_moe.rs:531-549) */
FTM_API int ftm_bank_ptrs(const ftm_handle* h, uint64_t out[FTM_NUM_BANKS]);
/* bytes of one expert's row in bank b (ExpertShapes::bank_row_bytes) */
FTM_API size_t ftm_bank_row_bytes(const ftm_handle* h, int bank);
/* slot holding (layer, expert), or -1 */
FTM_API int32_t ftm_slot_of(const ftm_handle* h, int32_t layer, int32_t expert);

/* ---- ExpertCache, the host slot machine (src/domain/expert_cache.rs:8-134) -------------- */
/* ensure_experts(layer, routed): marks hits used, assigns LRU victims to the misses
 * (ascending expert id) and rewrites every routed id to its slot.  Returns FTM_OK and
 * *n_miss; misses / write_slots need room for n entries.  Purely a plan: the caller
 * performs the loads (run_experts, src/application/run_experts.rs:209-246). */
FTM_API int ftm_ensure_experts(ftm_handle* h, int32_t layer, const uint32_t* routed, size_t n,
                       uint32_t* misses, uint32_t* write_slots, int32_t* rewrites, size_t* n_miss);

/* ---- router (src/models/qwen3_6/forward_cudarc.rs:1403-1435) ---------------------------- */
/* Fused gate projection + softmax + top-k + renormalise.  x [T, hidden] bf16 dev,
 * gate_w [experts, hidden] bf16 dev -> ids [T, top_k] i32 dev, weights [T, top_k] f32 dev.
 * Logits are f32 sums taken over k in ascending order, so the selected ids equal the host
 * path's (forward.rs:162-179, :793-830); equal probabilities go to the lowest expert index.
 * Asynchronous. */
FTM_API int ftm_router(ftm_handle* h, const void* x_bf16, const void* gate_w_bf16, int32_t tokens,
               int32_t* ids_out, float* weights_out, void* stream);
/* Tensor::fused_topk_softmax(k) (src/infrastructure/cudarc.rs:1147-1171;
 * python/ferrum_kernel/elementwise.py:350-382): logits [T, experts] f32 dev. */
FTM_API int ftm_router_from_logits(ftm_handle* h, const float* logits, int32_t tokens, int32_t* ids_out,
                           float* weights_out, void* stream);

/* ---- permutation (src/infrastructure/cuda_moe.rs:1198-1253, :2328-2362) ----------------- */
/* csr_build: route_slot [R] i32 dev -> seg [bins+1] i32 dev (exclusive prefix of per-bin
 * counts) and route_idx [R] i32 dev (route ids sorted by bin, ascending route id inside a
 * bin).  A slot outside [0, bins) raises the device flag read by ftm_csr_bad.  Asynchronous. */
FTM_API int ftm_csr_build(ftm_handle* h, const int32_t* route_slot, int32_t routes, int32_t bins,
                  int32_t* seg_out, int32_t* route_idx_out, void* stream);
/* synchronises the stream and returns the flag (0 = all routes were in range) */
FTM_API int ftm_csr_bad(ftm_handle* h, void* stream, int32_t* bad_out);
/* No counterpart in the reference.  The same permutation build for callers that cannot allocate device
 * memory (an engine running under a fixed memory plan whose allocator is locked after start-up, or
 * a call site where allocation is forbidden): it takes no handle, and its scratch (per-CTA histograms
 * and the out-of-range flag) is a fixed array inside the library image, held by every GPU that loads
 * the library until the process exits.  Limits: routes <= 262144, bins <= 1024; larger sizes return
 * FTM_ERR_BAD.  It calls no allocating routine.  The first call on a device looks up the array's
 * device address (with that device current): make it before any stream capture.  Calls on one
 * device share the array, so two calls that overlap on the GPU race.  bad_out (device pointer, may
 * be NULL) receives 1 when a slot was outside [0, bins).  Asynchronous on `stream`. */
FTM_API int ftm_csr_build_noalloc(const int32_t* route_slot, int32_t routes, int32_t bins, int32_t* seg_out,
                                  int32_t* route_idx_out, int32_t* bad_out, void* stream);

/* ---- ExpertGemm (src/domain/expert_kernel.rs:246-294) ----------------------------------- */
/* grouped_moe(&MoEGroup, &mut [f32]): host hand-off.  x [T, hidden] f32 host (narrowed to bf16
 * like the reference adapter, cuda_moe.rs:1022-1045), routes [T*top_k] i32 slot ids (-1 = not
 * resident, contributes nothing), weights [T*top_k] f32, out [T, hidden] f32 host.  Synchronous. */
FTM_API int ftm_grouped_moe_host(ftm_handle* h, const float* x, size_t x_len, int32_t top_k,
                         const int32_t* routes, size_t routes_len, const float* weights,
                         size_t weights_len, float* out, size_t out_len);
/* grouped_moe_dev: x / weights / out on the device, routes (slot ids) on the host
 * (expert_kernel.rs:345-352, cuda_moe.rs:1531-1539).  Asynchronous after the routes upload. */
FTM_API int ftm_grouped_moe_dev(ftm_handle* h, const void* x, int x_dtype, int32_t tokens, int32_t top_k,
                        const int32_t* routes_host, size_t routes_len, const float* weights_dev,
                        void* out, int out_dtype, void* stream);
/* grouped_moe_staged(&MoEDeviceRequest, out): THE SERVING CALL (expert_kernel.rs:261-273,
 * :332-340; cuda_moe.rs:1545-1622).  experts [T, top_k] are the router's dense expert ids of
 * `layer` (i32 or i64 dev); the adapter maps them to slots on the device through its residency
 * table and works on its own copy.  x bf16 or f32, weights f32, out bf16 or f32, exact shape
 * [T, hidden].  out receives the routed sum only.  Asynchronous, capturable. */
FTM_API int ftm_moe_layer_staged(ftm_handle* h, int32_t layer, const void* x, int x_dtype,
                         const void* expert_ids, int ids_dtype, const float* weights,
                         int32_t tokens, void* out, int out_dtype, int path, void* stream);
/* begin_staged / PendingMoE::finish (expert_kernel.rs:275-281, :359-361).  With every expert
 * resident there is no miss copy to overlap, so begin answers FTM_ERR_NOT_SUPPORTED, the
 * reference's `Ok(None)`: call ftm_moe_layer_staged. */
FTM_API int ftm_moe_begin(ftm_handle* h, int32_t layer, const void* x, int x_dtype, const void* expert_ids,
                  int ids_dtype, const float* weights, int32_t tokens, void* stream);
FTM_API int ftm_moe_finish(ftm_handle* h, void* out, int out_dtype, void* stream);
/* staged_route_cap (expert_kernel.rs:283-287): largest tokens * top_k of one staged call */
FTM_API size_t ftm_route_cap(const ftm_handle* h);
/* reset_staging (expert_kernel.rs:289-293): forgets residency; the banks keep their bytes */
FTM_API int ftm_reset_staging(ftm_handle* h);
/* Waits for `stream` and reports what the asynchronous calls could not: an expert id outside the
 * layer (the reference's device `bad` flag, python/ferrum_kernel/moe_prefill.py:49-56) or a kernel
 * that gave up a bounded wait.  FTM_OK when the steps since the last call were clean. */
FTM_API int ftm_sync_status(ftm_handle* h, void* stream);
/* MoEExecutor::steps (expert_kernel.rs:390-395): routed steps run since creation */
FTM_API uint64_t ftm_steps(const ftm_handle* h);

/* ---- shared expert and combine (forward_cudarc.rs:1455-1562, :1590) --------------------- */
/* SharedExpertFused::{phase1, phase2} (src/infrastructure/cuda_linear.rs:391-450) and the
 * T > 1 path (forward_cudarc.rs:1541-1561): shared[t] = down_s(silu(gate_s x) * up_s x),
 * se_gate[t] = sigmoid(x . shared_gate).  gate_up [2*shared_inter, hidden], down [hidden,
 * shared_inter], shared_gate [hidden], all bf16 dev.  shared_out [T, hidden] f32 dev receives the
 * UNGATED shared-expert output, se_gate_out [T] f32 dev the gate.  Asynchronous. */
FTM_API int ftm_shared_expert(ftm_handle* h, const void* x_bf16, int32_t tokens, const void* gate_up_bf16,
                      const void* down_bf16, const void* shared_gate_bf16, float* shared_out,
                      float* se_gate_out, void* stream);
/* out[t] = se_gate[t] * shared[t] + routed[t]  (forward.rs:737-742, :785-787; `se.add(&routed)`).
 * routed is [T, hidden] bf16 or f32.  Asynchronous. */
FTM_API int ftm_combine(ftm_handle* h, const void* routed, int routed_dtype, const float* shared,
                const float* se_gate, int32_t tokens, void* out, int out_dtype, void* stream);

/* ---- the whole block (moe_parts, forward_cudarc.rs:1388-1591; moe_block, forward.rs:716-791) */
/* router -> residency rewrite -> routed experts -> fused weighted combine + gated shared
 * expert, with the shared expert overlapped on a second stream.  ids_out / weights_out may
 * be NULL.  out [T, hidden] bf16 or f32 dev.  Asynchronous. */
FTM_API int ftm_moe_block(ftm_handle* h, int32_t layer, const void* x_bf16, int32_t tokens,
                  const void* gate_w_bf16, const void* sh_gate_up_bf16, const void* sh_down_bf16,
                  const void* sh_gate_bf16, void* out, int out_dtype, int32_t* ids_out,
                  float* weights_out, int path, void* stream);

/* ---- the steps either side of the block ------------------------------------------------------- */
/* Fused residual add + RMSNorm (python/ferrum_kernel/norm.py:35-110 `_add_rmsnorm_kernel`; the
 * post-attention site src/models/qwen3_6/forward.rs:942-953): per row of `hidden` elements
 *   sum_out = bf16(f32(x) + f32(residual)),   out = bf16(f32(sum_out) * (1 / sqrt(mean(sum_out^2) + eps)) * f32(norm_w))
 * x, residual, sum_out, out [T, hidden] bf16 dev, norm_w [hidden] bf16 dev (the baked 1 + weight vector).
 * sum_out is the next layer's residual.  hidden a multiple of 8, at most 4096.  Asynchronous. */
FTM_API int ftm_add_rmsnorm(ftm_handle* h, const void* x_bf16, const void* residual_bf16, const void* norm_w_bf16, float eps,
                            int32_t tokens, void* sum_out_bf16, void* out_bf16, void* stream);
/* The post-attention norm and the block in one call (forward.rs:942-953 then moe_block(&h2), :716-791):
 * sum_out = attn_out + residual, h2 = rms_norm(sum_out), out = moe_block(h2).  The normalised rows are
 * written once to the adapter's scratch (or to h2_out when it is not NULL), which at decode sizes stays
 * in L2 until the router, the expert kernels and the shared expert have read it; the caller never
 * materialises h2 or runs a separate norm launch chain.  Other arguments as ftm_moe_block. */
FTM_API int ftm_moe_block_prenorm(ftm_handle* h, int32_t layer, const void* attn_out_bf16, const void* residual_bf16,
                                  const void* norm_w_bf16, float eps, int32_t tokens, const void* gate_w_bf16,
                                  const void* sh_gate_up_bf16, const void* sh_down_bf16, const void* sh_gate_bf16,
                                  void* sum_out_bf16, void* h2_out_bf16, void* out, int out_dtype, int32_t* ids_out,
                                  float* weights_out, int path, void* stream);
/* DenseGemv::gemv (src/infrastructure/cuda_linear.rs:48-175; kernel python/ferrum_kernel/linear.py:41-150):
 * c = a @ dequant(packed, scale, global)^T for the lm_head.  a [M, K] bf16 or f32 dev; the weight is the
 * engine's K-major resident bank: packed [K/8, N] int32 (word (w, n) = the eight e2m1 codes k = 8w .. 8w+7
 * of row n, nibble j -> k = 8w + j), scale [K/16, N] uint8 (e4m3), global [N] f16; c [M, N] f32 dev, fully
 * overwritten.  N a multiple of 4, K a multiple of 32.  The weight is streamed once per sixteen rows of a.
 * Asynchronous. */
FTM_API int ftm_dense_gemv(ftm_handle* h, const void* a, int a_dtype, const void* packed_kmajor_i32, const void* scale_kmajor_u8,
                           const void* global_f16, int32_t m, int32_t n, int32_t k, float* c, void* stream);

/* ---- FTW checkpoint: index and expert banks ---------------------------------------------------
 * The checkpoint the reference engine loads (src/infrastructure/ftw.rs): a JSON index
 * `freetoken_weight.json` over one logical byte region cut into shard files.  Host code only; none of
 * these calls needs a CUDA device except ftm_load_layer_from_ftw. */
typedef struct ftm_ftw ftm_ftw;
/* FtwReader::open (ftw.rs:397-440): parses `dir`/freetoken_weight.json (FtwIndex::parse, ftw.rs:95-252: format
 * tag, version 1, 4096 alignment, contiguous shards covering total_bytes, every tensor aligned, non-empty,
 * in range and shape * element size == nbytes) and opens every shard (a shard shorter than the index says is
 * refused).  Errors: FTM_ERR_READ for I/O and JSON syntax, FTM_ERR_BAD for an invalid index. */
FTM_API int ftm_ftw_open(const char* dir, ftm_ftw** out);
/* FtwIndex::parse alone, from the document text: entry / pieces work, reads fail (no shard is open) */
FTM_API int ftm_ftw_parse(const char* json_doc, ftm_ftw** out);
FTM_API void ftm_ftw_close(ftm_ftw* f);
/* message of the last failed call on f; ftm_ftw_last_error(NULL): of the last failed open / parse on this thread */
FTM_API const char* ftm_ftw_last_error(const ftm_ftw* f);
FTM_API int64_t ftm_ftw_tensor_count(const ftm_ftw* f);
FTM_API int64_t ftm_ftw_shard_count(const ftm_ftw* f);
FTM_API uint64_t ftm_ftw_total_bytes(const ftm_ftw* f);
/* FtwIndex::entry (ftw.rs:254-256): FTM_ERR_MISSING when the index has no such tensor.  shape receives at most
 * eight dimensions; is_experts_bank = the entry's kind is "experts_bank". */
FTM_API int ftm_ftw_entry(const ftm_ftw* f, const char* name, uint64_t* global_off, uint64_t* nbytes, uint64_t shape[8],
                          int32_t* ndim, int32_t* is_experts_bank);
/* FtwIndex::pieces (ftw.rs:262-302): the per-shard copies of the byte range [global_off, global_off + nbytes);
 * *n_pieces receives their number, the arrays at most max_pieces of them. */
FTM_API int ftm_ftw_pieces(const ftm_ftw* f, uint64_t global_off, uint64_t nbytes, int32_t max_pieces, int32_t* shard_index,
                           uint64_t* file_off, uint64_t* dest_off, uint64_t* length, int32_t* n_pieces);
/* WeightsReader::read_range (ftw.rs:505-520) */
FTM_API int ftm_ftw_read_range(ftm_ftw* f, uint64_t global_off, uint64_t nbytes, void* dst, size_t dst_len);
/* FtwBanks::slab (src/infrastructure/banks.rs:95-199): one expert's packed / scale / global bytes of
 * `{prefix}{gate_up|down}_{packed,scale,global}#L{layer:05}` (part 0 = gate_up, 1 = down; prefix NULL or ""
 * for the target's layers, "draft_" for the MTP draft's).  cap / lens: capacity of the three buffers and the
 * bytes written.  FTM_ERR_MISSING for a layer without entries, FTM_ERR_BAD when the expert is past the bank
 * or the three entries do not agree with the packed entry's shape, FTM_ERR_READ for a failed read. */
FTM_API int ftm_ftw_expert_slab(ftm_ftw* f, const char* bank_prefix, int32_t layer, uint32_t expert, int32_t part,
                                uint8_t* packed, uint8_t* scale, uint8_t* global, const size_t cap[3], size_t lens[3],
                                int32_t* rows_out, int32_t* cols_out);
/* Experts first_expert .. first_expert + n_experts - 1 of `layer` straight from the checkpoint into slots
 * slot0, slot0 + 1, ..: FtwBanks::slab for both parts, then ExpertSlotStore::load (cuda_moe.rs:552-576).
 * Synchronous.  The reference stages experts on demand because they do not fit its card; with every expert
 * resident this is the whole load path. */
FTM_API int ftm_load_layer_from_ftw(ftm_handle* h, ftm_ftw* f, const char* bank_prefix, int32_t layer, int32_t first_expert,
                                    int32_t n_experts, int32_t slot0);

/* ---- per-kernel timing (the reference's FT_PROFILE stage timer, src/infrastructure/profile.rs:1-14) */
/* While enabled, every kernel launch of h is bracketed by CUDA events on its stream.  Enabling
 * resets the accumulators; both calls synchronise the device.  Not for use under stream capture. */
FTM_API int ftm_profile_enable(ftm_handle* h, int on);
/* accumulated device time and launch count of one kernel kind since profiling was enabled */
FTM_API int ftm_profile_read(ftm_handle* h, int kind, double* total_ms, uint64_t* launches);
/* name of kernel kind 0, 1, ..; NULL past the last kind */
FTM_API const char* ftm_profile_kind_name(int kind);

/* ---- expert parallelism (no counterpart in the reference, which is single-GPU: README.md:132) ------
 * The layer is split over ep_size GPUs, rank p owning experts [p*E/n, (p+1)*E/n) of every layer.
 * ftm_ep_pack sorts this rank's T*top_k routes by global expert id (hence by owning rank, ascending
 * route id inside an expert: the CSR order) and fills the send buffers: send_x [R, hidden] bf16 (the
 * token's row), send_expert [R] (global expert id), send_weight [R], route_idx [R] (the route at each
 * position) and counts [ep_size] (routes per owning rank), all device memory.  After the all-to-all
 * the owner runs ftm_moe_layer_staged on a handle created with top_k = 1 (one received route = one
 * token, ids = the received global expert ids, only its own experts resident) and sends the weighted
 * rows back.  ftm_ep_combine is the fused weighted un-permute + gated shared-expert add:
 * out[t] = se_gate[t] * shared[t] + sum_j y[position of route t*top_k + j]; y is [R, hidden] bf16 or
 * f32 in send order; shared may be NULL.  Both asynchronous. */
FTM_API int ftm_ep_pack(ftm_handle* h, const void* x_bf16, const int32_t* ids, const float* weights, int32_t tokens,
                        int32_t ep_size, void* send_x, int32_t* send_expert, float* send_weight, int32_t* route_idx,
                        int32_t* counts, void* stream);
/* The same exchange over peer memory (NVLink loads and stores instead of a collective library).
 * counts_all [ep_size][ep_size] (device): row s = the counts of rank s, gathered by the caller.
 *   ftm_ep_plan      sorts this rank's routes by (owner, expert): route_idx [R], counts [ep_size].
 *   ftm_ep_dispatch  stores every route's activation row, expert id and weight straight into its
 *                    owner's receive buffers: peer_x / peer_meta are device arrays of ep_size pointers
 *                    ([capacity_rows, hidden] bf16 and [capacity_rows] (i32 id, f32 bits)); a rank's
 *                    rows follow those of the ranks before it, in its send order.  Call after
 *                    ftm_ep_plan on the same handle and stream.
 *   ftm_ep_return    the owner stores row i of y [rows, hidden] bf16 (receive order) into the source's
 *                    back buffer (peer_back: ep_size pointers to [capacity_rows, hidden] bf16) at the
 *                    position the source packed that route.
 * The caller orders the ranks (a barrier after the dispatch and after the return).  A row that would
 * fall outside a buffer is not stored and ftm_sync_status reports it. */
FTM_API int ftm_ep_plan(ftm_handle* h, const int32_t* ids, int32_t tokens, int32_t ep_size, int32_t* route_idx,
                        int32_t* counts, void* stream);
FTM_API int ftm_ep_dispatch(ftm_handle* h, const void* x_bf16, const int32_t* ids, const float* weights,
                            const int32_t* route_idx, int32_t tokens, int32_t ep_size, int32_t ep_rank,
                            const int32_t* counts_all, const uint64_t* peer_x, const uint64_t* peer_meta,
                            int64_t capacity_rows, void* stream);
FTM_API int ftm_ep_return(ftm_handle* h, const void* y_bf16, int32_t rows, int32_t ep_size, int32_t ep_rank,
                          const int32_t* counts_all, const uint64_t* peer_back, int64_t capacity_rows, void* stream);
/* The owner's step without its last pass.  ftm_moe_layer_staged on an owner adapter (top_k = 1) sorts the
 * received rows by expert, runs the grouped GEMMs and copies the results back into receive order; that copy
 * is only there to be read again by ftm_ep_return.  ftm_ep_experts_sorted stops before it (x [rows, hidden]
 * bf16, expert_ids / weights [rows], all device) and ftm_ep_return_sorted stores every row from where the GEMM
 * left it straight into its source's back buffer.  FTM_ERR_NOT_SUPPORTED for steps too small for the grouped
 * GEMM (at most 2048 rows): use ftm_moe_layer_staged and ftm_ep_return there.  Both asynchronous, same stream. */
FTM_API int ftm_ep_experts_sorted(ftm_handle* h, int32_t layer, const void* x_bf16, const int32_t* expert_ids,
                                  const float* weights, int32_t rows, void* stream);
FTM_API int ftm_ep_return_sorted(ftm_handle* h, int32_t rows, int32_t ep_size, int32_t ep_rank, const int32_t* counts_all,
                                 const uint64_t* peer_back, int64_t capacity_rows, void* stream);
/* The owner's step with the return inside it: as ftm_ep_experts_sorted, but the down GEMM's epilogue stores every
 * finished row straight into row r of peer_back[s], where s is the rank the row came from and r its position in
 * that rank's send order (plain stores over peer memory while the GEMM runs, no return pass and no copy of the
 * rows in this GPU's memory).  A received row whose expert is not resident returns zeros.  Same limits and
 * FTM_ERR_NOT_SUPPORTED rule as ftm_ep_experts_sorted; the caller's barrier follows it as it follows ftm_ep_return. */
FTM_API int ftm_ep_experts_return(ftm_handle* h, int32_t layer, const void* x_bf16, const int32_t* expert_ids,
                                  const float* weights, int32_t rows, int32_t ep_size, int32_t ep_rank,
                                  const int32_t* counts_all, const uint64_t* peer_back, int64_t capacity_rows,
                                  void* stream);
/* The exchange without a permutation build or a gather pass on the owner.  ftm_ep_plan_seg is ftm_ep_plan that
 * also hands out the prefix of the send order over the layer's experts (seg_out [experts + 1], device); the
 * caller all-gathers those prefixes into seg_all [ep_size, experts + 1].  From seg_all every rank knows where
 * each of its routes lands in the owner's activation matrix sorted by expert (within an expert: source rank,
 * then the source's send order), and ftm_ep_dispatch_sorted stores there, over peer memory, the token's row as
 * f16 scaled by a power of two (the layout the grouped GEMM's activation tiles are read from), its route weight
 * and its row scale: peer_xg / peer_weight / peer_row_scale are device tables of ep_size base addresses of
 * [capacity_rows, hidden] f16 and [capacity_rows] f32 buffers.  hidden 2048.  After the caller's barrier the owner
 * runs ftm_ep_experts_presorted on its own three buffers (xg 128-byte aligned, xg_capacity_rows rows long): groups
 * from seg_all, both GEMMs, every finished row stored by the down GEMM at row (prefix of its expert in the
 * source's send order + its index) of peer_back[source], i.e. at the position the source sent it from.  rows =
 * the rows this owner received (more than 0); an expert that is not resident returns zero rows. */
FTM_API int ftm_ep_plan_seg(ftm_handle* h, const int32_t* ids, int32_t tokens, int32_t* route_idx, int32_t* seg_out,
                            void* stream);
FTM_API int ftm_ep_dispatch_sorted(ftm_handle* h, const void* x_bf16, const int32_t* ids, const float* weights,
                                   const int32_t* route_idx, int32_t tokens, int32_t ep_size, int32_t ep_rank,
                                   const int32_t* seg_all, const uint64_t* peer_xg, const uint64_t* peer_weight,
                                   const uint64_t* peer_row_scale, int64_t capacity_rows, void* stream);
FTM_API int ftm_ep_experts_presorted(ftm_handle* h, int32_t layer, const void* xg_f16, const float* weights,
                                     const float* row_scale, int32_t rows, int64_t xg_capacity_rows, int32_t ep_size,
                                     int32_t ep_rank, const int32_t* seg_all, const uint64_t* peer_back,
                                     int64_t back_capacity_rows, void* stream);
FTM_API int ftm_ep_combine(ftm_handle* h, const void* y, int y_dtype, const int32_t* route_idx, const float* shared,
                           const float* se_gate, int32_t tokens, void* out, int out_dtype, void* stream);

/* SMs that the persistent expert kernels of h may occupy (0 = all of the device).  The expert kernels
 * run one CTA per SM for their whole duration; an expert-parallel caller that wants its exchange kernels
 * (NCCL) to run at the same time leaves them a few SMs.  No counterpart in the reference (one GPU). */
FTM_API int ftm_set_sm_budget(ftm_handle* h, int32_t sms);

/* number of this library's kernels launched on h since creation (a diagnostics counter) */
FTM_API uint64_t ftm_kernel_launches(const ftm_handle* h);

#ifdef __cplusplus
}
#endif
#endif /* FTMOE_H */
