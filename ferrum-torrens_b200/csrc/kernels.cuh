// Launchers of the MoE kernels; each returns the number of kernel launches it enqueued.
#pragma once

#include <cuda.h>

#include <atomic>

#include "common.cuh"

namespace ftm {

// kinds of kernels, for the per-kernel CUDA-event profile (ftm_profile_*)
enum Kind {
    K_ROUTER_LOGITS = 0,
    K_ROUTER_TOPK,
    K_SLOT_REWRITE,
    K_CSR,
    K_EXPERT_GATE_UP,
    K_EXPERT_DOWN,
    K_SUM_ROUTES,
    K_SHARED_PHASE1,
    K_SHARED_PHASE2,
    K_CAST,
    K_COMBINE,
    K_GROUPED_GATE_UP,
    K_GROUPED_DOWN,
    K_PERMUTE_ACT,
    K_DECODE_PLAN,
    K_EP_PACK,
    K_EP_COMBINE,
    K_PREFILL_RESCALE,
    K_DENSE_GEMV,
    K_ADD_RMSNORM,
    K_NUM_KINDS
};

struct Profiler;

// what every launcher gets: the stream, and the profiler when one is recording
struct Ctx {
    cudaStream_t s;
    Profiler* prof;
    void begin(int kind) const;  // records an event before a launch when profiling
    void end() const;            // and one after it
};

// Programmatic dependent launch for chains of small dependent kernels (the decode step): the next kernel of the
// stream may be scheduled while its predecessor drains; it calls pdl_wait() before it reads what the
// predecessor wrote.  Both calls are no-ops for a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// The opt-in to more than 48 KB of dynamic shared memory is a per-device property of a kernel, and one
// process may hold adapters on several devices: every launcher remembers, per device ordinal, whether
// the current device has been opted in.  Safe to call from several threads (the attribute call is
// idempotent; the mask only saves repeating it).
struct PerDeviceOnce {
    std::atomic<uint64_t> mask{0};
};
template <typename KernelT>
inline cudaError_t allow_dyn_smem(PerDeviceOnce& once, KernelT kernel, size_t bytes) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const uint64_t bit = 1ull << (dev & 63);
    if (once.mask.load(std::memory_order_acquire) & bit) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess) once.mask.fetch_or(bit, std::memory_order_release);
    return e;
}

// router.cu
int launch_router_logits(const __nv_bfloat16* x, const __nv_bfloat16* gate_w, int tokens, int experts,
                         int hidden, float* logits, const Ctx& c);
int launch_router_topk(const float* logits, int tokens, int experts, int top_k, int32_t* ids,
                       float* weights, const Ctx& c);

// logits and top-k in one cluster launch (256 experts, fewer than 1024 tokens)
bool router_fused_supported(int tokens, int experts, int hidden, int top_k);
int launch_router_fused(const __nv_bfloat16* x, const __nv_bfloat16* gate_w, int tokens, int hidden, int top_k,
                        int32_t* ids, float* weights, const Ctx& c);

// permute.cu
// scratch: cta_hist needs csr_scratch_ints(routes, bins) int32 entries
size_t csr_scratch_ints(int routes, int bins);
// optional second output of the permutation build: every bin cut into passes of at most `group` routes
struct CsrGroups {
    const int32_t* slot_of_bin = nullptr;   // bin -> slot (null: the bin is the slot); bins of slots outside [0, slots) are skipped
    int slots = 0, group = 0;
    int4* groups = nullptr;
    int32_t* n_groups = nullptr;
    int32_t* pos_of_route = nullptr;        // optional: route -> sorted position, written by the scatter pass
};
// optional first step of the permutation build: dense expert ids of a layer -> slots (route_slot) and bins (route_expert:
// the expert id, -1 when not resident); the build then buckets by route_expert
struct SlotRewrite {
    const void* expert_ids = nullptr;
    int ids_dtype = 0, layer = 0, experts = 0;
    const int32_t* slot_for_id = nullptr;
    int n_ids = 0;
    int32_t* route_slot = nullptr;
    int32_t* route_expert = nullptr;
    int32_t* bad_flag = nullptr;
};
int launch_csr_build(const int32_t* route_bin, int routes, int bins, int32_t* seg, int32_t* route_idx,
                     int32_t* scratch, int32_t* bad_flag, const Ctx& c, bool coarse = false, const CsrGroups* groups = nullptr,
                     const SlotRewrite* rewrite = nullptr);
int launch_slot_rewrite(const void* expert_ids, int ids_dtype, int routes, int layer, int experts,
                        const int32_t* slot_for_id, int n_ids, int32_t* route_slot, int32_t* route_expert,
                        int32_t* bad_flag, const Ctx& c);

// decode_gemv.cu
int launch_decode_routes(const BankView& b, const __nv_bfloat16* x, const int32_t* route_slot,
                         const float* route_weight, int tokens, int top_k, float* ic2, float* yroute,
                         const Ctx& c);

// decode_mma.cu: grouped decode path (plan + k-permuted activations + TMA/mma.sync expert kernels)
struct DecodeScratch {
    float* ic2p;            // [routes, inter] f32
    int4* groups;           // [routes] (slot, first sorted position, count, 0)
    int32_t* sorted_route;  // [routes]
    int32_t* n_groups;      // [1]
    float* yroute;          // [routes, hidden] f32
    int32_t* err;           // raised when a bounded wait gives up
    // large batches: buckets through the multi-CTA CSR build
    int32_t* route_bin;     // [routes]
    int32_t* seg;           // [bins + 1]
    int32_t* csr_scratch;
    int32_t* csr_flag;
};
// where the routes of a decode step come from: slot ids as given, or dense expert ids of one layer
// that the plan maps to slots through the residency table
struct DecodeRoutes {
    const int32_t* route_slot_in;
    const void* expert_ids;
    int ids_dtype, layer, experts, n_ids;
    const int32_t* slot_for_id;
    int32_t* route_slot_out;
    int32_t* bad_flag;
};
bool decode_mma_supported(int hidden, int inter, int routes, int slots, int experts, bool have_expert_ids);
int launch_decode_mma(const BankView& b, const void* x, int x_dtype, const DecodeRoutes& rt,
                      const float* route_weight, int tokens, int top_k, DecodeScratch sc, int sm_count,
                      const Ctx& c);

// fragment-ordered copy of one slot's block scales (both projections), after the slot's bytes have landed
int launch_scale_repack(const BankView& b, int slot, uint8_t* gu_scale_frag, uint8_t* dn_scale_frag, const Ctx& c);

int launch_groups_from_csr(const int32_t* seg, int bins, const int32_t* slot_of_bin, int slots, int group,
                           int4* groups, int32_t* n_groups, const Ctx& c);

// prefill_umma.cu: grouped GEMM on tcgen05 tensor cores for large batches
struct PrefillScratch {
    int32_t* route_bin;      // [routes]
    int32_t* seg;            // [bins + 1]
    int32_t* route_idx;      // [routes] sorted position -> route
    int32_t* pos_of_route;   // [routes]
    int32_t* csr_scratch;
    int32_t* csr_flag;
    int4* groups;            // [routes / 1 ..] (slot, first sorted row, rows, 0)
    int32_t* n_groups;
    __half* xg;              // [routes, hidden] sorted activations, scaled f16
    float* row_scale;        // [routes]
    float* ic1;              // [routes, 2 * inter] f32: gate | up of every sorted row
    __half* ic2h;            // [routes, inter]
    float* row_scale2;       // [routes]
    void* y;                 // [routes, hidden] weighted expert outputs, sorted rows: bf16, or f32 for f32 outputs
    int32_t* err;
};
// tensor maps of the grouped GEMMs, encoded once per adapter (activation boxes of 32 / 64 / 96 / 128 rows)
struct PrefillMaps {
    CUtensorMap x[4], h[4], gp, gs, dp, ds;
    bool ok = false;
};
// expert-parallel owner: where the down GEMM stores its finished rows instead of the adapter's own scratch.
// Received row i came from source rank s at row r of that rank's send order; its output row goes to row r of
// peer_back[s] ([capacity, hidden] bf16 in that rank's memory), by plain stores of the GEMM's epilogue.
struct EpReturnTo {
    int world, rank;
    const int32_t* counts_all;   // [world, world] routes source -> owner
    const uint64_t* peer_back;   // [world] base addresses of the back buffers
    long long capacity;          // rows of every back buffer
};
bool prefill_umma_supported(int hidden, int inter, int slots, int experts, bool have_expert_ids);
bool prefill_build_maps(const BankView& b, const __half* xg, const __half* ic2h, size_t rows, PrefillMaps* out);
int launch_prefill_umma(const BankView& b, const void* x, int x_dtype, const DecodeRoutes& rt,
                        const float* route_weight, int tokens, int top_k, PrefillScratch sc, int sm_count,
                        const float* shared, const float* se_gate, cudaEvent_t join, void* out, int out_dtype,
                        const PrefillMaps& maps, const Ctx& c, const EpReturnTo* ret = nullptr);
int launch_prefill_umma_presorted(const BankView& b, const float* row_scale, const float* route_weight, int rows,
                                  const int32_t* seg_all, int experts, const int32_t* slot_of_bin, PrefillScratch sc,
                                  int sm_count, const EpReturnTo& ret, const PrefillMaps& maps, const Ctx& c);

// shared_expert.cu
int launch_shared_expert(const __nv_bfloat16* x, int tokens, int hidden, int shared_inter,
                         const __nv_bfloat16* gate_up, const __nv_bfloat16* down,
                         const __nv_bfloat16* shared_gate, float* ic2s, float* shared_out,
                         float* se_gate, int32_t* err, const Ctx& c);
// shared_umma.cu: the same on tcgen05 tensor cores, for batches of 256 tokens and more
bool shared_umma_supported(int tokens, int hidden, int shared_inter);
int launch_shared_umma(const __nv_bfloat16* x, int tokens, int hidden, int shared_inter, const __nv_bfloat16* gate_up,
                       const __nv_bfloat16* down, const __nv_bfloat16* shared_gate, __nv_bfloat16* ic2b, float* shared_out,
                       float* se_gate, int32_t* err, const Ctx& c);

// combine.cu
int launch_sum_routes(const float* yroute, int tokens, int top_k, int hidden, const float* shared,
                      const float* se_gate, void* out, int out_dtype, const Ctx& c);
int launch_combine(const void* routed, int routed_dtype, const float* shared, const float* se_gate,
                   int tokens, int hidden, void* out, int out_dtype, const Ctx& c);
int launch_ep_pack(const __nv_bfloat16* x, const int32_t* ids, const float* weights, const int32_t* route_idx,
                   const int32_t* seg, int tokens, int top_k, int hidden, int experts, int ranks,
                   __nv_bfloat16* send_x, int32_t* send_expert, float* send_weight, int32_t* counts, const Ctx& c);
int launch_ep_combine(const void* y, int y_dtype, const int32_t* route_idx, int32_t* pos_scratch, int tokens,
                      int top_k, int hidden, const float* shared, const float* se_gate, void* out, int out_dtype,
                      const Ctx& c);
int launch_ep_counts(const int32_t* seg, int experts, int ranks, int32_t* counts, const Ctx& c);
int launch_ep_dispatch_sorted(const __nv_bfloat16* x, const int32_t* ids, const float* weights, const int32_t* route_idx,
                              const int32_t* seg_all, int tokens, int top_k, int experts, int world, int rank,
                              const uint64_t* peer_xg, const uint64_t* peer_w, const uint64_t* peer_rs, long long capacity,
                              int32_t* err, const Ctx& c);
int launch_ep_dispatch(const __nv_bfloat16* x, const int32_t* ids, const float* weights, const int32_t* route_idx,
                       const int32_t* seg, int tokens, int top_k, int hidden, int experts, int world, int rank,
                       const int32_t* counts_all, const uint64_t* peer_x, const uint64_t* peer_meta, long long capacity,
                       int32_t* err, const Ctx& c);
// pos_of_route / route_slot null: y is in receive order; else y is still sorted by expert (see the kernel)
int launch_ep_return(const __nv_bfloat16* y, const int32_t* pos_of_route, const int32_t* route_slot, int n, int hidden,
                     int world, int rank, const int32_t* counts_all, const uint64_t* peer_back, long long capacity,
                     int32_t* err, const Ctx& c);
int launch_cast_to_bf16(const void* src, int src_dtype, size_t n, __nv_bfloat16* dst, const Ctx& c);
// fused residual add + RMSNorm in front of the block: sum_out = bf16(x + r), out = bf16(sum * rsqrt(mean(sum^2) + eps) * w)
int launch_add_rmsnorm(const __nv_bfloat16* x, const __nv_bfloat16* r, const __nv_bfloat16* w, float eps, int tokens,
                       int hidden, __nv_bfloat16* sum_out, __nv_bfloat16* out, const Ctx& c);

// dense_gemv.cu: K-major NVFP4 GEMV of the decode tail (lm_head)
bool dense_gemv_supported(int N, int K);
int launch_dense_gemv(const void* a, int a_dtype, const uint32_t* packed, const uint8_t* scale, const uint16_t* global,
                      int M, int N, int K, float* c, int sm_count, int32_t* err, const Ctx& ctx);

}  // namespace ftm
