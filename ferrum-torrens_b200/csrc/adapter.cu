// The device MoE adapter behind the C ABI of include/ftmoe.h.
//
// It plays the role of the reference's `CudaMoE` (src/infrastructure/cuda_moe.rs:145-195): it owns
// the six expert banks (slot-major, stable addresses for the adapter's life), the residency table,
// the per-step scratch, and it launches the kernels.  With every expert resident in HBM the
// reference's host-offload slot cache collapses to an identity indirection, which is kept: routes
// name slots, a slot of -1 contributes nothing, and the dense expert ids of the serving call are
// mapped to slots on the device.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/ftmoe.h"
#include "expert_cache.hpp"
#include "kernels.cuh"

using namespace ftm;

namespace {

thread_local std::string g_create_error;

const char* const kKindNames[K_NUM_KINDS] = {
    "router_logits", "router_topk", "slot_rewrite", "csr_build", "expert_gate_up", "expert_down", "sum_routes",
    "shared_phase1", "shared_phase2", "cast_bf16",   "combine",  "grouped_gate_up", "grouped_down",
    "permute_act",   "decode_plan",   "ep_pack",         "ep_combine", "prefill_rescale", "dense_gemv",
    "add_rmsnorm"};

}  // namespace

// CUDA-event timing of every kernel launch while enabled (the counterpart of the reference's
// FT_PROFILE stage timer, src/infrastructure/profile.rs:1-14).  Off by default: no events.
struct ftm::Profiler {
    struct Rec {
        int kind;
        cudaEvent_t a, b;
    };
    bool on = false;
    std::vector<Rec> recs;
    std::vector<cudaEvent_t> pool;
    double total_ms[K_NUM_KINDS] = {};
    uint64_t count[K_NUM_KINDS] = {};
    cudaEvent_t get() {
        if (!pool.empty()) {
            cudaEvent_t e = pool.back();
            pool.pop_back();
            return e;
        }
        cudaEvent_t e = nullptr;
        cudaEventCreate(&e);
        return e;
    }
    void drain() {  // caller has synchronised the streams
        for (auto& r : recs) {
            float ms = 0.f;
            if (cudaEventElapsedTime(&ms, r.a, r.b) == cudaSuccess) {
                total_ms[r.kind] += ms;
                count[r.kind]++;
            }
            pool.push_back(r.a);
            pool.push_back(r.b);
        }
        recs.clear();
    }
    ~Profiler() {
        for (auto& r : recs) {
            cudaEventDestroy(r.a);
            cudaEventDestroy(r.b);
        }
        for (auto e : pool) cudaEventDestroy(e);
    }
};

void ftm::Ctx::begin(int kind) const {
    if (!prof || !prof->on) return;
    Profiler::Rec r{kind, prof->get(), prof->get()};
    cudaEventRecord(r.a, s);
    prof->recs.push_back(r);
}

void ftm::Ctx::end() const {
    if (!prof || !prof->on || prof->recs.empty()) return;
    cudaEventRecord(prof->recs.back().b, s);
}

struct ftm_handle {
    ftm_config cfg{};
    cudaStream_t stream = nullptr;
    cudaStream_t aux = nullptr;  // shared expert runs here, ordered by events
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    mutable std::mutex mu;
    mutable std::string err;

    size_t row_bytes[FTM_NUM_BANKS]{};
    void* banks[FTM_NUM_BANKS]{};
    // the block scales of both projections once more, in the order the decode kernels' lanes read them
    // (same bytes, reordered by launch_scale_repack whenever a slot is loaded); null for shapes those
    // kernels do not take
    void* scale_frag[2]{};
    bool resident = false;

    std::vector<int32_t> slot_for_id;  // host mirror, [layers * experts]
    std::vector<int32_t> id_of_slot;   // [slots]
    int32_t* d_slot_for_id = nullptr;
    std::unique_ptr<ExpertCache> cache;

    // scratch, sized for cfg.max_tokens at creation (the serving call never allocates)
    __nv_bfloat16* x_bf16 = nullptr;
    int32_t *route_slot = nullptr, *route_expert = nullptr, *seg = nullptr, *route_idx = nullptr;
    int32_t *csr_scratch = nullptr, *flags = nullptr, *ids = nullptr;
    float *ic2 = nullptr, *yroute = nullptr, *logits = nullptr, *rweights = nullptr;
    float *ic2s = nullptr, *shared_out = nullptr, *se_gate = nullptr, *routed_f32 = nullptr;
    __half* xh = nullptr;
    float *tok_scale = nullptr, *ic2p = nullptr;
    __half* xg = nullptr;        // [R, H] sorted activations of the grouped GEMM
    float *row_scale = nullptr, *row_scale2 = nullptr;
    int4* groups = nullptr;
    int32_t *sorted_route = nullptr, *n_groups = nullptr;
    PrefillMaps maps;     // tensor maps of the grouped GEMMs (fixed addresses: encoded once)
    PrefillMaps maps_ext; // the same with the activation maps on a caller's matrix (expert-parallel owner)
    const void* maps_ext_xg = nullptr;
    int64_t maps_ext_rows = 0;
    int sm_count = 148;   // CTAs of the persistent kernels (ftm_set_sm_budget)
    int sm_total = 148;
    std::vector<void*> allocs;

    uint64_t steps = 0;
    uint64_t launches = 0;
    Profiler prof;
    Ctx ctx(cudaStream_t s) { return Ctx{s, &prof}; }
};

namespace {

// Makes the adapter's device current for one call and restores the caller's on the way out: a host
// thread that drives adapters on several devices need not switch devices itself.
struct DeviceGuard {
    int prev = -1;
    bool switched = false;
    explicit DeviceGuard(int want) {
        if (cudaGetDevice(&prev) == cudaSuccess && prev != want) switched = cudaSetDevice(want) == cudaSuccess;
    }
    ~DeviceGuard() {
        if (switched) cudaSetDevice(prev);
    }
    DeviceGuard(const DeviceGuard&) = delete;
    DeviceGuard& operator=(const DeviceGuard&) = delete;
};

int fail(const ftm_handle* h, int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (h)
        h->err = buf;
    else
        g_create_error = buf;
    return code;
}

int cuda_fail(const ftm_handle* h, cudaError_t e, const char* what) {
    if (e == cudaErrorMemoryAllocation)
        return fail(h, FTM_ERR_OUT_OF_MEMORY, "moe: out of device memory: %s: out of memory", what);
    return fail(h, FTM_ERR_CUDA, "moe: driver: %s: %s", what, cudaGetErrorString(e));
}

#define CU(h, call)                                       \
    do {                                                  \
        cudaError_t e__ = (call);                         \
        if (e__ != cudaSuccess) return cuda_fail(h, e__, #call); \
    } while (0)

template <typename T>
int dev_alloc(ftm_handle* h, T** out, size_t count) {
    void* p = nullptr;
    size_t bytes = (count ? count : 1) * sizeof(T);
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) return cuda_fail(h, e, "cudaMalloc(scratch)");
    h->allocs.push_back(p);
    *out = reinterpret_cast<T*>(p);
    return FTM_OK;
}

void free_banks(ftm_handle* h) {
    for (int b = 0; b < FTM_NUM_BANKS; b++) {
        if (h->banks[b]) cudaFree(h->banks[b]);
        h->banks[b] = nullptr;
    }
    for (int q = 0; q < 2; q++) {
        if (h->scale_frag[q]) cudaFree(h->scale_frag[q]);
        h->scale_frag[q] = nullptr;
    }
}

int alloc_banks(ftm_handle* h) {
    for (int b = 0; b < FTM_NUM_BANKS; b++) {
        size_t bytes = h->row_bytes[b] * (size_t)h->cfg.slots;
        cudaError_t e = cudaMalloc(&h->banks[b], bytes);
        if (e != cudaSuccess) {
            for (int q = 0; q < b; q++) {
                cudaFree(h->banks[q]);
                h->banks[q] = nullptr;
            }
            h->banks[b] = nullptr;
            return cuda_fail(h, e, "cudaMalloc(expert bank)");
        }
    }
    // fragment-ordered scale copies (11 % more device memory) for the shapes the decode kernels take
    if (h->cfg.hidden % 512 == 0 && h->cfg.inter % 512 == 0) {
        for (int q = 0; q < 2; q++) {
            cudaError_t e = cudaMalloc(&h->scale_frag[q], h->row_bytes[q ? 4 : 1] * (size_t)h->cfg.slots);
            if (e != cudaSuccess) {
                free_banks(h);
                return cuda_fail(h, e, "cudaMalloc(expert scale copy)");
            }
        }
    }
    h->resident = true;
    return FTM_OK;
}

BankView bank_view(const ftm_handle* h) {
    BankView v;
    v.gu_packed = (const uint8_t*)h->banks[0];
    v.gu_scale = (const uint8_t*)h->banks[1];
    v.gu_global = (const uint16_t*)h->banks[2];
    v.dn_packed = (const uint8_t*)h->banks[3];
    v.dn_scale = (const uint8_t*)h->banks[4];
    v.dn_global = (const uint16_t*)h->banks[5];
    v.gu_scale_frag = (const uint8_t*)h->scale_frag[0];
    v.dn_scale_frag = (const uint8_t*)h->scale_frag[1];
    v.hidden = h->cfg.hidden;
    v.inter = h->cfg.inter;
    v.slots = h->cfg.slots;
    return v;
}

// (re)encodes the grouped GEMM's tensor maps; the shapes the tcgen05 path does not cover need none
void build_maps(ftm_handle* h) {
    h->maps.ok = false;
    h->maps_ext.ok = false;     // encoded on the old bank addresses
    if (!h->resident || !h->xg || !h->ic2) return;
    if (!prefill_umma_supported(h->cfg.hidden, h->cfg.inter, 1, 1, true)) return;
    prefill_build_maps(bank_view(h), h->xg, reinterpret_cast<const __half*>(h->ic2),
                       (size_t)h->cfg.max_tokens * h->cfg.top_k, &h->maps);
}

void clear_residency(ftm_handle* h) {
    std::fill(h->slot_for_id.begin(), h->slot_for_id.end(), -1);
    std::fill(h->id_of_slot.begin(), h->id_of_slot.end(), -1);
    if (h->cache) h->cache->reset();
}

cudaStream_t pick(const ftm_handle* h, void* s) { return s ? (cudaStream_t)s : h->stream; }

// the checks of check_batch (src/infrastructure/cuda_moe.rs:959-1003)
int check_tokens(const ftm_handle* h, int64_t tokens, int top_k) {
    if (top_k != h->cfg.top_k)
        return fail(h, FTM_ERR_BAD, "moe: the adapter was built for top_k %d, got %d", h->cfg.top_k, top_k);
    if (tokens <= 0) return fail(h, FTM_ERR_BAD, "moe: grouped_moe: %lld tokens", (long long)tokens);
    if (tokens > h->cfg.max_tokens)
        return fail(h, FTM_ERR_BAD, "moe: %lld tokens exceed the adapter's max_tokens %d", (long long)tokens,
                    h->cfg.max_tokens);
    if (!h->resident) return fail(h, FTM_ERR_BAD, "moe: grouped_moe while the expert banks are released");
    return FTM_OK;
}

int stage_x(ftm_handle* h, const void* x, int x_dtype, int tokens, const __nv_bfloat16** out, cudaStream_t s);

// above this many routes FTM_PATH_AUTO takes the tcgen05 grouped GEMM instead of the decode kernels
constexpr int kGroupedMinRoutes = 2048;

// routed experts -> out (routed sum only when shared == nullptr).  The routes are slot ids in
// h->route_slot, or, when `expert_ids` is set, dense expert ids of `layer` still to be mapped.
// `join`, when set, is waited on just before the pass that reads `shared`.
int run_routed(ftm_handle* h, const void* x, int x_dtype, const void* expert_ids, int ids_dtype, int layer,
               const float* weights, int tokens, const float* shared, const float* se_gate, cudaEvent_t join,
               void* out, int out_dtype, int path, cudaStream_t s, const EpReturnTo* ret = nullptr) {
    BankView b = bank_view(h);
    const int routes = tokens * h->cfg.top_k;
    // large batches (or FTM_PATH_GROUPED): the tcgen05 grouped GEMM, which also does the combine
    if ((path == FTM_PATH_GROUPED || (path == FTM_PATH_AUTO && routes > kGroupedMinRoutes)) && h->maps.ok &&
        prefill_umma_supported(h->cfg.hidden, h->cfg.inter, h->cfg.slots, h->cfg.experts, expert_ids != nullptr)) {
        PrefillScratch sc{};
        sc.route_bin = h->route_expert; sc.seg = h->seg; sc.route_idx = h->sorted_route; sc.pos_of_route = h->route_idx;
        sc.csr_scratch = h->csr_scratch; sc.csr_flag = h->flags + 3; sc.groups = h->groups; sc.n_groups = h->n_groups;
        sc.xg = h->xg; sc.row_scale = h->row_scale; sc.ic1 = h->ic2p; sc.ic2h = reinterpret_cast<__half*>(h->ic2);
        sc.row_scale2 = h->row_scale2; sc.y = h->yroute; sc.err = h->flags + 2;
        DecodeRoutes rt{expert_ids ? nullptr : h->route_slot, expert_ids, ids_dtype, layer, h->cfg.experts,
                        (int)h->slot_for_id.size(), h->d_slot_for_id, h->route_slot, h->flags + 1};
        int n = launch_prefill_umma(b, x, x_dtype, rt, weights, tokens, h->cfg.top_k, sc, h->sm_count, shared, se_gate, join,
                                    out, out_dtype, h->maps, h->ctx(s), ret);
        if (n < 0) return fail(h, FTM_ERR_CUDA, "moe: driver: cuTensorMapEncodeTiled failed");
        h->launches += n;
        return FTM_OK;
    }
    if (path != FTM_PATH_SCALAR &&
        decode_mma_supported(h->cfg.hidden, h->cfg.inter, routes, h->cfg.slots, h->cfg.experts, expert_ids != nullptr)) {
        DecodeScratch sc{h->ic2p, h->groups, h->sorted_route, h->n_groups, h->yroute, h->flags + 2,
                         h->route_expert, h->seg, h->csr_scratch, h->flags + 3};
        DecodeRoutes rt{expert_ids ? nullptr : h->route_slot, expert_ids, ids_dtype, layer, h->cfg.experts,
                        (int)h->slot_for_id.size(), h->d_slot_for_id, h->route_slot, h->flags + 1};
        h->launches += launch_decode_mma(b, x, x_dtype, rt, weights, tokens, h->cfg.top_k, sc, h->sm_count, h->ctx(s));
    } else {
        const __nv_bfloat16* xb = nullptr;
        int rc = stage_x(h, x, x_dtype, tokens, &xb, s);
        if (rc != FTM_OK) return rc;
        if (expert_ids)
            h->launches += launch_slot_rewrite(expert_ids, ids_dtype, routes, layer, h->cfg.experts, h->d_slot_for_id,
                                               (int)h->slot_for_id.size(), h->route_slot, h->route_expert,
                                               h->flags + 1, h->ctx(s));
        h->launches += launch_decode_routes(b, xb, h->route_slot, weights, tokens, h->cfg.top_k, h->ic2, h->yroute,
                                            h->ctx(s));
    }
    if (join) CU(h, cudaStreamWaitEvent(s, join, 0));
    h->launches += launch_sum_routes(h->yroute, tokens, h->cfg.top_k, h->cfg.hidden, shared, se_gate, out, out_dtype, h->ctx(s));
    return FTM_OK;
}

// activations as bf16: the caller's buffer when it already is, else a cast into scratch
int stage_x(ftm_handle* h, const void* x, int x_dtype, int tokens, const __nv_bfloat16** out, cudaStream_t s) {
    if (x_dtype == FTM_BF16) {
        *out = (const __nv_bfloat16*)x;
        return FTM_OK;
    }
    if (x_dtype != FTM_F32) return fail(h, FTM_ERR_BAD, "moe: activations cannot be dtype %d", x_dtype);
    h->launches += launch_cast_to_bf16(x, x_dtype, (size_t)tokens * h->cfg.hidden, h->x_bf16, h->ctx(s));
    *out = h->x_bf16;
    return FTM_OK;
}

}  // namespace

extern "C" {

FTM_API int ftm_abi_version(void) { return FTM_ABI_VERSION; }

FTM_API const char* ftm_last_error(const ftm_handle* h) { return h ? h->err.c_str() : g_create_error.c_str(); }

FTM_API int ftm_create(const ftm_config* c, void* stream, ftm_handle** out) {
    if (!c || !out) return fail(nullptr, FTM_ERR_BAD, "moe: null config or output");
    *out = nullptr;
    if (c->hidden <= 0 || c->inter <= 0 || c->hidden % 16 || c->inter % 16)
        return fail(nullptr, FTM_ERR_BAD, "moe: expert shapes hidden %d inter %d must be nonzero multiples of 16",
                    c->hidden, c->inter);
    if (c->slots < 1) return fail(nullptr, FTM_ERR_BAD, "moe: the slot cache needs at least one slot");
    if (c->experts < 1 || c->experts > 512 || c->layers < 1)
        return fail(nullptr, FTM_ERR_BAD, "moe: experts %d (1..512) layers %d", c->experts, c->layers);
    if (c->top_k < 1 || c->top_k > 32 || c->top_k > c->experts)
        return fail(nullptr, FTM_ERR_BAD, "moe: top_k %d for %d experts", c->top_k, c->experts);
    if (c->max_tokens < 1) return fail(nullptr, FTM_ERR_BAD, "moe: max_tokens %d", c->max_tokens);
    if (c->shared_inter < 0 || c->shared_inter % 16)
        return fail(nullptr, FTM_ERR_BAD, "moe: shared_inter %d must be a multiple of 16", c->shared_inter);
    if (c->ep_size < 1 || c->ep_rank < 0 || c->ep_rank >= c->ep_size)
        return fail(nullptr, FTM_ERR_BAD, "moe: expert-parallel rank %d of %d", c->ep_rank, c->ep_size);
    int ndev = 0;
    cudaError_t e = cudaGetDeviceCount(&ndev);
    if (e != cudaSuccess || ndev == 0)
        return fail(nullptr, FTM_ERR_CUDA, "moe: driver: no CUDA device (%s); this library has no CPU path",
                    cudaGetErrorString(e));
    if (c->ordinal < 0 || c->ordinal >= ndev)
        return fail(nullptr, FTM_ERR_BAD, "moe: device ordinal %d of %d", c->ordinal, ndev);
    DeviceGuard dg(c->ordinal);
    int cur = -1;
    e = cudaGetDevice(&cur);
    if (e != cudaSuccess || cur != c->ordinal)
        return cuda_fail(nullptr, e == cudaSuccess ? cudaErrorInvalidDevice : e, "cudaSetDevice");

    std::unique_ptr<ftm_handle> h(new ftm_handle);
    h->cfg = *c;
    h->stream = (cudaStream_t)stream;
    const size_t H = c->hidden, I = c->inter;
    h->row_bytes[0] = 2 * I * H / 2;
    h->row_bytes[1] = 2 * I * H / 16;
    h->row_bytes[2] = 2 * I * 2;
    h->row_bytes[3] = H * I / 2;
    h->row_bytes[4] = H * I / 16;
    h->row_bytes[5] = H * 2;
    int rc = alloc_banks(h.get());
    if (rc != FTM_OK) {
        g_create_error = h->err;
        return rc;
    }
    const size_t n_ids = (size_t)c->layers * c->experts;
    h->slot_for_id.assign(n_ids, -1);
    h->id_of_slot.assign(c->slots, -1);
    h->cache.reset(new ExpertCache(c->layers, c->experts, c->slots));

    const size_t T = c->max_tokens, R = T * c->top_k, SI = c->shared_inter;
    const int bins = c->experts > c->slots ? c->experts : (c->slots < 1024 ? c->slots : c->experts);
    ftm_handle* hp = h.get();
    auto A = [&](int r) {
        if (r != FTM_OK && rc == FTM_OK) rc = r;
    };
    A(dev_alloc(hp, &h->d_slot_for_id, n_ids));
    A(dev_alloc(hp, &h->x_bf16, T * H));
    A(dev_alloc(hp, &h->route_slot, R));
    A(dev_alloc(hp, &h->route_expert, R));
    A(dev_alloc(hp, &h->seg, (size_t)1024 + 1));
    A(dev_alloc(hp, &h->route_idx, R));
    A(dev_alloc(hp, &h->csr_scratch, csr_scratch_ints((int)R, 1024)));
    A(dev_alloc(hp, &h->flags, 8));
    A(dev_alloc(hp, &h->ids, R));
    A(dev_alloc(hp, &h->rweights, R));
    A(dev_alloc(hp, &h->ic2, R * I));
    A(dev_alloc(hp, &h->yroute, R * H));
    A(dev_alloc(hp, &h->logits, T * c->experts));
    A(dev_alloc(hp, &h->ic2s, T * (SI ? SI : 1)));
    A(dev_alloc(hp, &h->shared_out, T * H));
    A(dev_alloc(hp, &h->se_gate, T));
    A(dev_alloc(hp, &h->routed_f32, T * H));
    A(dev_alloc(hp, &h->xh, T * H));
    A(dev_alloc(hp, &h->tok_scale, T));
    A(dev_alloc(hp, &h->ic2p, R * 2 * I));  // also gate | up of the grouped GEMM
    A(dev_alloc(hp, &h->groups, R));
    A(dev_alloc(hp, &h->sorted_route, R));
    A(dev_alloc(hp, &h->n_groups, 1));
    A(dev_alloc(hp, &h->xg, R * H));
    A(dev_alloc(hp, &h->row_scale, R));
    A(dev_alloc(hp, &h->row_scale2, R));
    cudaDeviceGetAttribute(&h->sm_total, cudaDevAttrMultiProcessorCount, c->ordinal);
    h->sm_count = h->sm_total;
    (void)bins;
    if (rc == FTM_OK) {
        e = cudaMemset(h->d_slot_for_id, 0xff, n_ids * sizeof(int32_t));
        if (e == cudaSuccess) e = cudaMemset(h->flags, 0, 8 * sizeof(int32_t));
        if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&h->aux, cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->ev_fork, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->ev_join, cudaEventDisableTiming);
        if (e != cudaSuccess) rc = cuda_fail(hp, e, "adapter setup");
    }
    if (rc == FTM_OK) build_maps(hp);
    if (rc != FTM_OK) {
        g_create_error = h->err;
        ftm_destroy(h.release());
        return rc;
    }
    *out = h.release();
    return FTM_OK;
}

FTM_API void ftm_destroy(ftm_handle* h) {
    if (!h) return;
    DeviceGuard dg(h->cfg.ordinal);
    cudaDeviceSynchronize();
    for (void* p : h->allocs) cudaFree(p);
    free_banks(h);
    if (h->aux) cudaStreamDestroy(h->aux);
    if (h->ev_fork) cudaEventDestroy(h->ev_fork);
    if (h->ev_join) cudaEventDestroy(h->ev_join);
    delete h;
}

// ---- ExpertSlotStore ------------------------------------------------------------------------

static int load_common(ftm_handle* h, int32_t layer, int32_t expert, int32_t slot, const void* const fields[],
                       const size_t lens[], cudaMemcpyKind kind) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    if (!h->resident) return fail(h, FTM_ERR_BAD, "moe: load while the expert banks are released");
    if (layer < 0 || layer >= h->cfg.layers || expert < 0 || expert >= h->cfg.experts)
        return fail(h, FTM_ERR_MISSING, "moe: no expert bank entry L%05d expert %d", layer, expert);
    if (slot < 0 || slot >= h->cfg.slots)
        return fail(h, FTM_ERR_SLOT_OUT_OF_RANGE, "moe: slot %d out of range (capacity %d)", slot, h->cfg.slots);
    if (!fields || !lens) return fail(h, FTM_ERR_BAD, "moe: null expert fields");
    for (int b = 0; b < FTM_NUM_BANKS; b++) {
        if (!fields[b]) return fail(h, FTM_ERR_BAD, "moe: expert field %d is null", b);
        if (lens[b] != h->row_bytes[b])
            return fail(h, FTM_ERR_BAD, "moe: expert field %d has %zu bytes, the bank row is %zu", b, lens[b],
                        h->row_bytes[b]);
    }
    for (int b = 0; b < FTM_NUM_BANKS; b++) {
        uint8_t* dst = (uint8_t*)h->banks[b] + (size_t)slot * h->row_bytes[b];
        if (fields[b] == dst) continue;  // the bytes were written in place through ftm_bank_ptrs
        CU(h, cudaMemcpyAsync(dst, fields[b], lens[b], kind, h->stream));
    }
    if (h->scale_frag[0]) {
        h->launches += launch_scale_repack(bank_view(h), slot, (uint8_t*)h->scale_frag[0], (uint8_t*)h->scale_frag[1],
                                           h->ctx(h->stream));
        CU(h, cudaGetLastError());
    }
    // residency: the slot's previous occupant leaves, the expert's previous slot empties
    const int32_t id = layer * h->cfg.experts + expert;
    int32_t old_id = h->id_of_slot[slot];
    if (old_id >= 0 && old_id != id) {
        h->slot_for_id[old_id] = -1;
        CU(h, cudaMemcpyAsync(h->d_slot_for_id + old_id, &h->slot_for_id[old_id], sizeof(int32_t),
                              cudaMemcpyHostToDevice, h->stream));
    }
    int32_t old_slot = h->slot_for_id[id];
    if (old_slot >= 0 && old_slot != slot) h->id_of_slot[old_slot] = -1;
    h->id_of_slot[slot] = id;
    h->slot_for_id[id] = slot;
    CU(h, cudaMemcpyAsync(h->d_slot_for_id + id, &h->slot_for_id[id], sizeof(int32_t), cudaMemcpyHostToDevice,
                          h->stream));
    if (kind == cudaMemcpyHostToDevice) CU(h, cudaStreamSynchronize(h->stream));
    return FTM_OK;
}

FTM_API int ftm_load_expert(ftm_handle* h, int32_t layer, int32_t expert, int32_t slot,
                    const uint8_t* const host_fields[FTM_NUM_BANKS], const size_t lens[FTM_NUM_BANKS]) {
    return load_common(h, layer, expert, slot, (const void* const*)host_fields, lens, cudaMemcpyHostToDevice);
}

FTM_API int ftm_load_expert_dev(ftm_handle* h, int32_t layer, int32_t expert, int32_t slot,
                        const void* const dev_fields[FTM_NUM_BANKS], const size_t lens[FTM_NUM_BANKS]) {
    int rc = load_common(h, layer, expert, slot, dev_fields, lens, cudaMemcpyDeviceToDevice);
    // the table entry was copied from host memory that may change: make it land before returning
    if (rc == FTM_OK) cudaStreamSynchronize(h->stream);
    return rc;
}

FTM_API int ftm_slots(const ftm_handle* h) { return h ? h->cfg.slots : 0; }

FTM_API int ftm_release_banks(ftm_handle* h) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    if (!h->resident) return FTM_OK;
    CU(h, cudaDeviceSynchronize());
    free_banks(h);
    h->resident = false;
    clear_residency(h);
    CU(h, cudaMemset(h->d_slot_for_id, 0xff, h->slot_for_id.size() * sizeof(int32_t)));
    return FTM_OK;
}

FTM_API int ftm_rehydrate_banks(ftm_handle* h) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    if (h->resident) return FTM_OK;
    int rc = alloc_banks(h);
    if (rc == FTM_OK) build_maps(h);   // the banks have new addresses
    return rc;
}

FTM_API int ftm_banks_resident(const ftm_handle* h) { return h && h->resident ? 1 : 0; }

FTM_API int ftm_bank_ptrs(const ftm_handle* h, uint64_t out[FTM_NUM_BANKS]) {
    if (!h || !out) return FTM_ERR_BAD;
    if (!h->resident) return fail(h, FTM_ERR_BAD, "moe: the expert banks are released");
    for (int b = 0; b < FTM_NUM_BANKS; b++) out[b] = (uint64_t)(uintptr_t)h->banks[b];
    return FTM_OK;
}

FTM_API size_t ftm_bank_row_bytes(const ftm_handle* h, int bank) {
    return (h && bank >= 0 && bank < FTM_NUM_BANKS) ? h->row_bytes[bank] : 0;
}

FTM_API int32_t ftm_slot_of(const ftm_handle* h, int32_t layer, int32_t expert) {
    if (!h || layer < 0 || layer >= h->cfg.layers || expert < 0 || expert >= h->cfg.experts) return -1;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    return h->slot_for_id[(size_t)layer * h->cfg.experts + expert];
}

FTM_API int ftm_ensure_experts(ftm_handle* h, int32_t layer, const uint32_t* routed, size_t n, uint32_t* misses,
                       uint32_t* write_slots, int32_t* rewrites, size_t* n_miss) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    if (layer < 0 || layer >= h->cfg.layers) return fail(h, FTM_ERR_BAD, "moe: layer %d of %d", layer, h->cfg.layers);
    if ((n && !routed) || !n_miss) return fail(h, FTM_ERR_BAD, "moe: null routed ids");
    for (size_t i = 0; i < n; i++)
        if (routed[i] >= (uint32_t)h->cfg.experts)
            return fail(h, FTM_ERR_BAD, "moe: routed expert %u of %d", routed[i], h->cfg.experts);
    ExpertPlan p = h->cache->ensure_experts((size_t)layer, routed, n);
    *n_miss = p.misses.size();
    for (size_t i = 0; i < p.misses.size(); i++) {
        if (misses) misses[i] = p.misses[i];
        if (write_slots) write_slots[i] = p.write_slots[i];
    }
    if (rewrites)
        for (size_t i = 0; i < n; i++) rewrites[i] = p.rewrites[i];
    return FTM_OK;
}

// ---- router ---------------------------------------------------------------------------------

FTM_API int ftm_router_from_logits(ftm_handle* h, const float* logits, int32_t tokens, int32_t* ids_out,
                           float* weights_out, void* stream) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    if (!logits || !ids_out || !weights_out) return fail(h, FTM_ERR_BAD, "moe: router: null buffer");
    if (tokens <= 0) return fail(h, FTM_ERR_BAD, "moe: router: %d tokens", tokens);
    h->launches += launch_router_topk(logits, tokens, h->cfg.experts, h->cfg.top_k, ids_out, weights_out, h->ctx(pick(h, stream)));
    CU(h, cudaGetLastError());
    return FTM_OK;
}

static int router_locked(ftm_handle* h, const void* x, const void* gate_w, int32_t tokens, int32_t* ids_out,
                         float* weights_out, cudaStream_t s) {
    if (!x || !gate_w || !ids_out || !weights_out) return fail(h, FTM_ERR_BAD, "moe: router: null buffer");
    if (tokens <= 0 || tokens > h->cfg.max_tokens)
        return fail(h, FTM_ERR_BAD, "moe: router: %d tokens (max_tokens %d)", tokens, h->cfg.max_tokens);
    if (router_fused_supported(tokens, h->cfg.experts, h->cfg.hidden, h->cfg.top_k)) {
        h->launches += launch_router_fused((const __nv_bfloat16*)x, (const __nv_bfloat16*)gate_w, tokens, h->cfg.hidden,
                                           h->cfg.top_k, ids_out, weights_out, h->ctx(s));
    } else {
        h->launches += launch_router_logits((const __nv_bfloat16*)x, (const __nv_bfloat16*)gate_w, tokens, h->cfg.experts,
                                            h->cfg.hidden, h->logits, h->ctx(s));
        h->launches += launch_router_topk(h->logits, tokens, h->cfg.experts, h->cfg.top_k, ids_out, weights_out, h->ctx(s));
    }
    CU(h, cudaGetLastError());
    return FTM_OK;
}

FTM_API int ftm_router(ftm_handle* h, const void* x_bf16, const void* gate_w_bf16, int32_t tokens, int32_t* ids_out,
               float* weights_out, void* stream) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    return router_locked(h, x_bf16, gate_w_bf16, tokens, ids_out, weights_out, pick(h, stream));
}

// ---- permutation ----------------------------------------------------------------------------

FTM_API int ftm_csr_build(ftm_handle* h, const int32_t* route_slot, int32_t routes, int32_t bins, int32_t* seg_out,
                  int32_t* route_idx_out, void* stream) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    if (!route_slot || !seg_out || !route_idx_out) return fail(h, FTM_ERR_BAD, "moe: csr: null buffer");
    if (routes <= 0 || (int64_t)routes > (int64_t)h->cfg.max_tokens * h->cfg.top_k)
        return fail(h, FTM_ERR_BAD, "moe: csr: %d routes (cap %lld)", routes,
                    (long long)h->cfg.max_tokens * h->cfg.top_k);
    if (bins < 1 || bins > 1024) return fail(h, FTM_ERR_BAD, "moe: csr: %d bins (1..1024)", bins);
    cudaStream_t s = pick(h, stream);
    CU(h, cudaMemsetAsync(h->flags, 0, sizeof(int32_t), s));
    h->launches += launch_csr_build(route_slot, routes, bins, seg_out, route_idx_out, h->csr_scratch, h->flags, h->ctx(s));
    CU(h, cudaGetLastError());
    return FTM_OK;
}

FTM_API int ftm_csr_bad(ftm_handle* h, void* stream, int32_t* bad_out) {
    if (!h || !bad_out) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    cudaStream_t s = pick(h, stream);
    CU(h, cudaMemcpyAsync(bad_out, h->flags, sizeof(int32_t), cudaMemcpyDeviceToHost, s));
    CU(h, cudaStreamSynchronize(s));
    return FTM_OK;
}

// ---- ExpertGemm -----------------------------------------------------------------------------

static int check_host_routes(const ftm_handle* h, const int32_t* routes, size_t n) {
    for (size_t i = 0; i < n; i++)
        if (routes[i] >= h->cfg.slots)
            return fail(h, FTM_ERR_SLOT_OUT_OF_RANGE, "moe: slot %d out of range (capacity %d)", routes[i],
                        h->cfg.slots);
    return FTM_OK;
}

FTM_API int ftm_grouped_moe_host(ftm_handle* h, const float* x, size_t x_len, int32_t top_k, const int32_t* routes,
                         size_t routes_len, const float* weights, size_t weights_len, float* out, size_t out_len) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    if (!x || !routes || !weights || !out) return fail(h, FTM_ERR_BAD, "moe: grouped_moe: null buffer");
    const size_t H = h->cfg.hidden;
    if (x_len == 0 || x_len % H) return fail(h, FTM_ERR_BAD, "moe: grouped_moe: %zu activations for hidden %zu", x_len, H);
    const size_t tokens = x_len / H;
    int rc = check_tokens(h, (int64_t)tokens, top_k);
    if (rc != FTM_OK) return rc;
    const size_t R = tokens * top_k;
    if (routes_len != R || weights_len < R)
        return fail(h, FTM_ERR_BAD, "moe: grouped_moe: %zu routes and %zu weights for %zu tokens x top_k %d",
                    routes_len, weights_len, tokens, top_k);
    if (out_len < tokens * H) return fail(h, FTM_ERR_BAD, "moe: grouped_moe: out holds %zu, needs %zu", out_len, tokens * H);
    if ((rc = check_host_routes(h, routes, R)) != FTM_OK) return rc;
    cudaStream_t s = h->stream;
    // narrow to bf16 on the host, as the reference adapter does before its upload
    std::vector<uint16_t> xb(x_len);
    for (size_t i = 0; i < x_len; i++) xb[i] = ftm_f32_to_bf16_bits(x[i]);
    CU(h, cudaMemcpyAsync(h->x_bf16, xb.data(), x_len * 2, cudaMemcpyHostToDevice, s));
    CU(h, cudaMemcpyAsync(h->route_slot, routes, R * sizeof(int32_t), cudaMemcpyHostToDevice, s));
    CU(h, cudaMemcpyAsync(h->rweights, weights, R * sizeof(float), cudaMemcpyHostToDevice, s));
    rc = run_routed(h, h->x_bf16, FTM_BF16, nullptr, 0, 0, h->rweights, (int)tokens, nullptr, nullptr, nullptr,
                    h->routed_f32, FTM_F32, FTM_PATH_AUTO, s);
    if (rc != FTM_OK) return rc;
    CU(h, cudaGetLastError());
    CU(h, cudaMemcpyAsync(out, h->routed_f32, tokens * H * sizeof(float), cudaMemcpyDeviceToHost, s));
    CU(h, cudaStreamSynchronize(s));
    h->steps++;
    return FTM_OK;
}

FTM_API int ftm_grouped_moe_dev(ftm_handle* h, const void* x, int x_dtype, int32_t tokens, int32_t top_k,
                        const int32_t* routes_host, size_t routes_len, const float* weights_dev, void* out,
                        int out_dtype, void* stream) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    if (!x || !routes_host || !weights_dev || !out) return fail(h, FTM_ERR_BAD, "moe: grouped_moe_dev: null buffer");
    int rc = check_tokens(h, tokens, top_k);
    if (rc != FTM_OK) return rc;
    const size_t R = (size_t)tokens * top_k;
    if (routes_len != R)
        return fail(h, FTM_ERR_BAD, "moe: grouped_moe: %zu routes for %d tokens x top_k %d", routes_len, tokens, top_k);
    if (out_dtype != FTM_BF16 && out_dtype != FTM_F32) return fail(h, FTM_ERR_BAD, "moe: out cannot be dtype %d", out_dtype);
    if ((rc = check_host_routes(h, routes_host, R)) != FTM_OK) return rc;
    cudaStream_t s = pick(h, stream);
    if (x_dtype != FTM_BF16 && x_dtype != FTM_F32) return fail(h, FTM_ERR_BAD, "moe: activations cannot be dtype %d", x_dtype);
    CU(h, cudaMemcpyAsync(h->route_slot, routes_host, R * sizeof(int32_t), cudaMemcpyHostToDevice, s));
    rc = run_routed(h, x, x_dtype, nullptr, 0, 0, weights_dev, tokens, nullptr, nullptr, nullptr, out, out_dtype,
                    FTM_PATH_AUTO, s);
    if (rc != FTM_OK) return rc;
    CU(h, cudaGetLastError());
    h->steps++;
    return FTM_OK;
}

static int staged_locked(ftm_handle* h, int32_t layer, const void* x, int x_dtype, const void* expert_ids,
                         int ids_dtype, const float* weights, int32_t tokens, const float* shared,
                         const float* se_gate, cudaEvent_t join, void* out, int out_dtype, int path,
                         cudaStream_t s) {
    if (!x || !expert_ids || !weights || !out) return fail(h, FTM_ERR_BAD, "moe: grouped_moe_staged: null buffer");
    if (layer < 0 || layer >= h->cfg.layers) return fail(h, FTM_ERR_BAD, "moe: layer %d of %d", layer, h->cfg.layers);
    int rc = check_tokens(h, tokens, h->cfg.top_k);
    if (rc != FTM_OK) return rc;
    if (ids_dtype != FTM_I32 && ids_dtype != FTM_I64 && ids_dtype != FTM_F32)
        return fail(h, FTM_ERR_BAD, "moe: expert ids cannot be dtype %d", ids_dtype);
    if (out_dtype != FTM_BF16 && out_dtype != FTM_F32) return fail(h, FTM_ERR_BAD, "moe: out cannot be dtype %d", out_dtype);
    if (path < FTM_PATH_AUTO || path > FTM_PATH_SCALAR) return fail(h, FTM_ERR_BAD, "moe: unknown path %d", path);
    if (x_dtype != FTM_BF16 && x_dtype != FTM_F32) return fail(h, FTM_ERR_BAD, "moe: activations cannot be dtype %d", x_dtype);
    // the adapter keeps its own copy of the ids, rewritten to slots through the residency table
    rc = run_routed(h, x, x_dtype, expert_ids, ids_dtype, layer, weights, tokens, shared, se_gate, join, out,
                    out_dtype, path, s);
    if (rc != FTM_OK) return rc;
    CU(h, cudaGetLastError());
    h->steps++;
    return FTM_OK;
}

FTM_API int ftm_moe_layer_staged(ftm_handle* h, int32_t layer, const void* x, int x_dtype, const void* expert_ids,
                         int ids_dtype, const float* weights, int32_t tokens, void* out, int out_dtype, int path,
                         void* stream) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    return staged_locked(h, layer, x, x_dtype, expert_ids, ids_dtype, weights, tokens, nullptr, nullptr, nullptr,
                         out, out_dtype, path, pick(h, stream));
}

FTM_API int ftm_moe_begin(ftm_handle* h, int32_t, const void*, int, const void*, int, const float*, int32_t, void*) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    return fail(h, FTM_ERR_NOT_SUPPORTED,
                "moe: no overlapped path: every expert is resident, call ftm_moe_layer_staged");
}

FTM_API int ftm_moe_finish(ftm_handle* h, void*, int, void*) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    return fail(h, FTM_ERR_NOT_SUPPORTED, "moe: no pending step");
}

FTM_API size_t ftm_route_cap(const ftm_handle* h) { return h ? (size_t)h->cfg.max_tokens * h->cfg.top_k : 0; }

FTM_API int ftm_reset_staging(ftm_handle* h) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    clear_residency(h);
    CU(h, cudaMemsetAsync(h->d_slot_for_id, 0xff, h->slot_for_id.size() * sizeof(int32_t), h->stream));
    CU(h, cudaStreamSynchronize(h->stream));
    return FTM_OK;
}

FTM_API uint64_t ftm_steps(const ftm_handle* h) { return h ? h->steps : 0; }

FTM_API int ftm_sync_status(ftm_handle* h, void* stream) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    cudaStream_t s = pick(h, stream);
    int32_t f[8] = {};
    CU(h, cudaMemcpyAsync(f, h->flags, sizeof f, cudaMemcpyDeviceToHost, s));
    CU(h, cudaStreamSynchronize(s));
    if (f[2]) {
        cudaMemsetAsync(h->flags + 2, 0, sizeof(int32_t), s);
        if (f[2] == 4)
            return fail(h, FTM_ERR_BAD, "moe: an expert-parallel exchange row fell outside its buffer and was dropped; "
                                        "the step's output is invalid");
        return fail(h, FTM_ERR_CUDA, "moe: driver: a kernel gave up a bounded wait (code %d); the step's output is invalid",
                    f[2]);
    }
    if (f[1]) {
        cudaMemsetAsync(h->flags + 1, 0, sizeof(int32_t), s);
        return fail(h, FTM_ERR_BAD, "moe: an expert id was outside [0, %d)", h->cfg.experts);
    }
    return FTM_OK;
}

FTM_API int ftm_profile_enable(ftm_handle* h, int on) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    CU(h, cudaDeviceSynchronize());
    h->prof.drain();
    if (on) {
        for (int k = 0; k < K_NUM_KINDS; k++) {
            h->prof.total_ms[k] = 0;
            h->prof.count[k] = 0;
        }
    }
    h->prof.on = on != 0;
    return FTM_OK;
}

FTM_API int ftm_profile_read(ftm_handle* h, int kind, double* total_ms, uint64_t* launches) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    if (kind < 0 || kind >= K_NUM_KINDS) return fail(h, FTM_ERR_BAD, "moe: profile kind %d", kind);
    CU(h, cudaDeviceSynchronize());
    h->prof.drain();
    if (total_ms) *total_ms = h->prof.total_ms[kind];
    if (launches) *launches = h->prof.count[kind];
    return FTM_OK;
}

FTM_API const char* ftm_profile_kind_name(int kind) {
    return (kind >= 0 && kind < K_NUM_KINDS) ? kKindNames[kind] : nullptr;
}
FTM_API int ftm_set_sm_budget(ftm_handle* h, int32_t sms) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    if (sms < 0 || sms > h->sm_total) return fail(h, FTM_ERR_BAD, "moe: sm budget %d of %d SMs", sms, h->sm_total);
    h->sm_count = sms ? sms : h->sm_total;
    return FTM_OK;
}

FTM_API uint64_t ftm_kernel_launches(const ftm_handle* h) { return h ? h->launches : 0; }

// ---- expert-parallel dispatch / combine -------------------------------------------------------

FTM_API int ftm_ep_pack(ftm_handle* h, const void* x_bf16, const int32_t* ids, const float* weights, int32_t tokens,
                        int32_t ep_size, void* send_x, int32_t* send_expert, float* send_weight, int32_t* route_idx,
                        int32_t* counts, void* stream) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    if (!x_bf16 || !ids || !weights || !send_x || !send_expert || !send_weight || !route_idx || !counts)
        return fail(h, FTM_ERR_BAD, "moe: ep_pack: null buffer");
    if (tokens <= 0 || tokens > h->cfg.max_tokens)
        return fail(h, FTM_ERR_BAD, "moe: ep_pack: %d tokens (max_tokens %d)", tokens, h->cfg.max_tokens);
    if (ep_size < 1 || ep_size > 32 || h->cfg.experts % ep_size)
        return fail(h, FTM_ERR_BAD, "moe: ep_pack: %d experts do not split over %d ranks", h->cfg.experts, ep_size);
    cudaStream_t s = pick(h, stream);
    const int routes = tokens * h->cfg.top_k;
    CU(h, cudaMemsetAsync(h->flags + 1, 0, sizeof(int32_t), s));
    // positions the permutation build leaves unwritten (a route whose expert id is out of range) read as -1
    CU(h, cudaMemsetAsync(route_idx, 0xff, (size_t)routes * sizeof(int32_t), s));
    h->launches += launch_csr_build(ids, routes, h->cfg.experts, h->seg, route_idx, h->csr_scratch, h->flags + 1, h->ctx(s));
    h->launches += launch_ep_pack((const __nv_bfloat16*)x_bf16, ids, weights, route_idx, h->seg, tokens, h->cfg.top_k,
                                  h->cfg.hidden, h->cfg.experts, ep_size, (__nv_bfloat16*)send_x, send_expert,
                                  send_weight, counts, h->ctx(s));
    CU(h, cudaGetLastError());
    return FTM_OK;
}

FTM_API int ftm_ep_plan(ftm_handle* h, const int32_t* ids, int32_t tokens, int32_t ep_size, int32_t* route_idx,
                        int32_t* counts, void* stream) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    if (!ids || !route_idx || !counts) return fail(h, FTM_ERR_BAD, "moe: ep_plan: null buffer");
    if (tokens <= 0 || tokens > h->cfg.max_tokens)
        return fail(h, FTM_ERR_BAD, "moe: ep_plan: %d tokens (max_tokens %d)", tokens, h->cfg.max_tokens);
    if (ep_size < 1 || ep_size > 32 || h->cfg.experts % ep_size)
        return fail(h, FTM_ERR_BAD, "moe: ep_plan: %d experts do not split over %d ranks", h->cfg.experts, ep_size);
    cudaStream_t s = pick(h, stream);
    const int routes = tokens * h->cfg.top_k;
    CU(h, cudaMemsetAsync(h->flags + 1, 0, sizeof(int32_t), s));
    // positions the permutation build leaves unwritten (a route whose expert id is out of range) read as -1
    CU(h, cudaMemsetAsync(route_idx, 0xff, (size_t)routes * sizeof(int32_t), s));
    h->launches += launch_csr_build(ids, routes, h->cfg.experts, h->seg, route_idx, h->csr_scratch, h->flags + 1, h->ctx(s));
    h->launches += launch_ep_counts(h->seg, h->cfg.experts, ep_size, counts, h->ctx(s));
    CU(h, cudaGetLastError());
    return FTM_OK;
}

FTM_API int ftm_ep_dispatch(ftm_handle* h, const void* x_bf16, const int32_t* ids, const float* weights,
                            const int32_t* route_idx, int32_t tokens, int32_t ep_size, int32_t ep_rank,
                            const int32_t* counts_all, const uint64_t* peer_x, const uint64_t* peer_meta,
                            int64_t capacity_rows, void* stream) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    if (!x_bf16 || !ids || !weights || !route_idx || !counts_all || !peer_x || !peer_meta)
        return fail(h, FTM_ERR_BAD, "moe: ep_dispatch: null buffer");
    if (tokens <= 0 || tokens > h->cfg.max_tokens)
        return fail(h, FTM_ERR_BAD, "moe: ep_dispatch: %d tokens (max_tokens %d)", tokens, h->cfg.max_tokens);
    if (ep_size < 1 || ep_size > 32 || h->cfg.experts % ep_size || ep_rank < 0 || ep_rank >= ep_size || capacity_rows < 1)
        return fail(h, FTM_ERR_BAD, "moe: ep_dispatch: rank %d of %d, capacity %lld", ep_rank, ep_size, (long long)capacity_rows);
    h->launches += launch_ep_dispatch((const __nv_bfloat16*)x_bf16, ids, weights, route_idx, h->seg, tokens, h->cfg.top_k,
                                      h->cfg.hidden, h->cfg.experts, ep_size, ep_rank, counts_all, peer_x, peer_meta,
                                      capacity_rows, h->flags + 2, h->ctx(pick(h, stream)));
    CU(h, cudaGetLastError());
    return FTM_OK;
}

FTM_API int ftm_ep_return(ftm_handle* h, const void* y_bf16, int32_t rows, int32_t ep_size, int32_t ep_rank,
                          const int32_t* counts_all, const uint64_t* peer_back, int64_t capacity_rows, void* stream) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    if (!y_bf16 || !counts_all || !peer_back) return fail(h, FTM_ERR_BAD, "moe: ep_return: null buffer");
    if (rows < 0 || ep_size < 1 || ep_size > 32 || ep_rank < 0 || ep_rank >= ep_size || capacity_rows < 1)
        return fail(h, FTM_ERR_BAD, "moe: ep_return: %d rows, rank %d of %d", rows, ep_rank, ep_size);
    if (rows == 0) return FTM_OK;
    h->launches += launch_ep_return((const __nv_bfloat16*)y_bf16, nullptr, nullptr, rows, h->cfg.hidden, ep_size, ep_rank, counts_all, peer_back,
                                    capacity_rows, h->flags + 2, h->ctx(pick(h, stream)));
    CU(h, cudaGetLastError());
    return FTM_OK;
}

FTM_API int ftm_ep_experts_sorted(ftm_handle* h, int32_t layer, const void* x_bf16, const int32_t* expert_ids,
                                  const float* weights, int32_t rows, void* stream) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    if (!x_bf16 || !expert_ids || !weights) return fail(h, FTM_ERR_BAD, "moe: ep_experts_sorted: null buffer");
    if (layer < 0 || layer >= h->cfg.layers) return fail(h, FTM_ERR_BAD, "moe: layer %d of %d", layer, h->cfg.layers);
    if (h->cfg.top_k != 1)
        return fail(h, FTM_ERR_BAD, "moe: ep_experts_sorted needs an owner adapter (top_k 1), this one has top_k %d", h->cfg.top_k);
    int rc = check_tokens(h, rows, 1);
    if (rc != FTM_OK) return rc;
    // only the grouped GEMM leaves its rows sorted; small steps take the ordinary call and ftm_ep_return
    if (rows <= kGroupedMinRoutes || !h->maps.ok ||
        !prefill_umma_supported(h->cfg.hidden, h->cfg.inter, h->cfg.slots, h->cfg.experts, true))
        return fail(h, FTM_ERR_NOT_SUPPORTED, "moe: ep_experts_sorted: %d rows take the ordinary staged call", rows);
    rc = run_routed(h, x_bf16, FTM_BF16, expert_ids, FTM_I32, layer, weights, rows, nullptr, nullptr, nullptr, nullptr,
                    FTM_BF16, FTM_PATH_GROUPED, pick(h, stream));
    if (rc != FTM_OK) return rc;
    CU(h, cudaGetLastError());
    h->steps++;
    return FTM_OK;
}

FTM_API int ftm_ep_experts_return(ftm_handle* h, int32_t layer, const void* x_bf16, const int32_t* expert_ids,
                                  const float* weights, int32_t rows, int32_t ep_size, int32_t ep_rank,
                                  const int32_t* counts_all, const uint64_t* peer_back, int64_t capacity_rows,
                                  void* stream) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    if (!x_bf16 || !expert_ids || !weights || !counts_all || !peer_back)
        return fail(h, FTM_ERR_BAD, "moe: ep_experts_return: null buffer");
    if (layer < 0 || layer >= h->cfg.layers) return fail(h, FTM_ERR_BAD, "moe: layer %d of %d", layer, h->cfg.layers);
    if (h->cfg.top_k != 1)
        return fail(h, FTM_ERR_BAD, "moe: ep_experts_return needs an owner adapter (top_k 1), this one has top_k %d", h->cfg.top_k);
    if (ep_size < 1 || ep_size > 32 || ep_rank < 0 || ep_rank >= ep_size || capacity_rows < 1)
        return fail(h, FTM_ERR_BAD, "moe: ep_experts_return: rank %d of %d, capacity %lld", ep_rank, ep_size, (long long)capacity_rows);
    int rc = check_tokens(h, rows, 1);
    if (rc != FTM_OK) return rc;
    // only the grouped GEMM's epilogue stores to the source ranks; small steps take the ordinary call and ftm_ep_return
    if (rows <= kGroupedMinRoutes || !h->maps.ok ||
        !prefill_umma_supported(h->cfg.hidden, h->cfg.inter, h->cfg.slots, h->cfg.experts, true))
        return fail(h, FTM_ERR_NOT_SUPPORTED, "moe: ep_experts_return: %d rows take the ordinary staged call", rows);
    EpReturnTo ret{ep_size, ep_rank, counts_all, peer_back, (long long)capacity_rows};
    rc = run_routed(h, x_bf16, FTM_BF16, expert_ids, FTM_I32, layer, weights, rows, nullptr, nullptr, nullptr, nullptr,
                    FTM_BF16, FTM_PATH_GROUPED, pick(h, stream), &ret);
    if (rc != FTM_OK) return rc;
    CU(h, cudaGetLastError());
    h->steps++;
    return FTM_OK;
}

FTM_API int ftm_ep_plan_seg(ftm_handle* h, const int32_t* ids, int32_t tokens, int32_t* route_idx, int32_t* seg_out,
                            void* stream) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    if (!ids || !route_idx || !seg_out) return fail(h, FTM_ERR_BAD, "moe: ep_plan_seg: null buffer");
    if (tokens <= 0 || tokens > h->cfg.max_tokens)
        return fail(h, FTM_ERR_BAD, "moe: ep_plan_seg: %d tokens (max_tokens %d)", tokens, h->cfg.max_tokens);
    cudaStream_t s = pick(h, stream);
    const int routes = tokens * h->cfg.top_k;
    CU(h, cudaMemsetAsync(h->flags + 1, 0, sizeof(int32_t), s));
    // positions the permutation build leaves unwritten (a route whose expert id is out of range) read as -1
    CU(h, cudaMemsetAsync(route_idx, 0xff, (size_t)routes * sizeof(int32_t), s));
    h->launches += launch_csr_build(ids, routes, h->cfg.experts, h->seg, route_idx, h->csr_scratch, h->flags + 1, h->ctx(s));
    CU(h, cudaMemcpyAsync(seg_out, h->seg, (size_t)(h->cfg.experts + 1) * sizeof(int32_t), cudaMemcpyDeviceToDevice, s));
    CU(h, cudaGetLastError());
    return FTM_OK;
}

FTM_API int ftm_ep_dispatch_sorted(ftm_handle* h, const void* x_bf16, const int32_t* ids, const float* weights,
                                   const int32_t* route_idx, int32_t tokens, int32_t ep_size, int32_t ep_rank,
                                   const int32_t* seg_all, const uint64_t* peer_xg, const uint64_t* peer_weight,
                                   const uint64_t* peer_row_scale, int64_t capacity_rows, void* stream) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    if (!x_bf16 || !ids || !weights || !route_idx || !seg_all || !peer_xg || !peer_weight || !peer_row_scale)
        return fail(h, FTM_ERR_BAD, "moe: ep_dispatch_sorted: null buffer");
    if (tokens <= 0 || tokens > h->cfg.max_tokens)
        return fail(h, FTM_ERR_BAD, "moe: ep_dispatch_sorted: %d tokens (max_tokens %d)", tokens, h->cfg.max_tokens);
    if (ep_size < 1 || ep_size > 32 || h->cfg.experts % ep_size || ep_rank < 0 || ep_rank >= ep_size || capacity_rows < 1)
        return fail(h, FTM_ERR_BAD, "moe: ep_dispatch_sorted: rank %d of %d, capacity %lld", ep_rank, ep_size, (long long)capacity_rows);
    if (h->cfg.hidden != 2048)
        return fail(h, FTM_ERR_NOT_SUPPORTED, "moe: ep_dispatch_sorted is built for hidden 2048, this adapter has %d", h->cfg.hidden);
    h->launches += launch_ep_dispatch_sorted((const __nv_bfloat16*)x_bf16, ids, weights, route_idx, seg_all, tokens, h->cfg.top_k,
                                             h->cfg.experts, ep_size, ep_rank, peer_xg, peer_weight, peer_row_scale,
                                             capacity_rows, h->flags + 2, h->ctx(pick(h, stream)));
    CU(h, cudaGetLastError());
    return FTM_OK;
}

FTM_API int ftm_ep_experts_presorted(ftm_handle* h, int32_t layer, const void* xg_f16, const float* weights,
                                     const float* row_scale, int32_t rows, int64_t xg_capacity_rows, int32_t ep_size,
                                     int32_t ep_rank, const int32_t* seg_all, const uint64_t* peer_back,
                                     int64_t back_capacity_rows, void* stream) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    if (!xg_f16 || !weights || !row_scale || !seg_all || !peer_back)
        return fail(h, FTM_ERR_BAD, "moe: ep_experts_presorted: null buffer");
    if (layer < 0 || layer >= h->cfg.layers) return fail(h, FTM_ERR_BAD, "moe: layer %d of %d", layer, h->cfg.layers);
    if (h->cfg.top_k != 1)
        return fail(h, FTM_ERR_BAD, "moe: ep_experts_presorted needs an owner adapter (top_k 1), this one has top_k %d", h->cfg.top_k);
    if (ep_size < 1 || ep_size > 32 || h->cfg.experts % ep_size || ep_rank < 0 || ep_rank >= ep_size || back_capacity_rows < 1 ||
        xg_capacity_rows < rows)
        return fail(h, FTM_ERR_BAD, "moe: ep_experts_presorted: rank %d of %d, %d rows in a matrix of %lld", ep_rank, ep_size, rows,
                    (long long)xg_capacity_rows);
    int rc = check_tokens(h, rows, 1);
    if (rc != FTM_OK) return rc;
    if (!h->maps.ok || !prefill_umma_supported(h->cfg.hidden, h->cfg.inter, h->cfg.slots, h->cfg.experts, true))
        return fail(h, FTM_ERR_NOT_SUPPORTED, "moe: ep_experts_presorted needs the grouped GEMM (hidden 2048, inter 512)");
    if ((reinterpret_cast<uintptr_t>(xg_f16) & 127) != 0)
        return fail(h, FTM_ERR_BAD, "moe: ep_experts_presorted: the activation matrix must be 128-byte aligned");
    // the activation maps follow the caller's matrix; its address does not change between steps
    if (h->maps_ext_xg != xg_f16 || h->maps_ext_rows != xg_capacity_rows || !h->maps_ext.ok) {
        if (!prefill_build_maps(bank_view(h), (const __half*)xg_f16, reinterpret_cast<const __half*>(h->ic2), (size_t)xg_capacity_rows,
                                &h->maps_ext))
            return fail(h, FTM_ERR_CUDA, "moe: driver: cuTensorMapEncodeTiled failed");
        h->maps_ext_xg = xg_f16;
        h->maps_ext_rows = xg_capacity_rows;
    }
    PrefillScratch sc{};
    sc.seg = h->seg; sc.groups = h->groups; sc.n_groups = h->n_groups; sc.ic1 = h->ic2p;
    sc.ic2h = reinterpret_cast<__half*>(h->ic2); sc.row_scale2 = h->row_scale2; sc.y = h->yroute; sc.err = h->flags + 2;
    const int per = h->cfg.experts / ep_size;
    const int32_t* slot_of_bin = h->d_slot_for_id + (size_t)layer * h->cfg.experts + (size_t)ep_rank * per;
    EpReturnTo ret{ep_size, ep_rank, nullptr, peer_back, (long long)back_capacity_rows};
    int n = launch_prefill_umma_presorted(bank_view(h), row_scale, weights, rows, seg_all, h->cfg.experts, slot_of_bin, sc,
                                          h->sm_count, ret, h->maps_ext, h->ctx(pick(h, stream)));
    if (n < 0) return fail(h, FTM_ERR_CUDA, "moe: the grouped GEMM's tensor maps are not built");
    h->launches += n;
    CU(h, cudaGetLastError());
    h->steps++;
    return FTM_OK;
}

FTM_API int ftm_ep_return_sorted(ftm_handle* h, int32_t rows, int32_t ep_size, int32_t ep_rank, const int32_t* counts_all,
                                 const uint64_t* peer_back, int64_t capacity_rows, void* stream) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    if (!counts_all || !peer_back) return fail(h, FTM_ERR_BAD, "moe: ep_return_sorted: null buffer");
    if (rows <= 0 || rows > h->cfg.max_tokens || ep_size < 1 || ep_size > 32 || ep_rank < 0 || ep_rank >= ep_size ||
        capacity_rows < 1 || h->cfg.top_k != 1)
        return fail(h, FTM_ERR_BAD, "moe: ep_return_sorted: %d rows, rank %d of %d", rows, ep_rank, ep_size);
    // the rows ftm_ep_experts_sorted left in the adapter: y sorted by expert, the position of every received row,
    // and its slot (a row whose expert is not resident returns zeros)
    h->launches += launch_ep_return((const __nv_bfloat16*)h->yroute, h->route_idx, h->route_slot, rows, h->cfg.hidden, ep_size,
                                    ep_rank, counts_all, peer_back, capacity_rows, h->flags + 2, h->ctx(pick(h, stream)));
    CU(h, cudaGetLastError());
    return FTM_OK;
}

FTM_API int ftm_ep_combine(ftm_handle* h, const void* y, int y_dtype, const int32_t* route_idx, const float* shared,
                           const float* se_gate, int32_t tokens, void* out, int out_dtype, void* stream) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    if (!y || !route_idx || !out || (shared && !se_gate)) return fail(h, FTM_ERR_BAD, "moe: ep_combine: null buffer");
    if (tokens <= 0 || tokens > h->cfg.max_tokens)
        return fail(h, FTM_ERR_BAD, "moe: ep_combine: %d tokens (max_tokens %d)", tokens, h->cfg.max_tokens);
    if ((y_dtype != FTM_BF16 && y_dtype != FTM_F32) || (out_dtype != FTM_BF16 && out_dtype != FTM_F32))
        return fail(h, FTM_ERR_BAD, "moe: ep_combine: dtypes %d -> %d", y_dtype, out_dtype);
    h->launches += launch_ep_combine(y, y_dtype, route_idx, h->route_expert, tokens, h->cfg.top_k, h->cfg.hidden, shared,
                                     se_gate, out, out_dtype, h->ctx(pick(h, stream)));
    CU(h, cudaGetLastError());
    return FTM_OK;
}

// ---- shared expert, combine, whole block ----------------------------------------------------

static int shared_locked(ftm_handle* h, const void* x, int32_t tokens, const void* gate_up, const void* down,
                         const void* shared_gate, float* shared_out, float* se_gate_out, cudaStream_t s) {
    if (!x || !gate_up || !down || !shared_gate || !shared_out || !se_gate_out)
        return fail(h, FTM_ERR_BAD, "moe: shared expert: null buffer");
    if (h->cfg.shared_inter <= 0) return fail(h, FTM_ERR_BAD, "moe: the adapter was built without a shared expert");
    if (tokens <= 0 || tokens > h->cfg.max_tokens)
        return fail(h, FTM_ERR_BAD, "moe: shared expert: %d tokens (max_tokens %d)", tokens, h->cfg.max_tokens);
    h->launches += launch_shared_expert((const __nv_bfloat16*)x, tokens, h->cfg.hidden, h->cfg.shared_inter,
                                        (const __nv_bfloat16*)gate_up, (const __nv_bfloat16*)down,
                                        (const __nv_bfloat16*)shared_gate, h->ic2s, shared_out, se_gate_out, h->flags + 2,
                                        h->ctx(s));
    CU(h, cudaGetLastError());
    return FTM_OK;
}

FTM_API int ftm_shared_expert(ftm_handle* h, const void* x_bf16, int32_t tokens, const void* gate_up_bf16,
                      const void* down_bf16, const void* shared_gate_bf16, float* shared_out, float* se_gate_out,
                      void* stream) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    return shared_locked(h, x_bf16, tokens, gate_up_bf16, down_bf16, shared_gate_bf16, shared_out, se_gate_out,
                         pick(h, stream));
}

FTM_API int ftm_combine(ftm_handle* h, const void* routed, int routed_dtype, const float* shared, const float* se_gate,
                int32_t tokens, void* out, int out_dtype, void* stream) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    if (!routed || !shared || !se_gate || !out) return fail(h, FTM_ERR_BAD, "moe: combine: null buffer");
    if (tokens <= 0) return fail(h, FTM_ERR_BAD, "moe: combine: %d tokens", tokens);
    if ((routed_dtype != FTM_BF16 && routed_dtype != FTM_F32) || (out_dtype != FTM_BF16 && out_dtype != FTM_F32))
        return fail(h, FTM_ERR_BAD, "moe: combine: dtypes %d -> %d", routed_dtype, out_dtype);
    h->launches += launch_combine(routed, routed_dtype, shared, se_gate, tokens, h->cfg.hidden, out, out_dtype, h->ctx(pick(h, stream)));
    CU(h, cudaGetLastError());
    return FTM_OK;
}

static int block_locked(ftm_handle* h, int32_t layer, const void* x_bf16, int32_t tokens, const void* gate_w_bf16,
                        const void* sh_gate_up_bf16, const void* sh_down_bf16, const void* sh_gate_bf16, void* out,
                        int out_dtype, int32_t* ids_out, float* weights_out, int path, cudaStream_t s) {
    // shared expert on the second stream, forked from and joined back into s
    CU(h, cudaEventRecord(h->ev_fork, s));
    CU(h, cudaStreamWaitEvent(h->aux, h->ev_fork, 0));
    int rc = shared_locked(h, x_bf16, tokens, sh_gate_up_bf16, sh_down_bf16, sh_gate_bf16, h->shared_out, h->se_gate,
                           h->aux);
    CU(h, cudaEventRecord(h->ev_join, h->aux));
    if (rc != FTM_OK) {
        cudaStreamWaitEvent(s, h->ev_join, 0);
        return rc;
    }
    int32_t* ids = ids_out ? ids_out : h->ids;
    float* w = weights_out ? weights_out : h->rweights;
    rc = router_locked(h, x_bf16, gate_w_bf16, tokens, ids, w, s);
    if (rc == FTM_OK)
        rc = staged_locked(h, layer, x_bf16, FTM_BF16, ids, FTM_I32, w, tokens, h->shared_out, h->se_gate,
                           h->ev_join, out, out_dtype, path, s);
    if (rc != FTM_OK) cudaStreamWaitEvent(s, h->ev_join, 0);  // never leave the fork unjoined
    return rc;
}

FTM_API int ftm_moe_block(ftm_handle* h, int32_t layer, const void* x_bf16, int32_t tokens, const void* gate_w_bf16,
                  const void* sh_gate_up_bf16, const void* sh_down_bf16, const void* sh_gate_bf16, void* out,
                  int out_dtype, int32_t* ids_out, float* weights_out, int path, void* stream) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    cudaStream_t s = pick(h, stream);
    if (!x_bf16 || !out) return fail(h, FTM_ERR_BAD, "moe: moe_block: null buffer");
    int rc = check_tokens(h, tokens, h->cfg.top_k);
    if (rc != FTM_OK) return rc;
    return block_locked(h, layer, x_bf16, tokens, gate_w_bf16, sh_gate_up_bf16, sh_down_bf16, sh_gate_bf16, out,
                        out_dtype, ids_out, weights_out, path, s);
}

// ---- the steps either side of the block -----------------------------------------------------

static int add_rmsnorm_locked(ftm_handle* h, const void* x, const void* r, const void* w, float eps, int32_t tokens,
                              void* sum_out, void* out, cudaStream_t s) {
    if (!x || !r || !w || !sum_out || !out) return fail(h, FTM_ERR_BAD, "moe: add_rmsnorm: null buffer");
    if (tokens <= 0) return fail(h, FTM_ERR_BAD, "moe: add_rmsnorm: %d tokens", tokens);
    if (h->cfg.hidden % 8 || h->cfg.hidden > 4096)
        return fail(h, FTM_ERR_BAD, "moe: add_rmsnorm: hidden %d (a multiple of 8, at most 4096)", h->cfg.hidden);
    if (!(eps >= 0.f)) return fail(h, FTM_ERR_BAD, "moe: add_rmsnorm: eps %g", (double)eps);
    h->launches += launch_add_rmsnorm((const __nv_bfloat16*)x, (const __nv_bfloat16*)r, (const __nv_bfloat16*)w, eps, tokens,
                                      h->cfg.hidden, (__nv_bfloat16*)sum_out, (__nv_bfloat16*)out, h->ctx(s));
    CU(h, cudaGetLastError());
    return FTM_OK;
}

FTM_API int ftm_add_rmsnorm(ftm_handle* h, const void* x_bf16, const void* residual_bf16, const void* norm_w_bf16, float eps,
                            int32_t tokens, void* sum_out_bf16, void* out_bf16, void* stream) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    return add_rmsnorm_locked(h, x_bf16, residual_bf16, norm_w_bf16, eps, tokens, sum_out_bf16, out_bf16, pick(h, stream));
}

FTM_API int ftm_moe_block_prenorm(ftm_handle* h, int32_t layer, const void* attn_out_bf16, const void* residual_bf16,
                                  const void* norm_w_bf16, float eps, int32_t tokens, const void* gate_w_bf16,
                                  const void* sh_gate_up_bf16, const void* sh_down_bf16, const void* sh_gate_bf16,
                                  void* sum_out_bf16, void* h2_out_bf16, void* out, int out_dtype, int32_t* ids_out,
                                  float* weights_out, int path, void* stream) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    cudaStream_t s = pick(h, stream);
    if (!out) return fail(h, FTM_ERR_BAD, "moe: moe_block_prenorm: null buffer");
    int rc = check_tokens(h, tokens, h->cfg.top_k);
    if (rc != FTM_OK) return rc;
    // the normalised rows go to the adapter's own scratch (or to the caller's buffer when it wants them): at
    // decode sizes they never leave L2 before the router, the expert kernels and the shared expert read them
    void* h2 = h2_out_bf16 ? h2_out_bf16 : (void*)h->x_bf16;
    rc = add_rmsnorm_locked(h, attn_out_bf16, residual_bf16, norm_w_bf16, eps, tokens, sum_out_bf16, h2, s);
    if (rc != FTM_OK) return rc;
    return block_locked(h, layer, h2, tokens, gate_w_bf16, sh_gate_up_bf16, sh_down_bf16, sh_gate_bf16, out, out_dtype,
                        ids_out, weights_out, path, s);
}

// ---- dense NVFP4 GEMV of the decode tail ----------------------------------------------------

FTM_API int ftm_dense_gemv(ftm_handle* h, const void* a, int a_dtype, const void* packed_kmajor_i32, const void* scale_kmajor_u8,
                           const void* global_f16, int32_t m, int32_t n, int32_t k, float* c, void* stream) {
    if (!h) return FTM_ERR_BAD;
    std::lock_guard<std::mutex> lk(h->mu);
    DeviceGuard dg(h->cfg.ordinal);
    const char* shapes = "the dense gemv kernel was built for %s, not the shapes handed in";
    if (!a || !packed_kmajor_i32 || !scale_kmajor_u8 || !global_f16 || !c)
        return fail(h, FTM_ERR_BAD, "moe: dense gemv: null buffer");
    if (a_dtype != FTM_BF16 && a_dtype != FTM_F32) return fail(h, FTM_ERR_BAD, "moe: dense gemv: activations cannot be dtype %d", a_dtype);
    if (m <= 0 || n <= 0 || k <= 0) return fail(h, FTM_ERR_BAD, shapes, "a = [M, K] and packed = [K // 8, N]");
    if (!dense_gemv_supported(n, k))
        return fail(h, FTM_ERR_BAD, shapes, "N a multiple of 4 and K a multiple of 32 (at most 3136)");
    h->launches += launch_dense_gemv(a, a_dtype, (const uint32_t*)packed_kmajor_i32, (const uint8_t*)scale_kmajor_u8,
                                     (const uint16_t*)global_f16, m, n, k, c, h->sm_count, h->flags + 2, h->ctx(pick(h, stream)));
    CU(h, cudaGetLastError());
    return FTM_OK;
}

}  // extern "C"
