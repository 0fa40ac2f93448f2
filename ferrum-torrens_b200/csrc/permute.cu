// Token permutation for the routed experts: per-bin histogram, prefix scan, stable scatter.
//
// Reference behaviour (src/infrastructure/cuda_moe.rs:2328-2362 `build_grouped_csr_host`,
// python/ferrum_kernel/moe_prefill.py:30-89): seg[b] .. seg[b+1] indexes route_idx, which holds the
// original route ids of bin b in ascending order; a route whose bin is outside [0, bins) raises a
// device flag.  The reference scans all R routes once per bin (O(bins * R)); here every route is
// read twice in total.
//
// Layout of the work: the routes are cut into chunks of kChunkRoutes, one CTA per chunk, and each
// warp of a CTA owns a contiguous sub-range, so "ascending route id" is "CTA order, then warp
// order, then lane order".  Pass 1 counts per (CTA, bin); pass 2 (one CTA) turns the counts into
// per-(CTA, bin) start offsets; pass 3 recounts per warp and scatters with a warp-level rank.
// When everything fits one CTA the three passes run inside a single launch.
#include <mutex>

#include "../../include/ftmoe.h"
#include "kernels.cuh"

namespace ftm {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kChunkRoutes = 2048;                    // routes per CTA
constexpr int kWarpRoutes = kChunkRoutes / kWarps;    // contiguous routes per warp
constexpr int kMaxBins = 1024;

// (route_bin is not declared restrict: the counting kernel may have written this chunk's bins itself just before)
__device__ __forceinline__ void count_chunk(const int32_t* route_bin, int routes, int bins,
                                            int chunk_begin, int warp_routes, int* whist /* [kWarps][bins] smem */,
                                            int32_t* bad_flag) {
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    for (int i = threadIdx.x; i < kWarps * bins; i += kThreads) whist[i] = 0;
    __syncthreads();
    const int begin = min(chunk_begin + warp * warp_routes, routes);
    const int end = min(begin + warp_routes, routes);
    for (int r = begin + lane; r < end; r += 32) {
        int b = route_bin[r];
        if (b < 0 || b >= bins) {
            atomicExch(bad_flag, 1);
            continue;
        }
        atomicAdd(&whist[warp * bins + b], 1);
    }
    __syncthreads();
}

// stable scatter of this CTA's chunk; wbase[w][b] = first output position of warp w's routes of bin b
__device__ __forceinline__ void scatter_chunk(const int32_t* __restrict__ route_bin, int routes, int bins,
                                              int chunk_begin, int warp_routes, int* wbase, int32_t* __restrict__ route_idx,
                                              int32_t* __restrict__ pos_of_route) {
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int begin = min(chunk_begin + warp * warp_routes, routes);
    const int end = min(begin + warp_routes, routes);
    int* mine = wbase + warp * bins;
    for (int r0 = begin; r0 < end; r0 += 32) {
        int r = r0 + lane;
        int b = (r < end) ? route_bin[r] : -1;
        bool ok = b >= 0 && b < bins;
        unsigned peers = __match_any_sync(0xffffffffu, ok ? b : -1 - lane);
        if (ok) {
            int rank = __popc(peers & ((1u << lane) - 1u));
            int pos = mine[b] + rank;
            route_idx[pos] = r;
            if (pos_of_route) pos_of_route[r] = pos;      // the inverse, for callers that walk the routes in their own order
        }
        __syncwarp();
        if (ok && lane == 31 - __clz(peers)) mine[b] += __popc(peers);
        __syncwarp();
    }
}

// single-CTA build: routes <= kChunkRoutes
__global__ void __launch_bounds__(kThreads)
csr_small_kernel(const int32_t* __restrict__ route_bin, int routes, int bins, int32_t* __restrict__ seg,
                 int32_t* __restrict__ route_idx, int32_t* bad_flag, int32_t* __restrict__ pos_of_route) {
    extern __shared__ int sm[];
    int* whist = sm;                   // [kWarps][bins]
    int* binbase = sm + kWarps * bins; // [bins + 1]
    count_chunk(route_bin, routes, bins, 0, kWarpRoutes, whist, bad_flag);
    // per-bin totals, then an exclusive scan over bins by warp 0
    for (int b = threadIdx.x; b < bins; b += kThreads) {
        int tot = 0;
        for (int w = 0; w < kWarps; w++) tot += whist[w * bins + b];
        binbase[b] = tot;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        int lane = threadIdx.x, carry = 0;
        for (int b0 = 0; b0 < bins; b0 += 32) {
            int b = b0 + lane;
            int c = (b < bins) ? binbase[b] : 0;
            int incl = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                int n = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += n;
            }
            if (b < bins) {
                binbase[b] = carry + incl - c;
                seg[b] = carry + incl - c;
            }
            carry += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) seg[bins] = carry;
    }
    __syncthreads();
    // warp bases: bin start + counts of earlier warps
    for (int b = threadIdx.x; b < bins; b += kThreads) {
        int run = binbase[b];
        for (int w = 0; w < kWarps; w++) {
            int c = whist[w * bins + b];
            whist[w * bins + b] = run;
            run += c;
        }
    }
    __syncthreads();
    scatter_chunk(route_bin, routes, bins, 0, kWarpRoutes, whist, route_idx, pos_of_route);
}

// dense expert id of route r -> slot through the residency table; writes the route's slot and its bin (the expert id,
// -1 when the expert is not resident)
__device__ __forceinline__ void rewrite_route(const SlotRewrite& w, int r) {
    // ids arrive as i32, i64 or f32 (src/infrastructure/cuda_moe.rs:67-86 accepts all three)
    long long e;
    if (w.ids_dtype == 3)
        e = reinterpret_cast<const long long*>(w.expert_ids)[r];
    else if (w.ids_dtype == 1)
        e = (long long)reinterpret_cast<const float*>(w.expert_ids)[r];
    else
        e = (long long)reinterpret_cast<const int32_t*>(w.expert_ids)[r];
    int slot = -1;
    if (e >= 0 && e < w.experts) {
        long long id = (long long)w.layer * w.experts + e;
        if (id < w.n_ids) slot = w.slot_for_id[id];
    } else {
        atomicExch(w.bad_flag, 1);
    }
    w.route_slot[r] = slot;
    if (w.route_expert) w.route_expert[r] = (slot >= 0) ? (int32_t)e : -1;
}

// dense expert ids of one layer -> slot ids through the residency table
__global__ void slot_rewrite_kernel(SlotRewrite w, int routes) {
    int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < routes) rewrite_route(w, r);
}

// pass 1: per-(CTA, bin) counts -> cta_hist[cta][bin].  With `w.expert_ids` set the CTA first maps its chunk's dense
// expert ids to slots and bins (what slot_rewrite_kernel does in a launch of its own): route_bin is then w.route_expert.
__global__ void __launch_bounds__(kThreads)
csr_count_kernel(const int32_t* route_bin, int routes, int bins, int chunk, int32_t* __restrict__ cta_hist,
                 int32_t* bad_flag, SlotRewrite w) {
    extern __shared__ int sm[];
    if (w.expert_ids) {
        const int begin = blockIdx.x * chunk, end = min(begin + chunk, routes);
        for (int r = begin + threadIdx.x; r < end; r += kThreads) rewrite_route(w, r);
        __syncthreads();     // the chunk's bins are read back by this CTA only
    }
    count_chunk(route_bin, routes, bins, blockIdx.x * chunk, chunk / kWarps, sm, bad_flag);
    for (int b = threadIdx.x; b < bins; b += kThreads) {
        int tot = 0;
        for (int w = 0; w < kWarps; w++) tot += sm[w * bins + b];
        cta_hist[(size_t)blockIdx.x * bins + b] = tot;
    }
}

// pass 2 (one CTA): cta_hist[c][b] <- seg[b] + sum of counts of CTAs before c; writes seg
// With `g.groups` set the same CTA also cuts every bin into passes of at most g.group routes (what
// groups_from_csr_kernel does in a launch of its own): (slot, first sorted row, rows, 0) per pass, bins whose slot
// is not resident skipped, the number of passes in *g.n_groups.
__global__ void __launch_bounds__(kMaxBins)
csr_scan_kernel(int32_t* __restrict__ cta_hist, int nctas, int bins, int32_t* __restrict__ seg, CsrGroups g) {
    __shared__ int wsum[32];
    const int b = threadIdx.x;
    int total = 0;
    if (b < bins)
        for (int c = 0; c < nctas; c++) total += cta_hist[(size_t)c * bins + b];
    // exclusive scan over bins (block-wide: warp scan + scan of warp totals)
    const int lane = b % 32, warp = b / 32;
    int incl = (b < bins) ? total : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int n = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += n;
    }
    if (lane == 31) wsum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int v = (lane < (int)(blockDim.x / 32)) ? wsum[lane] : 0;
        int inc2 = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int n = __shfl_up_sync(0xffffffffu, inc2, o);
            if (lane >= o) inc2 += n;
        }
        wsum[lane] = inc2 - v;
    }
    __syncthreads();
    int excl = wsum[warp] + incl - ((b < bins) ? total : 0);
    if (b < bins) {
        seg[b] = excl;
        if (b == bins - 1) seg[bins] = excl + total;
        int run = excl;
        for (int c = 0; c < nctas; c++) {
            int v = cta_hist[(size_t)c * bins + b];
            cta_hist[(size_t)c * bins + b] = run;
            run += v;
        }
    }
    if (!g.groups) return;
    int cnt = 0, slot = -1;
    if (b < bins) {
        cnt = total;
        slot = g.slot_of_bin ? g.slot_of_bin[b] : b;
        if (slot < 0 || slot >= g.slots) cnt = 0;
    }
    const int ng = (cnt + g.group - 1) / g.group;
    int gi = ng;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int n = __shfl_up_sync(0xffffffffu, gi, o);
        if (lane >= o) gi += n;
    }
    __syncthreads();     // wsum is reused
    if (lane == 31) wsum[warp] = gi;
    __syncthreads();
    if (warp == 0) {
        int v = (lane < (int)(blockDim.x / 32)) ? wsum[lane] : 0;
        int j = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int n = __shfl_up_sync(0xffffffffu, j, o);
            if (lane >= o) j += n;
        }
        wsum[lane] = j - v;
        if (lane == 31) *g.n_groups = j;
    }
    __syncthreads();
    const int base = wsum[warp] + gi - ng;
    for (int q = 0; q < ng; q++) g.groups[base + q] = make_int4(slot, excl + q * g.group, min(g.group, cnt - q * g.group), 0);
}

// pass 3: recount per warp, then ranked scatter from the CTA's bases
__global__ void __launch_bounds__(kThreads)
csr_scatter_kernel(const int32_t* __restrict__ route_bin, int routes, int bins, int chunk,
                   const int32_t* __restrict__ cta_base, int32_t* __restrict__ route_idx, int32_t* scratch_flag,
                   int32_t* __restrict__ pos_of_route) {
    extern __shared__ int sm[];
    count_chunk(route_bin, routes, bins, blockIdx.x * chunk, chunk / kWarps, sm, scratch_flag);
    for (int b = threadIdx.x; b < bins; b += kThreads) {
        int run = cta_base[(size_t)blockIdx.x * bins + b];
        for (int w = 0; w < kWarps; w++) {
            int c = sm[w * bins + b];
            sm[w * bins + b] = run;
            run += c;
        }
    }
    __syncthreads();
    scatter_chunk(route_bin, routes, bins, blockIdx.x * chunk, chunk / kWarps, sm, route_idx, pos_of_route);
}

}  // namespace

// ---- permutation build without any allocation ------------------------------------------------
// Scratch of the multi-CTA build (per-CTA histograms and the out-of-range flag) for callers that
// must not allocate.  It lives in the library image: every GPU that loads the library carries these
// bytes until the process exits.
constexpr int kNoAllocMaxRoutes = 262144;                                // 128 chunks of 2048 routes
constexpr int kNoAllocMaxBins = 1024;
constexpr int kNoAllocScratchInts = (kNoAllocMaxRoutes / 2048) * kNoAllocMaxBins;  // 512 KiB
static __device__ __align__(256) int32_t g_noalloc_scratch[kNoAllocScratchInts + 64];

namespace {

// device address of g_noalloc_scratch per device ordinal, looked up once with that device current
constexpr int kMaxDevices = 64;
int32_t* g_noalloc_ptr[kMaxDevices] = {};
std::mutex g_noalloc_mu;

}  // namespace

// the adapter's builds cut the routes into chunks of kFineChunk per CTA (more CTAs in flight for the two passes
// that read every route); the allocation-free entry keeps chunks of kChunkRoutes, which its fixed scratch is sized for
constexpr int kFineChunk = 512;
size_t csr_scratch_ints(int routes, int bins) {
    size_t nctas = ((size_t)routes + kFineChunk - 1) / kFineChunk;
    return (nctas ? nctas : 1) * (size_t)bins;
}

int launch_csr_build(const int32_t* route_bin, int routes, int bins, int32_t* seg, int32_t* route_idx,
                     int32_t* scratch, int32_t* bad_flag, const Ctx& c, bool coarse, const CsrGroups* groups,
                     const SlotRewrite* rewrite) {
    if (routes <= kChunkRoutes) {
        int pre = 0;
        if (rewrite) {
            c.begin(K_SLOT_REWRITE);
            slot_rewrite_kernel<<<(routes + 255) / 256, 256, 0, c.s>>>(*rewrite, routes);
            c.end();
            pre = 1;
        }
        size_t smem = ((size_t)kWarps * bins + bins + 1) * sizeof(int);
        c.begin(K_CSR);
        csr_small_kernel<<<1, kThreads, smem, c.s>>>(route_bin, routes, bins, seg, route_idx, bad_flag,
                                                     groups ? groups->pos_of_route : nullptr);
        c.end();
        if (groups)
            return pre + 1 + launch_groups_from_csr(seg, bins, groups->slot_of_bin, groups->slots, groups->group, groups->groups,
                                              groups->n_groups, c);
        return pre + 1;
    }
    const int chunk = coarse ? kChunkRoutes : kFineChunk;
    int nctas = (routes + chunk - 1) / chunk;
    size_t smem = (size_t)kWarps * bins * sizeof(int);
    c.begin(K_CSR);
    csr_count_kernel<<<nctas, kThreads, smem, c.s>>>(route_bin, routes, bins, chunk, scratch, bad_flag,
                                                     rewrite ? *rewrite : SlotRewrite{});
    int scan_threads = ((bins + 31) / 32) * 32;
    csr_scan_kernel<<<1, scan_threads, 0, c.s>>>(scratch, nctas, bins, seg, groups ? *groups : CsrGroups{});
    csr_scatter_kernel<<<nctas, kThreads, smem, c.s>>>(route_bin, routes, bins, chunk, scratch, route_idx, bad_flag,
                                                       groups ? groups->pos_of_route : nullptr);
    c.end();
    return 3;
}

int launch_slot_rewrite(const void* expert_ids, int ids_dtype, int routes, int layer, int experts,
                        const int32_t* slot_for_id, int n_ids, int32_t* route_slot, int32_t* route_expert,
                        int32_t* bad_flag, const Ctx& c) {
    int threads = 256;
    const SlotRewrite w{expert_ids, ids_dtype, layer, experts, slot_for_id, n_ids, route_slot, route_expert, bad_flag};
    c.begin(K_SLOT_REWRITE);
    slot_rewrite_kernel<<<(routes + threads - 1) / threads, threads, 0, c.s>>>(w, routes);
    c.end();
    return 1;
}

}  // namespace ftm

// The permutation build for callers that cannot allocate device memory: an engine that runs under
// a fixed memory plan (every byte handed out at start-up, the allocator then locked), or a call site
// inside a region where allocation is forbidden.  It needs no adapter handle: the per-CTA histograms
// and the out-of-range flag live in g_noalloc_scratch above.
//
//  - Limits: routes <= 262144 and bins <= 1024 (the array's size); anything larger is refused.
//  - The first call on a device looks the array's device address up (cudaGetSymbolAddress, with that
//    device current) and keeps it; make that first call before any stream capture begins.
//  - All calls on one device share the array.  The flag is cleared at the start of every call, the
//    histograms are fully rewritten by the first pass; two calls that overlap on the GPU (different
//    streams) race on it.
//  - bad_out (device, may be NULL) receives 1 when a slot was outside [0, bins), else 0.
extern "C" FTM_API int ftm_csr_build_noalloc(const int32_t* route_slot, int32_t routes, int32_t bins,
                                             int32_t* seg_out, int32_t* route_idx_out, int32_t* bad_out,
                                             void* stream) {
    using namespace ftm;
    if (!route_slot || !seg_out || !route_idx_out) return FTM_ERR_BAD;
    if (routes <= 0 || routes > kNoAllocMaxRoutes || bins < 1 || bins > kNoAllocMaxBins) return FTM_ERR_BAD;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return FTM_ERR_CUDA;
    int32_t* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_noalloc_mu);
        if (!g_noalloc_ptr[dev]) {
            void* p = nullptr;
            if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || !p) return FTM_ERR_CUDA;
            g_noalloc_ptr[dev] = reinterpret_cast<int32_t*>(p);
        }
        scratch = g_noalloc_ptr[dev];
    }
    cudaStream_t s = (cudaStream_t)stream;
    int32_t* flag = scratch + kNoAllocScratchInts;  // the last 256 bytes of the array
    if (cudaMemsetAsync(flag, 0, sizeof(int32_t), s) != cudaSuccess) return FTM_ERR_CUDA;
    Ctx c{s, nullptr};
    launch_csr_build(route_slot, routes, bins, seg_out, route_idx_out, scratch, flag, c, /*coarse=*/true);
    if (bad_out && cudaMemcpyAsync(bad_out, flag, sizeof(int32_t), cudaMemcpyDeviceToDevice, s) != cudaSuccess)
        return FTM_ERR_CUDA;
    return cudaGetLastError() == cudaSuccess ? FTM_OK : FTM_ERR_CUDA;
}

