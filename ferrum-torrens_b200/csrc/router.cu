// Router: gate projection with the host path's summation order, then softmax / top-k /
// renormalise.
//
// Reference behaviour (src/models/qwen3_6/forward.rs:162-179, :721-723, :793-830):
//   logit[t,e] = sum over k = 0..H-1, left to right, of x[t,k] * w[e,k]   (f32)
//   p = exp(logit - max) * (1 / sum_e exp(..))   with the sum taken over e ascending
//   top-k by p descending, equal p to the lowest index, weights p * (1 / sum of the k).
// The selected ids must equal the host path's bit for bit, so the k-sum is kept sequential:
// a bf16 x bf16 product is exact in f32, hence fma(x, w, acc) rounds exactly like the host's
// separate multiply and add, and one thread walks one (token, expert) chain in k order.
#include <cooperative_groups.h>

#include "kernels.cuh"

namespace ftm {

namespace {

constexpr int kExpertsPerCta = 32;  // threadIdx.x
constexpr int kTokGroups = 8;       // threadIdx.y
constexpr int kChunk = 512;         // k staged per pass

// Each thread owns TT (token, expert) chains: one expert, TT tokens.
template <int TT>
__global__ void __launch_bounds__(kExpertsPerCta* kTokGroups)
router_logits_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gate_w,
                     int tokens, int experts, int hidden, float* __restrict__ logits) {
    extern __shared__ float xs[];  // [kTokGroups * TT][kChunk] f32
    const int e = blockIdx.x * kExpertsPerCta + threadIdx.x;
    const int tok0 = blockIdx.y * (kTokGroups * TT);
    const int tid = threadIdx.y * kExpertsPerCta + threadIdx.x;
    const int nthreads = kExpertsPerCta * kTokGroups;
    const bool live = e < experts;
    const uint4* wrow = reinterpret_cast<const uint4*>(gate_w + (size_t)(live ? e : 0) * hidden);

    float acc[TT];
#pragma unroll
    for (int i = 0; i < TT; i++) acc[i] = 0.0f;

    for (int k0 = 0; k0 < hidden; k0 += kChunk) {
        const int kc = min(kChunk, hidden - k0);
        __syncthreads();
        // stage x[tok0 .. tok0 + 8*TT) [k0 .. k0+kc) as f32; tokens past the end read as zero
        for (int i = tid; i < kTokGroups * TT * (kChunk / 2); i += nthreads) {
            int tl = i / (kChunk / 2), kk = (i % (kChunk / 2)) * 2;
            int t = tok0 + tl;
            float2 v = make_float2(0.f, 0.f);
            if (t < tokens && kk < kc)
                v = bf16x2_to_f32(*reinterpret_cast<const uint32_t*>(x + (size_t)t * hidden + k0 + kk));
            *reinterpret_cast<float2*>(&xs[tl * kChunk + kk]) = v;
        }
        __syncthreads();
        const float* xt = xs + (threadIdx.y * TT) * kChunk;
        uint4 wv = wrow[k0 / 8];
        for (int kk = 0; kk < kc; kk += 8) {
            uint4 cur = wv;
            if (kk + 8 < kc) wv = wrow[(k0 + kk) / 8 + 1];
            float w[8];
            float2 p;
            p = bf16x2_to_f32(cur.x); w[0] = p.x; w[1] = p.y;
            p = bf16x2_to_f32(cur.y); w[2] = p.x; w[3] = p.y;
            p = bf16x2_to_f32(cur.z); w[4] = p.x; w[5] = p.y;
            p = bf16x2_to_f32(cur.w); w[6] = p.x; w[7] = p.y;
#pragma unroll
            for (int i = 0; i < TT; i++) {
                const float4 a = *reinterpret_cast<const float4*>(&xt[i * kChunk + kk]);
                const float4 b = *reinterpret_cast<const float4*>(&xt[i * kChunk + kk + 4]);
                float s = acc[i];
                s = __fmaf_rn(a.x, w[0], s);
                s = __fmaf_rn(a.y, w[1], s);
                s = __fmaf_rn(a.z, w[2], s);
                s = __fmaf_rn(a.w, w[3], s);
                s = __fmaf_rn(b.x, w[4], s);
                s = __fmaf_rn(b.y, w[5], s);
                s = __fmaf_rn(b.z, w[6], s);
                s = __fmaf_rn(b.w, w[7], s);
                acc[i] = s;
            }
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < TT; i++) {
            int t = tok0 + threadIdx.y * TT + i;
            if (t < tokens) logits[(size_t)t * experts + e] = acc[i];
        }
    }
}

// ---- tiled variant for hidden % 256 == 0 -----------------------------------------------------
// CTA = 4 warps, tile = 32 experts x 16 tokens; lane = expert, each warp owns 4 tokens, so a thread
// walks 4 independent chains (enough to cover the FMA latency).  The gate rows stream through a
// double-buffered shared tile filled with 16-byte cp.async; the activations are widened to f32
// and stored k-major so that one broadcast 128-bit load feeds the warp's 4 tokens.
constexpr int kTileE = 32, kTileT = 16, kKC = 256;
constexpr int kWStride = kKC * 2 + 16;  // bytes per expert row in shared memory (conflict-free 128-bit reads)

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

__global__ void __launch_bounds__(128)
router_logits_tiled_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gate_w,
                           int tokens, int experts, int hidden, float* __restrict__ logits) {
    extern __shared__ __align__(16) uint8_t rsm[];
    uint8_t* const wbuf = rsm;                                                  // [2][32][kWStride]
    float* const xbuf = reinterpret_cast<float*>(rsm + 2 * kTileE * kWStride);  // [2][kKC][16]
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const int e0 = blockIdx.x * kTileE, t0 = blockIdx.y * kTileT;
    const int nchunks = hidden / kKC;
    const uint32_t wbase = (uint32_t)__cvta_generic_to_shared(wbuf);

    auto issue_w = [&](int c, int b) {
        for (int i = tid; i < kTileE * (kKC / 8); i += 128) {
            const int row = i / (kKC / 8), piece = i % (kKC / 8);
            const int e = min(e0 + row, experts - 1);
            cp_async16(wbase + b * kTileE * kWStride + row * kWStride + piece * 16,
                       gate_w + (size_t)e * hidden + c * kKC + piece * 8);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // activations: thread -> token tid % 16, 16-byte pieces tid / 16 + 8 * i
    const int xtl = tid % 16, xpc = tid / 16;
    uint4 xr[4];
    auto load_x = [&](int c) {
        const int t = t0 + xtl;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            xr[i] = make_uint4(0, 0, 0, 0);
            if (t < tokens)
                xr[i] = *reinterpret_cast<const uint4*>(x + (size_t)t * hidden + c * kKC + (xpc + 8 * i) * 8);
        }
    };
    auto store_x = [&](int b) {
        float* xs = xbuf + b * kKC * kTileT;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int k = (xpc + 8 * i) * 8;
            const uint32_t w[4] = {xr[i].x, xr[i].y, xr[i].z, xr[i].w};
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float2 v = bf16x2_to_f32(w[q]);
                xs[(k + 2 * q) * kTileT + xtl] = v.x;
                xs[(k + 2 * q + 1) * kTileT + xtl] = v.y;
            }
        }
    };

    issue_w(0, 0);
    load_x(0);
    store_x(0);
    const bool active = t0 + warp * 4 < tokens;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int c = 0; c < nchunks; c++) {
        const int b = c & 1;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        if (c + 1 < nchunks) {
            issue_w(c + 1, b ^ 1);
            load_x(c + 1);
        }
        if (active) {
            const uint32_t wrow = wbase + b * kTileE * kWStride + lane * kWStride;
            const float* xs = xbuf + b * kKC * kTileT + warp * 4;
            // operands of the next eight k are fetched while the current eight are multiplied
            uint4 wc;
            float4 xc[8];
            auto fetch = [&](int kk, uint4& wv, float4 (&xv)[8]) {
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                             : "=r"(wv.x), "=r"(wv.y), "=r"(wv.z), "=r"(wv.w)
                             : "r"(wrow + kk * 2));
#pragma unroll
                for (int q = 0; q < 8; q++) xv[q] = *reinterpret_cast<const float4*>(xs + (kk + q) * kTileT);
            };
            fetch(0, wc, xc);
#pragma unroll 2
            for (int kk = 0; kk < kKC; kk += 8) {
                uint4 wn = wc;
                float4 xn[8];
#pragma unroll
                for (int q = 0; q < 8; q++) xn[q] = xc[q];
                if (kk + 8 < kKC) fetch(kk + 8, wn, xn);
                const uint32_t ww[4] = {wc.x, wc.y, wc.z, wc.w};
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const float2 w2 = bf16x2_to_f32(ww[q]);
                    const float4 xa = xc[2 * q], xb = xc[2 * q + 1];
                    acc[0] = __fmaf_rn(xa.x, w2.x, acc[0]);
                    acc[1] = __fmaf_rn(xa.y, w2.x, acc[1]);
                    acc[2] = __fmaf_rn(xa.z, w2.x, acc[2]);
                    acc[3] = __fmaf_rn(xa.w, w2.x, acc[3]);
                    acc[0] = __fmaf_rn(xb.x, w2.y, acc[0]);
                    acc[1] = __fmaf_rn(xb.y, w2.y, acc[1]);
                    acc[2] = __fmaf_rn(xb.z, w2.y, acc[2]);
                    acc[3] = __fmaf_rn(xb.w, w2.y, acc[3]);
                }
                wc = wn;
#pragma unroll
                for (int q = 0; q < 8; q++) xc[q] = xn[q];
            }
        }
        if (c + 1 < nchunks) store_x(b ^ 1);
    }
    const int e = e0 + lane;
    if (active && e < experts) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int t = t0 + warp * 4 + i;
            if (t < tokens) logits[(size_t)t * experts + e] = acc[i];
        }
    }
}

// One warp per token; lane owns PER contiguous experts (experts <= 32 * PER), so "lowest index"
// is "lowest lane, then lowest position in the lane".
constexpr int kTopkWarps = 4;

// one warp: softmax over the row's logits, top-k by probability (ties: lowest index), renormalise.
// `row` may point to global or shared memory.
template <int PER>
__device__ __forceinline__ void warp_topk_row(const float* row, int experts, int top_k, int lane,
                                              int32_t* __restrict__ ids_row, float* __restrict__ weights_row) {
    float v[PER];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < PER; i++) {
        const int e = lane * PER + i;
        v[i] = (e < experts) ? row[e] : -INFINITY;
        mx = fmaxf(mx, v[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
#pragma unroll
    for (int i = 0; i < PER; i++)
        if (lane * PER + i < experts) v[i] = ftm_expf(__fadd_rn(v[i], -mx));
    // the host sums the exponentials over e ascending: the running sum is handed from lane to lane,
    // each adding its own experts in order
    float sum = 0.0f;
    for (int l = 0; l < 32; l++) {
        float s2 = sum;
#pragma unroll
        for (int i = 0; i < PER; i++)
            if (lane * PER + i < experts) s2 = __fadd_rn(s2, v[i]);
        sum = __shfl_sync(0xffffffffu, s2, l);
    }
    const float inv = __fdiv_rn(1.0f, sum);
    // probabilities are >= 0, so their bit patterns order like the values: one integer warp-max
    // finds the largest, one warp-min the lowest index holding it
    uint32_t pb[PER];
#pragma unroll
    for (int i = 0; i < PER; i++)
        pb[i] = (lane * PER + i < experts) ? __float_as_uint(__fmul_rn(v[i], inv)) : 0u;
    uint32_t taken = 0;  // bit i: this lane's expert i was already selected
    float my_p = 0.0f;
    int my_id = 0;
    float topsum = 0.0f;
    for (int j = 0; j < top_k; j++) {
        uint32_t best = 0;
        int best_i = -1;
#pragma unroll
        for (int i = 0; i < PER; i++) {
            const bool ok = !((taken >> i) & 1u) && (lane * PER + i < experts);
            if (ok && (best_i < 0 || pb[i] > best)) {
                best = pb[i];
                best_i = i;
            }
        }
        const uint32_t wmax = __reduce_max_sync(0xffffffffu, best_i >= 0 ? best : 0u);
        const uint32_t cand = (best_i >= 0 && best == wmax) ? (uint32_t)(lane * PER + best_i) : 0xffffffffu;
        const uint32_t win = __reduce_min_sync(0xffffffffu, cand);
        const float p = __uint_as_float(wmax);
        topsum = __fadd_rn(topsum, p);
        if (lane == j) {
            my_p = p;
            my_id = (int)win;
        }
        if ((int)(win / PER) == lane) taken |= 1u << (win % PER);
    }
    const float inv2 = __fdiv_rn(1.0f, topsum);
    if (lane < top_k) {
        ids_row[lane] = my_id;
        weights_row[lane] = __fmul_rn(my_p, inv2);
    }
}

template <int PER>
__global__ void __launch_bounds__(kTopkWarps * 32)
router_topk_kernel(const float* __restrict__ logits, int tokens, int experts, int top_k,
                   int32_t* __restrict__ ids, float* __restrict__ weights) {
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int t = blockIdx.x * kTopkWarps + warp;
    if (t >= tokens) return;
    warp_topk_row<PER>(logits + (size_t)t * experts, experts, top_k, lane, ids + (size_t)t * top_k, weights + (size_t)t * top_k);
}

// ---- fused router for decode batches: logits and top-k in one launch --------------------------
// 256 experts, hidden % 256 == 0.  A cluster of 8 CTAs covers the 256 experts of 4 tokens: CTA r computes
// the logits of experts 32r..32r+31 (lane = expert, warp = token, ONE chain per thread, so the launch has
// tokens/4 x 8 CTAs and the chain of 2048 dependent FMAs is the only long latency), stores them into the
// first CTA's shared memory (distributed shared memory), and after the cluster barrier the first CTA's four
// warps run the top-k of the four tokens.  Same arithmetic, same order as the two separate kernels.
constexpr int kFusedTok = 4, kFusedK = 256;
constexpr int kFusedWStride = kFusedK * 2 + 16;

__global__ void __cluster_dims__(8, 1, 1) __launch_bounds__(128)
router_fused_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gate_w, int tokens,
                    int hidden, int top_k, int32_t* __restrict__ ids, float* __restrict__ weights) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ __align__(16) uint8_t wbuf[2][32 * kFusedWStride];
    __shared__ __align__(16) float xbuf[2][kFusedTok][kFusedK];
    __shared__ float slog[kFusedTok][256];       // used in the cluster's first CTA
    pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const int rank = (int)cluster.block_rank();   // = blockIdx.x: experts 32 * rank ..
    const int e0 = rank * 32, t0 = blockIdx.y * kFusedTok;
    const int nchunks = hidden / kFusedK;
    const uint32_t wbase = (uint32_t)__cvta_generic_to_shared(&wbuf[0][0]);

    auto issue_w = [&](int c, int b) {
        for (int i = tid; i < 32 * (kFusedK / 8); i += 128) {
            const int row = i / (kFusedK / 8), piece = i % (kFusedK / 8);
            cp_async16(wbase + b * 32 * kFusedWStride + row * kFusedWStride + piece * 16,
                       gate_w + (size_t)(e0 + row) * hidden + c * kFusedK + piece * 8);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // activations of the chunk: thread -> token tid / 32, 8 k at lane * 8
    uint4 xr;
    auto load_x = [&](int c) {
        const int t = t0 + warp;
        xr = make_uint4(0, 0, 0, 0);
        if (t < tokens) xr = *reinterpret_cast<const uint4*>(x + (size_t)t * hidden + c * kFusedK + lane * 8);
    };
    auto store_x = [&](int b) {
        const uint32_t w[4] = {xr.x, xr.y, xr.z, xr.w};
        float* dst = &xbuf[b][warp][lane * 8];
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const float2 v = bf16x2_to_f32(w[q]);
            dst[2 * q] = v.x;
            dst[2 * q + 1] = v.y;
        }
    };
    issue_w(0, 0);
    load_x(0);
    store_x(0);
    float acc = 0.f;
    for (int c = 0; c < nchunks; c++) {
        const int b = c & 1;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        if (c + 1 < nchunks) {
            issue_w(c + 1, b ^ 1);
            load_x(c + 1);
        }
        const uint32_t wrow = wbase + b * 32 * kFusedWStride + lane * kFusedWStride;
        const float* xs = &xbuf[b][warp][0];
#pragma unroll 4
        for (int kk = 0; kk < kFusedK; kk += 8) {
            uint4 wv;
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(wv.x), "=r"(wv.y), "=r"(wv.z), "=r"(wv.w) : "r"(wrow + kk * 2));
            const float4 xa = *reinterpret_cast<const float4*>(xs + kk), xb = *reinterpret_cast<const float4*>(xs + kk + 4);
            const float2 w01 = bf16x2_to_f32(wv.x), w23 = bf16x2_to_f32(wv.y), w45 = bf16x2_to_f32(wv.z), w67 = bf16x2_to_f32(wv.w);
            acc = __fmaf_rn(xa.x, w01.x, acc);
            acc = __fmaf_rn(xa.y, w01.y, acc);
            acc = __fmaf_rn(xa.z, w23.x, acc);
            acc = __fmaf_rn(xa.w, w23.y, acc);
            acc = __fmaf_rn(xb.x, w45.x, acc);
            acc = __fmaf_rn(xb.y, w45.y, acc);
            acc = __fmaf_rn(xb.z, w67.x, acc);
            acc = __fmaf_rn(xb.w, w67.y, acc);
        }
        if (c + 1 < nchunks) store_x(b ^ 1);
    }
    // hand the logit to the cluster's first CTA
    float* remote = cluster.map_shared_rank(&slog[0][0], 0);
    remote[warp * 256 + e0 + lane] = acc;
    cluster.sync();
    if (rank == 0) {
        const int t = t0 + warp;
        if (t < tokens) warp_topk_row<8>(&slog[warp][0], 256, top_k, lane, ids + (size_t)t * top_k, weights + (size_t)t * top_k);
    }
}



// ---- wide variant for large batches --------------------------------------------------------
// CTA = 4 warps, tile = 64 experts x 32 tokens; a lane owns experts lane and lane + 32, a warp 8 tokens:
// 16 independent chains per thread and 10 shared-memory loads per 64 FMAs, so the kernel is bound by the
// FP32 pipe instead of by load issue.  Every chain still walks k in order with one fma per k.
constexpr int kBE = 64, kBT = 32, kBK = 128;
constexpr int kBWStride = kBK * 2 + 16;

__global__ void __launch_bounds__(128, 2)
router_logits_wide_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gate_w,
                          int tokens, int experts, int hidden, float* __restrict__ logits) {
    extern __shared__ __align__(16) uint8_t rsm[];
    uint8_t* const wbuf = rsm;                                               // [2][64][kBWStride]
    float* const xbuf = reinterpret_cast<float*>(rsm + 2 * kBE * kBWStride);  // [2][kBK][32]
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const int e0 = blockIdx.x * kBE, t0 = blockIdx.y * kBT;
    const int nchunks = hidden / kBK;
    const uint32_t wbase = (uint32_t)__cvta_generic_to_shared(wbuf);

    auto issue_w = [&](int c, int b) {
        for (int i = tid; i < kBE * (kBK / 8); i += 128) {
            const int row = i / (kBK / 8), piece = i % (kBK / 8);
            const int e = min(e0 + row, experts - 1);
            cp_async16(wbase + b * kBE * kBWStride + row * kBWStride + piece * 16,
                       gate_w + (size_t)e * hidden + c * kBK + piece * 8);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // activations: thread -> token lane, 16-byte pieces warp + 4 * i
    uint4 xr[4];
    auto load_x = [&](int c) {
        const int t = t0 + lane;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            xr[i] = make_uint4(0, 0, 0, 0);
            if (t < tokens) xr[i] = *reinterpret_cast<const uint4*>(x + (size_t)t * hidden + c * kBK + (warp + 4 * i) * 8);
        }
    };
    auto store_x = [&](int b) {
        float* xs = xbuf + b * kBK * kBT;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int k = (warp + 4 * i) * 8;
            const uint32_t w[4] = {xr[i].x, xr[i].y, xr[i].z, xr[i].w};
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float2 v = bf16x2_to_f32(w[q]);
                xs[(k + 2 * q) * kBT + lane] = v.x;
                xs[(k + 2 * q + 1) * kBT + lane] = v.y;
            }
        }
    };

    issue_w(0, 0);
    load_x(0);
    store_x(0);
    float acc[2][8];
#pragma unroll
    for (int i = 0; i < 8; i++) acc[0][i] = acc[1][i] = 0.f;
    for (int c = 0; c < nchunks; c++) {
        const int b = c & 1;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        if (c + 1 < nchunks) {
            issue_w(c + 1, b ^ 1);
            load_x(c + 1);
        }
        const uint32_t wrow = wbase + b * kBE * kBWStride + lane * kBWStride;
        const float* xs = xbuf + b * kBK * kBT + warp * 8;
#pragma unroll 4
        for (int kk = 0; kk < kBK; kk += 4) {
            uint2 wa, wb;
            asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(wa.x), "=r"(wa.y) : "r"(wrow + kk * 2));
            asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(wb.x), "=r"(wb.y) : "r"(wrow + 32 * kBWStride + kk * 2));
            const float2 a01 = bf16x2_to_f32(wa.x), a23 = bf16x2_to_f32(wa.y);
            const float2 b01 = bf16x2_to_f32(wb.x), b23 = bf16x2_to_f32(wb.y);
            const float wa4[4] = {a01.x, a01.y, a23.x, a23.y}, wb4[4] = {b01.x, b01.y, b23.x, b23.y};
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float4 x0 = *reinterpret_cast<const float4*>(xs + (kk + q) * kBT);
                const float4 x1 = *reinterpret_cast<const float4*>(xs + (kk + q) * kBT + 4);
                const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    acc[0][i] = __fmaf_rn(xv[i], wa4[q], acc[0][i]);
                    acc[1][i] = __fmaf_rn(xv[i], wb4[q], acc[1][i]);
                }
            }
        }
        if (c + 1 < nchunks) store_x(b ^ 1);
    }
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int e = e0 + lane + 32 * h;
        if (e < experts) {
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int t = t0 + warp * 8 + i;
                if (t < tokens) logits[(size_t)t * experts + e] = acc[h][i];
            }
        }
    }
}

// ---- big variant for batches of 4096 tokens and more -------------------------------------------
// The wide kernel reads a shared-memory wavefront per four FMAs and is bound by that pipe.  Here a lane owns
// four experts (lane, lane + 32, lane + 64, lane + 96) and a warp eight tokens: 32 independent chains per
// thread; per eight k a warp reads four 16-byte weight pieces (eight k of one expert each) and sixteen
// broadcast activation vectors for 256 FMAs, half the shared-memory traffic per FMA.  Every chain still
// walks k in order with one fma per k.  Needs enough tokens to fill the device with 32-token tiles.
constexpr int kGE = 128, kGT = 32, kGK = 64;
constexpr int kGWStride = kGK * 2 + 16;

__global__ void __launch_bounds__(128, 4)
router_logits_big_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gate_w,
                         int tokens, int experts, int hidden, float* __restrict__ logits) {
    extern __shared__ __align__(16) uint8_t rsm[];
    uint8_t* const wbuf = rsm;                                               // [2][128][kGWStride]
    float* const xbuf = reinterpret_cast<float*>(rsm + 2 * kGE * kGWStride);  // [2][kGK][32]
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const int e0 = blockIdx.x * kGE, t0 = blockIdx.y * kGT;
    const int nchunks = hidden / kGK;
    const uint32_t wbase = (uint32_t)__cvta_generic_to_shared(wbuf);

    auto issue_w = [&](int c, int b) {
        for (int i = tid; i < kGE * (kGK / 8); i += 128) {
            const int row = i / (kGK / 8), piece = i % (kGK / 8);
            const int e = min(e0 + row, experts - 1);
            cp_async16(wbase + b * kGE * kGWStride + row * kGWStride + piece * 16,
                       gate_w + (size_t)e * hidden + c * kGK + piece * 8);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // activations: thread -> token lane, 16-byte pieces warp + 4 * i
    uint4 xr[kGK / 32];
    auto load_x = [&](int c) {
        const int t = t0 + lane;
#pragma unroll
        for (int i = 0; i < kGK / 32; i++) {
            xr[i] = make_uint4(0, 0, 0, 0);
            if (t < tokens) xr[i] = *reinterpret_cast<const uint4*>(x + (size_t)t * hidden + c * kGK + (warp + 4 * i) * 8);
        }
    };
    auto store_x = [&](int b) {
        float* xs = xbuf + b * kGK * kGT;
#pragma unroll
        for (int i = 0; i < kGK / 32; i++) {
            const int k = (warp + 4 * i) * 8;
            const uint32_t w[4] = {xr[i].x, xr[i].y, xr[i].z, xr[i].w};
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float2 v = bf16x2_to_f32(w[q]);
                xs[(k + 2 * q) * kGT + lane] = v.x;
                xs[(k + 2 * q + 1) * kGT + lane] = v.y;
            }
        }
    };

    issue_w(0, 0);
    load_x(0);
    store_x(0);
    float acc[4][8];
#pragma unroll
    for (int j = 0; j < 4; j++)
#pragma unroll
        for (int i = 0; i < 8; i++) acc[j][i] = 0.f;
    for (int c = 0; c < nchunks; c++) {
        const int b = c & 1;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        if (c + 1 < nchunks) {
            issue_w(c + 1, b ^ 1);
            load_x(c + 1);
        }
        const uint32_t wrow = wbase + b * kGE * kGWStride + lane * kGWStride;
        const float* xs = xbuf + b * kGK * kGT + warp * 8;
#pragma unroll 2
        for (int kk = 0; kk < kGK; kk += 8) {
            uint4 wq[4];
#pragma unroll
            for (int j = 0; j < 4; j++)
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                             : "=r"(wq[j].x), "=r"(wq[j].y), "=r"(wq[j].z), "=r"(wq[j].w)
                             : "r"(wrow + j * 32 * kGWStride + kk * 2));
#pragma unroll
            for (int q = 0; q < 8; q++) {
                const float4 x0 = *reinterpret_cast<const float4*>(xs + (kk + q) * kGT);
                const float4 x1 = *reinterpret_cast<const float4*>(xs + (kk + q) * kGT + 4);
                const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const uint32_t pair = (q < 2) ? wq[j].x : (q < 4) ? wq[j].y : (q < 6) ? wq[j].z : wq[j].w;
                    const float wv = (q & 1) ? __uint_as_float(pair & 0xffff0000u) : __uint_as_float(pair << 16);
#pragma unroll
                    for (int i = 0; i < 8; i++) acc[j][i] = __fmaf_rn(xv[i], wv, acc[j][i]);
                }
            }
        }
        if (c + 1 < nchunks) store_x(b ^ 1);
    }
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int e = e0 + lane + 32 * j;
        if (e < experts) {
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int t = t0 + warp * 8 + i;
                if (t < tokens) logits[(size_t)t * experts + e] = acc[j][i];
            }
        }
    }
}

}  // namespace

int launch_router_logits(const __nv_bfloat16* x, const __nv_bfloat16* gate_w, int tokens, int experts,
                         int hidden, float* logits, const Ctx& c) {
    if (hidden % kGK == 0 && tokens >= 4096 && experts >= kGE) {
        dim3 grid((experts + kGE - 1) / kGE, (tokens + kGT - 1) / kGT);
        const size_t smem = 2 * kGE * kGWStride + 2 * kGK * kGT * sizeof(float);
        static PerDeviceOnce once;
        allow_dyn_smem(once, router_logits_big_kernel, smem);
        c.begin(K_ROUTER_LOGITS);
        router_logits_big_kernel<<<grid, 128, smem, c.s>>>(x, gate_w, tokens, experts, hidden, logits);
        c.end();
        return 1;
    }
    if (hidden % kBK == 0 && tokens >= 768) {      // below that the 32 x 16 tiles fill the device better
        dim3 grid((experts + kBE - 1) / kBE, (tokens + kBT - 1) / kBT);
        const size_t smem = 2 * kBE * kBWStride + 2 * kBK * kBT * sizeof(float);
        static PerDeviceOnce once;
        allow_dyn_smem(once, router_logits_wide_kernel, smem);
        c.begin(K_ROUTER_LOGITS);
        router_logits_wide_kernel<<<grid, 128, smem, c.s>>>(x, gate_w, tokens, experts, hidden, logits);
        c.end();
        return 1;
    }
    if (hidden % kKC == 0) {
        dim3 grid((experts + kTileE - 1) / kTileE, (tokens + kTileT - 1) / kTileT);
        const size_t smem = 2 * kTileE * kWStride + 2 * kKC * kTileT * sizeof(float);
        static PerDeviceOnce once;
        allow_dyn_smem(once, router_logits_tiled_kernel, smem);
        c.begin(K_ROUTER_LOGITS);
        router_logits_tiled_kernel<<<grid, 128, smem, c.s>>>(x, gate_w, tokens, experts, hidden, logits);
        c.end();
        return 1;
    }
    dim3 block(kExpertsPerCta, kTokGroups);
    int etiles = (experts + kExpertsPerCta - 1) / kExpertsPerCta;
    if (tokens <= kTokGroups) {
        dim3 grid(etiles, 1);
        size_t smem = (size_t)kTokGroups * 1 * kChunk * sizeof(float);
        c.begin(K_ROUTER_LOGITS);
        router_logits_kernel<1><<<grid, block, smem, c.s>>>(x, gate_w, tokens, experts, hidden, logits);
        c.end();
    } else {
        constexpr int TT = 4;
        dim3 grid(etiles, (tokens + kTokGroups * TT - 1) / (kTokGroups * TT));
        size_t smem = (size_t)kTokGroups * TT * kChunk * sizeof(float);
        static PerDeviceOnce once;
        allow_dyn_smem(once, router_logits_kernel<TT>, smem);
        c.begin(K_ROUTER_LOGITS);
        router_logits_kernel<TT><<<grid, block, smem, c.s>>>(x, gate_w, tokens, experts, hidden, logits);
        c.end();
    }
    return 1;
}

bool router_fused_supported(int tokens, int experts, int hidden, int top_k) {
    // measured per whole block (Zipf routing): 128 tokens 105 us fused against 115 us with the tiled kernel + top-k,
    // 256 tokens 157 against 147, 512 tokens 194 against 189: the cluster kernel re-reads the gate weight once per
    // four tokens and walks one chain per thread, which stops paying at about 200 tokens
    return experts == 256 && hidden % kFusedK == 0 && tokens < 256 && top_k <= 32;
}

int launch_router_fused(const __nv_bfloat16* x, const __nv_bfloat16* gate_w, int tokens, int hidden, int top_k,
                        int32_t* ids, float* weights, const Ctx& c) {
    dim3 grid(8, (tokens + kFusedTok - 1) / kFusedTok);
    c.begin(K_ROUTER_LOGITS);
    router_fused_kernel<<<grid, 128, 0, c.s>>>(x, gate_w, tokens, hidden, top_k, ids, weights);
    c.end();
    return 1;
}

int launch_router_topk(const float* logits, int tokens, int experts, int top_k, int32_t* ids,
                       float* weights, const Ctx& c) {
    int grid = (tokens + kTopkWarps - 1) / kTopkWarps;
    c.begin(K_ROUTER_TOPK);
    if (experts <= 256)
        router_topk_kernel<8><<<grid, kTopkWarps * 32, 0, c.s>>>(logits, tokens, experts, top_k, ids, weights);
    else
        router_topk_kernel<16><<<grid, kTopkWarps * 32, 0, c.s>>>(logits, tokens, experts, top_k, ids, weights);
    c.end();
    return 1;
}

}  // namespace ftm
