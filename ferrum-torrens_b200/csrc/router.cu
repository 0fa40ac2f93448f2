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

// One warp per token.  experts <= 32 * kMaxPerLane.
constexpr int kMaxPerLane = 16;
constexpr int kTopkWarps = 4;

__global__ void __launch_bounds__(kTopkWarps * 32)
router_topk_kernel(const float* __restrict__ logits, int tokens, int experts, int top_k,
                   int32_t* __restrict__ ids, float* __restrict__ weights) {
    extern __shared__ float es[];  // [kTopkWarps][experts]
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int t = blockIdx.x * kTopkWarps + warp;
    if (t >= tokens) return;
    float* e_row = es + warp * experts;
    const float* row = logits + (size_t)t * experts;
    const int per = (experts + 31) / 32;

    // lane owns experts lane*per .. lane*per+per-1 (contiguous, so "lowest index" is
    // "lowest lane, then lowest local position")
    float v[kMaxPerLane];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; i++) {
        int e = lane * per + i;
        v[i] = (i < per && e < experts) ? row[e] : -INFINITY;
        mx = fmaxf(mx, v[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
#pragma unroll
    for (int i = 0; i < kMaxPerLane; i++) {
        int e = lane * per + i;
        if (i < per && e < experts) {
            v[i] = ftm_expf(__fadd_rn(v[i], -mx));
            e_row[e] = v[i];
        }
    }
    __syncwarp();
    // the host sums the exponentials over e ascending; one lane repeats that order
    float sum = 0.0f;
    if (lane == 0)
        for (int e = 0; e < experts; e++) sum = __fadd_rn(sum, e_row[e]);
    sum = __shfl_sync(0xffffffffu, sum, 0);
    const float inv = __fdiv_rn(1.0f, sum);
#pragma unroll
    for (int i = 0; i < kMaxPerLane; i++) {
        int e = lane * per + i;
        v[i] = (i < per && e < experts) ? __fmul_rn(v[i], inv) : -INFINITY;
    }
    // top_k passes of (largest p, lowest index)
    float my_p = 0.0f;   // lane j keeps the j-th pick
    int my_id = 0;
    float topsum = 0.0f;
    for (int j = 0; j < top_k; j++) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < kMaxPerLane; i++) {
            if (i < per && v[i] > best) {
                best = v[i];
                best_e = lane * per + i;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ob = __shfl_xor_sync(0xffffffffu, best, o);
            int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) {
                best = ob;
                best_e = oe;
            }
        }
        topsum = __fadd_rn(topsum, best);
        if (lane == j) {
            my_p = best;
            my_id = best_e;
        }
        if (best_e / per == lane) {
#pragma unroll
            for (int i = 0; i < kMaxPerLane; i++)
                if (i == best_e - lane * per) v[i] = -INFINITY;
        }
    }
    const float inv2 = __fdiv_rn(1.0f, topsum);
    if (lane < top_k) {
        ids[(size_t)t * top_k + lane] = my_id;
        weights[(size_t)t * top_k + lane] = __fmul_rn(my_p, inv2);
    }
}

}  // namespace

int launch_router_logits(const __nv_bfloat16* x, const __nv_bfloat16* gate_w, int tokens, int experts,
                         int hidden, float* logits, const Ctx& c) {
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
        static bool attr = false;
        if (!attr) {
            cudaFuncSetAttribute(router_logits_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem);
            attr = true;
        }
        c.begin(K_ROUTER_LOGITS);
        router_logits_kernel<TT><<<grid, block, smem, c.s>>>(x, gate_w, tokens, experts, hidden, logits);
        c.end();
    }
    return 1;
}

int launch_router_topk(const float* logits, int tokens, int experts, int top_k, int32_t* ids,
                       float* weights, const Ctx& c) {
    int grid = (tokens + kTopkWarps - 1) / kTopkWarps;
    size_t smem = (size_t)kTopkWarps * experts * sizeof(float);
    c.begin(K_ROUTER_TOPK);
    router_topk_kernel<<<grid, kTopkWarps * 32, smem, c.s>>>(logits, tokens, experts, top_k, ids, weights);
    c.end();
    return 1;
}

}  // namespace ftm
