// Shared expert (dense bf16 SwiGLU) and its sigmoid gate.
//
// Reference behaviour (src/models/qwen3_6/forward.rs:684-714 with the bf16 projection of
// :162-179, :727-742; device form src/infrastructure/cuda_linear.rs:391-450 and
// src/models/qwen3_6/forward_cudarc.rs:1541-1561):
//   ic1 = gate_up_s x            [2*SI]
//   ic2 = silu(ic1[:SI]) * ic1[SI:]
//   shared = down_s ic2          [H]
//   se_gate = sigmoid(x . shared_gate)
// f32 accumulation throughout.
#include "kernels.cuh"

namespace ftm {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kTokTile = 8;  // tokens per CTA, activations staged in shared memory as f32

// dot of one bf16 weight row with kTokTile activation rows held in shared memory
template <int NT>
__device__ __forceinline__ void row_dots(const __nv_bfloat16* __restrict__ wrow, const float* __restrict__ xs,
                                         int K, int lane, float (&acc)[NT]) {
#pragma unroll
    for (int t = 0; t < NT; t++) acc[t] = 0.f;
    for (int k = lane * 8; k < K; k += 32 * 8) {
        uint4 wv = *reinterpret_cast<const uint4*>(wrow + k);
        float w[8];
        float2 p;
        p = bf16x2_to_f32(wv.x); w[0] = p.x; w[1] = p.y;
        p = bf16x2_to_f32(wv.y); w[2] = p.x; w[3] = p.y;
        p = bf16x2_to_f32(wv.z); w[4] = p.x; w[5] = p.y;
        p = bf16x2_to_f32(wv.w); w[6] = p.x; w[7] = p.y;
#pragma unroll
        for (int t = 0; t < NT; t++) {
            const float4 a = *reinterpret_cast<const float4*>(xs + (size_t)t * K + k);
            const float4 b = *reinterpret_cast<const float4*>(xs + (size_t)t * K + k + 4);
            acc[t] += a.x * w[0] + a.y * w[1] + a.z * w[2] + a.w * w[3] + b.x * w[4] + b.y * w[5] +
                      b.z * w[6] + b.w * w[7];
        }
    }
#pragma unroll
    for (int t = 0; t < NT; t++) acc[t] = warp_sum(acc[t]);
}

// grid (ceil(T / kTokTile), SI / rows_per_cta).  K = hidden must be a multiple of 8.
__global__ void __launch_bounds__(kThreads)
shared_phase1_kernel(const __nv_bfloat16* __restrict__ x, int tokens, int H, int SI,
                     const __nv_bfloat16* __restrict__ gate_up, const __nv_bfloat16* __restrict__ shared_gate,
                     int rows_per_cta, float* __restrict__ ic2s, float* __restrict__ se_gate) {
    extern __shared__ float xs[];  // [kTokTile][H]
    const int t0 = blockIdx.x * kTokTile;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    for (int i = threadIdx.x; i < kTokTile * H; i += kThreads) {
        int t = t0 + i / H;
        xs[i] = (t < tokens) ? __bfloat162float(x[(size_t)t * H + i % H]) : 0.f;
    }
    __syncthreads();
    const int n0 = blockIdx.y * rows_per_cta;
    float ag[kTokTile], au[kTokTile];
    for (int i = warp; i < rows_per_cta && n0 + i < SI; i += kWarps) {
        const int n = n0 + i;
        row_dots<kTokTile>(gate_up + (size_t)n * H, xs, H, lane, ag);
        row_dots<kTokTile>(gate_up + (size_t)(SI + n) * H, xs, H, lane, au);
        if (lane == 0) {
#pragma unroll
            for (int t = 0; t < kTokTile; t++)
                if (t0 + t < tokens) ic2s[(size_t)(t0 + t) * SI + n] = (ag[t] / (1.0f + expf(-ag[t]))) * au[t];
        }
    }
    // the first row-tile also produces the sigmoid gate
    if (blockIdx.y == 0 && warp == 0) {
        row_dots<kTokTile>(shared_gate, xs, H, lane, ag);
        if (lane == 0) {
#pragma unroll
            for (int t = 0; t < kTokTile; t++)
                if (t0 + t < tokens) se_gate[t0 + t] = 1.0f / (1.0f + expf(-ag[t]));
        }
    }
}

// grid (ceil(T / kTokTile), H / rows_per_cta)
__global__ void __launch_bounds__(kThreads)
shared_phase2_kernel(const float* __restrict__ ic2s, int tokens, int H, int SI,
                     const __nv_bfloat16* __restrict__ down, int rows_per_cta, float* __restrict__ shared_out) {
    extern __shared__ float xs[];  // [kTokTile][SI]
    const int t0 = blockIdx.x * kTokTile;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    for (int i = threadIdx.x; i < kTokTile * SI; i += kThreads) {
        int t = t0 + i / SI;
        xs[i] = (t < tokens) ? ic2s[(size_t)t * SI + i % SI] : 0.f;
    }
    __syncthreads();
    const int d0 = blockIdx.y * rows_per_cta;
    float a[kTokTile];
    for (int i = warp; i < rows_per_cta && d0 + i < H; i += kWarps) {
        const int d = d0 + i;
        row_dots<kTokTile>(down + (size_t)d * SI, xs, SI, lane, a);
        if (lane == 0) {
#pragma unroll
            for (int t = 0; t < kTokTile; t++)
                if (t0 + t < tokens) shared_out[(size_t)(t0 + t) * H + d] = a[t];
        }
    }
}

}  // namespace

int launch_shared_expert(const __nv_bfloat16* x, int tokens, int hidden, int shared_inter,
                         const __nv_bfloat16* gate_up, const __nv_bfloat16* down,
                         const __nv_bfloat16* shared_gate, float* ic2s, float* shared_out, float* se_gate,
                         const Ctx& c) {
    const int ttiles = (tokens + kTokTile - 1) / kTokTile;
    const int r1 = 16, r2 = 64;
    size_t sm1 = (size_t)kTokTile * hidden * sizeof(float), sm2 = (size_t)kTokTile * shared_inter * sizeof(float);
    static bool attr = false;
    if (!attr) {
        cudaFuncSetAttribute(shared_phase1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(shared_phase2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        attr = true;
    }
    dim3 g1(ttiles, (shared_inter + r1 - 1) / r1);
    c.begin(K_SHARED_PHASE1);
    shared_phase1_kernel<<<g1, kThreads, sm1, c.s>>>(x, tokens, hidden, shared_inter, gate_up, shared_gate, r1, ic2s,
                                                     se_gate);
    c.end();
    dim3 g2(ttiles, (hidden + r2 - 1) / r2);
    c.begin(K_SHARED_PHASE2);
    shared_phase2_kernel<<<g2, kThreads, sm2, c.s>>>(ic2s, tokens, hidden, shared_inter, down, r2, shared_out);
    c.end();
    return 2;
}

}  // namespace ftm
