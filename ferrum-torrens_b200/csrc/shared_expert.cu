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

// ---- tensor-core variant for small batches --------------------------------------------------
// The weights are the A operand of mma.sync.m16n8k16 (16 rows x 16 k, bf16), the tokens the N
// dimension (eight per tile).  A lane reads 16 contiguous bytes of a weight row (eight k) and the
// same eight k of its token row; the k slots of two MMAs are fed from those eight k in order, for
// both operands alike, so any assignment is consistent.  Each weight byte is read once.
constexpr int kMaxTokTiles = 8;  // up to 64 tokens per pass

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// partial products of one warp: rows (row_lo + g8, row_hi + g8) x tokens [tok0, tok0 + 8*NT) over
// k in [k_begin, k_end), 32 k per step
template <int NT>
__device__ __forceinline__ void warp_rows_x_tokens(const __nv_bfloat16* __restrict__ w_lo,
                                                   const __nv_bfloat16* __restrict__ w_hi,
                                                   const __nv_bfloat16* __restrict__ x, int ldx, int tok0, int tokens,
                                                   int k_begin, int k_end, int lane, float (&acc)[NT][4],
                                                   bool init = true) {
    const int g8 = lane >> 2, t4 = lane & 3;
    if (init) {
#pragma unroll
        for (int n = 0; n < NT; n++)
#pragma unroll
            for (int q = 0; q < 4; q++) acc[n][q] = 0.f;
    }
    const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll 2
    for (int k = k_begin + t4 * 8; k < k_end; k += 32) {
        const uint4 alo = *reinterpret_cast<const uint4*>(w_lo + k);
        const uint4 ahi = *reinterpret_cast<const uint4*>(w_hi + k);
#pragma unroll
        for (int n = 0; n < NT; n++) {
            const int t = tok0 + n * 8 + g8;
            const uint4 b = (t < tokens) ? *reinterpret_cast<const uint4*>(x + (size_t)t * ldx + k) : zero;
            mma_bf16_16816(acc[n], alo.x, ahi.x, alo.y, ahi.y, b.x, b.y);
            mma_bf16_16816(acc[n], alo.z, ahi.z, alo.w, ahi.w, b.z, b.w);
        }
    }
}

// phase 1: grid (SI / 8, ceil(T / 64)); 8 warps split K; rows = 8 gate rows + the 8 matching up rows
__global__ void __launch_bounds__(256)
shared_phase1_mma_kernel(const __nv_bfloat16* __restrict__ x, int tokens, int H, int SI,
                         const __nv_bfloat16* __restrict__ gate_up, const __nv_bfloat16* __restrict__ shared_gate,
                         __nv_bfloat16* __restrict__ ic2b, float* __restrict__ se_gate) {
    __shared__ float red[8][kMaxTokTiles][32][4];
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int g8 = lane >> 2, t4 = lane & 3;
    const int pair0 = blockIdx.x * 8, tok0 = blockIdx.y * 64;
    const int kper = H / 8;
    float acc[kMaxTokTiles][4];
    warp_rows_x_tokens<kMaxTokTiles>(gate_up + (size_t)(pair0 + g8) * H, gate_up + (size_t)(SI + pair0 + g8) * H, x, H,
                                     tok0, tokens, warp * kper, (warp + 1) * kper, lane, acc);
#pragma unroll
    for (int n = 0; n < kMaxTokTiles; n++)
        *reinterpret_cast<float4*>(red[warp][n][lane]) = make_float4(acc[n][0], acc[n][1], acc[n][2], acc[n][3]);
    __syncthreads();
    // warp n finishes token tile n: sum the K partials, silu(gate) * up
    {
        const int n = warp;
        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int w = 0; w < 8; w++) {
            const float4 v = *reinterpret_cast<const float4*>(red[w][n][lane]);
            c[0] += v.x; c[1] += v.y; c[2] += v.z; c[3] += v.w;
        }
#pragma unroll
        for (int q = 0; q < 2; q++) {
            const int t = tok0 + n * 8 + 2 * t4 + q;
            if (t < tokens) {
                // ic2 leaves as a bf16 pair hi + lo (16 significant bits), two planes [tokens, SI]
                const float g = c[q], u = c[2 + q];
                const float v = (g / (1.0f + expf(-g))) * u;
                const __nv_bfloat16 hi = __float2bfloat16_rn(v);
                ic2b[(size_t)t * SI + pair0 + g8] = hi;
                ic2b[(size_t)(tokens + t) * SI + pair0 + g8] = __float2bfloat16_rn(v - __bfloat162float(hi));
            }
        }
    }
    // the first row block also produces the sigmoid gate: one warp per token
    if (blockIdx.x == 0) {
        for (int tl = warp; tl < 64; tl += 8) {
            const int t = tok0 + tl;
            if (t >= tokens) break;
            float a = 0.f;
            for (int k = lane * 8; k < H; k += 256) {
                const uint4 wv = *reinterpret_cast<const uint4*>(shared_gate + k);
                const uint4 xv = *reinterpret_cast<const uint4*>(x + (size_t)t * H + k);
                const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w}, xx[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const float2 w2 = bf16x2_to_f32(ww[q]), x2 = bf16x2_to_f32(xx[q]);
                    a += w2.x * x2.x + w2.y * x2.y;
                }
            }
            a = warp_sum(a);
            if (lane == 0) se_gate[t] = 1.0f / (1.0f + expf(-a));
        }
    }
}

// phase 2: grid (H / 16, ceil(T / 64)); 2 warps split K = SI
__global__ void __launch_bounds__(64)
shared_phase2_mma_kernel(const __nv_bfloat16* __restrict__ ic2b, int tokens, int H, int SI,
                         const __nv_bfloat16* __restrict__ down, float* __restrict__ shared_out) {
    __shared__ float red[kMaxTokTiles][32][4];
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int g8 = lane >> 2, t4 = lane & 3;
    const int d0 = blockIdx.x * 16, tok0 = blockIdx.y * 64;
    const int kper = SI / 2;
    float acc[kMaxTokTiles][4];
    warp_rows_x_tokens<kMaxTokTiles>(down + (size_t)(d0 + g8) * SI, down + (size_t)(d0 + 8 + g8) * SI, ic2b, SI, tok0,
                                     tokens, warp * kper, (warp + 1) * kper, lane, acc);
    warp_rows_x_tokens<kMaxTokTiles>(down + (size_t)(d0 + g8) * SI, down + (size_t)(d0 + 8 + g8) * SI,
                                     ic2b + (size_t)tokens * SI, SI, tok0, tokens, warp * kper, (warp + 1) * kper, lane,
                                     acc, false);
    if (warp == 1) {
#pragma unroll
        for (int n = 0; n < kMaxTokTiles; n++)
            *reinterpret_cast<float4*>(red[n][lane]) = make_float4(acc[n][0], acc[n][1], acc[n][2], acc[n][3]);
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
        for (int n = 0; n < kMaxTokTiles; n++) {
            const float4 v = *reinterpret_cast<const float4*>(red[n][lane]);
#pragma unroll
            for (int q = 0; q < 2; q++) {
                const int t = tok0 + n * 8 + 2 * t4 + q;
                if (t < tokens) {
                    shared_out[(size_t)t * H + d0 + g8] = acc[n][q] + (q ? v.y : v.x);
                    shared_out[(size_t)t * H + d0 + 8 + g8] = acc[n][2 + q] + (q ? v.w : v.z);
                }
            }
        }
    }
}

}  // namespace

int launch_shared_expert(const __nv_bfloat16* x, int tokens, int hidden, int shared_inter,
                         const __nv_bfloat16* gate_up, const __nv_bfloat16* down,
                         const __nv_bfloat16* shared_gate, float* ic2s, float* shared_out, float* se_gate,
                         int32_t* err, const Ctx& c) {
    if (shared_umma_supported(tokens, hidden, shared_inter)) {
        const int n = launch_shared_umma(x, tokens, hidden, shared_inter, gate_up, down, shared_gate,
                                         reinterpret_cast<__nv_bfloat16*>(ic2s), shared_out, se_gate, err, c);
        if (n >= 0) return n;
    }
    // tensor-core path: K splits must be multiples of 32
    if (hidden % 256 == 0 && shared_inter % 64 == 0 && hidden % 16 == 0 && shared_inter % 8 == 0) {
        __nv_bfloat16* ic2b = reinterpret_cast<__nv_bfloat16*>(ic2s);
        dim3 g1(shared_inter / 8, (tokens + 63) / 64);
        c.begin(K_SHARED_PHASE1);
        shared_phase1_mma_kernel<<<g1, 256, 0, c.s>>>(x, tokens, hidden, shared_inter, gate_up, shared_gate, ic2b, se_gate);
        c.end();
        dim3 g2(hidden / 16, (tokens + 63) / 64);
        c.begin(K_SHARED_PHASE2);
        shared_phase2_mma_kernel<<<g2, 64, 0, c.s>>>(ic2b, tokens, hidden, shared_inter, down, shared_out);
        c.end();
        return 2;
    }
    const int ttiles = (tokens + kTokTile - 1) / kTokTile;
    const int r1 = 16, r2 = 64;
    size_t sm1 = (size_t)kTokTile * hidden * sizeof(float), sm2 = (size_t)kTokTile * shared_inter * sizeof(float);
    static PerDeviceOnce once1, once2;
    allow_dyn_smem(once1, shared_phase1_kernel, 200 * 1024);
    allow_dyn_smem(once2, shared_phase2_kernel, 200 * 1024);
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
