// Routed experts, per-route GEMV form (small batches).
//
// Reference behaviour (src/domain/expert_kernel.rs:547-618 `gemv_rows`,
// python/ferrum_kernel/nvfp4_moe.py:186-294): for each route r with slot s >= 0
//   ic1[n]  = global_gu[s,n] * sum_k x[token(r),k] * fp4(gu[s,n,k]) * e4m3(gu_scale[s,n,k/16])
//   ic2[i]  = silu(ic1[i]) * ic1[I+i]                       (gate = first half of the rows)
//   y[r,d]  = w[r] * global_dn[s,d] * sum_k ic2[k] * fp4(dn[s,d,k]) * e4m3(dn_scale[s,d,k/16])
// and a route with slot -1 contributes zeros.  Accumulation is f32; the f16 row global is applied
// once after the K reduction.
#include "kernels.cuh"

namespace ftm {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

// dot of one scale block: 16 consecutive k (8 packed bytes, low nibble = even k) with
// activations in shared memory
__device__ __forceinline__ float dot16(uint2 p, uint32_t sc, const float* __restrict__ xs) {
    const uint32_t w[2] = {p.x, p.y};
    float a = 0.f;
#pragma unroll
    for (int q = 0; q < 2; q++)
#pragma unroll
        for (int j = 0; j < 8; j++) a = fmaf(xs[q * 8 + j], e2m1_to_f32((w[q] >> (4 * j)) & 0xfu), a);
    return a * e4m3_to_f32(sc);
}

// grid (routes, I / rows_per_cta); each warp computes (gate row n, up row I+n) pairs
__global__ void __launch_bounds__(kThreads)
route_gate_up_kernel(BankView b, const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ route_slot,
                     int top_k, int rows_per_cta, float* __restrict__ ic2) {
    extern __shared__ float xs[];  // [hidden]
    const int r = blockIdx.x;
    const int slot = route_slot[r];
    const int H = b.hidden, I = b.inter;
    const int n0 = blockIdx.y * rows_per_cta;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    if (slot < 0) {
        for (int i = threadIdx.x; i < rows_per_cta && n0 + i < I; i += kThreads) ic2[(size_t)r * I + n0 + i] = 0.f;
        return;
    }
    const __nv_bfloat16* xr = x + (size_t)(r / top_k) * H;
    for (int k = threadIdx.x * 2; k < H; k += kThreads * 2) {
        float2 v = bf16x2_to_f32(*reinterpret_cast<const uint32_t*>(xr + k));
        xs[k] = v.x;
        xs[k + 1] = v.y;
    }
    __syncthreads();
    const size_t prow = H / 2, srow = H / 16;
    const uint8_t* P = b.gu_packed + (size_t)slot * 2 * I * prow;
    const uint8_t* S = b.gu_scale + (size_t)slot * 2 * I * srow;
    const uint16_t* G = b.gu_global + (size_t)slot * 2 * I;
    for (int i = warp; i < rows_per_cta && n0 + i < I; i += kWarps) {
        const int n = n0 + i;
        float ag = 0.f, au = 0.f;
        for (int c = lane; c < H / 16; c += 32) {
            uint2 pg = *reinterpret_cast<const uint2*>(P + (size_t)n * prow + c * 8);
            uint2 pu = *reinterpret_cast<const uint2*>(P + (size_t)(I + n) * prow + c * 8);
            ag += dot16(pg, S[(size_t)n * srow + c], xs + c * 16);
            au += dot16(pu, S[(size_t)(I + n) * srow + c], xs + c * 16);
        }
        ag = warp_sum(ag);
        au = warp_sum(au);
        if (lane == 0) {
            float g = ag * f16_global_to_f32(G[n]);
            float u = au * f16_global_to_f32(G[I + n]);
            ic2[(size_t)r * I + n] = (g / (1.0f + expf(-g))) * u;
        }
    }
}

// grid (routes, H / rows_per_cta); one warp per output row
__global__ void __launch_bounds__(kThreads)
route_down_kernel(BankView b, const float* __restrict__ ic2, const int32_t* __restrict__ route_slot,
                  const float* __restrict__ route_weight, int rows_per_cta, float* __restrict__ yroute) {
    extern __shared__ float xs[];  // [inter]
    const int r = blockIdx.x;
    const int slot = route_slot[r];
    const int H = b.hidden, I = b.inter;
    const int d0 = blockIdx.y * rows_per_cta;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    if (slot < 0) {
        for (int i = threadIdx.x; i < rows_per_cta && d0 + i < H; i += kThreads) yroute[(size_t)r * H + d0 + i] = 0.f;
        return;
    }
    for (int k = threadIdx.x; k < I; k += kThreads) xs[k] = ic2[(size_t)r * I + k];
    __syncthreads();
    const float w = route_weight[r];
    const size_t prow = I / 2, srow = I / 16;
    const uint8_t* P = b.dn_packed + (size_t)slot * H * prow;
    const uint8_t* S = b.dn_scale + (size_t)slot * H * srow;
    const uint16_t* G = b.dn_global + (size_t)slot * H;
    for (int i = warp; i < rows_per_cta && d0 + i < H; i += kWarps) {
        const int d = d0 + i;
        float a = 0.f;
        for (int c = lane; c < I / 16; c += 32)
            a += dot16(*reinterpret_cast<const uint2*>(P + (size_t)d * prow + c * 8), S[(size_t)d * srow + c],
                       xs + c * 16);
        a = warp_sum(a);
        if (lane == 0) yroute[(size_t)r * H + d] = w * (a * f16_global_to_f32(G[d]));
    }
}

}  // namespace

int launch_decode_routes(const BankView& b, const __nv_bfloat16* x, const int32_t* route_slot,
                         const float* route_weight, int tokens, int top_k, float* ic2, float* yroute,
                         const Ctx& c) {
    const int routes = tokens * top_k;
    const int gu_rows = 64, dn_rows = 256;
    dim3 g1(routes, (b.inter + gu_rows - 1) / gu_rows);
    c.begin(K_EXPERT_GATE_UP);
    route_gate_up_kernel<<<g1, kThreads, b.hidden * sizeof(float), c.s>>>(b, x, route_slot, top_k,
                                                                          min(gu_rows, b.inter), ic2);
    c.end();
    dim3 g2(routes, (b.hidden + dn_rows - 1) / dn_rows);
    c.begin(K_EXPERT_DOWN);
    route_down_kernel<<<g2, kThreads, b.inter * sizeof(float), c.s>>>(b, ic2, route_slot, route_weight,
                                                                      min(dn_rows, b.hidden), yroute);
    c.end();
    return 2;
}

}  // namespace ftm
