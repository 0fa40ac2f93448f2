// Weighted un-permute / combine and the gated shared-expert add.
//
// Reference behaviour (src/models/qwen3_6/forward.rs:737-742, :785-787; device form
// python/ferrum_kernel/nvfp4_moe.py:423-445 `_sum_reduce_kernel` followed by `se.add(&routed)`,
// src/models/qwen3_6/forward_cudarc.rs:1590):
//   out[t] = se_gate[t] * shared[t] + sum_{j < top_k} w[t,j] * ic3[t,j]
// with the routes added in j order.  The route weights were applied by the down projection, so
// this pass reads each per-route row once and writes the token row once.
#include "kernels.cuh"

namespace ftm {

namespace {

// yroute [T*top_k, H] f32 (already weighted); shared / se_gate may be null (routed sum only)
__global__ void sum_routes_kernel(const float* __restrict__ yroute, int tokens, int top_k, int H,
                                  const float* __restrict__ shared, const float* __restrict__ se_gate,
                                  void* __restrict__ out, int out_dtype) {
    const int t = blockIdx.x;  // tokens on x: the owner side of expert parallelism runs > 65535 rows
    const int d = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
    if (d >= H) return;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (shared) {
        const float g = se_gate[t];
        const float4 sv = *reinterpret_cast<const float4*>(shared + (size_t)t * H + d);
        acc = make_float4(sv.x * g, sv.y * g, sv.z * g, sv.w * g);
    }
    for (int j = 0; j < top_k; j++) {
        const float4 y = *reinterpret_cast<const float4*>(yroute + ((size_t)t * top_k + j) * H + d);
        acc.x += y.x; acc.y += y.y; acc.z += y.z; acc.w += y.w;
    }
    const size_t o = (size_t)t * H + d;
    if (out_dtype == 0) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
        uint2 pk = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(out) + o) = pk;
    } else {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + o) = acc;
    }
}

__global__ void combine_kernel(const void* __restrict__ routed, int routed_dtype, const float* __restrict__ shared,
                               const float* __restrict__ se_gate, int tokens, int H, void* __restrict__ out,
                               int out_dtype) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)tokens * H) return;
    int t = (int)(i / H);
    float v = shared[i] * se_gate[t] + load_act(routed, routed_dtype, i);
    store_act(out, out_dtype, i, v);
}

__global__ void cast_to_bf16_kernel(const void* __restrict__ src, int src_dtype, size_t n,
                                    __nv_bfloat16* __restrict__ dst) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = __float2bfloat16_rn(load_act(src, src_dtype, i));
}

// ---- fused residual add + RMSNorm in front of the block -------------------------------------
// Reference: python/ferrum_kernel/norm.py:35-110 (`_add_rmsnorm_kernel`, `add_rmsnorm_reference`), the
// post-attention site src/models/qwen3_6/forward.rs:942-953:
//   s = bf16(f32(x) + f32(r))                    the new residual, bf16 like the stream
//   var = mean(f32(s)^2)                         f32
//   y = bf16((f32(s) * (1 / sqrt(var + eps))) * f32(w))      w is the baked 1 + weight vector
// One warp per row; a lane keeps its elements in registers between the two passes.
template <int kPerLane>
__global__ void __launch_bounds__(128)
add_rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ r,
                   const __nv_bfloat16* __restrict__ w, float eps, int tokens, int H,
                   __nv_bfloat16* __restrict__ sum_out, __nv_bfloat16* __restrict__ out) {
    const int row = blockIdx.x * 4 + threadIdx.x / 32, lane = threadIdx.x % 32;
    if (row >= tokens) return;
    // chunk c of the lane: eight consecutive elements at (c * 32 + lane) * 8
    float sf[kPerLane][8];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < kPerLane; c++) {
        const int k = (c * 32 + lane) * 8;
        if (k < H) {
            const uint4 xv = *reinterpret_cast<const uint4*>(x + (size_t)row * H + k);
            const uint4 rv = *reinterpret_cast<const uint4*>(r + (size_t)row * H + k);
            const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w}, rw[4] = {rv.x, rv.y, rv.z, rv.w};
            uint32_t sw[4];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float2 a = bf16x2_to_f32(xw[q]), b = bf16x2_to_f32(rw[q]);
                const __nv_bfloat162 s2 = __floats2bfloat162_rn(a.x + b.x, a.y + b.y);
                sw[q] = *reinterpret_cast<const uint32_t*>(&s2);
                const float2 f = bf16x2_to_f32(sw[q]);
                sf[c][2 * q] = f.x;
                sf[c][2 * q + 1] = f.y;
                ss += f.x * f.x;
                ss += f.y * f.y;
            }
            *reinterpret_cast<uint4*>(sum_out + (size_t)row * H + k) = make_uint4(sw[0], sw[1], sw[2], sw[3]);
        }
    }
    ss = warp_sum(ss);
    const float var = ss * (1.0f / (float)H);
    const float recip = 1.0f / sqrtf(var + eps);
#pragma unroll
    for (int c = 0; c < kPerLane; c++) {
        const int k = (c * 32 + lane) * 8;
        if (k < H) {
            const uint4 wv = *reinterpret_cast<const uint4*>(w + k);
            const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
            uint32_t yw[4];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float2 g = bf16x2_to_f32(ww[q]);
                const __nv_bfloat162 y2 = __floats2bfloat162_rn((sf[c][2 * q] * recip) * g.x, (sf[c][2 * q + 1] * recip) * g.y);
                yw[q] = *reinterpret_cast<const uint32_t*>(&y2);
            }
            *reinterpret_cast<uint4*>(out + (size_t)row * H + k) = make_uint4(yw[0], yw[1], yw[2], yw[3]);
        }
    }
}

// ---- expert-parallel dispatch / combine ----------------------------------------------------
// pack: position i of the send buffers takes route r = route_idx[i] (routes sorted by global expert
// id, hence by owning rank): the token's activation row, the expert id and the route weight
__global__ void ep_pack_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ ids,
                               const float* __restrict__ weights, const int32_t* __restrict__ route_idx, int routes,
                               int top_k, int H, __nv_bfloat16* __restrict__ send_x, int32_t* __restrict__ send_expert,
                               float* __restrict__ send_weight) {
    const int i = blockIdx.x;
    const int r = route_idx[i];
    if (r < 0 || r >= routes) return;   // a route the permutation build dropped (expert id out of range, flagged there)
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(r / top_k) * H);
    uint4* dst = reinterpret_cast<uint4*>(send_x + (size_t)i * H);
    for (int c = threadIdx.x; c < H / 8; c += blockDim.x) dst[c] = src[c];
    if (threadIdx.x == 0) {
        send_expert[i] = ids[r];
        send_weight[i] = weights[r];
    }
}

// routes per owning rank from the per-expert prefix: rank p owns experts [p*per, (p+1)*per)
__global__ void ep_rank_counts_kernel(const int32_t* __restrict__ seg, int experts, int ranks,
                                      int32_t* __restrict__ counts) {
    const int p = threadIdx.x;
    if (p < ranks) {
        const int per = experts / ranks;
        counts[p] = seg[(p + 1) * per] - seg[p * per];
    }
}

__global__ void ep_invert_kernel(const int32_t* __restrict__ route_idx, int routes, int32_t* __restrict__ pos_of_route) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < routes) pos_of_route[route_idx[i]] = i;
}

// out[t] = se_gate[t] * shared[t] + sum_j y[pos_of_route[t*k + j]]   (weights were applied by the owner)
__global__ void ep_combine_kernel(const void* __restrict__ y, int y_dtype, const int32_t* __restrict__ pos_of_route,
                                  int top_k, int H, const float* __restrict__ shared, const float* __restrict__ se_gate,
                                  void* __restrict__ out, int out_dtype) {
    const int t = blockIdx.x;
    const int d = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
    if (d >= H) return;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (shared) {
        const float g = se_gate[t];
        const float4 sv = *reinterpret_cast<const float4*>(shared + (size_t)t * H + d);
        acc = make_float4(sv.x * g, sv.y * g, sv.z * g, sv.w * g);
    }
    for (int j = 0; j < top_k; j++) {
        const size_t row = (size_t)pos_of_route[t * top_k + j] * H + d;
        if (y_dtype == 0) {
            const uint2 pk = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(y) + row);
            const float2 a = bf16x2_to_f32(pk.x), b = bf16x2_to_f32(pk.y);
            acc.x += a.x; acc.y += a.y; acc.z += b.x; acc.w += b.y;
        } else {
            const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(y) + row);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
    }
    const size_t o = (size_t)t * H + d;
    if (out_dtype == 0) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(out) + o) =
            make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    } else {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + o) = acc;
    }
}

// ---- expert-parallel exchange over peer memory -------------------------------------------------
// counts_all[s * world + p] = routes that rank s sends to owner p.  An owner's receive buffer holds the
// sources in rank order, each source's routes in its send order (sorted by expert).

// Both kernels move whole rows between GPUs with plain 16-byte peer stores.  A CTA takes kEpRows rows and
// issues all their loads before the first store, so that every thread keeps several stores in flight on the
// link (one row per CTA reached 0.71 of the measured peer-copy rate).
constexpr int kEpRows = 4;

// dispatch: position i of this rank's send order goes straight into the owner's receive buffers
__global__ void __launch_bounds__(128)
ep_dispatch_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ ids, const float* __restrict__ weights,
                   const int32_t* __restrict__ route_idx, const int32_t* __restrict__ seg, int routes, int top_k, int H,
                   int per, int world, int rank, const int32_t* __restrict__ counts_all,
                   const uint64_t* __restrict__ peer_x, const uint64_t* __restrict__ peer_meta, long long capacity,
                   int32_t* err) {
    // CTAs walk the send order starting at the next rank's block, so that at any time every owner is written
    // by one source (all ranks starting at owner 0 would share that owner's ingress bandwidth)
    const int first = seg[((rank + 1) % world) * per];
    const uint4* src[kEpRows];
    uint4* dst[kEpRows];
#pragma unroll
    for (int q = 0; q < kEpRows; q++) {
        src[q] = nullptr;
        dst[q] = nullptr;
        int i = blockIdx.x * kEpRows + q;
        if (i >= routes) continue;
        i += first;
        if (i >= routes) i -= routes;
        // every index is checked before the load that depends on it: a route the permutation build dropped
        // (route_idx left at -1) or an expert id outside the layer raises the error flag, it is never followed
        const int r = (i >= 0 && i < routes) ? route_idx[i] : -1;
        const int e = (r >= 0 && r < routes) ? ids[r] : -1;
        if (e < 0 || e >= per * world) {
            if (threadIdx.x == 0) atomicExch(err, 4);
            continue;
        }
        const int p = e / per;
        long long row = i - seg[p * per];
        for (int s = 0; s < rank; s++) row += counts_all[s * world + p];
        if (row < 0 || row >= capacity) {   // never store outside the owner's buffer
            if (threadIdx.x == 0) atomicExch(err, 4);
            continue;
        }
        src[q] = reinterpret_cast<const uint4*>(x + (size_t)(r / top_k) * H);
        dst[q] = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(peer_x[p]) + (size_t)row * H);
        if (threadIdx.x == 0)
            reinterpret_cast<int2*>(peer_meta[p])[row] = make_int2(e, __float_as_int(weights[r]));
    }
    for (int c = threadIdx.x; c < H / 8; c += blockDim.x) {
        uint4 v[kEpRows];
#pragma unroll
        for (int q = 0; q < kEpRows; q++)
            if (src[q]) v[q] = src[q][c];
#pragma unroll
        for (int q = 0; q < kEpRows; q++)
            if (dst[q]) dst[q][c] = v[q];
    }
}


// ---- dispatch into the owner's sorted activation matrix -----------------------------------------
// seg_all[s * (experts + 1) + e] = first position of expert e in rank s's send order (its permutation build's
// prefix over the layer's experts), all-gathered.  From it every rank knows where each of its routes lands in
// the owner's matrix SORTED BY EXPERT (within an expert: source rank, then the source's send order), so the
// owner needs neither a permutation build nor a gather pass: this kernel reads a token's row once, scales it
// to f16 exactly as the owner's gather would (largest magnitude into [2^14, 2^15), a power of two) and stores
// row, route weight and row scale at that position over peer memory.  One warp per route, hidden = 2048.
__device__ __forceinline__ long long ep_sorted_row(const int32_t* __restrict__ seg_all, int experts, int per, int world, int rank,
                                                   int e, int lane) {
    // rows of the owner's experts before e from every source, plus the rows of e from the sources before this one
    const int p0 = (e / per) * per;
    long long v = 0;
    if (lane < world) {
        const int32_t* sg = seg_all + (size_t)lane * (experts + 1);
        v = sg[e] - sg[p0];
        if (lane < rank) v += sg[e + 1] - sg[e];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__global__ void __launch_bounds__(128)
ep_dispatch_sorted_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ ids, const float* __restrict__ weights,
                          const int32_t* __restrict__ route_idx, const int32_t* __restrict__ seg_all, int routes, int top_k,
                          int experts, int per, int world, int rank, const uint64_t* __restrict__ peer_xg,
                          const uint64_t* __restrict__ peer_w, const uint64_t* __restrict__ peer_rs, long long capacity,
                          int32_t* err) {
    constexpr int H = 2048, kChunks = 8;     // a lane holds 8 chunks of 8 k
    const int lane = threadIdx.x % 32;
    const int32_t* const seg = seg_all + (size_t)rank * (experts + 1);
    int i = blockIdx.x * 4 + threadIdx.x / 32;
    if (i >= routes) return;
    // walk the send order starting at the next rank's block (see ep_dispatch_kernel)
    i += seg[((rank + 1) % world) * per];
    if (i >= routes) i -= routes;
    const int r = (i >= 0 && i < routes) ? route_idx[i] : -1;
    const int e = (r >= 0 && r < routes) ? ids[r] : -1;
    if (e < 0 || e >= per * world) {
        if (lane == 0) atomicExch(err, 4);
        return;
    }
    const int p = e / per;
    const long long row = ep_sorted_row(seg_all, experts, per, world, rank, e, lane) + (i - seg[e]);
    if (row < 0 || row >= capacity || i < seg[e]) {   // never store outside the owner's buffers
        if (lane == 0) atomicExch(err, 4);
        return;
    }
    const __nv_bfloat16* const src = x + (size_t)(r / top_k) * H;
    uint4 raw[kChunks];
#pragma unroll
    for (int c = 0; c < kChunks; c++) raw[c] = *reinterpret_cast<const uint4*>(src + (c * 32 + lane) * 8);
    float v[kChunks][8];
    float m = 0.f;
#pragma unroll
    for (int c = 0; c < kChunks; c++) {
        const uint32_t w[4] = {raw[c].x, raw[c].y, raw[c].z, raw[c].w};
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const float2 f = bf16x2_to_f32(w[q]);
            v[c][2 * q] = f.x;
            v[c][2 * q + 1] = f.y;
            m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const int ex = max((int)((__float_as_uint(m) >> 23) & 0xff), 15);
    float inv = 1.0f, sc = 1.0f;
    if (ex < 255) {
        inv = __uint_as_float((uint32_t)(127 + 14 - (ex - 127)) << 23);
        sc = __uint_as_float((uint32_t)(127 - 14 + (ex - 127)) << 23);
    }
    __half* const dst = reinterpret_cast<__half*>(peer_xg[p]) + (size_t)row * H;
#pragma unroll
    for (int c = 0; c < kChunks; c++) {
        __half2 h[4];
#pragma unroll
        for (int q = 0; q < 4; q++) h[q] = __floats2half2_rn(v[c][2 * q] * inv, v[c][2 * q + 1] * inv);
        *reinterpret_cast<uint4*>(dst + (c * 32 + lane) * 8) =
            make_uint4(*reinterpret_cast<uint32_t*>(&h[0]), *reinterpret_cast<uint32_t*>(&h[1]),
                       *reinterpret_cast<uint32_t*>(&h[2]), *reinterpret_cast<uint32_t*>(&h[3]));
    }
    if (lane == 0) {
        reinterpret_cast<float*>(peer_w[p])[row] = weights[r];
        reinterpret_cast<float*>(peer_rs[p])[row] = sc;
    }
}

// return: row i of the owner's output (receive order) goes to the position its source packed it at.  With
// pos_of_route the owner's rows are still sorted by expert (y row pos_of_route[i] belongs to received row i,
// a received row whose expert is not resident returns zeros): the un-permute pass and its extra read and
// write of every row are skipped.
__global__ void __launch_bounds__(128)
ep_return_kernel(const __nv_bfloat16* __restrict__ y, const int32_t* __restrict__ pos_of_route,
                 const int32_t* __restrict__ route_slot, int n, int H, int world, int rank,
                 const int32_t* __restrict__ counts_all, const uint64_t* __restrict__ peer_back, long long capacity,
                 int32_t* err) {
    // rows are walked starting at the next rank's block (see ep_dispatch_kernel)
    int first = 0;
    for (int q = 0; q < (rank + 1) % world; q++) first += counts_all[q * world + rank];
    const uint4* src[kEpRows];
    uint4* dst[kEpRows];
    bool zero[kEpRows];
#pragma unroll
    for (int q = 0; q < kEpRows; q++) {
        src[q] = nullptr;
        dst[q] = nullptr;
        zero[q] = false;
        int i = blockIdx.x * kEpRows + q;
        if (i >= n) continue;
        i += first;
        if (i >= n) i -= n;
        int s = 0, roff = 0;
        for (; s < world; s++) {
            const int c = counts_all[s * world + rank];
            if (i < roff + c) break;
            roff += c;
        }
        long long row = i - roff;
        if (s < world)
            for (int p = 0; p < rank; p++) row += counts_all[s * world + p];
        if (s >= world || row < 0 || row >= capacity) {
            if (threadIdx.x == 0) atomicExch(err, 4);
            continue;
        }
        long long from = i;
        if (pos_of_route) {
            if (route_slot[i] < 0)
                zero[q] = true;
            else
                from = pos_of_route[i];
        }
        src[q] = reinterpret_cast<const uint4*>(y + (size_t)from * H);
        dst[q] = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(peer_back[s]) + (size_t)row * H);
    }
    for (int c = threadIdx.x; c < H / 8; c += blockDim.x) {
        uint4 v[kEpRows];
#pragma unroll
        for (int q = 0; q < kEpRows; q++)
            if (src[q]) v[q] = zero[q] ? make_uint4(0, 0, 0, 0) : src[q][c];
#pragma unroll
        for (int q = 0; q < kEpRows; q++)
            if (dst[q]) dst[q][c] = v[q];
    }
}

}  // namespace

int launch_ep_dispatch(const __nv_bfloat16* x, const int32_t* ids, const float* weights, const int32_t* route_idx,
                       const int32_t* seg, int tokens, int top_k, int hidden, int experts, int world, int rank,
                       const int32_t* counts_all, const uint64_t* peer_x, const uint64_t* peer_meta, long long capacity,
                       int32_t* err, const Ctx& c) {
    c.begin(K_EP_PACK);
    ep_dispatch_kernel<<<(tokens * top_k + kEpRows - 1) / kEpRows, 128, 0, c.s>>>(x, ids, weights, route_idx, seg, tokens * top_k, top_k, hidden,
                                                       experts / world, world, rank, counts_all, peer_x, peer_meta, capacity,
                                                       err);
    c.end();
    return 1;
}

int launch_ep_return(const __nv_bfloat16* y, const int32_t* pos_of_route, const int32_t* route_slot, int n, int hidden,
                     int world, int rank, const int32_t* counts_all, const uint64_t* peer_back, long long capacity,
                     int32_t* err, const Ctx& c) {
    c.begin(K_EP_COMBINE);
    ep_return_kernel<<<(n + kEpRows - 1) / kEpRows, 128, 0, c.s>>>(y, pos_of_route, route_slot, n, hidden, world, rank, counts_all,
                                                                  peer_back, capacity, err);
    c.end();
    return 1;
}

int launch_ep_dispatch_sorted(const __nv_bfloat16* x, const int32_t* ids, const float* weights, const int32_t* route_idx,
                              const int32_t* seg_all, int tokens, int top_k, int experts, int world, int rank,
                              const uint64_t* peer_xg, const uint64_t* peer_w, const uint64_t* peer_rs, long long capacity,
                              int32_t* err, const Ctx& c) {
    const int routes = tokens * top_k;
    c.begin(K_EP_PACK);
    ep_dispatch_sorted_kernel<<<(routes + 3) / 4, 128, 0, c.s>>>(x, ids, weights, route_idx, seg_all, routes, top_k, experts,
                                                               experts / world, world, rank, peer_xg, peer_w, peer_rs, capacity,
                                                               err);
    c.end();
    return 1;
}

int launch_ep_counts(const int32_t* seg, int experts, int ranks, int32_t* counts, const Ctx& c) {
    c.begin(K_EP_PACK);
    ep_rank_counts_kernel<<<1, 32, 0, c.s>>>(seg, experts, ranks, counts);
    c.end();
    return 1;
}

int launch_sum_routes(const float* yroute, int tokens, int top_k, int hidden, const float* shared,
                      const float* se_gate, void* out, int out_dtype, const Ctx& c) {
    int threads = 128;
    dim3 grid(tokens, (hidden / 4 + threads - 1) / threads);
    c.begin(K_SUM_ROUTES);
    sum_routes_kernel<<<grid, threads, 0, c.s>>>(yroute, tokens, top_k, hidden, shared, se_gate, out, out_dtype);
    c.end();
    return 1;
}

int launch_combine(const void* routed, int routed_dtype, const float* shared, const float* se_gate, int tokens,
                   int hidden, void* out, int out_dtype, const Ctx& c) {
    size_t n = (size_t)tokens * hidden;
    c.begin(K_COMBINE);
    combine_kernel<<<(unsigned)((n + 255) / 256), 256, 0, c.s>>>(routed, routed_dtype, shared, se_gate, tokens, hidden,
                                                               out, out_dtype);
    c.end();
    return 1;
}

int launch_add_rmsnorm(const __nv_bfloat16* x, const __nv_bfloat16* r, const __nv_bfloat16* w, float eps, int tokens,
                       int hidden, __nv_bfloat16* sum_out, __nv_bfloat16* out, const Ctx& c) {
    // hidden is a multiple of 8 and at most 4096 (32 lanes x 8 elements x 16 chunks), checked by the caller
    const int chunks = (hidden + 255) / 256;
    const int grid = (tokens + 3) / 4;
    c.begin(K_ADD_RMSNORM);
    if (chunks <= 8)
        add_rmsnorm_kernel<8><<<grid, 128, 0, c.s>>>(x, r, w, eps, tokens, hidden, sum_out, out);
    else
        add_rmsnorm_kernel<16><<<grid, 128, 0, c.s>>>(x, r, w, eps, tokens, hidden, sum_out, out);
    c.end();
    return 1;
}

int launch_cast_to_bf16(const void* src, int src_dtype, size_t n, __nv_bfloat16* dst, const Ctx& c) {
    c.begin(K_CAST);
    cast_to_bf16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, c.s>>>(src, src_dtype, n, dst);
    c.end();
    return 1;
}

int launch_ep_pack(const __nv_bfloat16* x, const int32_t* ids, const float* weights, const int32_t* route_idx,
                   const int32_t* seg, int tokens, int top_k, int hidden, int experts, int ranks,
                   __nv_bfloat16* send_x, int32_t* send_expert, float* send_weight, int32_t* counts, const Ctx& c) {
    const int routes = tokens * top_k;
    c.begin(K_EP_PACK);
    ep_pack_kernel<<<routes, 128, 0, c.s>>>(x, ids, weights, route_idx, routes, top_k, hidden, send_x, send_expert,
                                           send_weight);
    ep_rank_counts_kernel<<<1, 32, 0, c.s>>>(seg, experts, ranks, counts);
    c.end();
    return 2;
}

int launch_ep_combine(const void* y, int y_dtype, const int32_t* route_idx, int32_t* pos_scratch, int tokens,
                      int top_k, int hidden, const float* shared, const float* se_gate, void* out, int out_dtype,
                      const Ctx& c) {
    const int routes = tokens * top_k;
    c.begin(K_EP_COMBINE);
    ep_invert_kernel<<<(routes + 255) / 256, 256, 0, c.s>>>(route_idx, routes, pos_scratch);
    dim3 grid(tokens, (hidden / 4 + 127) / 128);
    ep_combine_kernel<<<grid, 128, 0, c.s>>>(y, y_dtype, pos_scratch, top_k, hidden, shared, se_gate, out, out_dtype);
    c.end();
    return 2;
}

}  // namespace ftm
