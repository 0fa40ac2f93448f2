// Routed experts for small batches (decode): a bandwidth-bound grouped GEMV.
//
// Same arithmetic as the per-route kernels in decode_gemv.cu (reference:
// src/domain/expert_kernel.rs:547-618, python/ferrum_kernel/nvfp4_moe.py:186-294), organised so
// that every expert byte is read from HBM once per step however many tokens route to it:
//
//   plan      one CTA sorts the routes by slot (counting sort), cuts every slot's run into groups of at
//             most 8 routes and writes the group list.  No host round trip: the expert kernels read
//             the group count from device memory.  Batches of more than 2048 routes take the multi-CTA
//             permutation build of permute.cu and groups of 16.
//   experts   persistent CTAs, one per SM, each owning a contiguous range of (group, row-block) items.
//             Every warp is an independent worker on one item at a time: it issues the bulk async
//             copies (TMA engine, mbarrier transaction count) of its own packed E2M1 rows and E4M3
//             scales into a private double-buffered ring, reads 128-bit fragments from there, converts
//             in registers with the hardware conversions (e2m1x2 -> f16x2, e4m3x2 -> f16x2; the product
//             with the block scale is exact in f16) and feeds mma.sync.m16n8k16 with the group's tokens
//             as the N dimension, f32 accumulate.  There is no producer warp and no cross-warp
//             reduction; the warps of a CTA share only the group's activation tile (f16, scaled per
//             token by a power of two, k-permuted so that B fragments are conflict-free 128-bit loads).
//             gate_up pairs 8 gate rows with their 8 up rows in one tile, so global scale and
//             silu(gate) * up are a per-thread epilogue that writes ic2 (f32); down applies global scale
//             and route weight and writes one f32 row per route.
//
// The weights stay in the reference's bank layout (row-major packed nibbles, low nibble = even k).
#include <cstdlib>

#include "kernels.cuh"

namespace ftm {

namespace {

// ------------------------------------------------------------------------------------------
// k-permutation shared by the activation matrices and the kernels.
//
// Inside every window of 128 k, logical k = 32*t + 8*j + n (t, j in 0..3, n in 0..7) is stored at
// position 8*(4*j + t) + n.  Lane t of a fragment group then finds, for step j, its eight k as one
// contiguous chunk, and the four lanes' chunks are contiguous too (conflict-free 128-bit shared
// loads).  A lane's eight k are the eight nibbles of one packed weight word.
// ------------------------------------------------------------------------------------------
__host__ __device__ __forceinline__ int perm_k(int k) {
    const int w = k & ~127, r = k & 127;
    const int t = r >> 5, j = (r >> 3) & 3, n = r & 7;
    return w + 8 * (4 * j + t) + n;
}

// ------------------------------------------------------------------------------------------
// plan: bucket the routes by slot, cut every slot's bucket into groups of <= 8 routes
//
// One CTA.  A counting sort over the slot range (histogram in shared memory, prefix sums of the
// counts and of the group counts, scatter through the claimed positions).  Which routes of a slot
// share a group depends on the order the atomics land in, which does not matter: every route's
// result is computed from its own activations only.  The same pass maps dense expert ids to slots
// through the residency table (the serving call) and clears the output rows of routes whose expert
// is not resident.
// ------------------------------------------------------------------------------------------
constexpr int kPlanThreads = 1024;
constexpr int kPlanMaxRoutes = 2048;

struct PlanArgs {
    const int32_t* route_slot_in;  // slot ids, or null when expert ids are given
    const void* expert_ids;        // dense expert ids of `layer` (i32 / i64 / f32)
    int ids_dtype, layer, experts, n_ids;
    const int32_t* slot_for_id;
    int32_t* route_slot_out;       // slot per route (-1 = not resident); may alias route_slot_in
    int routes, slots, hidden;
    int4* groups;
    int32_t* sorted_route;
    int32_t* n_groups;
    float* yroute;
    int32_t* bad_flag;
};

__global__ void __launch_bounds__(kPlanThreads) decode_plan_kernel(PlanArgs a) {
    pdl_launch_dependents();
    pdl_wait();     // the router's ids
    extern __shared__ int psm[];
    int* const cnt = psm;                 // [slots]
    int* const pos_base = cnt + a.slots;  // [slots]
    int* const grp_base = pos_base + a.slots;
    __shared__ int wsum_pos[32], wsum_grp[32];
    __shared__ int s_missing[kPlanMaxRoutes];
    __shared__ int s_nmissing;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int i = tid; i < a.slots; i += kPlanThreads) cnt[i] = 0;
    if (tid == 0) s_nmissing = 0;
    __syncthreads();
    // each thread owns up to two routes
    int slot[2], claim[2];
#pragma unroll
    for (int q = 0; q < 2; q++) {
        const int r = tid + q * kPlanThreads;
        slot[q] = -2;
        claim[q] = 0;
        if (r < a.routes) {
            int sl;
            if (a.route_slot_in) {
                sl = a.route_slot_in[r];
            } else {
                long long e;
                if (a.ids_dtype == 3)
                    e = reinterpret_cast<const long long*>(a.expert_ids)[r];
                else if (a.ids_dtype == 1)
                    e = (long long)reinterpret_cast<const float*>(a.expert_ids)[r];
                else
                    e = (long long)reinterpret_cast<const int32_t*>(a.expert_ids)[r];
                sl = -1;
                if (e >= 0 && e < a.experts) {
                    const long long id = (long long)a.layer * a.experts + e;
                    if (id < a.n_ids) sl = a.slot_for_id[id];
                } else {
                    atomicExch(a.bad_flag, 1);
                }
            }
            if (sl >= a.slots) sl = -1;
            if (a.route_slot_out) a.route_slot_out[r] = sl;
            slot[q] = sl;
            if (sl >= 0)
                claim[q] = atomicAdd(&cnt[sl], 1);
            else
                s_missing[atomicAdd(&s_nmissing, 1)] = r;
        }
    }
    __syncthreads();
    // prefix sums over the slots: thread t scans slots [t*per, (t+1)*per)
    const int per = (a.slots + kPlanThreads - 1) / kPlanThreads;
    const int s0 = tid * per, s1 = min(s0 + per, a.slots);
    int lp = 0, lg = 0;
    for (int i = s0; i < s1; i++) {
        lp += cnt[i];
        lg += (cnt[i] + 7) >> 3;
    }
    int ip = lp, ig = lg;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int vp = __shfl_up_sync(0xffffffffu, ip, o), vg = __shfl_up_sync(0xffffffffu, ig, o);
        if (lane >= o) {
            ip += vp;
            ig += vg;
        }
    }
    if (lane == 31) {
        wsum_pos[warp] = ip;
        wsum_grp[warp] = ig;
    }
    __syncthreads();
    if (warp == 0) {
        const int vp = wsum_pos[lane], vg = wsum_grp[lane];
        int jp = vp, jg = vg;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, jp, o), ug = __shfl_up_sync(0xffffffffu, jg, o);
            if (lane >= o) {
                jp += up;
                jg += ug;
            }
        }
        wsum_pos[lane] = jp - vp;
        wsum_grp[lane] = jg - vg;
        if (lane == 31) *a.n_groups = jg;
    }
    __syncthreads();
    int bp = wsum_pos[warp] + ip - lp, bg = wsum_grp[warp] + ig - lg;
    for (int i = s0; i < s1; i++) {
        pos_base[i] = bp;
        grp_base[i] = bg;
        bp += cnt[i];
        bg += (cnt[i] + 7) >> 3;
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < 2; q++) {
        const int r = tid + q * kPlanThreads;
        if (slot[q] >= 0) {
            const int sl = slot[q], c = claim[q];
            a.sorted_route[pos_base[sl] + c] = r;
            if ((c & 7) == 0) a.groups[grp_base[sl] + (c >> 3)] = make_int4(sl, pos_base[sl] + c, min(8, cnt[sl] - c), 0);
        }
    }
    // routes without a resident expert contribute zeros
    const int nm = s_nmissing;
    for (int m = 0; m < nm; m++) {
        float* row = a.yroute + (size_t)s_missing[m] * a.hidden;
        for (int d = tid; d < a.hidden; d += kPlanThreads) row[d] = 0.f;
    }
}

// ------------------------------------------------------------------------------------------
// PTX helpers: mbarrier, bulk async copy, mma
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after kSpinLimit polls, raises the error flag and reports failure, so a
// lost completion can never hang the GPU.
constexpr uint32_t kSpinLimit = 1u << 18;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int32_t* err) {
    for (uint32_t i = 0; i < kSpinLimit; i++)
        if (mbar_try_wait(bar, parity)) return true;
    atomicExch(err, 2);
    return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t hmul2_f16(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
// The same MMA and shared load without `volatile`: the compiler may then move them freely between the
// ordering points that matter (the mbarrier wait before a piece and the refill after it, both volatile
// with a memory clobber), hoisting the next step's fragment loads above the current step's MMAs.
__device__ __forceinline__ void mma_f16_free(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                             uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Eight E2M1 codes of one packed word -> four f16x2, one hardware conversion per byte.  Byte b holds
// k = 2b (low nibble, low half of the result) and k = 2b + 1.  The values 0, 0.5 .. 6 are exact.
__device__ __forceinline__ void e2m1x8_to_f16x2(uint32_t w, uint32_t (&q)[4]) {
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
        "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
        "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
        "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
        : "=r"(q[0]), "=r"(q[1]), "=r"(q[2]), "=r"(q[3])
        : "r"(w));
}

// Two E4M3 block scales (low byte = first block) -> two f16x2 with the scale in both halves.
// e2m1 * e4m3 needs at most 6 significant bits and stays inside [2^-10, 2688]: exact in f16.
__device__ __forceinline__ void e4m3x2_to_f16_scales(uint32_t two, uint32_t& s0, uint32_t& s1) {
    uint32_t h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"((uint16_t)two));
    s0 = __byte_perm(h2, h2, 0x1010);
    s1 = __byte_perm(h2, h2, 0x3232);
}

// ------------------------------------------------------------------------------------------
// the expert kernel
//
// Every warp is an independent worker: a warp item is one 16-row MMA tile over the full K, for one
// group (<= 8 tokens).  The warp streams its own packed rows and scales through a private
// double-buffered ring with bulk async copies that it issues itself (one mbarrier per buffer, the
// TMA engine signals the bytes), so there is no producer warp, no cross-warp reduction and no
// per-item handshake between warps.  The warps of a CTA share only the group's activation tile:
// when the CTA's contiguous item range crosses into a new group, warp t converts token t's row
// (power-of-two scale into the f16 range, k-permuted) into shared memory between two CTA barriers.
// ------------------------------------------------------------------------------------------
constexpr int kGroupTokens = 8;

struct ExpertArgs {
    const uint8_t* packed;      // bank base [slots, N, K/2]
    const uint8_t* scale;       // [slots, N, K/16]
    const uint8_t* scale_frag;  // the same scales in fragment order (register-streaming kernel), or null
    const uint16_t* global;     // [slots, N]
    const void* act;            // gate_up: the layer input [tokens, K] (bf16 or f32); down: ic2 f32 [routes, K]
    int act_dtype;
    const int4* groups;
    const int32_t* sorted_route;
    const int32_t* n_groups;
    const float* route_weight;  // down only
    float* ic2;                 // gate_up out: [routes, inter] f32
    float* yroute;              // down out: [routes, hidden] f32, weighted
    int32_t* err;
    int N, top_k;
};

// The group's activation tile: warp t converts token t (t, t + kWarps, ..) of the group into shared memory as
// f16, scaled per token by a power of two so that its largest magnitude lies in [2^14, 2^15) (exact: f16 keeps
// every bit of a bf16 input and 11 bits of an f32 one), in the k-permuted order of perm_k.  Also notes the
// token's scale, route and (down projection) route weight.
template <bool GATE_UP, int K, int kWarps>
__device__ __forceinline__ void convert_group_tokens(const ExpertArgs& a, const int4 grp, uint8_t* xtile, int RSX,
                                                     float* s_xscale, int* s_route, float* s_factor, int warp, int lane) {
    for (int tk = warp; tk < grp.z; tk += kWarps) {
        const int route = a.sorted_route[grp.y + tk];
        const size_t row = GATE_UP ? (size_t)(route / a.top_k) : (size_t)route;
        const bool is_bf16 = GATE_UP && a.act_dtype == 0;
        // the lane's K / 32 values, eight consecutive k at a time, kept in registers
        float v[K / 256][8];
#pragma unroll
        for (int c8 = 0; c8 < K / 256; c8++) {
            const size_t k = row * K + c8 * 256 + lane * 8;
            if (is_bf16) {
                const uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(a.act) + k);
                const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const float2 f = bf16x2_to_f32(w[q]);
                    v[c8][2 * q] = f.x;
                    v[c8][2 * q + 1] = f.y;
                }
            } else {
                const float4 f0 = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.act) + k);
                const float4 f1 = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.act) + k + 4);
                v[c8][0] = f0.x; v[c8][1] = f0.y; v[c8][2] = f0.z; v[c8][3] = f0.w;
                v[c8][4] = f1.x; v[c8][5] = f1.y; v[c8][6] = f1.z; v[c8][7] = f1.w;
            }
        }
        float m = 0.f;
#pragma unroll
        for (int c8 = 0; c8 < K / 256; c8++)
#pragma unroll
            for (int q = 0; q < 8; q++) m = fmaxf(m, fabsf(v[c8][q]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        // largest magnitude into [2^14, 2^15): exact power-of-two scaling, f16 keeps every bit of
        // a bf16 input and 11 bits of an f32 one
        const int e = (int)((__float_as_uint(m) >> 23) & 0xff);
        float inv = 1.0f, sc = 1.0f;
        if (e > 0 && e < 255) {
            inv = __uint_as_float((uint32_t)(127 + 14 - (e - 127)) << 23);
            sc = __uint_as_float((uint32_t)(127 - 14 + (e - 127)) << 23);
        }
        __half* xrow = reinterpret_cast<__half*>(xtile + (size_t)tk * RSX);
#pragma unroll
        for (int c8 = 0; c8 < K / 256; c8++) {
            __half2 h[4];
#pragma unroll
            for (int q = 0; q < 4; q++) h[q] = __floats2half2_rn(v[c8][2 * q] * inv, v[c8][2 * q + 1] * inv);
            // eight consecutive k are one 16-byte chunk of the k-permuted row
            *reinterpret_cast<uint4*>(xrow + perm_k(c8 * 256 + lane * 8)) =
                make_uint4(*reinterpret_cast<uint32_t*>(&h[0]), *reinterpret_cast<uint32_t*>(&h[1]),
                           *reinterpret_cast<uint32_t*>(&h[2]), *reinterpret_cast<uint32_t*>(&h[3]));
        }
        if (lane == 0) {
            s_xscale[tk] = sc;
            s_route[tk] = route;
            s_factor[tk] = GATE_UP ? 1.0f : a.route_weight[route];
        }
    }
}

// GATE_UP: K = hidden, a warp item is 8 gate rows and the 8 matching up rows, so that the
// silu(gate) * up epilogue stays inside one thread; K is streamed in SUB pieces.  Otherwise
// K = inter and a warp item is 16 consecutive rows in one piece.
template <bool GATE_UP, int K_, int NT_>
struct Cfg {
    static constexpr int K = K_;
    static constexpr int NT = NT_;                       // token tiles of 8 per group
    static constexpr int kWarps = GATE_UP ? 8 : 16;      // independent workers per CTA
    static constexpr int kThreads = kWarps * 32;
    static constexpr int SUB = GATE_UP ? (NT == 1 ? 2 : 4) : 1;  // pieces of K per item
    static constexpr int D = 2;            // ring depth: pieces in flight per warp
    static constexpr int KSUB = K / SUB;
    static constexpr int WIN = KSUB / 128;               // 128-k windows per piece
    // gate_up rows are copied one by one with 64 B of padding (conflict-free 128-bit reads); down
    // rows are contiguous in the bank and arrive with one copy (two-way conflicts on the reads)
    static constexpr int RSA = GATE_UP ? KSUB / 2 + 64 : KSUB / 2;
    static constexpr int RSS = K / 16;                   // scale row: the whole K
    static constexpr int kStageBytes = 16 * RSA;
    static constexpr int kScaleBytes = 16 * RSS;
    // scales travel with an item's first piece; an item's scales must outlive all its pieces
    static constexpr int NSB = (D + SUB - 2) / SUB + 1;
    static constexpr int kWarpBytes = D * kStageBytes + NSB * kScaleBytes;
    static constexpr int RSX = K * 2 + 64;               // f16 activation row, padded
    static constexpr int kXBytes = kGroupTokens * NT * RSX;
    static constexpr size_t kSmem = (size_t)kWarps * kWarpBytes + kXBytes + 96 * NT + 8 * kWarps * D + 32;
};

// the items of one warp inside its CTA's contiguous range [ib, ie): within every group segment the
// warp takes items first + w, first + w + 8, ...
struct ItemIter {
    int g, it, ie, blocks, w, nw;
    __device__ __forceinline__ void start(int ib, int ie_, int blocks_, int w_, int nw_) {
        ie = ie_; blocks = blocks_; w = w_; nw = nw_;
        g = ib / blocks;
        it = ib + w;
        settle(ib);
    }
    // moves to the next group segment until `it` lies inside [segment begin, segment end)
    __device__ __forceinline__ void settle(int ib) {
        while (g * blocks < ie && it >= min(ie, (g + 1) * blocks)) {
            g++;
            it = max(ib, g * blocks) + w;
        }
    }
    __device__ __forceinline__ bool valid() const { return g * blocks < ie && it < ie; }
    __device__ __forceinline__ void next(int ib) {
        it += nw;
        settle(ib);
    }
};

template <bool GATE_UP, int K_, int NT, int OCC, int VAR>
__global__ void __launch_bounds__(Cfg<GATE_UP, K_, NT>::kThreads, OCC) expert_mma_kernel(ExpertArgs a) {
    using C = Cfg<GATE_UP, K_, NT>;
    constexpr int kWarps = C::kWarps;
    constexpr int kTok = kGroupTokens * NT;  // tokens per group
    constexpr int K = C::K, SUB = C::SUB, D = C::D, NSB = C::NSB, KSUB = C::KSUB, WIN = C::WIN, RSA = C::RSA, RSS = C::RSS,
                  RSX = C::RSX;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t smem_base = smem_u32(smem);
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int g8 = lane >> 2, t4 = lane & 3;
    uint8_t* const wbase = smem + (size_t)warp * C::kWarpBytes;   // [2 stages | 2 scale buffers]
    uint8_t* const xtile = smem + (size_t)kWarps * C::kWarpBytes;
    float* const s_xscale = reinterpret_cast<float*>(xtile + C::kXBytes);  // [kTok] token scales
    float* const s_factor = s_xscale + kTok;                               // [kTok] route weights (down)
    int* const s_route = reinterpret_cast<int*>(s_factor + kTok);          // [kTok] routes of the group
    uint64_t* const bars = reinterpret_cast<uint64_t*>(s_route + kTok);    // [kWarps][D]
    const uint32_t full0 = smem_u32(bars) + 8u * D * warp;
    if (lane == 0) {
        for (int q = 0; q < D; q++) mbar_init(full0 + 8u * q, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_launch_dependents();
    pdl_wait();     // the plan (groups, sorted routes) and, for the down kernel, ic2

    // contiguous item range of this CTA: item = group * blocks + block
    const int n_groups = *a.n_groups;
    const int blocks = (GATE_UP ? a.N / 2 : a.N) / (GATE_UP ? 8 : 16);
    const long long total = (long long)n_groups * blocks;
    const int ib = (int)(total * blockIdx.x / gridDim.x);
    const int ie = (int)(total * (blockIdx.x + 1) / gridDim.x);
    if (ib >= ie) return;

    // ---- copy issue: piece `half` of item `it` (group descriptor `grp`) into ring position n % D ----
    auto issue = [&](const int4 grp, int it, int half, int n) {
        const int blk = it % blocks;
        const size_t slot_rows = (size_t)grp.x * a.N;
        const uint32_t bar = full0 + 8u * (n % D);
        uint8_t* const sp = wbase + (size_t)(n % D) * C::kStageBytes;
        uint8_t* const sc = wbase + D * C::kStageBytes + (size_t)((n / SUB) % NSB) * C::kScaleBytes;
        const uint32_t bytes = 16 * (KSUB / 2) + (half == 0 ? 16 * RSS : 0);
        if (lane == 0) mbar_expect_tx(bar, bytes);
        __syncwarp();
        if (GATE_UP) {
            // ring row m: m < 8 gate row, m >= 8 the matching up row
            if (lane < 16) {
                const int pair = blk * 8 + (lane & 7);
                const int nrow = (lane < 8) ? pair : a.N / 2 + pair;
                bulk_g2s(smem_u32(sp + (size_t)lane * RSA),
                         a.packed + (slot_rows + nrow) * (size_t)(K / 2) + (size_t)half * (KSUB / 2), (uint32_t)(KSUB / 2), bar);
            } else if (lane < 18 && half == 0) {
                const int up = lane - 16;
                const int nrow = (up ? a.N / 2 : 0) + blk * 8;
                bulk_g2s(smem_u32(sc + (size_t)up * 8 * RSS), a.scale + (slot_rows + nrow) * (size_t)RSS, (uint32_t)(8 * RSS), bar);
            }
        } else {
            const size_t nrow = slot_rows + (size_t)blk * 16;
            if (lane == 0) bulk_g2s(smem_u32(sp), a.packed + nrow * (size_t)(K / 2), (uint32_t)(16 * (K / 2)), bar);
            if (lane == 1) bulk_g2s(smem_u32(sc), a.scale + nrow * (size_t)RSS, (uint32_t)(16 * RSS), bar);
        }
    };

    ItemIter cur, pre;   // the item being computed, and the one whose copies are issued next
    cur.start(ib, ie, blocks, warp, kWarps);
    pre = cur;
    int pre_half = 0, n_issued = 0, n_done = 0;
    int pre_g = -1;
    int4 pre_grp = make_int4(0, 0, 0, 0);
    auto issue_next = [&]() {
        if (!pre.valid()) return;
        if (pre.g != pre_g) {
            pre_g = pre.g;
            pre_grp = a.groups[pre_g];
        }
        issue(pre_grp, pre.it, pre_half, n_issued++);
        if (++pre_half == SUB) {
            pre_half = 0;
            pre.next(ib);
        }
    };
    // prologue: D pieces in flight
    for (int q = 0; q < D; q++) issue_next();

    // A warp whose bounded wait gave up stops working but keeps meeting the CTA barriers below.
    bool dead = false;
    const int g_first = ib / blocks, g_last = (ie - 1) / blocks;
    for (int g = g_first; g <= g_last; g++) {
        const int4 grp = a.groups[g];
        // ---- the group's activation tile: warp t converts token t ----
        __syncthreads();  // every warp is done with the previous group's tile
        convert_group_tokens<GATE_UP, K, kWarps>(a, grp, xtile, RSX, s_xscale, s_route, s_factor, warp, lane);
        __syncthreads();

        // ---- this warp's items of the group ----
        const int seg_end = min(ie, (g + 1) * blocks);
        while (!dead && cur.valid() && cur.g == g && cur.it < seg_end) {
            const int blk = cur.it % blocks;
            const size_t slot_rows = (size_t)grp.x * a.N;
            // the two rows' f16 globals: requested now (raw), converted after the MMAs
            uint16_t graw_a, graw_b;
            if (GATE_UP) {
                graw_a = a.global[slot_rows + blk * 8 + g8];
                graw_b = a.global[slot_rows + a.N / 2 + blk * 8 + g8];
            } else {
                graw_a = a.global[slot_rows + blk * 16 + g8];
                graw_b = a.global[slot_rows + blk * 16 + 8 + g8];
            }
            float acc[NT][4][4];
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int q = 0; q < 4; q++)
#pragma unroll
                    for (int r = 0; r < 4; r++) acc[nt][q][r] = 0.f;
#pragma unroll
            for (int half = 0; half < SUB; half++) {
                const int n = n_done;
                if (!mbar_wait(full0 + 8u * (n % D), (n / D) & 1, a.err)) {
                    dead = true;
                    break;
                }
                // byte offsets inside the CTA's shared memory of this lane's fragments
                const uint32_t o_sp = (uint32_t)(warp * C::kWarpBytes + (n % D) * C::kStageBytes);
                const uint32_t o_sc = (uint32_t)(warp * C::kWarpBytes + D * C::kStageBytes + ((n / SUB) % NSB) * C::kScaleBytes);
                const uint32_t row_lo = o_sp + g8 * RSA + t4 * 16, row_hi = row_lo + 8 * RSA;
                const uint32_t sc_lo = o_sc + g8 * RSS + half * (KSUB / 16), sc_hi = sc_lo + 8 * RSS;
                const uint32_t xa = (uint32_t)(kWarps * C::kWarpBytes) + g8 * RSX + t4 * 16 + half * (KSUB * 2);
                // VAR bit 0: ordinary loads and a non-volatile MMA, which the compiler may reorder inside the piece
                auto LD = [&](uint32_t off) -> uint4 {
                    if (VAR & 1) return *reinterpret_cast<const uint4*>(smem + off);
                    return lds128(smem_base + off);
                };
                {
#pragma unroll
                    for (int w2 = 0; w2 < WIN / 2; w2++) {
                        // scales of two windows: 16 bytes per row
                        const uint4 sl4 = LD(sc_lo + w2 * 16), sh4 = LD(sc_hi + w2 * 16);
                        const uint32_t slw[4] = {sl4.x, sl4.y, sl4.z, sl4.w}, shw[4] = {sh4.x, sh4.y, sh4.z, sh4.w};
#pragma unroll
                        for (int wq = 0; wq < 2; wq++) {
                            const int wi = w2 * 2 + wq;
                            const uint4 plo = LD(row_lo + wi * 64), phi = LD(row_hi + wi * 64);
                            // the lane's two scale bytes of this window: bytes 2*t4, 2*t4+1 of the window's eight
                            const uint32_t wl2 = (t4 & 2) ? slw[wq * 2 + 1] : slw[wq * 2];
                            const uint32_t wh2 = (t4 & 2) ? shw[wq * 2 + 1] : shw[wq * 2];
                            uint32_t slo0, slo1, shi0, shi1;
                            e4m3x2_to_f16_scales((t4 & 1) ? (wl2 >> 16) : (wl2 & 0xffffu), slo0, slo1);
                            e4m3x2_to_f16_scales((t4 & 1) ? (wh2 >> 16) : (wh2 & 0xffffu), shi0, shi1);
                            const uint32_t wl[4] = {plo.x, plo.y, plo.z, plo.w};
                            const uint32_t wh[4] = {phi.x, phi.y, phi.z, phi.w};
                            // VAR bit 1: the window's activation fragments are requested before its conversions
                            uint4 xpre[NT][4];
                            if (VAR & 2) {
#pragma unroll
                                for (int nt = 0; nt < NT; nt++)
#pragma unroll
                                    for (int j = 0; j < 4; j++) xpre[nt][j] = LD(xa + nt * 8 * RSX + wi * 256 + j * 64);
                            }
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                uint32_t ql[4], qh[4];
                                e2m1x8_to_f16x2(wl[j], ql);
                                e2m1x8_to_f16x2(wh[j], qh);
                                const uint32_t sl = (j < 2) ? slo0 : slo1, sh = (j < 2) ? shi0 : shi1;
#pragma unroll
                                for (int q = 0; q < 4; q++) {
                                    ql[q] = hmul2_f16(ql[q], sl);
                                    qh[q] = hmul2_f16(qh[q], sh);
                                }
                                // k slots (2t, 2t+1 | 2t+8, 2t+9) of the two MMAs <- the word's k (0,1 | 2,3), (4,5 | 6,7);
                                // the dequantised fragments serve every token tile of the group
#pragma unroll
                                for (int nt = 0; nt < NT; nt++) {
                                    const uint4 xb = (VAR & 2) ? xpre[nt][j] : LD(xa + nt * 8 * RSX + wi * 256 + j * 64);
                                    if (VAR & 1) {
                                        mma_f16_free(acc[nt][(j & 1) * 2], ql[0], qh[0], ql[1], qh[1], xb.x, xb.y);
                                        mma_f16_free(acc[nt][(j & 1) * 2 + 1], ql[2], qh[2], ql[3], qh[3], xb.z, xb.w);
                                    } else {
                                        mma_f16(acc[nt][(j & 1) * 2], ql[0], qh[0], ql[1], qh[1], xb.x, xb.y);
                                        mma_f16(acc[nt][(j & 1) * 2 + 1], ql[2], qh[2], ql[3], qh[3], xb.z, xb.w);
                                    }
                                }
                            }
                        }
                    }
                }
                n_done++;
                // every lane's reads of the buffer have returned (their values fed the MMAs above), so the
                // refill may be issued: a write-after-read across the proxies needs no fence
                __syncwarp();
                issue_next();
            }
            if (dead) break;
            // ---- epilogue: rows g8 (acc[.][0..1]) and g8 + 8 (acc[.][2..3]), tokens 2*t4, 2*t4 + 1 ----
            const float ga = f16_global_to_f32(graw_a), gb = f16_global_to_f32(graw_b);
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                float c4[4];
#pragma unroll
                for (int r = 0; r < 4; r++) c4[r] = (acc[nt][0][r] + acc[nt][1][r]) + (acc[nt][2][r] + acc[nt][3][r]);
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    const int tok = nt * 8 + 2 * t4 + c;
                    if (tok < grp.z) {
                        const float ts = s_xscale[tok];
                        const int route = s_route[tok];
                        if (GATE_UP) {
                            const float gate = c4[c] * ga * ts, up = c4[2 + c] * gb * ts;
                            a.ic2[(size_t)route * (a.N / 2) + blk * 8 + g8] = (gate / (1.0f + __expf(-gate))) * up;
                        } else {
                            const float wr = s_factor[tok];
                            a.yroute[(size_t)route * a.N + blk * 16 + g8] = wr * ((c4[c] * ts) * ga);
                            a.yroute[(size_t)route * a.N + blk * 16 + 8 + g8] = wr * ((c4[2 + c] * ts) * gb);
                        }
                    }
                }
            }
            cur.next(ib);
        }
    }
}

// ------------------------------------------------------------------------------------------
// the expert kernel, register-streaming form
//
// Same items, same fragments, same arithmetic and epilogue as expert_mma_kernel, but no shared-memory
// ring: every lane fetches its own fragments of the packed rows straight from global memory with 128-bit
// loads (a warp-wide load covers 8 rows x 64 contiguous bytes) and its block scales with 32-bit loads,
// kPre windows ahead of the window it is converting, in a rotating register buffer.  Nothing waits on a
// barrier, the only shared memory is the group's activation tile, so two CTAs (16 warps) fit an SM and
// the conversions of one warp run under the memory latency of the others.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 ldg_stream128(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
// the same with a 256-byte L2 fill: a miss brings the row's next three 64-byte windows along
__device__ __forceinline__ uint4 ldg_stream128_wide(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::256B.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ldg_nc128(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ldg_u32(const void* p) {
    uint32_t v;
    asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

template <bool GATE_UP, int K_, int NT_>
struct LdgCfg {
    static constexpr int K = K_, NT = NT_;
    static constexpr int kWarps = GATE_UP ? 10 : 8, kThreads = kWarps * 32;   // gate_up: 96 registers at 10 warps, two CTAs per SM (12 warps spill)
    static constexpr int WINS = K / 128;
    static constexpr int kPre = WINS < 4 ? WINS : 4;     // windows in flight per warp
    static constexpr int RSX = K * 2 + 64;
    static constexpr int kXBytes = kGroupTokens * NT * RSX;
    static constexpr size_t kSmem = (size_t)kXBytes + 96 * NT + 32;    // the group's activation tile and its per-token notes
};

template <bool GATE_UP, int K_, int NT, int OCC, int LV>
__global__ void __launch_bounds__((LdgCfg<GATE_UP, K_, NT>::kThreads), OCC) expert_ldg_kernel(ExpertArgs a) {
    using C = LdgCfg<GATE_UP, K_, NT>;
    constexpr int kWarps = C::kWarps, kTok = kGroupTokens * NT, K = C::K, WINS = C::WINS, P = C::kPre, RSX = C::RSX;
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int g8 = lane >> 2, t4 = lane & 3;
    uint8_t* const xtile = smem;
    float* const s_xscale = reinterpret_cast<float*>(xtile + C::kXBytes);
    float* const s_factor = s_xscale + kTok;
    int* const s_route = reinterpret_cast<int*>(s_factor + kTok);
    pdl_launch_dependents();
    pdl_wait();     // the plan (groups, sorted routes) and, for the down kernel, ic2

    const int n_groups = *a.n_groups;
    const int blocks = (GATE_UP ? a.N / 2 : a.N) / (GATE_UP ? 8 : 16);
    const long long total = (long long)n_groups * blocks;
    const int ib = (int)(total * blockIdx.x / gridDim.x);
    const int ie = (int)(total * (blockIdx.x + 1) / gridDim.x);
    if (ib >= ie) return;

    // this lane's fragment rows of an item: rows g8 and g8 + 8 of the tile, as row indices into the bank (they
    // fit 32 bits; the 64-bit addresses are formed where they are used, which keeps the register count down)
    auto rows_of = [&](int slot, int it, int& r_lo, int& r_hi) {
        const int blk = it % blocks;
        const int slot_rows = slot * a.N;
        r_lo = slot_rows + (GATE_UP ? blk * 8 + g8 : blk * 16 + g8);
        r_hi = slot_rows + (GATE_UP ? a.N / 2 + blk * 8 + g8 : blk * 16 + 8 + g8);
    };
    uint4 bl[P], bh[P];
    uint32_t cl[P], ch[P];
    // LV bit 0: the scales of two windows (16 bytes per row) come with one 128-bit load per row instead of a
    // 32-bit load per row and window: half the requests to the L1, where a load that touches eight rows costs
    // eight tag look-ups whatever its width.  LV bit 1: 256-byte L2 fill on the packed rows.
    // LV bit 2: fragment-ordered scales.  The adapter keeps a second copy of every expert's block scales in
    // the order this kernel's lanes consume them: for tile t of a slot and every group of four windows
    // (512 k), 32 lanes x 16 bytes, lane (g8, t4) holding for each of the four windows the two scale bytes
    // of its low row (blocks 2*t4, 2*t4 + 1 of the window) and the two of its high row.  One fully coalesced
    // 128-bit load per lane then serves four windows of both rows: a quarter of a load instruction and one
    // L1 tag look-up per window instead of two loads that each touch eight rows.
    constexpr bool kFragScales = (LV & 4) != 0;
    constexpr bool kPairScales = (LV & 1) != 0 && !kFragScales;
    constexpr int kGroups = WINS / 4;     // groups of four windows per item
    uint4 dl[P / 2 > 0 ? P / 2 : 1], dh[P / 2 > 0 ? P / 2 : 1];
    uint4 sf[2];
    // window w of the item whose fragment rows are r_lo / r_hi into slot sl: 16 bytes per 64-byte window step
    // of each packed row, and the 32-bit word holding scale bytes 2*t4, 2*t4 + 1 of the window's eight
    auto fetch = [&](int r_lo, int r_hi, int w, int sl) {
        const uint8_t* const q_lo = a.packed + (size_t)r_lo * (K / 2) + t4 * 16 + w * 64;
        const uint8_t* const q_hi = a.packed + (size_t)r_hi * (K / 2) + t4 * 16 + w * 64;
        bl[sl] = (LV & 2) ? ldg_stream128_wide(q_lo) : ldg_stream128(q_lo);
        bh[sl] = (LV & 2) ? ldg_stream128_wide(q_hi) : ldg_stream128(q_hi);
        if (kFragScales) {
            // loaded per group of four windows, see the item loop
        } else if (!kPairScales) {
            cl[sl] = ldg_u32(a.scale + (size_t)r_lo * (K / 16) + (t4 >> 1) * 4 + w * 8);
            ch[sl] = ldg_u32(a.scale + (size_t)r_hi * (K / 16) + (t4 >> 1) * 4 + w * 8);
        } else if ((w & 1) == 1) {
            // with the pair's second window: by then the pair that held these registers has been consumed
            dl[(sl >> 1)] = ldg_nc128(a.scale + (size_t)r_lo * (K / 16) + (w - 1) * 8);
            dh[(sl >> 1)] = ldg_nc128(a.scale + (size_t)r_hi * (K / 16) + (w - 1) * 8);
        }
    };

    ItemIter cur;
    cur.start(ib, ie, blocks, warp, kWarps);
    int cr_lo = 0, cr_hi = 0;
    const int g_first = ib / blocks, g_last = (ie - 1) / blocks;
    for (int g = g_first; g <= g_last; g++) {
        const int4 grp = a.groups[g];
        __syncthreads();  // every warp is done with the previous group's tile
        convert_group_tokens<GATE_UP, K, kWarps>(a, grp, xtile, RSX, s_xscale, s_route, s_factor, warp, lane);
        __syncthreads();
        const int seg_end = min(ie, (g + 1) * blocks);
        while (cur.valid() && cur.g == g && cur.it < seg_end) {
            const int blk = cur.it % blocks;
            rows_of(grp.x, cur.it, cr_lo, cr_hi);
#pragma unroll
            for (int p = 0; p < P; p++) fetch(cr_lo, cr_hi, p, p);
            const uint8_t* const fr = a.scale_frag + ((size_t)grp.x * blocks + blk) * (size_t)(kGroups * 512) + lane * 16;
            if (kFragScales) {
                sf[0] = ldg_nc128(fr);
                if (kGroups > 1) sf[1] = ldg_nc128(fr + 512);
            }
            const uint16_t graw_a = a.global[cr_lo], graw_b = a.global[cr_hi];
            float acc[NT][4][4];
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int q = 0; q < 4; q++)
#pragma unroll
                    for (int r = 0; r < 4; r++) acc[nt][q][r] = 0.f;
            const uint8_t* const xa = xtile + g8 * RSX + t4 * 16;
#pragma unroll
            for (int wi = 0; wi < WINS; wi++) {
                const int sl = wi % P;
                const uint4 plo = bl[sl], phi = bh[sl];
                uint32_t wl2 = 0, wh2 = 0, lo16, hi16;   // the lane's two scale bytes of the low and of the high row
                if (kFragScales) {
                    // word wi % 4 of the group's sixteen bytes: low row's two bytes | high row's two bytes
                    const uint4 g4 = sf[(wi >> 2) & 1];
                    const uint32_t word = (wi & 3) == 0 ? g4.x : (wi & 3) == 1 ? g4.y : (wi & 3) == 2 ? g4.z : g4.w;
                    lo16 = word;
                    hi16 = word >> 16;
                    // the group after next, once this group's last window has taken its word
                    if ((wi & 3) == 3 && (wi >> 2) + 2 < kGroups) sf[(wi >> 2) & 1] = ldg_nc128(fr + ((wi >> 2) + 2) * 512);
                } else if (!kPairScales) {
                    wl2 = cl[sl];
                    wh2 = ch[sl];
                } else {
                    // word (wi & 1) * 2 + (t4 >> 1) of the pair's sixteen bytes
                    const uint4 ql4 = dl[sl >> 1], qh4 = dh[sl >> 1];
                    wl2 = (wi & 1) ? ((t4 & 2) ? ql4.w : ql4.z) : ((t4 & 2) ? ql4.y : ql4.x);
                    wh2 = (wi & 1) ? ((t4 & 2) ? qh4.w : qh4.z) : ((t4 & 2) ? qh4.y : qh4.x);
                }
                // refill the slot with the window kPre ahead
                if (wi + P < WINS) fetch(cr_lo, cr_hi, wi + P, sl);
                if (!kFragScales) {
                    lo16 = (t4 & 1) ? (wl2 >> 16) : wl2;
                    hi16 = (t4 & 1) ? (wh2 >> 16) : wh2;
                }
                uint32_t slo0, slo1, shi0, shi1;
                e4m3x2_to_f16_scales(lo16, slo0, slo1);   // (the conversion reads the low 16 bits)
                e4m3x2_to_f16_scales(hi16, shi0, shi1);
                const uint32_t wl[4] = {plo.x, plo.y, plo.z, plo.w};
                const uint32_t wh[4] = {phi.x, phi.y, phi.z, phi.w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    uint32_t ql[4], qh[4];
                    e2m1x8_to_f16x2(wl[j], ql);
                    e2m1x8_to_f16x2(wh[j], qh);
                    const uint32_t s0 = (j < 2) ? slo0 : slo1, s1 = (j < 2) ? shi0 : shi1;
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        ql[q] = hmul2_f16(ql[q], s0);
                        qh[q] = hmul2_f16(qh[q], s1);
                    }
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        const uint4 xb = *reinterpret_cast<const uint4*>(xa + nt * 8 * RSX + wi * 256 + j * 64);
                        mma_f16_free(acc[nt][(j & 1) * 2], ql[0], qh[0], ql[1], qh[1], xb.x, xb.y);
                        mma_f16_free(acc[nt][(j & 1) * 2 + 1], ql[2], qh[2], ql[3], qh[3], xb.z, xb.w);
                    }
                }
            }
            // ---- epilogue: rows g8 (acc[.][0..1]) and g8 + 8 (acc[.][2..3]), tokens 2*t4, 2*t4 + 1 ----
            const float ga = f16_global_to_f32(graw_a), gb = f16_global_to_f32(graw_b);
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                float c4[4];
#pragma unroll
                for (int r = 0; r < 4; r++) c4[r] = (acc[nt][0][r] + acc[nt][1][r]) + (acc[nt][2][r] + acc[nt][3][r]);
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    const int tok = nt * 8 + 2 * t4 + c;
                    if (tok < grp.z) {
                        const float ts = s_xscale[tok];
                        const int route = s_route[tok];
                        if (GATE_UP) {
                            const float gate = c4[c] * ga * ts, up = c4[2 + c] * gb * ts;
                            a.ic2[(size_t)route * (a.N / 2) + blk * 8 + g8] = (gate / (1.0f + __expf(-gate))) * up;
                        } else {
                            const float wr = s_factor[tok];
                            a.yroute[(size_t)route * a.N + blk * 16 + g8] = wr * ((c4[c] * ts) * ga);
                            a.yroute[(size_t)route * a.N + blk * 16 + 8 + g8] = wr * ((c4[2 + c] * ts) * gb);
                        }
                    }
                }
            }
            cur.next(ib);
        }
    }
}

template <bool GATE_UP, int K_, int NT, int OCC, int LV>
void launch_expert_ldg(ExpertArgs a, int sm_count, cudaStream_t s, bool pdl) {
    using C = LdgCfg<GATE_UP, K_, NT>;
    const size_t smem = C::kSmem;
    static PerDeviceOnce once;
    allow_dyn_smem(once, expert_ldg_kernel<GATE_UP, K_, NT, OCC, LV>, smem);
    if (pdl)
        launch_pdl(expert_ldg_kernel<GATE_UP, K_, NT, OCC, LV>, dim3(sm_count * OCC), dim3(C::kThreads), smem, s, a);
    else
        expert_ldg_kernel<GATE_UP, K_, NT, OCC, LV><<<sm_count * OCC, C::kThreads, smem, s>>>(a);
}

// ------------------------------------------------------------------------------------------
// fragment-ordered scales: the copy of a slot's block scales that expert_ldg_kernel reads
//
// dst[((tile * groups + q) * 32 + lane) * 16 + 4 * w + {0, 1, 2, 3}] =
//   scale[row_lo][8 * (4q + w) + 2 * t4 + {0, 1}], scale[row_hi][8 * (4q + w) + 2 * t4 + {0, 1}]
// with lane = 4 * g8 + t4 and (row_lo, row_hi) the two rows lane's fragments belong to: gate row 8 * tile + g8
// and its up row for gate_up, rows 16 * tile + g8 and + 8 for down.  One CTA per tile, one thread per
// (group, lane).  Same bytes as the bank's scale rows, only reordered.
// ------------------------------------------------------------------------------------------
template <bool GATE_UP>
__global__ void scale_repack_kernel(const uint8_t* __restrict__ scale /* the slot's [N, K/16] */, int N, int K,
                                    uint8_t* __restrict__ dst /* the slot's fragment-ordered copy */) {
    const int tile = blockIdx.x, groups = K / 512;
    const int q = threadIdx.x / 32, lane = threadIdx.x % 32;
    if (q >= groups) return;
    const int g8 = lane >> 2, t4 = lane & 3;
    const int r_lo = GATE_UP ? tile * 8 + g8 : tile * 16 + g8;
    const int r_hi = GATE_UP ? N / 2 + tile * 8 + g8 : tile * 16 + 8 + g8;
    const int rs = K / 16;
    uint32_t w4[4];
#pragma unroll
    for (int w = 0; w < 4; w++) {
        const int off = 8 * (4 * q + w) + 2 * t4;
        const uint32_t lo = *reinterpret_cast<const uint16_t*>(scale + (size_t)r_lo * rs + off);
        const uint32_t hi = *reinterpret_cast<const uint16_t*>(scale + (size_t)r_hi * rs + off);
        w4[w] = lo | (hi << 16);
    }
    *reinterpret_cast<uint4*>(dst + ((size_t)(tile * groups + q) * 32 + lane) * 16) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
}

// latency-bound steps (a handful of tokens) chain their kernels with programmatic dependent launch: measured
// 49 -> 43 us per block at one token; at 64 tokens the early-resident CTAs only get in the way of the shared
// expert that runs beside them, so larger steps launch the ordinary way
constexpr int kPdlMaxRoutes = 128;
constexpr int kDefaultVariant = 14;   // register-streaming kernels, fragment-ordered scales, 256-byte L2 fill

template <bool GATE_UP, int K_, int NT, int OCC, int VAR>
void launch_expert_var(ExpertArgs a, int sm_count, cudaStream_t s, bool pdl) {
    using C = Cfg<GATE_UP, K_, NT>;
    static PerDeviceOnce once;   // one per instantiation
    allow_dyn_smem(once, expert_mma_kernel<GATE_UP, K_, NT, OCC, VAR>, C::kSmem);
    if (pdl)
        launch_pdl(expert_mma_kernel<GATE_UP, K_, NT, OCC, VAR>, dim3(sm_count * OCC), dim3(C::kThreads), C::kSmem, s, a);
    else
        expert_mma_kernel<GATE_UP, K_, NT, OCC, VAR><<<sm_count * OCC, C::kThreads, C::kSmem, s>>>(a);
}

// instruction-scheduling variant of the expert kernels (see VAR in the kernel); FTM_DECODE_VARIANT overrides
// the default for experiments
int decode_variant() {
    static const int v = [] {
        const char* e = getenv("FTM_DECODE_VARIANT");
        return e ? atoi(e) & 15 : kDefaultVariant;
    }();
    return v;
}

template <bool GATE_UP, int K_, int NT, int OCC>
void launch_expert(ExpertArgs a, int sm_count, cudaStream_t s, bool pdl) {
    if (decode_variant() & 4) {
        // register-streaming kernels, two CTAs per SM.  Variant bits: 1 = paired scale loads, 2 = fragment-ordered
        // scales (when the adapter keeps that copy), 8 = 256-byte L2 fill
        const int v = decode_variant();
        const bool frag = (v & 2) && a.scale_frag != nullptr;
        const int lv = (frag ? 4 : (v & 1)) | ((v & 8) ? 2 : 0);
        switch (lv) {
            case 1: launch_expert_ldg<GATE_UP, K_, NT, 2, 1>(a, sm_count, s, pdl); break;
            case 3: launch_expert_ldg<GATE_UP, K_, NT, 2, 3>(a, sm_count, s, pdl); break;
            case 4: launch_expert_ldg<GATE_UP, K_, NT, 2, 4>(a, sm_count, s, pdl); break;
            case 6:
                // down with groups of at most eight tokens needs 80 registers: three CTAs (24 warps) per SM,
                // 36.1 -> 34.2 us at T = 64 (four CTAs spill and lose)
                if constexpr (!GATE_UP && NT == 1)
                    launch_expert_ldg<GATE_UP, K_, NT, 3, 6>(a, sm_count, s, pdl);
                else
                    launch_expert_ldg<GATE_UP, K_, NT, 2, 6>(a, sm_count, s, pdl);
                break;
            default: launch_expert_ldg<GATE_UP, K_, NT, 2, 0>(a, sm_count, s, pdl); break;
        }
        return;
    }
    launch_expert_var<GATE_UP, K_, NT, OCC, 0>(a, sm_count, s, pdl);   // the shared-memory ring kernels (variant 0)
}

// Large batches: the routes are bucketed by the multi-CTA CSR build (seg / route_idx); this turns every
// bucket into groups of at most `group` routes.  One CTA; bins <= 1024.
__global__ void __launch_bounds__(1024)
groups_from_csr_kernel(const int32_t* __restrict__ seg, int bins, const int32_t* __restrict__ slot_of_bin, int slots,
                       int group, int4* __restrict__ groups, int32_t* __restrict__ n_groups) {
    __shared__ int wsum[32];
    const int b = threadIdx.x, lane = b & 31, warp = b >> 5;
    int cnt = 0, slot = -1;
    if (b < bins) {
        cnt = seg[b + 1] - seg[b];
        slot = slot_of_bin ? slot_of_bin[b] : b;
        if (slot < 0 || slot >= slots) cnt = 0;
    }
    const int ng = (cnt + group - 1) / group;
    int incl = ng;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) wsum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        const int v = wsum[lane];
        int j = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int u = __shfl_up_sync(0xffffffffu, j, o);
            if (lane >= o) j += u;
        }
        wsum[lane] = j - v;
        if (lane == 31) *n_groups = j;
    }
    __syncthreads();
    int base = wsum[warp] + incl - ng;
    if (b < bins) {
        const int start = seg[b];
        for (int q = 0; q < ng; q++) groups[base + q] = make_int4(slot, start + q * group, min(group, cnt - q * group), 0);
    }
}

// rows whose slot is -1 contribute zeros: clear the per-route outputs that no group will write
__global__ void zero_missing_routes_kernel(const int32_t* __restrict__ route_slot, int routes, int H,
                                           float* __restrict__ yroute) {
    const int r = blockIdx.x;
    if (route_slot[r] >= 0) return;
    for (int d = threadIdx.x; d < H; d += blockDim.x) yroute[(size_t)r * H + d] = 0.f;
}

}  // namespace

int launch_groups_from_csr(const int32_t* seg, int bins, const int32_t* slot_of_bin, int slots, int group,
                           int4* groups, int32_t* n_groups, const Ctx& c) {
    c.begin(K_DECODE_PLAN);
    groups_from_csr_kernel<<<1, 1024, 0, c.s>>>(seg, bins, slot_of_bin, slots, group, groups, n_groups);
    c.end();
    return 1;
}

int launch_scale_repack(const BankView& b, int slot, uint8_t* gu_scale_frag, uint8_t* dn_scale_frag, const Ctx& c) {
    const int N1 = 2 * b.inter, K1 = b.hidden, N2 = b.hidden, K2 = b.inter;
    if (K1 % 512 || K2 % 512 || N1 % 16 || N2 % 16) return 0;   // shapes the register-streaming kernels do not take
    const size_t s1 = (size_t)N1 * K1 / 16, s2 = (size_t)N2 * K2 / 16;
    c.begin(K_CAST);
    scale_repack_kernel<true><<<N1 / 16, 32 * (K1 / 512), 0, c.s>>>(b.gu_scale + (size_t)slot * s1, N1, K1,
                                                                     gu_scale_frag + (size_t)slot * s1);
    scale_repack_kernel<false><<<N2 / 16, 32 * (K2 / 512), 0, c.s>>>(b.dn_scale + (size_t)slot * s2, N2, K2,
                                                                      dn_scale_frag + (size_t)slot * s2);
    c.end();
    return 2;
}

size_t decode_plan_smem(int slots) { return (size_t)3 * slots * sizeof(int); }

bool decode_mma_supported(int hidden, int inter, int routes, int slots, int experts, bool have_expert_ids) {
    // the tensor-core kernels are instantiated for the production expert shape; every other
    // multiple-of-16 shape takes the per-route kernels
    if (hidden != 2048 || inter != 512) return false;
    if (routes <= kPlanMaxRoutes) return decode_plan_smem(slots) <= 180 * 1024;
    // larger batches bucket by expert id (or by slot when slot ids were given): at most 1024 bins
    return have_expert_ids ? experts <= 1024 : slots <= 1024;
}

int launch_decode_mma(const BankView& b, const void* x, int x_dtype, const DecodeRoutes& rt,
                      const float* route_weight, int tokens, int top_k, DecodeScratch sc, int sm_count,
                      const Ctx& c) {
    const int routes = tokens * top_k;
    const bool small = routes <= kPlanMaxRoutes;
    int launches = 0;
    if (small) {
        PlanArgs pa{};
        pa.route_slot_in = rt.route_slot_in;
        pa.expert_ids = rt.expert_ids; pa.ids_dtype = rt.ids_dtype; pa.layer = rt.layer; pa.experts = rt.experts;
        pa.n_ids = rt.n_ids; pa.slot_for_id = rt.slot_for_id; pa.route_slot_out = rt.route_slot_out;
        pa.routes = routes; pa.slots = b.slots; pa.hidden = b.hidden;
        pa.groups = sc.groups; pa.sorted_route = sc.sorted_route; pa.n_groups = sc.n_groups; pa.yroute = sc.yroute;
        pa.bad_flag = rt.bad_flag;
        const size_t psmem = decode_plan_smem(b.slots);
        static PerDeviceOnce once;
        allow_dyn_smem(once, decode_plan_kernel, 200 * 1024);
        c.begin(K_DECODE_PLAN);
        if (routes <= kPdlMaxRoutes)
            launch_pdl(decode_plan_kernel, dim3(1), dim3(kPlanThreads), psmem, c.s, pa);
        else
            decode_plan_kernel<<<1, kPlanThreads, psmem, c.s>>>(pa);
        c.end();
        launches += 1;
    } else {
        // bucket by expert id of the layer (serving call) or by slot id, then cut into groups of 16
        const int32_t* bins_of_route;
        const int32_t* slot_of_bin = nullptr;
        int nbins;
        if (rt.expert_ids) {
            launches += launch_slot_rewrite(rt.expert_ids, rt.ids_dtype, routes, rt.layer, rt.experts, rt.slot_for_id,
                                            rt.n_ids, rt.route_slot_out, sc.route_bin, rt.bad_flag, c);
            bins_of_route = sc.route_bin;
            slot_of_bin = rt.slot_for_id + (size_t)rt.layer * rt.experts;
            nbins = rt.experts;
        } else {
            bins_of_route = rt.route_slot_in;
            nbins = b.slots;
        }
        launches += launch_csr_build(bins_of_route, routes, nbins, sc.seg, sc.sorted_route, sc.csr_scratch, sc.csr_flag, c);
        c.begin(K_DECODE_PLAN);
        groups_from_csr_kernel<<<1, 1024, 0, c.s>>>(sc.seg, nbins, slot_of_bin, b.slots, 16, sc.groups, sc.n_groups);
        zero_missing_routes_kernel<<<routes, 256, 0, c.s>>>(rt.expert_ids ? rt.route_slot_out : rt.route_slot_in, routes,
                                                           b.hidden, sc.yroute);
        c.end();
        launches += 2;
    }

    ExpertArgs a{};
    a.groups = sc.groups;
    a.sorted_route = sc.sorted_route;
    a.n_groups = sc.n_groups;
    a.err = sc.err;
    a.top_k = top_k;
    // gate_up: K = hidden, N = 2 * inter rows
    a.packed = b.gu_packed; a.scale = b.gu_scale; a.scale_frag = b.gu_scale_frag; a.global = b.gu_global;
    a.act = x; a.act_dtype = x_dtype; a.ic2 = sc.ic2p; a.N = 2 * b.inter;
    c.begin(K_EXPERT_GATE_UP);
    if (small)
        launch_expert<true, 2048, 1, 1>(a, sm_count, c.s, routes <= kPdlMaxRoutes);
    else
        launch_expert<true, 2048, 2, 1>(a, sm_count, c.s, false);
    c.end();
    // down: K = inter, N = hidden rows
    a.packed = b.dn_packed; a.scale = b.dn_scale; a.scale_frag = b.dn_scale_frag; a.global = b.dn_global;
    a.act = sc.ic2p; a.act_dtype = 1; a.yroute = sc.yroute; a.route_weight = route_weight; a.N = b.hidden;
    c.begin(K_EXPERT_DOWN);
    if (small)
        launch_expert<false, 512, 1, 1>(a, sm_count, c.s, routes <= kPdlMaxRoutes);
    else
        launch_expert<false, 512, 2, 1>(a, sm_count, c.s, false);
    c.end();
    return launches + 2;
}

}  // namespace ftm
