// Routed experts for small batches (decode): a bandwidth-bound grouped GEMV.
//
// Same arithmetic as the per-route kernels in decode_gemv.cu (reference:
// src/domain/expert_kernel.rs:547-618, python/ferrum_kernel/nvfp4_moe.py:186-294), organised so
// that every expert byte is read from HBM once per step however many tokens route to it:
//
//   plan      one CTA sorts the routes by slot (stable), cuts every slot's run into groups of at
//             most 8 routes and writes the group list.  No host round trip: the expert kernels
//             read the group count from device memory.
//   permute   activations are copied once into a k-permuted bf16 matrix whose rows can be fetched
//             with one bulk copy and read as tensor-core B fragments without bank conflicts.
//   experts   persistent CTAs, one per SM, each owning a contiguous range of (group, row-block)
//             items.  A producer warp streams the packed E2M1 rows and E4M3 scales of an item into
//             a ring of shared-memory stages with bulk async copies (TMA engine, mbarrier
//             completion); eight consumer warps read 128-bit fragments, dequantise in registers
//             (bit-placement E2M1 -> bf16, times the block scale, exact) and feed
//             mma.sync.m16n8k16 with the group's (<= 8) tokens as the N dimension, f32 accumulate.
//             K is split across the warps of a row tile and reduced through shared memory.
//             gate_up fuses global scale + silu(gate) * up and writes ic2 (bf16, k-permuted for the
//             down pass); down fuses global scale and route weight and writes one f32 row per route.
//
// The weights stay in the reference's bank layout (row-major packed nibbles, low nibble = even k).
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

// Activations -> f16, k-permuted, each token scaled by a power of two so that its largest
// magnitude lands in [2^14, 2^15): the tensor-core operands are f16 (the E2M1 -> f16 conversion is a
// hardware instruction), and the per-token scale keeps any bf16/f32 input inside the f16 range
// without losing bits (bf16 carries 8 significant bits, f16 11).  tok_scale[t] undoes it.
__global__ void __launch_bounds__(256)
prep_act_kernel(const void* __restrict__ x, int dtype, int K, __half* __restrict__ xh, float* __restrict__ tok_scale) {
    __shared__ float wmax[8];
    __shared__ float s_inv;
    const int t = blockIdx.x;
    const size_t base = (size_t)t * K;
    float m = 0.f;
    for (int k = threadIdx.x; k < K; k += 256) m = fmaxf(m, fabsf(load_act(x, dtype, base + k)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        float mm = 0.f;
        for (int w = 0; w < 8; w++) mm = fmaxf(mm, wmax[w]);
        // 2^(14 - floor(log2 mm)) by exponent arithmetic; zero, subnormal or non-finite rows keep scale 1
        const int e = (int)((__float_as_uint(mm) >> 23) & 0xff);
        float inv = 1.0f, sc = 1.0f;
        if (e > 0 && e < 255) {
            inv = __uint_as_float((uint32_t)(127 + 14 - (e - 127)) << 23);
            sc = __uint_as_float((uint32_t)(127 - 14 + (e - 127)) << 23);
        }
        s_inv = inv;
        tok_scale[t] = sc;
    }
    __syncthreads();
    const float inv = s_inv;
    for (int k = threadIdx.x; k < K; k += 256)
        xh[base + perm_k(k)] = __float2half_rn(load_act(x, dtype, base + k) * inv);
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
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
// ------------------------------------------------------------------------------------------
constexpr int kConsumerWarps = 8;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kGroupTokens = 8;

struct ExpertArgs {
    const uint8_t* packed;    // bank base [slots, N, K/2]
    const uint8_t* scale;     // [slots, N, K/16]
    const uint16_t* global;   // [slots, N]
    const void* act;          // k-permuted activations: gate_up f16 [tokens, K], down f32 [routes, K]
    const float* tok_scale;   // gate_up: per-token power-of-two scale of act
    const int4* groups;
    const int32_t* sorted_route;
    const int32_t* n_groups;
    const float* route_weight;  // down only
    float* ic2;                 // gate_up out: [routes, inter] f32, k-permuted
    float* yroute;              // down out: [routes, hidden] f32, weighted
    int32_t* err;
    int N, top_k, stages;
};

// GATE_UP: K = hidden, an item is ROWS/2 gate rows and the matching ROWS/2 up rows, so that the
// silu(gate) * up epilogue stays inside one thread.  Otherwise K = inter and an item is ROWS rows.
// KS warps split K for one 16-row tile; WIN = K / 128 / KS windows of 128 k per warp.
template <bool GATE_UP, int KS, int WIN>
struct Cfg {
    static constexpr int K = 128 * KS * WIN;
    static constexpr int kRowTiles = kConsumerWarps / KS;
    static constexpr int ROWS = 16 * kRowTiles;
    // gate_up rows are copied one by one with 64 B of padding (conflict-free 128-bit reads); down
    // rows are contiguous in the bank and arrive with one copy (two-way conflicts on the reads)
    static constexpr int RSA = GATE_UP ? K / 2 + 64 : K / 2;
    static constexpr int RSS = K / 16;
    static constexpr int kStageBytes = ROWS * (RSA + RSS);
};

template <bool GATE_UP, int KS, int WIN, int OCC>
__global__ void __launch_bounds__(kThreads, OCC) expert_mma_kernel(ExpertArgs a) {
    using C = Cfg<GATE_UP, KS, WIN>;
    constexpr int K = C::K, ROWS = C::ROWS, RSA = C::RSA, RSS = C::RSS;
    extern __shared__ __align__(128) uint8_t smem[];
    // layout: [stages][packed rows | scale rows] | reduce[2][warps][32 lanes][4 f32] | barriers
    uint8_t* const stage0 = smem;
    float* const red = reinterpret_cast<float*>(stage0 + (size_t)a.stages * C::kStageBytes);
    uint64_t* const bars = reinterpret_cast<uint64_t*>(red + 2 * kConsumerWarps * 128);
    // bars: full[stages], empty[stages], redfull[2], redempty[2]
    const uint32_t bar0 = smem_u32(bars);
    auto FULL = [&](int s) { return bar0 + 8u * s; };
    auto EMPTY = [&](int s) { return bar0 + 8u * (a.stages + s); };
    auto RFULL = [&](int s) { return bar0 + 8u * (2 * a.stages + s); };
    auto REMPTY = [&](int s) { return bar0 + 8u * (2 * a.stages + 2 + s); };

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; s++) {
            mbar_init(FULL(s), 1);
            mbar_init(EMPTY(s), kConsumerWarps);
        }
        for (int s = 0; s < 2; s++) {
            mbar_init(RFULL(s), KS > 1 ? (KS - 1) * C::kRowTiles : 1);
            mbar_init(REMPTY(s), C::kRowTiles);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // contiguous item range of this CTA: item = group * blocks + block
    const int n_groups = *a.n_groups;
    constexpr int kOutRows = GATE_UP ? ROWS / 2 : ROWS;  // output rows per item (pairs for gate_up)
    const int blocks = (GATE_UP ? a.N / 2 : a.N) / kOutRows;
    const long long total = (long long)n_groups * blocks;
    const int item_begin = (int)(total * blockIdx.x / gridDim.x);
    const int item_end = (int)(total * (blockIdx.x + 1) / gridDim.x);
    if (item_begin >= item_end) return;
    int g = item_begin / blocks, blk = item_begin % blocks;
    int4 grp = a.groups[g];

    if (warp == kConsumerWarps) {
        // ===================== producer: bulk copies of the packed rows and their scales ==========
        int st = 0, phase = 0;
        for (int item = item_begin; item < item_end; item++) {
            if (!mbar_wait(EMPTY(st), phase ^ 1, a.err)) return;
            if (lane == 0) mbar_expect_tx(FULL(st), (uint32_t)(ROWS * (K / 2 + K / 16)));
            __syncwarp();
            uint8_t* const sp = stage0 + (size_t)st * C::kStageBytes;
            const size_t slot_rows = (size_t)grp.x * a.N;
            if (GATE_UP) {
                // stage row r = tile * 16 + m: m < 8 gate row, m >= 8 the matching up row
                for (int r = lane; r < ROWS; r += 32) {
                    const int tile = r / 16, m = r % 16;
                    const int pair = blk * (ROWS / 2) + tile * 8 + (m & 7);
                    const int n = (m < 8) ? pair : a.N / 2 + pair;
                    bulk_g2s(smem_u32(sp + (size_t)r * RSA), a.packed + (slot_rows + n) * (size_t)(K / 2),
                             (uint32_t)(K / 2), FULL(st));
                }
                // scales: eight consecutive rows per copy
                for (int c8 = lane; c8 < ROWS / 8; c8 += 32) {
                    const int tile = c8 / 2, up = c8 & 1;
                    const int n = (up ? a.N / 2 : 0) + blk * (ROWS / 2) + tile * 8;
                    bulk_g2s(smem_u32(sp + (size_t)ROWS * RSA + (size_t)c8 * 8 * RSS),
                             a.scale + (slot_rows + n) * (size_t)(K / 16), (uint32_t)(8 * K / 16), FULL(st));
                }
            } else if (lane == 0) {
                const size_t n = slot_rows + (size_t)blk * ROWS;
                bulk_g2s(smem_u32(sp), a.packed + n * (size_t)(K / 2), (uint32_t)(ROWS * (K / 2)), FULL(st));
                bulk_g2s(smem_u32(sp + (size_t)ROWS * RSA), a.scale + n * (size_t)(K / 16), (uint32_t)(ROWS * (K / 16)),
                         FULL(st));
            }
            if (++st == a.stages) {
                st = 0;
                phase ^= 1;
            }
            if (++blk == blocks) {
                blk = 0;
                g++;
                if (item + 1 < item_end) grp = a.groups[g];
            }
        }
        return;
    }

    // ===================== consumers ==========================================================
    const int tile = warp / KS, ks = warp % KS;     // row tile of the item, K split index
    const int g8 = lane >> 2, t4 = lane & 3;        // fragment row group and k lane
    uint4 xf[WIN * 4];                              // this warp's B fragments of the current group
    float xscale = 1.0f;                            // down: this lane's token (g8) scale
    // per group, for the two token columns (2*t4, 2*t4+1) this lane's accumulators hold: the route
    // and its factor (gate_up: the token's activation scale; down: the route weight)
    int route0 = 0, route1 = 0;
    float rw0 = 0.f, rw1 = 0.f;
    int st = 0, phase = 0;
    int rs = 0, rphase = 0;
    bool new_group = true;
    for (int item = item_begin; item < item_end; item++) {
        if (new_group) {
            // Token g8's activations straight from global memory (they are small and L2-resident):
            // this warp's k slice, in the k-permuted layout, 16 bytes per (window, step).
            route0 = (2 * t4 < grp.z) ? a.sorted_route[grp.y + 2 * t4] : 0;
            route1 = (2 * t4 + 1 < grp.z) ? a.sorted_route[grp.y + 2 * t4 + 1] : 0;
            const int my_route = a.sorted_route[grp.y + (g8 < grp.z ? g8 : 0)];
            rw0 = GATE_UP ? a.tok_scale[route0 / a.top_k] : a.route_weight[route0];
            rw1 = GATE_UP ? a.tok_scale[route1 / a.top_k] : a.route_weight[route1];
            if (GATE_UP) {
                const uint4* xp = reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(a.act) +
                                                                 (size_t)(my_route / a.top_k) * K + ks * WIN * 128) + t4;
#pragma unroll
                for (int wi = 0; wi < WIN; wi++)
#pragma unroll
                    for (int j = 0; j < 4; j++) xf[wi * 4 + j] = xp[wi * 16 + j * 4];
            } else {
                // ic2 is f32: scale token g8 by a power of two into the f16 range and pack.  The
                // scale is taken over this warp's own k slice; the partial sums are rescaled before
                // they leave the warp.
                const uint4* xp = reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(a.act) +
                                                                 (size_t)my_route * K + ks * WIN * 128) + t4 * 2;
                uint4 raw[WIN * 8];
                float m = 0.f;
#pragma unroll
                for (int wi = 0; wi < WIN; wi++)
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        raw[(wi * 4 + j) * 2] = xp[wi * 32 + j * 8];
                        raw[(wi * 4 + j) * 2 + 1] = xp[wi * 32 + j * 8 + 1];
                    }
#pragma unroll
                for (int q = 0; q < WIN * 8; q++)
                    m = fmaxf(m, fmaxf(fmaxf(fabsf(__uint_as_float(raw[q].x)), fabsf(__uint_as_float(raw[q].y))),
                                       fmaxf(fabsf(__uint_as_float(raw[q].z)), fabsf(__uint_as_float(raw[q].w)))));
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
                const int e = (int)((__float_as_uint(m) >> 23) & 0xff);
                float inv = 1.0f;
                xscale = 1.0f;
                if (e > 0 && e < 255) {
                    inv = __uint_as_float((uint32_t)(127 + 14 - (e - 127)) << 23);
                    xscale = __uint_as_float((uint32_t)(127 - 14 + (e - 127)) << 23);
                }
#pragma unroll
                for (int q = 0; q < WIN * 4; q++) {
                    const uint4 u = raw[2 * q], v = raw[2 * q + 1];
                    __half2 h0 = __floats2half2_rn(__uint_as_float(u.x) * inv, __uint_as_float(u.y) * inv);
                    __half2 h1 = __floats2half2_rn(__uint_as_float(u.z) * inv, __uint_as_float(u.w) * inv);
                    __half2 h2 = __floats2half2_rn(__uint_as_float(v.x) * inv, __uint_as_float(v.y) * inv);
                    __half2 h3 = __floats2half2_rn(__uint_as_float(v.z) * inv, __uint_as_float(v.w) * inv);
                    xf[q] = make_uint4(*reinterpret_cast<uint32_t*>(&h0), *reinterpret_cast<uint32_t*>(&h1),
                                       *reinterpret_cast<uint32_t*>(&h2), *reinterpret_cast<uint32_t*>(&h3));
                }
            }
            new_group = false;
        }
        // the warp that gathers the K partials of this item and writes its outputs rotates, so the
        // extra work is spread over the KS warps of a row tile
        const int gatherer = (KS > 1) ? (item % KS) : 0;
        // the two rows' f16 globals: requested now (raw), converted after the MMAs
        uint16_t graw_a = 0, graw_b = 0;
        if (ks == gatherer) {
            const size_t slot_rows = (size_t)grp.x * a.N;
            if (GATE_UP) {
                const int pair = blk * (ROWS / 2) + tile * 8 + g8;
                graw_a = a.global[slot_rows + pair];
                graw_b = a.global[slot_rows + a.N / 2 + pair];
            } else {
                const int d = blk * ROWS + tile * 16 + g8;
                graw_a = a.global[slot_rows + d];
                graw_b = a.global[slot_rows + d + 8];
            }
        }

        if (!mbar_wait(FULL(st), phase, a.err)) return;
        const uint32_t sp = smem_u32(stage0 + (size_t)st * C::kStageBytes);
        const uint32_t row_lo = sp + (tile * 16 + g8) * RSA + t4 * 16 + ks * WIN * 64;
        const uint32_t row_hi = row_lo + 8 * RSA;
        // this warp's scale bytes of the two rows: WIN * 8 consecutive bytes each
        const uint32_t sc_lo = sp + ROWS * RSA + (tile * 16 + g8) * RSS + ks * WIN * 8;
        const uint32_t sc_hi = sc_lo + 8 * RSS;
        uint32_t scl[WIN * 2], sch[WIN * 2];
#pragma unroll
        for (int q = 0; q < WIN / 2; q++) {
            const uint4 v = lds128(sc_lo + q * 16), u = lds128(sc_hi + q * 16);
            scl[q * 4 + 0] = v.x; scl[q * 4 + 1] = v.y; scl[q * 4 + 2] = v.z; scl[q * 4 + 3] = v.w;
            sch[q * 4 + 0] = u.x; sch[q * 4 + 1] = u.y; sch[q * 4 + 2] = u.z; sch[q * 4 + 3] = u.w;
        }
        uint4 plo[WIN], phi[WIN];
#pragma unroll
        for (int wi = 0; wi < WIN; wi++) {
            plo[wi] = lds128(row_lo + wi * 64);
            phi[wi] = lds128(row_hi + wi * 64);
        }
        // everything this warp needs from the stage is in registers: hand the stage back now, so the
        // next copy overlaps the arithmetic
        __syncwarp();
        if (lane == 0) mbar_arrive(EMPTY(st));
        if (++st == a.stages) {
            st = 0;
            phase ^= 1;
        }
        float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int wi = 0; wi < WIN; wi++) {
            // the lane's two scale bytes of this window: bytes 2*t4, 2*t4+1 of the window's eight
            const uint32_t wl2 = (t4 & 2) ? scl[wi * 2 + 1] : scl[wi * 2];
            const uint32_t wh2 = (t4 & 2) ? sch[wi * 2 + 1] : sch[wi * 2];
            uint32_t slo0, slo1, shi0, shi1;
            e4m3x2_to_f16_scales((t4 & 1) ? (wl2 >> 16) : (wl2 & 0xffffu), slo0, slo1);
            e4m3x2_to_f16_scales((t4 & 1) ? (wh2 >> 16) : (wh2 & 0xffffu), shi0, shi1);
            const uint32_t wl[4] = {plo[wi].x, plo[wi].y, plo[wi].z, plo[wi].w};
            const uint32_t wh[4] = {phi[wi].x, phi[wi].y, phi[wi].z, phi[wi].w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint4 xb = xf[wi * 4 + j];
                uint32_t ql[4], qh[4];
                e2m1x8_to_f16x2(wl[j], ql);
                e2m1x8_to_f16x2(wh[j], qh);
                const uint32_t sl = (j < 2) ? slo0 : slo1, sh = (j < 2) ? shi0 : shi1;
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    ql[q] = hmul2_f16(ql[q], sl);
                    qh[q] = hmul2_f16(qh[q], sh);
                }
                // k slots (2t, 2t+1 | 2t+8, 2t+9) of the two MMAs <- the word's k (0,1 | 2,3) and (4,5 | 6,7)
                mma_f16(acc[0], ql[0], qh[0], ql[1], qh[1], xb.x, xb.y);
                mma_f16(acc[1], ql[2], qh[2], ql[3], qh[3], xb.z, xb.w);
            }
        }
        float c4[4];
#pragma unroll
        for (int q = 0; q < 4; q++) c4[q] = acc[0][q] + acc[1][q];
        if (!GATE_UP) {
            // undo this warp's token scales: columns 2*t4, 2*t4+1 belong to the lanes with g8 == column
            const float s0 = __shfl_sync(0xffffffffu, xscale, (2 * t4) * 4);
            const float s1 = __shfl_sync(0xffffffffu, xscale, (2 * t4 + 1) * 4);
            c4[0] *= s0; c4[1] *= s1; c4[2] *= s0; c4[3] *= s1;
        }

        // ---- K reduction across the warps of this row tile ----
        if (KS > 1) {
            float* const buf = red + (size_t)rs * kConsumerWarps * 128;
            if (ks != gatherer) {
                if (!mbar_wait(REMPTY(rs), rphase ^ 1, a.err)) return;
                *reinterpret_cast<float4*>(buf + warp * 128 + lane * 4) = make_float4(c4[0], c4[1], c4[2], c4[3]);
                __syncwarp();
                if (lane == 0) mbar_arrive(RFULL(rs));
            } else {
                // The gatherer changes from item to item, so it first observes that the previous use
                // of this buffer was drained (which implies that use's RFULL phase completed): a
                // parity wait is only meaningful when the waiter is at most one phase behind.
                if (!mbar_wait(REMPTY(rs), rphase ^ 1, a.err)) return;
                if (!mbar_wait(RFULL(rs), rphase, a.err)) return;
#pragma unroll
                for (int o = 0; o < KS; o++) {
                    if (o == gatherer) continue;
                    const float4 v = *reinterpret_cast<const float4*>(buf + (tile * KS + o) * 128 + lane * 4);
                    c4[0] += v.x; c4[1] += v.y; c4[2] += v.z; c4[3] += v.w;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(REMPTY(rs));
            }
            rs ^= 1;
            if (rs == 0) rphase ^= 1;
        }

        // ---- epilogue (the gathering warp of each row tile) ----
        // c4[0], c4[1]: fragment row g8, tokens 2*t4, 2*t4+1;  c4[2], c4[3]: row g8 + 8
        if (ks == gatherer) {
            const float ga = f16_global_to_f32(graw_a), gb = f16_global_to_f32(graw_b);
            if (GATE_UP) {
                const int pk = perm_k(blk * (ROWS / 2) + tile * 8 + g8);
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    if (2 * t4 + c < grp.z) {
                        const float ts = c ? rw1 : rw0;
                        const float gate = c4[c] * ga * ts, up = c4[2 + c] * gb * ts;
                        a.ic2[(size_t)(c ? route1 : route0) * (a.N / 2) + pk] = (gate / (1.0f + __expf(-gate))) * up;
                    }
                }
            } else {
                const int d = blk * ROWS + tile * 16 + g8;
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const float gd = h ? gb : ga;
#pragma unroll
                    for (int c = 0; c < 2; c++)
                        if (2 * t4 + c < grp.z)
                            a.yroute[(size_t)(c ? route1 : route0) * a.N + d + 8 * h] =
                                (c ? rw1 : rw0) * (c4[2 * h + c] * gd);
                }
            }
        }
        if (++blk == blocks) {
            blk = 0;
            g++;
            if (item + 1 < item_end) grp = a.groups[g];
            new_group = true;
        }
    }
}

template <bool GATE_UP, int KS, int WIN>
size_t expert_smem_bytes(int stages) {
    using C = Cfg<GATE_UP, KS, WIN>;
    return (size_t)stages * C::kStageBytes + 2 * kConsumerWarps * 128 * sizeof(float) +
           (2 * stages + 4) * sizeof(uint64_t) + 128;
}

// OCC persistent CTAs per SM share its shared memory: as many stages as fit in their share, at most 8
template <bool GATE_UP, int KS, int WIN, int OCC>
void launch_expert(ExpertArgs a, int sm_count, cudaStream_t s) {
    const size_t budget = (OCC == 1 ? 200 : 110) * 1024;
    int stages = 8;
    while (stages > 2 && expert_smem_bytes<GATE_UP, KS, WIN>(stages) > budget) stages--;
    a.stages = stages;
    const size_t smem = expert_smem_bytes<GATE_UP, KS, WIN>(stages);
    static bool attr = false;
    if (!attr) {
        cudaFuncSetAttribute(expert_mma_kernel<GATE_UP, KS, WIN, OCC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)(OCC == 1 ? 220 * 1024 : 112 * 1024));
        attr = true;
    }
    expert_mma_kernel<GATE_UP, KS, WIN, OCC><<<sm_count * OCC, kThreads, smem, s>>>(a);
}

}  // namespace

size_t decode_plan_smem(int slots) { return (size_t)3 * slots * sizeof(int); }

bool decode_mma_supported(int hidden, int inter, int routes, int slots) {
    // the tensor-core decode kernels are instantiated for the production expert shape; every other
    // multiple-of-16 shape takes the per-route kernels
    return hidden == 2048 && inter == 512 && routes <= kPlanMaxRoutes && decode_plan_smem(slots) <= 180 * 1024;
}

int launch_decode_mma(const BankView& b, const void* x, int x_dtype, const DecodeRoutes& rt,
                      const float* route_weight, int tokens, int top_k, DecodeScratch sc, int sm_count,
                      const Ctx& c) {
    const int routes = tokens * top_k;
    c.begin(K_PERMUTE_ACT);
    prep_act_kernel<<<tokens, 256, 0, c.s>>>(x, x_dtype, b.hidden, sc.xh, sc.tok_scale);
    c.end();
    PlanArgs pa{};
    pa.route_slot_in = rt.route_slot_in;
    pa.expert_ids = rt.expert_ids; pa.ids_dtype = rt.ids_dtype; pa.layer = rt.layer; pa.experts = rt.experts;
    pa.n_ids = rt.n_ids; pa.slot_for_id = rt.slot_for_id; pa.route_slot_out = rt.route_slot_out;
    pa.routes = routes; pa.slots = b.slots; pa.hidden = b.hidden;
    pa.groups = sc.groups; pa.sorted_route = sc.sorted_route; pa.n_groups = sc.n_groups; pa.yroute = sc.yroute;
    pa.bad_flag = rt.bad_flag;
    const size_t psmem = decode_plan_smem(b.slots);
    static bool pattr = false;
    if (!pattr) {
        cudaFuncSetAttribute(decode_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        pattr = true;
    }
    c.begin(K_DECODE_PLAN);
    decode_plan_kernel<<<1, kPlanThreads, psmem, c.s>>>(pa);
    c.end();

    ExpertArgs a{};
    a.groups = sc.groups;
    a.sorted_route = sc.sorted_route;
    a.n_groups = sc.n_groups;
    a.err = sc.err;
    a.top_k = top_k;
    // gate_up: K = hidden, N = 2 * inter rows
    a.packed = b.gu_packed; a.scale = b.gu_scale; a.global = b.gu_global;
    a.act = sc.xh; a.tok_scale = sc.tok_scale; a.ic2 = sc.ic2p; a.N = 2 * b.inter;
    c.begin(K_EXPERT_GATE_UP);
    launch_expert<true, 8, 2, 2>(a, sm_count, c.s);   // K = 2048: 8 warps x 2 windows, 16 rows per item
    c.end();
    // down: K = inter, N = hidden rows
    a.packed = b.dn_packed; a.scale = b.dn_scale; a.global = b.dn_global;
    a.act = sc.ic2p; a.yroute = sc.yroute; a.route_weight = route_weight; a.N = b.hidden;
    c.begin(K_EXPERT_DOWN);
    launch_expert<false, 2, 2, 2>(a, sm_count, c.s);  // K = 512: 2 warps x 2 windows, 64 rows per item
    c.end();
    return 4;
}

}  // namespace ftm
