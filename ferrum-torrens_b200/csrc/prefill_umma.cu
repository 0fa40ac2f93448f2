// Routed experts for large batches (prefill): a grouped SwiGLU GEMM on the 5th-generation tensor
// cores (tcgen05.mma, accumulators in tensor memory, activation tiles staged by TMA).
//
// Same arithmetic as the decode kernels (reference: src/domain/expert_kernel.rs:547-618,
// python/ferrum_kernel/nvfp4_moe.py:297-396 `_nvfp4_grouped_gemm_kernel`): per expert segment of the
// CSR, D[tokens, rows] = X[tokens, K] * W[rows, K]^T with W = e2m1 * e4m3 block scale, f32 accumulate,
// the f16 row global applied once after the K reduction.
//
//   gather    the routes are sorted by expert (CSR); xg[i] = f16(x[token of route_idx[i]] * 2^-e) with a
//             per-row power-of-two scale (exact, keeps any bf16 / f32 input inside the f16 range)
//   gemm      unit = (pass of <= 128 sorted rows of one expert, 256 weight rows = two tiles of 128);
//             persistent CTAs of 28 warps:
//               warp 0       TMA: activation tiles [32..128 tokens x 64 k] f16, 128-byte swizzle (B operand)
//               warp 2       TMA: packed weight rows (256 k = one 128-byte line per row, 128-byte swizzle)
//                            and block scales into a raw ring
//               warps 8..23  four dequantiser sets of four warps: hardware e2m1x2 / e4m3x2 -> f16x2, exact
//                            product with the block scale, stored into tensor memory (tcgen05.st).  The
//                            weights are the A operand, one TMEM lane per weight row, so the dequantised
//                            weights never cross shared memory
//               warps 1, 3   issue tcgen05.mma (TS form), one warp per row tile (M = 128, N = tokens
//                            rounded up to 16, K = 16 per instruction, f16 x f16 -> f32 in TMEM), commit
//                            to mbarriers
//               warps 4..7, 24..27  epilogue, one set per row tile: tcgen05.ld of the accumulators while
//                            the dequantisers already convert the next unit; a thread owns a weight row,
//                            so stores are coalesced over rows
//             The down GEMM (K = 512: a mainloop of eight pieces against an epilogue of the same length)
//             runs two dequantiser sets (warps 8..15, two weight buffers each) and gives warps 16..23
//             to the epilogue: two sets per row tile, alternate 16-token steps.
//             gate_up writes gate and up (globals and row scale applied) as f32; down applies global,
//             row scale and route weight and writes one row per route (bf16, or f32 for f32 outputs).
//             An expert-parallel owner's down GEMM (RET) stores every row at an address of its own (a
//             peer's back buffer): its epilogue passes 128 rows x 16 tokens through shared memory so that a
//             token's 128 columns leave as one 256-byte run of 16-byte stores.
//   rescale   silu(gate) * up -> f16 with a per-route power-of-two scale, between the two GEMMs
//   combine   out[t] = se_gate[t] * shared[t] + sum_j y[position of route (t, j)], j ascending
//
// Every mbarrier wait is bounded; a wait that gives up raises the error flag and the CTA drains.
#include <cuda.h>

#include "kernels.cuh"
#include "umma.cuh"

namespace ftm {

namespace {

using namespace umma;

constexpr int kTileM = 128;   // weight rows per tile (MMA M, one TMEM lane per row)
constexpr int kTileTok = 128; // most tokens per pass (MMA N <= 128, one TMEM column per token)
constexpr int kStepK = 64;    // k per pipeline step: one 128-byte swizzle atom of f16
constexpr int kXStages = 6;
constexpr int kTileBytes = kTileTok * kStepK * 2;  // 16 KiB activation tile
constexpr int kThreads = 896;
// instruction descriptor: f16 x f16 -> f32, both operands K-major, M = 128; N (bits 17..22, N >> 3) per unit
constexpr uint32_t kIdescBase = (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(kTileM >> 4) << 24);


// Eight E2M1 codes of one packed word -> four f16x2, one hardware conversion per byte.  Byte b holds
// k = 2b (low nibble, low half of the result) and k = 2b + 1.  (An integer-only unpack, shifts and masks
// into the f16 exponent field, was measured: same speed within 3 %, twice the instructions.)
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
__device__ __forceinline__ uint32_t hmul2_f16(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// ---- gather: sorted activations as scaled f16 ------------------------------------------------
// one warp per sorted position (no block-wide synchronisation); K == 2048: a lane holds 8 chunks of 8 k
__global__ void __launch_bounds__(256)
prefill_gather_kernel(const void* __restrict__ x, int x_dtype, const int32_t* __restrict__ route_idx,
                      const int32_t* __restrict__ n_sorted, int top_k, int K, __half* __restrict__ xg,
                      float* __restrict__ row_scale) {
    const int i = blockIdx.x * 8 + threadIdx.x / 32, lane = threadIdx.x % 32;
    if (i >= *n_sorted) return;   // routes of unknown experts are in no bucket
    const size_t src = (size_t)(route_idx[i] / top_k) * K;
    constexpr int kChunksPerLane = 8;   // 2048 / (32 lanes * 8 k)
    float v[kChunksPerLane][8];
    float m = 0.f;
    if (x_dtype == 0) {
        uint4 raw[kChunksPerLane];
#pragma unroll
        for (int c = 0; c < kChunksPerLane; c++)
            raw[c] = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(x) + src + (c * 32 + lane) * 8);
#pragma unroll
        for (int c = 0; c < kChunksPerLane; c++) {
            const uint32_t w[4] = {raw[c].x, raw[c].y, raw[c].z, raw[c].w};
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float2 f = bf16x2_to_f32(w[q]);
                v[c][2 * q] = f.x;
                v[c][2 * q + 1] = f.y;
            }
        }
    } else {
#pragma unroll
        for (int c = 0; c < kChunksPerLane; c++) {
            const float* p = reinterpret_cast<const float*>(x) + src + (c * 32 + lane) * 8;
            const float4 f0 = *reinterpret_cast<const float4*>(p), f1 = *reinterpret_cast<const float4*>(p + 4);
            v[c][0] = f0.x; v[c][1] = f0.y; v[c][2] = f0.z; v[c][3] = f0.w;
            v[c][4] = f1.x; v[c][5] = f1.y; v[c][6] = f1.z; v[c][7] = f1.w;
        }
    }
#pragma unroll
    for (int c = 0; c < kChunksPerLane; c++)
#pragma unroll
        for (int q = 0; q < 8; q++) m = fmaxf(m, fabsf(v[c][q]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    // largest magnitude into [2^14, 2^15): exact power-of-two scaling
    const int e = max((int)((__float_as_uint(m) >> 23) & 0xff), 15);
    float inv = 1.0f, sc = 1.0f;
    if (e < 255) {
        inv = __uint_as_float((uint32_t)(127 + 14 - (e - 127)) << 23);
        sc = __uint_as_float((uint32_t)(127 - 14 + (e - 127)) << 23);
    }
#pragma unroll
    for (int c = 0; c < kChunksPerLane; c++) {
        __half2 h[4];
#pragma unroll
        for (int q = 0; q < 4; q++) h[q] = __floats2half2_rn(v[c][2 * q] * inv, v[c][2 * q + 1] * inv);
        *reinterpret_cast<uint4*>(xg + (size_t)i * K + (c * 32 + lane) * 8) =
            make_uint4(*reinterpret_cast<uint32_t*>(&h[0]), *reinterpret_cast<uint32_t*>(&h[1]),
                       *reinterpret_cast<uint32_t*>(&h[2]), *reinterpret_cast<uint32_t*>(&h[3]));
    }
    if (lane == 0) row_scale[i] = sc;
}

// ic1 (f32, sorted rows: gate | up) -> ic2 = silu(gate) * up as f16 with a per-row power-of-two scale.
// One warp per row; K == 512.
__global__ void __launch_bounds__(256)
prefill_rescale_kernel(const float* __restrict__ ic1, const int32_t* __restrict__ n_sorted, int K,
                       __half* __restrict__ ic2h, float* __restrict__ row_scale) {
    const int row = blockIdx.x * 8 + threadIdx.x / 32, lane = threadIdx.x % 32;
    if (row >= *n_sorted) return;
    float v[16];
    float m = 0.f;
#pragma unroll
    for (int c = 0; c < 2; c++) {
        const float* g = ic1 + (size_t)row * 2 * K + c * 256 + lane * 8;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const float4 gv = *reinterpret_cast<const float4*>(g + 4 * h);
            const float4 uv = *reinterpret_cast<const float4*>(g + K + 4 * h);
            float* o = v + 8 * c + 4 * h;
            o[0] = (gv.x / (1.0f + __expf(-gv.x))) * uv.x;
            o[1] = (gv.y / (1.0f + __expf(-gv.y))) * uv.y;
            o[2] = (gv.z / (1.0f + __expf(-gv.z))) * uv.z;
            o[3] = (gv.w / (1.0f + __expf(-gv.w))) * uv.w;
        }
#pragma unroll
        for (int q = 0; q < 8; q++) m = fmaxf(m, fabsf(v[8 * c + q]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const int e = max((int)((__float_as_uint(m) >> 23) & 0xff), 15);
    float inv = 1.0f, sc = 1.0f;
    if (e < 255) {
        inv = __uint_as_float((uint32_t)(127 + 14 - (e - 127)) << 23);
        sc = __uint_as_float((uint32_t)(127 - 14 + (e - 127)) << 23);
    }
#pragma unroll
    for (int c = 0; c < 2; c++) {
        __half2 h[4];
#pragma unroll
        for (int q = 0; q < 4; q++) h[q] = __floats2half2_rn(v[8 * c + 2 * q] * inv, v[8 * c + 2 * q + 1] * inv);
        *reinterpret_cast<uint4*>(ic2h + (size_t)row * K + c * 256 + lane * 8) =
            make_uint4(*reinterpret_cast<uint32_t*>(&h[0]), *reinterpret_cast<uint32_t*>(&h[1]),
                       *reinterpret_cast<uint32_t*>(&h[2]), *reinterpret_cast<uint32_t*>(&h[3]));
    }
    if (lane == 0) row_scale[row] = sc;
}

// ---- the grouped GEMM ------------------------------------------------------------------------
struct UmmaArgs {
    const uint16_t* global;    // [slots, N] f16 row globals
    const int4* groups;        // (slot, first sorted row, rows <= 128, 0)
    const int32_t* n_groups;
    const int32_t* route_idx;  // sorted position -> route (null: the rows arrived sorted, position = route)
    const float* row_scale;    // per sorted row: power-of-two scale of the activations
    const float* route_weight; // down only, indexed by route
    float* ic1;                // gate_up out [rows, 2 * inter] f32 (sorted rows): gate | up, before silu
    void* y;                   // down out [rows, hidden], bf16 or f32 (sorted rows)
    int y_f32;
    const uint64_t* row_dest;  // down only, optional: address of the bf16 output row of every sorted row (0 = none)
    int32_t* err;
    int N;                     // rows of the weight matrix (2 * inter or hidden)
};

// warp roles of the GEMM CTA (28 warps)
constexpr int kWarpActTma = 0, kWarpMma = 1, kWarpRawTma = 2, kWarpMma1 = 3, kWarpEpi0 = 4, kWarpDeq0 = 8;
constexpr int kWarpEpi1 = 24;         // warps 4..7 read row tile 0, warps 24..27 row tile 1
constexpr int kMaxDeqSets = 4;                 // dequantiser sets of 4 warps (128 threads = 128 weight rows)
constexpr int kRawStages = 6;
constexpr int kRawPackedBytes = kTileM * 128;  // two chunks (256 k): 128 weight rows x 128 bytes, 128-byte swizzle
constexpr int kRawScaleBytes = kTileM * 16;    // 128 rows x 16 scale bytes (256 k)
constexpr int kRawStageBytes = kRawPackedBytes + kRawScaleBytes;
constexpr int kWBufs = kMaxDeqSets;            // dequantised weight chunks in tensor memory, 64 columns each
constexpr int kWCols = 64;
constexpr int kAccCol0 = kWBufs * kWCols;      // accumulators: a ring of two tiles of 128 f32 columns behind them

// activation tile maps by box height: 32, 64, 96 or 128 token rows, so that a small group does not
// pull 128 rows through L2
struct XMaps {
    CUtensorMap m[4];
};

// D[256 weight rows, n tokens] += W[256, K] * X[n, K]^T as two accumulator tiles of 128 rows.  The
// dequantised weights are the A operand in tensor memory (one lane per weight row, two f16 per 32-bit
// column), the activation tile is the B operand in shared memory and is read by both row tiles; n is
// the group's row count rounded up to 16.
template <bool GATE_UP, int K, bool RET>
__global__ void __launch_bounds__(kThreads, 1)
umma_grouped_gemm_kernel(const __grid_constant__ XMaps xmaps, const __grid_constant__ CUtensorMap tmap_packed,
                         const __grid_constant__ CUtensorMap tmap_scale, UmmaArgs a) {
    // Role map.  Two dequantiser sets (warps 8..15) with two weight buffers each, one being filled while the
    // other is multiplied, and four epilogue sets, two per row tile (warps 4..7 / 16..19 and 24..27 / 20..23)
    // taking alternate token steps: with four dequantiser sets and two epilogue sets the dequantisers idled two
    // thirds of the time while the MMA issuers waited for the accumulators to be read back.  The owner's
    // variant (RET) gives one raw stage to its epilogue sets' staging buffers.
    constexpr int kDeqSets = 2;
    constexpr int kEpiSets = 4;
    constexpr int kRS = RET ? kRawStages - 1 : kRawStages;   // the owner's variant gives a raw stage to its epilogue staging
    constexpr int kWarpEpi2 = kWarpDeq0 + 4 * kDeqSets;     // down: warps 16..19 row tile 0, 20..23 row tile 1
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment for the swizzled tiles
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* const x_tiles = smem;                                         // [kXStages][16 KiB]: 128 tokens x 64 k
    uint8_t* const raw_ring = x_tiles + kXStages * kTileBytes;             // [kRawStages][packed | scales]
    uint64_t* const bars = reinterpret_cast<uint64_t*>(raw_ring + kRS * kRawStageBytes);
    uint32_t* const s_tmem = reinterpret_cast<uint32_t*>(bars + 40);
    volatile int* const s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
    // (RET only) per-token factors [epilogue set][unit parity][128 tokens], bf16 staging [set][parity][16 tokens][128 rows]
    float* const s_fac = reinterpret_cast<float*>(s_tmem + 16);
    __nv_bfloat16* const s_stage = reinterpret_cast<__nv_bfloat16*>(s_fac + 8 * kTileTok);
    const uint32_t bar0 = smem_u32(bars);
    auto X_FULL = [&](int s) { return bar0 + 8u * s; };                 // kXStages <= 8
    auto X_EMPTY = [&](int s) { return bar0 + 8u * (8 + s); };
    auto RAW_FULL = [&](int s) { return bar0 + 8u * (16 + s); };         // kRawStages <= 6
    auto RAW_EMPTY = [&](int s) { return bar0 + 8u * (22 + s); };
    auto W_READY = [&](int s) { return bar0 + 8u * (28 + s); };          // kWBufs <= 4
    auto W_FREE = [&](int s) { return bar0 + 8u * (32 + s); };
    const uint32_t ACC_FULL = bar0 + 8u * 36, ACC_EMPTY = bar0 + 8u * 37;

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kXStages; s++) {
            mbar_init(X_FULL(s), 1);
            mbar_init(X_EMPTY(s), 2);
        }
        for (int s = 0; s < kRS; s++) {
            mbar_init(RAW_FULL(s), 1);
            mbar_init(RAW_EMPTY(s), 256);
        }
        for (int s = 0; s < kWBufs; s++) {
            mbar_init(W_READY(s), 128);
            mbar_init(W_FREE(s), 1);
        }
        mbar_init(ACC_FULL, 2);
        mbar_init(ACC_EMPTY, kEpiSets * 128);
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kWarpMma) {
        // all 512 columns of tensor memory: four weight buffers and two accumulator tiles
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(s_tmem)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *s_tmem;

    constexpr int kChunks = K / 128;
    constexpr int kItems = 2 * kChunks;   // (chunk, row tile) pieces of a unit, one weight buffer each
    static_assert(kItems % kDeqSets == 0, "every dequantiser set sees the same pieces of every unit");
    static_assert(kWBufs % kDeqSets == 0, "a weight buffer belongs to one dequantiser set");
    const int n_pairs = a.N / (2 * kTileM);
    const int n_units = *a.n_groups * n_pairs;

    if (warp == kWarpActTma) {
        // ===================== activation tiles: TMA, 128-byte swizzle ============================
        // (the whole warp walks the loop, one elected lane issues: see elect_one)
        {
            uint32_t it = 0;
            for (int u = blockIdx.x; u < n_units && !*s_abort; u += gridDim.x) {
                const int4 grp = a.groups[u / n_pairs];
                const int sel = (grp.z + 31) / 32 - 1;     // box of 32 * (sel + 1) rows
                const uint32_t bytes = (uint32_t)(sel + 1) * 32 * 128;
                bool ok = true;
                for (int ks = 0; ks < K / kStepK && ok; ks++, it++) {
                    const int st = it % kXStages;
                    ok = mbar_wait_warp(X_EMPTY(st), ((it / kXStages) & 1) ^ 1, s_abort, a.err);
                    if (!ok) break;
                    if (elect_one()) {
                        mbar_expect_tx(X_FULL(st), bytes);
                        tma_load_2d(smem_u32(x_tiles + (size_t)st * kTileBytes), &xmaps.m[sel], ks * kStepK, grp.y, X_FULL(st));
                    }
                    __syncwarp();
                }
                if (!ok) break;
            }
        }
    } else if (warp == kWarpRawTma) {
        // ===================== packed weights and block scales: TMA into the raw ring ===============
        {
            uint32_t it = 0;
            for (int u = blockIdx.x; u < n_units && !*s_abort; u += gridDim.x) {
                const int4 grp = a.groups[u / n_pairs];
                const int row0 = grp.x * a.N + (u % n_pairs) * 2 * kTileM;
                bool ok = true;
                // a stage = two chunks (256 k) of one row tile: full 128-byte lines per weight row
                for (int q = 0; q < kChunks && ok; q++, it++) {
                    const int cp = q >> 1, r = q & 1;
                    const int st = it % kRS;
                    ok = mbar_wait_warp(RAW_EMPTY(st), ((it / kRS) & 1) ^ 1, s_abort, a.err);
                    if (!ok) break;
                    if (elect_one()) {
                        const uint32_t dst = smem_u32(raw_ring + (size_t)st * kRawStageBytes);
                        mbar_expect_tx(RAW_FULL(st), kRawStageBytes);
                        tma_load_2d(dst, &tmap_packed, cp * 128, row0 + r * kTileM, RAW_FULL(st));
                        tma_load_2d(dst + kRawPackedBytes, &tmap_scale, cp * 16, row0 + r * kTileM, RAW_FULL(st));
                    }
                    __syncwarp();
                }
                if (!ok) break;
            }
        }
    } else if (warp == kWarpMma || warp == kWarpMma1) {
        // ===================== MMA issuers: one warp per row tile =================================
        // The whole warp walks the loop and one elected lane issues: the code stays warp-uniform.  Two
        // issuers on two schedulers, because issuing a tcgen05.mma costs more than the math of a small
        // token tile takes.
        {
            const int r = (warp == kWarpMma) ? 0 : 1;
            const uint32_t d_tmem = tmem_base + kAccCol0 + r * kTileTok;
            uint32_t it = 0, item = r, unit_i = 0;
            // Looking at a barrier costs a shared-memory round trip even when its phase completed long ago, and
            // this warp's chain (look, issue, look, issue ..) is what the tensor pipe waits for at small token
            // tiles.  So the barriers of the NEXT step are looked at (without suspending) just before this
            // step's MMAs are issued, and the blocking wait is taken only when that look came back empty.
            bool x_seen = false, w_seen = false;
            for (int u = blockIdx.x; u < n_units && !*s_abort; u += gridDim.x, unit_i++) {
                const int4 grp = a.groups[u / n_pairs];
                const int n_pad = max(16, (grp.z + 15) & ~15);
                const uint32_t idesc = kIdescBase | ((uint32_t)(n_pad >> 3) << 17);
                // the accumulators must have been read back
                bool ok = mbar_wait_warp(ACC_EMPTY, (unit_i & 1) ^ 1, s_abort, a.err);
                for (int ks = 0; ks < 2 * kChunks && ok; ks++, it++) {
                    const int h = ks & 1;                        // half of the 128-k weight piece
                    const int wb = item % kWBufs;
                    if (h == 0 && !w_seen) ok = mbar_wait_warp(W_READY(wb), (item / kWBufs) & 1, s_abort, a.err);
                    if (!ok) break;
                    const int st = it % kXStages;
                    if (!x_seen) ok = mbar_wait_warp(X_FULL(st), (it / kXStages) & 1, s_abort, a.err);
                    if (!ok) break;
                    {
                        const uint32_t it1 = it + 1;
                        x_seen = __all_sync(0xffffffffu, mbar_test_wait(X_FULL(it1 % kXStages), (it1 / kXStages) & 1));
                        if (h == 1) {
                            const uint32_t item1 = item + 2;
                            w_seen = __all_sync(0xffffffffu, mbar_test_wait(W_READY(item1 % kWBufs), (item1 / kWBufs) & 1));
                        }
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t w_addr = tmem_base + wb * kWCols;
                    const uint64_t xdesc = umma_desc(smem_u32(x_tiles + (size_t)st * kTileBytes));
                    if (elect_one()) {
#pragma unroll
                        for (int kk = 0; kk < 4; kk++)
                            umma_f16_ts(d_tmem, w_addr + (h * 4 + kk) * 8, xdesc + kk * 2, idesc, (ks > 0 || kk > 0) ? 1u : 0u);
                        umma_commit(X_EMPTY(st));    // the activation stage is free once both issuers' MMAs retire
                        if (h == 1) umma_commit(W_FREE(wb));   // and so is the weight buffer
                    }
                    __syncwarp();
                    if (h == 1) item += 2;
                }
                if (!ok) break;
                if (elect_one()) umma_commit(ACC_FULL);
                __syncwarp();
            }
        }
    } else if (warp >= kWarpDeq0 && warp < kWarpEpi2) {
        // ===================== dequantisers: raw ring -> f16 weights in tensor memory ================
        // Four sets of four warps; set s takes the pieces w = s (mod 4) of every unit (w = 2 * chunk +
        // row tile) and owns weight buffer s.  Warp quarter q may touch TMEM lanes 32q..32q+31; a thread
        // owns one weight row of the piece: 64 packed bytes, eight block scales, 64 columns.
        const int quarter = warp & 3, set = (warp - kWarpDeq0) >> 2;
        const int row = quarter * 32 + lane;
        const int sw = row & 7;             // 128-byte swizzle of the TMA box: 16-byte chunk index ^ (row & 7)
        const uint32_t tlane = tmem_base + ((uint32_t)(quarter * 32) << 16);
        uint32_t item0 = 0, stage0 = 0;     // pieces and raw stages before this unit
        for (int u = blockIdx.x; u < n_units && !*s_abort; u += gridDim.x, item0 += kItems, stage0 += kChunks) {
            bool ok = true;
            for (int w = set; w < kItems && ok; w += kDeqSets) {
                const uint32_t item = item0 + w;
                const int c = w >> 1;
                const uint32_t stage = stage0 + 2 * (c >> 1) + (w & 1);      // the raw stage holds chunks c & ~1 and c | 1
                const int st = stage % kRS;
                ok = mbar_wait(RAW_FULL(st), (stage / kRS) & 1, s_abort, a.err);
                if (!ok) break;
                const int wb = item % kWBufs;
                const uint32_t taddr = tlane + wb * kWCols;
                const uint8_t* const rp = raw_ring + (size_t)st * kRawStageBytes;
                const uint2 sc8 = *reinterpret_cast<const uint2*>(rp + kRawPackedBytes + row * 16 + (c & 1) * 8);
                uint4 raw[4];
#pragma unroll
                for (int g = 0; g < 4; g++) raw[g] = *reinterpret_cast<const uint4*>(rp + row * 128 + ((((c & 1) * 4 + g) ^ sw) << 4));
                // 32 k (one 16-byte piece, two block scales) -> 16 columns
                auto convert = [&](int g, uint32_t (&r)[16]) {
                    const uint32_t two = ((g & 2) ? sc8.y : sc8.x) >> ((g & 1) * 16);
                    uint32_t h2;
                    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"((uint16_t)(two & 0xffffu)));
                    const uint32_t s0 = __byte_perm(h2, h2, 0x1010), s1 = __byte_perm(h2, h2, 0x3232);
                    const uint32_t wd[4] = {raw[g].x, raw[g].y, raw[g].z, raw[g].w};
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        uint32_t q[4];
                        e2m1x8_to_f16x2(wd[j], q);
#pragma unroll
                        for (int e = 0; e < 4; e++) r[4 * j + e] = hmul2_f16(q[e], (j < 2) ? s0 : s1);
                    }
                };
                // the first half of the piece is converted before the buffer is known to be free: it waits in
                // registers, so the conversion is off the path between "buffer free" and "buffer ready"
                uint32_t r0[16], r1[16];
                convert(0, r0);
                convert(1, r1);
                ok = mbar_wait(W_FREE(wb), ((item / kWBufs) & 1) ^ 1, s_abort, a.err);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                tmem_st16(taddr, r0);
                tmem_st16(taddr + 16, r1);
                convert(2, r0);
                tmem_st16(taddr + 32, r0);
                convert(3, r1);
                tmem_st16(taddr + 48, r1);
                mbar_arrive(RAW_EMPTY(st));
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                mbar_arrive(W_READY(wb));
            }
            if (!ok) break;
        }
    } else if (warp >= kWarpEpi0) {
        if constexpr (!RET) {
            // ===================== epilogue (TMEM lane quarter = warp % 4) ================================
            // one thread = one weight row of its row tile; a column = one token of the group.  Lane l keeps
            // the per-token factors of tokens l, l + 32, l + 64, l + 96 and hands them out by shuffle.
            // With four sets (down) the two sets of a row tile take alternate 16-token steps.
            const int quarter = warp & 3;
            const int r = (warp < kWarpDeq0) ? 0 : (warp >= kWarpEpi1) ? 1 : ((warp - kWarpEpi2) >> 2);
            const int half = (warp >= kWarpDeq0 && warp < kWarpEpi1) ? 1 : 0;
            constexpr int kStride = 16 * (kEpiSets / 2);
            uint32_t unit_i = 0;
            for (int u = blockIdx.x; u < n_units && !*s_abort; u += gridDim.x, unit_i++) {
                const int4 grp = a.groups[u / n_pairs];
                const int cnt = grp.z, pos0 = grp.y;
                const int wrow = (u % n_pairs) * 2 * kTileM + r * kTileM + quarter * 32 + lane;
                const float gl = f16_global_to_f32(a.global[(size_t)grp.x * a.N + wrow]);
                float fac[4];
    #pragma unroll
                for (int q = 0; q < 4; q++) {
                    const int i = q * 32 + lane;
                    float f = 0.f;
                    if (i < cnt) {
                        f = a.row_scale[pos0 + i];
                        if (!GATE_UP) f *= a.route_weight[a.route_idx ? a.route_idx[pos0 + i] : pos0 + i];
                    }
                    fac[q] = f;
                }
                if (!mbar_wait(ACC_FULL, unit_i & 1, s_abort, a.err)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                {
                    const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + kAccCol0 + r * kTileTok;
    #pragma unroll 1
                    for (int c0 = 16 * half; c0 < cnt; c0 += kStride) {      // uniform over the warp
                        {
                            float v[16];
                            tmem_ld16(taddr + c0, v);
                            tmem_ld_wait();
                            const float fq = c0 < 32 ? fac[0] : c0 < 64 ? fac[1] : c0 < 96 ? fac[2] : fac[3];
    #pragma unroll
                            for (int j = 0; j < 16; j++) v[j] = (v[j] * gl) * __shfl_sync(0xffffffffu, fq, (c0 & 31) + j);
                            if (GATE_UP || a.y_f32) {
                                float* const dst = GATE_UP ? a.ic1 : reinterpret_cast<float*>(a.y);
    #pragma unroll
                                for (int j = 0; j < 16; j++)
                                    if (c0 + j < cnt) dst[(size_t)(pos0 + c0 + j) * a.N + wrow] = v[j];
                            } else {
                                // bf16 rows: neighbouring lanes swap so that every lane stores a pair of rows of one token
                                __nv_bfloat16* const dst = reinterpret_cast<__nv_bfloat16*>(a.y);
    #pragma unroll
                                for (int j = 0; j < 16; j += 2) {
                                    const float mine = (lane & 1) ? v[j + 1] : v[j];
                                    const float give = (lane & 1) ? v[j] : v[j + 1];
                                    const float got = __shfl_xor_sync(0xffffffffu, give, 1);
                                    const int tok = c0 + j + (lane & 1);
                                    const __nv_bfloat162 pr = (lane & 1) ? __floats2bfloat162_rn(got, mine) : __floats2bfloat162_rn(mine, got);
                                    if (tok < cnt)
                                        *reinterpret_cast<__nv_bfloat162*>(dst + (size_t)(pos0 + tok) * a.N + (wrow & ~1)) = pr;
                                }
                            }
                        }
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                mbar_arrive(ACC_EMPTY);
            }
    
        } else {
            // ===================== epilogue (warps 4..7 and 24..27: TMEM lane quarters 0..3) ==============
            // one thread = one weight row of its row tile; a column = one token of the group.  The per-token
            // factors of a unit are computed once per set (thread t: token t), left in shared memory and read
            // back as broadcasts; the accumulators are read 32 columns per wait.
            // Four sets: the two sets of a row tile take alternate 32-token chunks, each with its own factors,
            // staging buffers and named barrier.
            const int quarter = warp & 3;
            const int r = (warp < kWarpDeq0) ? 0 : (warp >= kWarpEpi1) ? 1 : ((warp - kWarpEpi2) >> 2);
            const int half = (warp >= kWarpDeq0 && warp < kWarpEpi1) ? 1 : 0;
            const int es = r + 2 * half;
            const int tid = quarter * 32 + lane;
            uint32_t unit_i = 0, stage_i = 0;
            for (int u = blockIdx.x; u < n_units; u += gridDim.x, unit_i++) {     // (the abort flag is seen inside the wait)
                const int4 grp = a.groups[u / n_pairs];
                const int cnt = grp.z, pos0 = grp.y;
                const int wrow0 = (u % n_pairs) * 2 * kTileM + r * kTileM;
                const int wrow = wrow0 + tid;
                const float gl = f16_global_to_f32(a.global[(size_t)grp.x * a.N + wrow]);
                float* const fac = s_fac + (es * 2 + (unit_i & 1)) * kTileTok;
                {
                    float f = 0.f;
                    if (tid < cnt) {
                        f = a.row_scale[pos0 + tid];
                        if (!GATE_UP) f *= a.route_weight[a.route_idx ? a.route_idx[pos0 + tid] : pos0 + tid];
                    }
                    fac[tid] = f;
                }
                // One answer for the 128 threads of this set: they meet at named barriers below, so none may leave
                // alone.  The same barrier publishes the factors (their buffer alternates by unit, so one barrier
                // per unit is enough).
                const bool mine = mbar_wait(ACC_FULL, unit_i & 1, s_abort, a.err);
                uint32_t all_ok;
                asm volatile(
                    "{\n\t.reg .pred p, q;\n\t"
                    "setp.ne.u32 q, %1, 0;\n\t"
                    "bar.red.and.pred p, %2, 128, q;\n\t"
                    "selp.u32 %0, 1, 0, p;\n\t}"
                    : "=r"(all_ok)
                    : "r"((uint32_t)mine), "r"(1 + es)
                    : "memory");
                if (!all_ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                {
                    const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + kAccCol0 + r * kTileTok;
    #pragma unroll 1
                    for (int c0 = 32 * half; c0 < cnt; c0 += 64) {      // uniform over the warp
                        float v[2][16];
                        tmem_ld16(taddr + c0, v[0]);
                        tmem_ld16(taddr + c0 + 16, v[1]);
                        tmem_ld_wait();
    #pragma unroll
                        for (int h = 0; h < 2; h++) {
                            const int cb = c0 + 16 * h;
                            if (cb >= cnt) break;
    #pragma unroll
                            for (int j = 0; j < 16; j += 4) {
                                const float4 f4 = *reinterpret_cast<const float4*>(fac + cb + j);
                                v[h][j] = (v[h][j] * gl) * f4.x; v[h][j + 1] = (v[h][j + 1] * gl) * f4.y;
                                v[h][j + 2] = (v[h][j + 2] * gl) * f4.z; v[h][j + 3] = (v[h][j + 3] * gl) * f4.w;
                            }
                            if (GATE_UP || a.y_f32) {
                                float* const dst = GATE_UP ? a.ic1 : reinterpret_cast<float*>(a.y);
    #pragma unroll
                                for (int j = 0; j < 16; j++)
                                    if (cb + j < cnt) dst[(size_t)(pos0 + cb + j) * a.N + wrow] = v[h][j];
                            } else {
                                // bf16 rows: the set's 128 rows x 16 tokens go through shared memory, so that every
                                // thread stores 16 bytes of one token's row and a token's 128 columns leave as one
                                // 256-byte run (the layout the peer stores of the expert-parallel return want too)
                                __nv_bfloat16* const st = s_stage + ((es * 2 + (stage_i & 1)) * 16) * kTileM;
                                stage_i++;
    #pragma unroll
                                for (int j = 0; j < 16; j++) st[j * kTileM + tid] = __float2bfloat16_rn(v[h][j]);
                                asm volatile("bar.sync %0, 128;" ::"r"(1 + es) : "memory");
    #pragma unroll
                                for (int q = 0; q < 2; q++) {
                                    const int piece = tid + q * 128, tok = cb + piece / 16, c8 = (piece % 16) * 8;
                                    if (tok < cnt) {
                                        __nv_bfloat16* const row = reinterpret_cast<__nv_bfloat16*>(__ldg(a.row_dest + pos0 + tok));
                                        if (row)
                                            *reinterpret_cast<uint4*>(row + wrow0 + c8) =
                                                *reinterpret_cast<const uint4*>(st + (piece / 16) * kTileM + c8);
                                    }
                                }
                            }
                        }
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                mbar_arrive(ACC_EMPTY);
            }
    
        }
    }
    // drain: nobody frees tensor memory while another role may still touch it
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == kWarpMma) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
    }
}

// the owner's variant (RET) adds the per-token factors and the bf16 staging of its epilogue
constexpr size_t kUmmaSmemLocal = 1024 + (size_t)kXStages * kTileBytes + (size_t)kRawStages * kRawStageBytes + 40 * 8 + 64 + 64;
constexpr size_t kUmmaSmem = kUmmaSmemLocal - kRawStageBytes + 8 * kTileTok * sizeof(float) + 8 * 16 * kTileM * sizeof(__nv_bfloat16);
static_assert(kUmmaSmem <= 227 * 1024, "shared memory of the grouped GEMM CTA");

// f16 matrix [rows, K] row-major, box = 64 k x box_rows, 128-byte swizzle
bool make_act_map(CUtensorMap* map, const void* base, size_t rows, int K, int box_rows) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)kStepK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Expert-parallel owner, one thread per received row i: the address of its output row in the source rank's back
// buffer goes into row_dest at the row's sorted position, where the down GEMM's epilogue finds it.  A row whose
// expert is not resident takes no part in the GEMM: its output row is zero-filled here.
__global__ void __launch_bounds__(128)
ep_row_dest_kernel(const int32_t* __restrict__ pos_of_route, const int32_t* __restrict__ route_slot, int n, int H,
                   int world, int rank, const int32_t* __restrict__ counts_all, const uint64_t* __restrict__ peer_back,
                   long long capacity, uint64_t* __restrict__ row_dest, int32_t* err) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const int lane = threadIdx.x & 31;
    uint64_t dest = 0;
    bool dropped = false;
    if (i < n) {
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
            atomicExch(err, 4);
        } else {
            dest = peer_back[s] + (uint64_t)row * H * sizeof(__nv_bfloat16);
            if (route_slot[i] < 0)
                dropped = true;
            else
                row_dest[pos_of_route[i]] = dest;
        }
    }
    unsigned todo = __ballot_sync(0xffffffffu, dropped);
    while (todo) {
        const int src = __ffs(todo) - 1;
        todo &= todo - 1;
        uint4* const z = reinterpret_cast<uint4*>(__shfl_sync(0xffffffffu, dest, src));
        for (int c = lane; c < H / 8; c += 32) z[c] = make_uint4(0, 0, 0, 0);
    }
}


// ---- expert-parallel owner whose rows arrived sorted (ep_dispatch_sorted_kernel) -------------------
// seg_owner[le] = first row of local expert le in the owner's matrix, le = 0 .. per (the total at per)
__global__ void ep_owner_seg_kernel(const int32_t* __restrict__ seg_all, int experts, int per, int world, int rank,
                                    int32_t* __restrict__ seg_owner) {
    const int le = blockIdx.x * blockDim.x + threadIdx.x;
    if (le > per) return;
    int v = 0;
    for (int s = 0; s < world; s++) {
        const int32_t* sg = seg_all + (size_t)s * (experts + 1);
        v += sg[rank * per + le] - sg[rank * per];
    }
    seg_owner[le] = v;
}

// One thread per sorted row: the address of its output row in its source's back buffer (row seg_s[e] + j of
// source s, the position the source sent it from).  A row of an expert that is not resident takes no part in
// the GEMM and is zero-filled there.
__global__ void __launch_bounds__(128)
ep_row_dest_sorted_kernel(const int32_t* __restrict__ seg_all, const int32_t* __restrict__ seg_owner,
                          const int32_t* __restrict__ slot_of_bin, int slots, int n, int H, int experts, int per, int world,
                          int rank, const uint64_t* __restrict__ peer_back, long long capacity,
                          uint64_t* __restrict__ row_dest, int32_t* err) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    const int lane = threadIdx.x & 31;
    uint64_t dest = 0;
    bool dropped = false;
    if (r < n) {
        int lo = 0, hi = per;              // largest le with seg_owner[le] <= r
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (seg_owner[mid] <= r) lo = mid; else hi = mid;
        }
        const int e = rank * per + lo;
        int j = r - seg_owner[lo], s = 0;
        for (; s < world; s++) {
            const int32_t* sg = seg_all + (size_t)s * (experts + 1);
            const int c = sg[e + 1] - sg[e];
            if (j < c) break;
            j -= c;
        }
        long long row = -1;
        if (s < world) row = (long long)seg_all[(size_t)s * (experts + 1) + e] + j;
        if (row < 0 || row >= capacity) {
            atomicExch(err, 4);
        } else {
            dest = peer_back[s] + (uint64_t)row * H * sizeof(__nv_bfloat16);
            const int slot = slot_of_bin[lo];
            if (slot < 0 || slot >= slots) dropped = true;
            row_dest[r] = dropped ? 0 : dest;
        }
    }
    unsigned todo = __ballot_sync(0xffffffffu, dropped);
    while (todo) {
        const int src = __ffs(todo) - 1;
        todo &= todo - 1;
        uint4* const z = reinterpret_cast<uint4*>(__shfl_sync(0xffffffffu, dest, src));
        for (int c = lane; c < H / 8; c += 32) z[c] = make_uint4(0, 0, 0, 0);
    }
}

// out[t] = se_gate[t] * shared[t] + sum over the resident routes j of y[pos_of_route[t*k + j]], j ascending
__global__ void prefill_combine_kernel(const void* __restrict__ y, int y_f32, const int32_t* __restrict__ pos_of_route,
                                       const int32_t* __restrict__ route_slot, int slots, int top_k, int H,
                                       const float* __restrict__ shared, const float* __restrict__ se_gate,
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
        const int slot = route_slot[t * top_k + j];
        if (slot < 0 || slot >= slots) continue;
        const size_t row = (size_t)pos_of_route[t * top_k + j] * H + d;
        if (y_f32) {
            const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(y) + row);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        } else {
            const uint2 pk = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(y) + row);
            const float2 a = bf16x2_to_f32(pk.x), b = bf16x2_to_f32(pk.y);
            acc.x += a.x; acc.y += a.y; acc.z += b.x; acc.w += b.y;
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

// u8 matrix [rows, row_bytes] row-major (packed nibbles or block scales), box = box_bytes x box_rows
bool make_raw_map(CUtensorMap* map, const void* base, size_t rows, int row_bytes, int box_bytes, int box_rows,
                  CUtensorMapSwizzle swizzle) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
    cuuint32_t box[2] = {(cuuint32_t)box_bytes, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// The tensor maps of the two grouped GEMMs.  Every address they hold (the sorted-activation scratch, the
// f16 intermediate, the four packed / scale banks) is fixed for the adapter's life, so they are encoded
// when the adapter is created (and again when its banks are reallocated), never per call.  `rows` is the
// scratch capacity in routes: a call with fewer routes reads stale rows past its own, whose columns the
// epilogue never stores.
bool prefill_build_maps(const BankView& b, const __half* xg, const __half* ic2h, size_t rows, PrefillMaps* out) {
    out->ok = false;
    if (!encode_tiled() || !b.gu_packed) return false;
    for (int q = 0; q < 4; q++)
        if (!make_act_map(&out->x[q], xg, rows, b.hidden, 32 * (q + 1)) ||
            !make_act_map(&out->h[q], ic2h, rows, b.inter, 32 * (q + 1)))
            return false;
    const size_t gu_rows = (size_t)b.slots * 2 * b.inter, dn_rows = (size_t)b.slots * b.hidden;
    if (!make_raw_map(&out->gp, b.gu_packed, gu_rows, b.hidden / 2, 128, kTileM, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_raw_map(&out->gs, b.gu_scale, gu_rows, b.hidden / 16, 16, kTileM, CU_TENSOR_MAP_SWIZZLE_NONE) ||
        !make_raw_map(&out->dp, b.dn_packed, dn_rows, b.inter / 2, 128, kTileM, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !make_raw_map(&out->ds, b.dn_scale, dn_rows, b.inter / 16, 16, kTileM, CU_TENSOR_MAP_SWIZZLE_NONE))
        return false;
    out->ok = true;
    return true;
}

bool prefill_umma_supported(int hidden, int inter, int slots, int experts, bool have_expert_ids) {
    if (hidden != 2048 || inter != 512) return false;
    if ((have_expert_ids ? experts : slots) > 1024) return false;
    return encode_tiled() != nullptr;
}

int launch_prefill_umma(const BankView& b, const void* x, int x_dtype, const DecodeRoutes& rt,
                        const float* route_weight, int tokens, int top_k, PrefillScratch sc, int sm_count,
                        const float* shared, const float* se_gate, cudaEvent_t join, void* out, int out_dtype,
                        const PrefillMaps& maps, const Ctx& c, const EpReturnTo* ret) {
    const int routes = tokens * top_k;
    int launches = 0;
    // 1. buckets, stable: by expert id of the layer (serving call) or by slot id
    const int32_t* bins_of_route;
    const int32_t* slot_of_bin = nullptr;
    const int32_t* route_slot;
    int nbins;
    SlotRewrite rewrite;      // the id -> slot mapping runs inside the permutation build's first pass
    if (rt.expert_ids) {
        rewrite = SlotRewrite{rt.expert_ids, rt.ids_dtype, rt.layer, rt.experts, rt.slot_for_id, rt.n_ids, rt.route_slot_out,
                              sc.route_bin, rt.bad_flag};
        bins_of_route = sc.route_bin;
        slot_of_bin = rt.slot_for_id + (size_t)rt.layer * rt.experts;
        route_slot = rt.route_slot_out;
        nbins = rt.experts;
    } else {
        bins_of_route = rt.route_slot_in;
        route_slot = rt.route_slot_in;
        nbins = b.slots;
    }
    // 1. + 2. buckets and, from the same scan, passes of <= 128 sorted rows per expert
    const CsrGroups cg{slot_of_bin, b.slots, kTileTok, sc.groups, sc.n_groups, sc.pos_of_route};
    launches += launch_csr_build(bins_of_route, routes, nbins, sc.seg, sc.route_idx, sc.csr_scratch, sc.csr_flag, c, false, &cg,
                                 rt.expert_ids ? &rewrite : nullptr);
    // 3. sorted, scaled f16 activations
    c.begin(K_PERMUTE_ACT);
    prefill_gather_kernel<<<(routes + 7) / 8, 256, 0, c.s>>>(x, x_dtype, sc.route_idx, sc.seg + nbins, top_k, b.hidden, sc.xg,
                                                   sc.row_scale);
    c.end();
    launches++;

    if (!maps.ok) return -1;
    XMaps map_x, map_h;
    for (int q = 0; q < 4; q++) {
        map_x.m[q] = maps.x[q];
        map_h.m[q] = maps.h[q];
    }
    const CUtensorMap &map_gp = maps.gp, &map_gs = maps.gs, &map_dp = maps.dp, &map_ds = maps.ds;
    static PerDeviceOnce once_gu, once_dn;
    allow_dyn_smem(once_gu, umma_grouped_gemm_kernel<true, 2048, false>, kUmmaSmem);
    allow_dyn_smem(once_dn, umma_grouped_gemm_kernel<false, 512, false>, kUmmaSmem);
    static PerDeviceOnce once_ret;
    allow_dyn_smem(once_ret, umma_grouped_gemm_kernel<false, 512, true>, kUmmaSmem);
    UmmaArgs a{};
    a.groups = sc.groups; a.n_groups = sc.n_groups; a.route_idx = sc.route_idx; a.err = sc.err;
    a.global = b.gu_global; a.row_scale = sc.row_scale;
    a.ic1 = sc.ic1; a.N = 2 * b.inter;
    c.begin(K_GROUPED_GATE_UP);
    umma_grouped_gemm_kernel<true, 2048, false><<<sm_count, kThreads, kUmmaSmemLocal, c.s>>>(map_x, map_gp, map_gs, a);
    c.end();
    c.begin(K_PREFILL_RESCALE);
    prefill_rescale_kernel<<<(routes + 7) / 8, 256, 0, c.s>>>(sc.ic1, sc.seg + nbins, b.inter, sc.ic2h, sc.row_scale2);
    c.end();
    a.global = b.dn_global; a.row_scale = sc.row_scale2;
    a.route_weight = route_weight; a.y = sc.y; a.y_f32 = (out_dtype == 1); a.N = b.hidden;
    if (ret) {
        // the finished rows go straight to their source ranks: the row addresses live in the scratch the rows
        // themselves would have taken
        uint64_t* const row_dest = reinterpret_cast<uint64_t*>(sc.y);
        c.begin(K_EP_COMBINE);
        ep_row_dest_kernel<<<(routes + 127) / 128, 128, 0, c.s>>>(sc.pos_of_route, route_slot, routes, b.hidden, ret->world, ret->rank,
                                                             ret->counts_all, ret->peer_back, ret->capacity, row_dest, sc.err);
        c.end();
        launches += 1;
        a.row_dest = row_dest;
        a.y = nullptr;
        a.y_f32 = 0;
    }
    c.begin(K_GROUPED_DOWN);
    if (ret)
        umma_grouped_gemm_kernel<false, 512, true><<<sm_count, kThreads, kUmmaSmem, c.s>>>(map_h, map_dp, map_ds, a);
    else
        umma_grouped_gemm_kernel<false, 512, false><<<sm_count, kThreads, kUmmaSmemLocal, c.s>>>(map_h, map_dp, map_ds, a);
    c.end();
    launches += 3;
    if (ret) return launches;
    // 4. un-permute and sum in route order; routes of experts that are not resident are skipped.  Without `out`
    // the rows stay sorted by expert (sc.y, with sc.pos_of_route to find them): the expert-parallel owner hands
    // them to the return kernel as they are.
    if (join) cudaStreamWaitEvent(c.s, join, 0);
    c.begin(K_SUM_ROUTES);
    if (out) {
        dim3 grid(tokens, (b.hidden / 4 + 127) / 128);
        prefill_combine_kernel<<<grid, 128, 0, c.s>>>(sc.y, out_dtype == 1, sc.pos_of_route, route_slot, b.slots, top_k, b.hidden, shared,
                                                      se_gate, out, out_dtype);
    }
    c.end();
    return launches + (out ? 1 : 0);
}

// The owner's step on rows that arrived sorted by expert as scaled f16 (xg, row_scale, route_weight: one entry per
// row, in this GPU's memory): no permutation build and no gather; groups from the all-gathered prefixes, the two
// GEMMs, every finished row stored by the down GEMM into its source's back buffer.  `maps` must hold activation
// maps encoded on xg.
int launch_prefill_umma_presorted(const BankView& b, const float* row_scale, const float* route_weight, int rows,
                                  const int32_t* seg_all, int experts, const int32_t* slot_of_bin, PrefillScratch sc,
                                  int sm_count, const EpReturnTo& ret, const PrefillMaps& maps, const Ctx& c) {
    if (!maps.ok) return -1;
    const int per = experts / ret.world;
    int launches = 0;
    c.begin(K_CSR);
    ep_owner_seg_kernel<<<(per + 1 + 127) / 128, 128, 0, c.s>>>(seg_all, experts, per, ret.world, ret.rank, sc.seg);
    c.end();
    launches += 1 + launch_groups_from_csr(sc.seg, per, slot_of_bin, b.slots, kTileTok, sc.groups, sc.n_groups, c);
    uint64_t* const row_dest = reinterpret_cast<uint64_t*>(sc.y);
    c.begin(K_EP_COMBINE);
    ep_row_dest_sorted_kernel<<<(rows + 127) / 128, 128, 0, c.s>>>(seg_all, sc.seg, slot_of_bin, b.slots, rows, b.hidden, experts, per,
                                                                 ret.world, ret.rank, ret.peer_back, ret.capacity, row_dest, sc.err);
    c.end();
    launches++;
    XMaps map_x, map_h;
    for (int q = 0; q < 4; q++) {
        map_x.m[q] = maps.x[q];
        map_h.m[q] = maps.h[q];
    }
    static PerDeviceOnce once_gu, once_ret;
    allow_dyn_smem(once_gu, umma_grouped_gemm_kernel<true, 2048, false>, kUmmaSmem);
    allow_dyn_smem(once_ret, umma_grouped_gemm_kernel<false, 512, true>, kUmmaSmem);
    UmmaArgs a{};
    a.groups = sc.groups; a.n_groups = sc.n_groups; a.route_idx = nullptr; a.err = sc.err;
    a.global = b.gu_global; a.row_scale = row_scale;
    a.ic1 = sc.ic1; a.N = 2 * b.inter;
    c.begin(K_GROUPED_GATE_UP);
    umma_grouped_gemm_kernel<true, 2048, false><<<sm_count, kThreads, kUmmaSmemLocal, c.s>>>(map_x, maps.gp, maps.gs, a);
    c.end();
    c.begin(K_PREFILL_RESCALE);
    prefill_rescale_kernel<<<(rows + 7) / 8, 256, 0, c.s>>>(sc.ic1, sc.seg + per, b.inter, sc.ic2h, sc.row_scale2);
    c.end();
    a.global = b.dn_global; a.row_scale = sc.row_scale2;
    a.route_weight = route_weight; a.y = nullptr; a.y_f32 = 0; a.N = b.hidden; a.row_dest = row_dest;
    c.begin(K_GROUPED_DOWN);
    umma_grouped_gemm_kernel<false, 512, true><<<sm_count, kThreads, kUmmaSmem, c.s>>>(map_h, maps.dp, maps.ds, a);
    c.end();
    return launches + 3;
}

}  // namespace ftm
