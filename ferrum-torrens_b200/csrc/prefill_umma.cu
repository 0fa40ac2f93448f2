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
//   gemm      persistent CTAs over (segment pass of <= 256 tokens, tile of 128 weight rows):
//               warp 0      TMA producer: activation tiles [128 tokens x 64 k] f16, 128-byte swizzle
//               warp 1      allocates tensor memory, issues tcgen05.mma (M = 128 tokens, N = 128 rows,
//                           K = 16 per instruction, f16 x f16 -> f32), commits to mbarriers
//               warps 2..5  dequantise the packed rows straight from global memory (hardware
//                           e2m1x2 / e4m3x2 -> f16x2 conversions, exact product with the block scale)
//                           into the K-major, 128-byte-swizzled B tile in shared memory; after the
//                           mainloop they read the accumulators back (tcgen05.ld) and run the epilogue
//             gate_up tiles hold 64 gate rows and the 64 matching up rows, so silu(gate) * up stays in
//             one thread; the epilogue applies the globals and the row scale and writes ic2 (f32).
//             down tiles apply global, row scale and route weight and write one bf16 row per route.
//   rescale   ic2 (f32) -> f16 with a per-route power-of-two scale, between the two GEMMs
//   combine   out[t] = se_gate[t] * shared[t] + sum_j y[position of route (t, j)]  (ep_combine_kernel)
//
// Every mbarrier wait is bounded; a wait that gives up raises the error flag and the CTA drains.
#include <cuda.h>

#include "kernels.cuh"

namespace ftm {

namespace {

constexpr int kTileM = 128;   // tokens per accumulator tile (MMA M, one TMEM lane per token)
constexpr int kTileN = 128;   // weight rows per tile (MMA N, one TMEM column per row)
constexpr int kStepK = 64;    // k per pipeline step: one 128-byte swizzle atom of f16
constexpr int kMaxTokTiles = 2;               // <= 256 tokens per pass
constexpr int kAStages = 3;
constexpr int kTileBytes = kTileM * kStepK * 2;  // 16 KiB, also the B tile
constexpr int kThreads = 512;
constexpr uint32_t kSpin = 1u << 20;

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
// bounded wait: false after kSpin polls or once another role has raised the abort flag
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int32_t* err) {
    for (uint32_t i = 0; i < kSpin; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1;
    atomicExch(err, 3);
    return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(map), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}

// shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 bytes, 8-row groups
// 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3ffffu) >> 4);   // start address
    d |= (uint64_t)1 << 16;                      // leading byte offset (unused with 128B swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;            // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                      // descriptor version
    d |= (uint64_t)2 << 61;                      // 128-byte swizzle
    return d;
}
// instruction descriptor: f16 x f16 -> f32, both operands K-major, M = 128, N = 128
constexpr uint32_t kIdesc = (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(kTileN >> 3) << 17) |
                            ((uint32_t)(kTileM >> 4) << 24);

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(kIdesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
#pragma unroll
    for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

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
// one CTA per sorted position; K % 256 == 0
__global__ void __launch_bounds__(256)
prefill_gather_kernel(const void* __restrict__ x, int x_dtype, const int32_t* __restrict__ route_idx,
                      const int32_t* __restrict__ n_sorted, int top_k, int K, __half* __restrict__ xg,
                      float* __restrict__ row_scale) {
    __shared__ float wmax[8];
    __shared__ float s_inv;
    const int i = blockIdx.x;
    if (i >= *n_sorted) return;   // routes of unknown experts are in no bucket
    const size_t src = (size_t)(route_idx[i] / top_k) * K;
    float v[8];
    float m = 0.f;
    const int k0 = threadIdx.x * 8;   // K == 2048: one pass
    for (int k = k0; k < K; k += 2048) {
#pragma unroll
        for (int q = 0; q < 8; q++) {
            v[q] = load_act(x, x_dtype, src + k + q);
            m = fmaxf(m, fabsf(v[q]));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        float mm = 0.f;
        for (int w = 0; w < 8; w++) mm = fmaxf(mm, wmax[w]);
        const int e = max((int)((__float_as_uint(mm) >> 23) & 0xff), 15);
        float inv = 1.0f, sc = 1.0f;
        if (e < 255) {
            inv = __uint_as_float((uint32_t)(127 + 14 - (e - 127)) << 23);
            sc = __uint_as_float((uint32_t)(127 - 14 + (e - 127)) << 23);
        }
        s_inv = inv;
        row_scale[i] = sc;
    }
    __syncthreads();
    const float inv = s_inv;
    for (int k = k0; k < K; k += 2048) {
        __half2 h[4];
#pragma unroll
        for (int q = 0; q < 4; q++) h[q] = __floats2half2_rn(v[2 * q] * inv, v[2 * q + 1] * inv);
        *reinterpret_cast<uint4*>(xg + (size_t)i * K + k) =
            make_uint4(*reinterpret_cast<uint32_t*>(&h[0]), *reinterpret_cast<uint32_t*>(&h[1]),
                       *reinterpret_cast<uint32_t*>(&h[2]), *reinterpret_cast<uint32_t*>(&h[3]));
    }
}

// ic2 (f32, sorted rows) -> f16 with a per-row power-of-two scale.  One warp per row; K == 512.
__global__ void __launch_bounds__(256)
prefill_rescale_kernel(const float* __restrict__ ic2, const int32_t* __restrict__ n_sorted, int K,
                       __half* __restrict__ ic2h, float* __restrict__ row_scale) {
    const int row = blockIdx.x * 8 + threadIdx.x / 32, lane = threadIdx.x % 32;
    if (row >= *n_sorted) return;
    float v[16];
    float m = 0.f;
#pragma unroll
    for (int c = 0; c < 4; c++) {
        const float4 f = *reinterpret_cast<const float4*>(ic2 + (size_t)row * K + c * 128 + lane * 4);
        v[4 * c] = f.x; v[4 * c + 1] = f.y; v[4 * c + 2] = f.z; v[4 * c + 3] = f.w;
        m = fmaxf(m, fmaxf(fmaxf(fabsf(f.x), fabsf(f.y)), fmaxf(fabsf(f.z), fabsf(f.w))));
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
    for (int c = 0; c < 4; c++) {
        __half2 a = __floats2half2_rn(v[4 * c] * inv, v[4 * c + 1] * inv);
        __half2 b = __floats2half2_rn(v[4 * c + 2] * inv, v[4 * c + 3] * inv);
        *reinterpret_cast<uint2*>(ic2h + (size_t)row * K + c * 128 + lane * 4) =
            make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
    }
    if (lane == 0) row_scale[row] = sc;
}

// ---- the grouped GEMM ------------------------------------------------------------------------
struct UmmaArgs {
    const uint16_t* global;    // [slots, N] f16 row globals
    const int4* groups;        // (slot, first sorted row, rows <= 256, 0)
    const int32_t* n_groups;
    const int32_t* route_idx;  // sorted position -> route
    const float* row_scale;    // per sorted row: power-of-two scale of the activations
    const float* route_weight; // down only, indexed by route
    float* ic2;                // gate_up out [rows, inter] f32 (sorted rows)
    void* y;                   // down out [rows, hidden], bf16 or f32 (sorted rows)
    int y_f32;
    int32_t* err;
    int N;                     // rows of the weight matrix (2 * inter or hidden)
};

// warp roles of the GEMM CTA (16 warps)
constexpr int kWarpActTma = 0, kWarpMma = 1, kWarpRawTma = 2, kWarpEpi0 = 4, kWarpDeq0 = 8;
constexpr int kDeqThreads = 256;
constexpr int kRawStages = 5;
constexpr int kRawPackedBytes = kTileN * 64;   // one chunk of 128 k: 128 rows x 64 bytes
constexpr int kRawScaleBytes = kTileN * 16;    // 128 rows x 16 scale bytes (256 k: the chunk's half is used)
constexpr int kRawStageBytes = kRawPackedBytes + kRawScaleBytes;
constexpr int kAccStages = 2;                  // accumulator sets in tensor memory (2 x 256 columns)

template <bool GATE_UP, int K>
__global__ void __launch_bounds__(kThreads, 1)
umma_grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_packed,
                         const __grid_constant__ CUtensorMap tmap_scale, UmmaArgs a) {
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment for the swizzled tiles
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* const a_tiles = smem;                                                  // [kAStages][kMaxTokTiles][16 KiB]
    uint8_t* const b_tiles = a_tiles + kAStages * kMaxTokTiles * kTileBytes;        // [2 buffers][2 k-steps][16 KiB]
    uint8_t* const raw_ring = b_tiles + 4 * kTileBytes;                              // [kRawStages][packed | scales]
    float* const s_glob = reinterpret_cast<float*>(raw_ring + kRawStages * kRawStageBytes);  // [4 epilogue warps][128]
    uint64_t* const bars = reinterpret_cast<uint64_t*>(s_glob + 4 * kTileN);
    uint32_t* const s_tmem = reinterpret_cast<uint32_t*>(bars + 32);
    volatile int* const s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
    const uint32_t bar0 = smem_u32(bars);
    auto A_FULL = [&](int s) { return bar0 + 8u * s; };
    auto A_EMPTY = [&](int s) { return bar0 + 8u * (3 + s); };
    auto B_READY = [&](int s) { return bar0 + 8u * (6 + s); };
    auto B_FREE = [&](int s) { return bar0 + 8u * (8 + s); };
    auto ACC_FULL = [&](int s) { return bar0 + 8u * (10 + s); };
    auto ACC_EMPTY = [&](int s) { return bar0 + 8u * (12 + s); };
    auto RAW_FULL = [&](int s) { return bar0 + 8u * (14 + s); };
    auto RAW_EMPTY = [&](int s) { return bar0 + 8u * (19 + s); };

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kAStages; s++) {
            mbar_init(A_FULL(s), 1);
            mbar_init(A_EMPTY(s), 1);
        }
        for (int s = 0; s < 2; s++) {
            mbar_init(B_READY(s), kDeqThreads);
            mbar_init(B_FREE(s), 1);
            mbar_init(ACC_FULL(s), 1);
            mbar_init(ACC_EMPTY(s), 128);
        }
        for (int s = 0; s < kRawStages; s++) {
            mbar_init(RAW_FULL(s), 1);
            mbar_init(RAW_EMPTY(s), kDeqThreads);
        }
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kWarpMma) {
        // all 512 columns of tensor memory: two accumulator sets of two 128-column f32 tiles
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(s_tmem)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *s_tmem;

    constexpr int kSteps = K / kStepK;
    constexpr int kChunks = K / 128;
    const int n_tiles = a.N / kTileN;
    const int n_units = *a.n_groups * n_tiles;
    // tile row n of tile nt -> weight row: gate_up tiles are 64 gate rows followed by the 64 matching up rows
    auto weight_row = [&](int nt, int n) -> int {
        if (GATE_UP) return (n < 64) ? nt * 64 + n : a.N / 2 + nt * 64 + (n - 64);
        return nt * kTileN + n;
    };

    if (warp == kWarpActTma) {
        // ===================== activation tiles: TMA, 128-byte swizzle ============================
        if (lane == 0) {
            uint32_t it = 0;
            for (int u = blockIdx.x; u < n_units && !*s_abort; u += gridDim.x) {
                const int4 grp = a.groups[u / n_tiles];
                const int ntt = (grp.z + kTileM - 1) / kTileM;
                bool ok = true;
                for (int ks = 0; ks < kSteps && ok; ks++, it++) {
                    const int st = it % kAStages;
                    ok = mbar_wait(A_EMPTY(st), ((it / kAStages) & 1) ^ 1, s_abort, a.err);
                    if (!ok) break;
                    mbar_expect_tx(A_FULL(st), (uint32_t)(ntt * kTileBytes));
                    for (int t = 0; t < ntt; t++)
                        tma_load_2d(smem_u32(a_tiles + (size_t)(st * kMaxTokTiles + t) * kTileBytes), &tmap_a, ks * kStepK,
                                    grp.y + t * kTileM, A_FULL(st));
                }
                if (!ok) break;
            }
        }
    } else if (warp == kWarpRawTma) {
        // ===================== packed weights and block scales: TMA into the raw ring ===============
        if (lane == 0) {
            uint32_t it = 0;
            for (int u = blockIdx.x; u < n_units && !*s_abort; u += gridDim.x) {
                const int4 grp = a.groups[u / n_tiles];
                const int nt = u % n_tiles;
                const int row0 = grp.x * a.N;
                bool ok = true;
                for (int c = 0; c < kChunks && ok; c++, it++) {
                    const int st = it % kRawStages;
                    ok = mbar_wait(RAW_EMPTY(st), ((it / kRawStages) & 1) ^ 1, s_abort, a.err);
                    if (!ok) break;
                    const uint32_t dst = smem_u32(raw_ring + (size_t)st * kRawStageBytes);
                    mbar_expect_tx(RAW_FULL(st), kRawStageBytes);
                    if (GATE_UP) {
                        // boxes of 64 rows: the gate rows, then the matching up rows
                        tma_load_2d(dst, &tmap_packed, c * 64, row0 + weight_row(nt, 0), RAW_FULL(st));
                        tma_load_2d(dst + kRawPackedBytes / 2, &tmap_packed, c * 64, row0 + weight_row(nt, 64), RAW_FULL(st));
                        tma_load_2d(dst + kRawPackedBytes, &tmap_scale, (c >> 1) * 16, row0 + weight_row(nt, 0), RAW_FULL(st));
                        tma_load_2d(dst + kRawPackedBytes + kRawScaleBytes / 2, &tmap_scale, (c >> 1) * 16,
                                    row0 + weight_row(nt, 64), RAW_FULL(st));
                    } else {
                        tma_load_2d(dst, &tmap_packed, c * 64, row0 + weight_row(nt, 0), RAW_FULL(st));
                        tma_load_2d(dst + kRawPackedBytes, &tmap_scale, (c >> 1) * 16, row0 + weight_row(nt, 0), RAW_FULL(st));
                    }
                }
                if (!ok) break;
            }
        }
    } else if (warp == kWarpMma) {
        // ===================== MMA issuer ======================================================
        if (lane == 0) {
            uint32_t it = 0, chunk = 0, unit_i = 0;
            for (int u = blockIdx.x; u < n_units && !*s_abort; u += gridDim.x, unit_i++) {
                const int4 grp = a.groups[u / n_tiles];
                const int ntt = (grp.z + kTileM - 1) / kTileM;
                const int acc = unit_i & 1;
                // this accumulator set must have been read back (two units ago)
                if (!mbar_wait(ACC_EMPTY(acc), ((unit_i >> 1) & 1) ^ 1, s_abort, a.err)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                bool ok = true;
                for (int ks = 0; ks < kSteps && ok; ks++, it++) {
                    const int st = it % kAStages;
                    const int buf = chunk & 1;
                    if ((ks & 1) == 0) ok = mbar_wait(B_READY(buf), (chunk >> 1) & 1, s_abort, a.err);
                    if (ok) ok = mbar_wait(A_FULL(st), (it / kAStages) & 1, s_abort, a.err);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t b_addr = smem_u32(b_tiles + (size_t)(buf * 2 + (ks & 1)) * kTileBytes);
                    for (int t = 0; t < ntt; t++) {
                        const uint32_t a_addr = smem_u32(a_tiles + (size_t)(st * kMaxTokTiles + t) * kTileBytes);
#pragma unroll
                        for (int kk = 0; kk < kStepK / 16; kk++)
                            umma_f16(tmem_base + acc * (kMaxTokTiles * kTileN) + t * kTileN, umma_desc(a_addr + kk * 32),
                                     umma_desc(b_addr + kk * 32), (ks > 0 || kk > 0) ? 1u : 0u);
                    }
                    umma_commit(A_EMPTY(st));            // the activation stage is free once these MMAs retire
                    if (ks & 1) {
                        umma_commit(B_FREE(buf));        // and so is the dequantised buffer
                        chunk++;
                    }
                }
                if (!ok) break;
                umma_commit(ACC_FULL(acc));
            }
        }
    } else if (warp >= kWarpDeq0) {
        // ===================== dequantisers (8 warps): raw ring -> swizzled f16 B tiles ==============
        const int tid = threadIdx.x - kWarpDeq0 * 32;   // 0..255
        uint32_t chunk = 0;
        for (int u = blockIdx.x; u < n_units && !*s_abort; u += gridDim.x) {
            bool ok = true;
            for (int c = 0; c < kChunks && ok; c++, chunk++) {
                const int buf = chunk & 1, st = chunk % kRawStages;
                ok = mbar_wait(RAW_FULL(st), (chunk / kRawStages) & 1, s_abort, a.err);
                if (ok) ok = mbar_wait(B_FREE(buf), ((chunk >> 1) & 1) ^ 1, s_abort, a.err);
                if (!ok) break;
                const uint8_t* const rp = raw_ring + (size_t)st * kRawStageBytes;
                // 128 rows x 4 pieces of 16 bytes (32 k, two scale blocks); four lanes share a row
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    const int unit = tid + kDeqThreads * i;
                    const int row = unit >> 2, piece = unit & 3;
                    const uint4 raw = *reinterpret_cast<const uint4*>(rp + row * 64 + piece * 16);
                    const uint16_t sc2 =
                        *reinterpret_cast<const uint16_t*>(rp + kRawPackedBytes + row * 16 + (c & 1) * 8 + piece * 2);
                    uint32_t h2;
                    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(sc2));
                    const uint32_t s0 = __byte_perm(h2, h2, 0x1010), s1 = __byte_perm(h2, h2, 0x3232);
                    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
                    // piece -> k-step (piece / 2) and 16-byte chunks (piece % 2) * 4 + j of the 128-byte row
                    uint8_t* const brow = b_tiles + (size_t)(buf * 2 + (piece >> 1)) * kTileBytes + row * 128;
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        uint32_t q[4];
                        e2m1x8_to_f16x2(w[j], q);
                        const uint32_t s = (j < 2) ? s0 : s1;
#pragma unroll
                        for (int r = 0; r < 4; r++) q[r] = hmul2_f16(q[r], s);
                        const int c16 = (piece & 1) * 4 + j;
                        *reinterpret_cast<uint4*>(brow + ((c16 ^ (row & 7)) << 4)) = make_uint4(q[0], q[1], q[2], q[3]);
                    }
                }
                mbar_arrive(RAW_EMPTY(st));
                // generic-proxy writes must be visible to the tensor core's async-proxy reads
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(B_READY(buf));
            }
            if (!ok) break;
        }
    } else if (warp >= kWarpEpi0) {
        // ===================== epilogue (warps 4..7: TMEM lane quarters 0..3) =======================
        const int quarter = warp & 3;
        float* const my_glob = s_glob + quarter * kTileN;   // private to this warp
        uint32_t unit_i = 0;
        for (int u = blockIdx.x; u < n_units && !*s_abort; u += gridDim.x, unit_i++) {
            const int4 grp = a.groups[u / n_tiles];
            const int nt = u % n_tiles;
            const int ntt = (grp.z + kTileM - 1) / kTileM;
            const int acc = unit_i & 1;
            __syncwarp();
#pragma unroll
            for (int q = 0; q < 4; q++)
                my_glob[lane + 32 * q] = f16_global_to_f32(a.global[(size_t)grp.x * a.N + weight_row(nt, lane + 32 * q)]);
            __syncwarp();
            if (!mbar_wait(ACC_FULL(acc), (unit_i >> 1) & 1, s_abort, a.err)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (int t = 0; t < ntt; t++) {
                const int row_in_pass = t * kTileM + quarter * 32 + lane;
                const bool valid = row_in_pass < grp.z;
                const int pos = grp.y + row_in_pass;
                const float rs = valid ? a.row_scale[pos] : 0.f;
                const uint32_t taddr =
                    tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * (kMaxTokTiles * kTileN) + t * kTileN;
                if (GATE_UP) {
#pragma unroll 1
                    for (int c0 = 0; c0 < 64; c0 += 16) {
                        float g[16], up[16];
                        tmem_ld16(taddr + c0, g);
                        tmem_ld16(taddr + 64 + c0, up);
                        tmem_ld_wait();
                        if (valid) {
                            float o[16];
#pragma unroll
                            for (int j = 0; j < 16; j++) {
                                const float gate = g[j] * my_glob[c0 + j] * rs, upv = up[j] * my_glob[64 + c0 + j] * rs;
                                o[j] = (gate / (1.0f + __expf(-gate))) * upv;
                            }
                            float4* dst = reinterpret_cast<float4*>(a.ic2 + (size_t)pos * (a.N / 2) + nt * 64 + c0);
#pragma unroll
                            for (int j = 0; j < 4; j++) dst[j] = make_float4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
                        }
                    }
                } else {
                    const float wr = valid ? a.route_weight[a.route_idx[pos]] : 0.f;
#pragma unroll 1
                    for (int c0 = 0; c0 < kTileN; c0 += 16) {
                        float v[16];
                        tmem_ld16(taddr + c0, v);
                        tmem_ld_wait();
                        if (valid) {
#pragma unroll
                            for (int j = 0; j < 16; j++) v[j] = wr * ((v[j] * rs) * my_glob[c0 + j]);
                            const size_t o = (size_t)pos * a.N + nt * kTileN + c0;
                            if (a.y_f32) {
                                float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(a.y) + o);
#pragma unroll
                                for (int j = 0; j < 4; j++) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                            } else {
                                uint32_t pk[8];
#pragma unroll
                                for (int j = 0; j < 8; j++) {
                                    __nv_bfloat162 b2 = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                                    pk[j] = *reinterpret_cast<uint32_t*>(&b2);
                                }
                                uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.y) + o);
                                dst[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                                dst[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                            }
                        }
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(ACC_EMPTY(acc));
        }
    }
    // drain: nobody frees tensor memory while another role may still touch it
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == kWarpMma) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
    }
}

constexpr size_t kUmmaSmem = 1024 + (size_t)(kAStages * kMaxTokTiles + 4) * kTileBytes + (size_t)kRawStages * kRawStageBytes +
                             4 * kTileN * 4 + 32 * 8 + 64;
static_assert(kUmmaSmem <= 227 * 1024, "shared memory of the grouped GEMM CTA");

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// f16 matrix [rows, K] row-major, box = 64 k x 128 rows, 128-byte swizzle
bool make_act_map(CUtensorMap* map, const void* base, size_t rows, int K) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)kStepK, (cuuint32_t)kTileM};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

__global__ void prefill_invert_kernel(const int32_t* __restrict__ route_idx, const int32_t* __restrict__ n_sorted,
                                      int32_t* __restrict__ pos_of_route) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < *n_sorted) pos_of_route[route_idx[i]] = i;
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

// u8 matrix [rows, row_bytes] row-major (packed nibbles or block scales), box = box_bytes x box_rows, no swizzle
bool make_raw_map(CUtensorMap* map, const void* base, size_t rows, int row_bytes, int box_bytes, int box_rows) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
    cuuint32_t box[2] = {(cuuint32_t)box_bytes, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

bool prefill_umma_supported(int hidden, int inter, int slots, int experts, bool have_expert_ids) {
    if (hidden != 2048 || inter != 512) return false;
    if ((have_expert_ids ? experts : slots) > 1024) return false;
    return encode_tiled() != nullptr;
}

int launch_prefill_umma(const BankView& b, const void* x, int x_dtype, const DecodeRoutes& rt,
                        const float* route_weight, int tokens, int top_k, PrefillScratch sc, int sm_count,
                        const float* shared, const float* se_gate, cudaEvent_t join, void* out, int out_dtype,
                        const Ctx& c) {
    const int routes = tokens * top_k;
    int launches = 0;
    // 1. buckets, stable: by expert id of the layer (serving call) or by slot id
    const int32_t* bins_of_route;
    const int32_t* slot_of_bin = nullptr;
    const int32_t* route_slot;
    int nbins;
    if (rt.expert_ids) {
        launches += launch_slot_rewrite(rt.expert_ids, rt.ids_dtype, routes, rt.layer, rt.experts, rt.slot_for_id, rt.n_ids,
                                        rt.route_slot_out, sc.route_bin, rt.bad_flag, c);
        bins_of_route = sc.route_bin;
        slot_of_bin = rt.slot_for_id + (size_t)rt.layer * rt.experts;
        route_slot = rt.route_slot_out;
        nbins = rt.experts;
    } else {
        bins_of_route = rt.route_slot_in;
        route_slot = rt.route_slot_in;
        nbins = b.slots;
    }
    launches += launch_csr_build(bins_of_route, routes, nbins, sc.seg, sc.route_idx, sc.csr_scratch, sc.csr_flag, c);
    // 2. passes of <= 256 sorted rows per expert
    launches += launch_groups_from_csr(sc.seg, nbins, slot_of_bin, b.slots, kMaxTokTiles * kTileM, sc.groups, sc.n_groups, c);
    // 3. sorted, scaled f16 activations
    c.begin(K_PERMUTE_ACT);
    prefill_gather_kernel<<<routes, 256, 0, c.s>>>(x, x_dtype, sc.route_idx, sc.seg + nbins, top_k, b.hidden, sc.xg,
                                                   sc.row_scale);
    c.end();
    launches++;

    CUtensorMap map_x, map_h, map_gp, map_gs, map_dp, map_ds;
    const size_t gu_rows = (size_t)b.slots * 2 * b.inter, dn_rows = (size_t)b.slots * b.hidden;
    if (!make_act_map(&map_x, sc.xg, (size_t)routes, b.hidden) || !make_act_map(&map_h, sc.ic2h, (size_t)routes, b.inter) ||
        !make_raw_map(&map_gp, b.gu_packed, gu_rows, b.hidden / 2, 64, 64) ||
        !make_raw_map(&map_gs, b.gu_scale, gu_rows, b.hidden / 16, 16, 64) ||
        !make_raw_map(&map_dp, b.dn_packed, dn_rows, b.inter / 2, 64, 128) ||
        !make_raw_map(&map_ds, b.dn_scale, dn_rows, b.inter / 16, 16, 128))
        return -1;
    static bool attr = false;
    if (!attr) {
        cudaFuncSetAttribute(umma_grouped_gemm_kernel<true, 2048>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kUmmaSmem);
        cudaFuncSetAttribute(umma_grouped_gemm_kernel<false, 512>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kUmmaSmem);
        attr = true;
    }
    UmmaArgs a{};
    a.groups = sc.groups; a.n_groups = sc.n_groups; a.route_idx = sc.route_idx; a.err = sc.err;
    a.global = b.gu_global; a.row_scale = sc.row_scale;
    a.ic2 = sc.ic2; a.N = 2 * b.inter;
    c.begin(K_GROUPED_GATE_UP);
    umma_grouped_gemm_kernel<true, 2048><<<sm_count, kThreads, kUmmaSmem, c.s>>>(map_x, map_gp, map_gs, a);
    c.end();
    c.begin(K_PREFILL_RESCALE);
    prefill_rescale_kernel<<<(routes + 7) / 8, 256, 0, c.s>>>(sc.ic2, sc.seg + nbins, b.inter, sc.ic2h, sc.row_scale2);
    c.end();
    a.global = b.dn_global; a.row_scale = sc.row_scale2;
    a.route_weight = route_weight; a.y = sc.y; a.y_f32 = (out_dtype == 1); a.N = b.hidden;
    c.begin(K_GROUPED_DOWN);
    umma_grouped_gemm_kernel<false, 512><<<sm_count, kThreads, kUmmaSmem, c.s>>>(map_h, map_dp, map_ds, a);
    c.end();
    launches += 3;
    // 4. un-permute and sum in route order; routes of experts that are not resident are skipped
    if (join) cudaStreamWaitEvent(c.s, join, 0);
    c.begin(K_SUM_ROUTES);
    prefill_invert_kernel<<<(routes + 255) / 256, 256, 0, c.s>>>(sc.route_idx, sc.seg + nbins, sc.pos_of_route);
    dim3 grid(tokens, (b.hidden / 4 + 127) / 128);
    prefill_combine_kernel<<<grid, 128, 0, c.s>>>(sc.y, out_dtype == 1, sc.pos_of_route, route_slot, b.slots, top_k, b.hidden, shared, se_gate,
                                                  out, out_dtype);
    c.end();
    return launches + 2;
}

}  // namespace ftm
