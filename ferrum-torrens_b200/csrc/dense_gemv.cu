// Dense NVFP4 GEMV for the decode tail (the lm_head): c[m, n] = global[n] * sum_k a[m, k] * W[n, k].
//
// Reference: python/ferrum_kernel/linear.py:41-150 (`_nvfp4_dense_gemv_kernel`, oracle
// `nvfp4_dense_gemv_reference`), launcher src/infrastructure/cuda_linear.rs:48-175 (`DenseGemv::gemv`).
// The weight is the engine's K-MAJOR resident bank, exactly as that launcher takes it:
//   packed [K/8, N] int32   word (w, n) holds the eight e2m1 codes k = 8w .. 8w+7 of row n, nibble j -> k = 8w + j
//   scale  [K/16, N] uint8  e4m3 block scale of block b of row n at (b, n)
//   global [N] f16
// 248 320 x 2048 is 254 MB of packed bytes and 32 MB of scales, streamed once per step: a pure
// HBM-bandwidth kernel.  Two kernels share the fragment mapping below: a register-streaming one (any N % 4,
// K % 32) and, for N % 16 == 0 and K % 256 == 0, one fed by tiled TMA through a shared-memory ring, which is
// the one the lm_head takes (2.3 times the rate of the first on that shape).
//
// Work item: 32 consecutive rows (n) x one half of K.  In a K-major bank four consecutive rows of one k-word
// are 16 contiguous bytes, so lane (g8, t4) of a warp loads, per step, k-word 4*s + t4 of rows
// n0 + 4*g8 .. + 3 with ONE 128-bit load (a warp-wide load is four full 128-byte lines) and the four rows'
// block scales with one 32-bit load.  Which actual row sits in which row of an MMA tile is free, as long as
// the four lanes of a quad agree, so the quad's rows (+0, +1) form one m16n8k16 tile and (+2, +3) another:
//   A (16 rows x 16 k)  row g8 = actual row n0 + 4*g8 (+2), row g8 + 8 = actual row n0 + 4*g8 + 1 (+3);
//                       the quad's four lanes supply k slots {2t, 2t+1, 2t+8, 2t+9} from half of their word
//   B (16 k x 8 tokens) the same eight k of the lane's word for token g8: one 128-bit shared load from the
//                       token's f16 row in natural k order
// Every word is converted with the hardware e2m1x2 -> f16x2 conversion, multiplied by its row's block
// scale (exact in f16) and used by two MMAs per row pair, f32 accumulate.  The two K halves of a row meet
// in `c` by atomic add (c is cleared first; two partial sums commute, so the result is deterministic).
// Loads run kPre steps ahead in a rotating register buffer; nothing waits on a barrier.
#include "kernels.cuh"
#include "umma.cuh"

namespace ftm {

namespace {

constexpr int kDgWarps = 8;
constexpr int kDgPre = 8;        // steps in flight per warp
constexpr int kDgTileRows = 32;

struct DenseArgs {
    const void* a;           // [M, K] bf16 or f32
    int a_dtype;
    const uint32_t* packed;  // [K/8, N]
    const uint8_t* scale;    // [K/16, N]
    const uint16_t* global;  // [N]
    float* c;                // [M, N], cleared before the launch
    int M, N, K, tok0, ntok, splits;
    int32_t* err;
};

__device__ __forceinline__ uint4 ldg_stream128(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ldg_u32(const void* p) {
    uint32_t v;
    asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
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
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NT token tiles of 8; dynamic shared memory: the tokens' f16 rows (padded by 64 bytes so that the eight
// token rows of a 128-bit fragment load fall into different banks) and their power-of-two scales
template <int NT>
__global__ void __launch_bounds__(kDgWarps * 32, 2) dense_gemv_kernel(DenseArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int K = a.K, N = a.N;
    const int rsx = K * 2 + 64;
    float* const s_xscale = reinterpret_cast<float*>(smem + (size_t)8 * NT * rsx);
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int g8 = lane >> 2, t4 = lane & 3;

    // ---- the activations: warp w converts tokens w, w + 8, .. ----
    for (int tk = warp; tk < 8 * NT; tk += kDgWarps) {
        __half* const xrow = reinterpret_cast<__half*>(smem + (size_t)tk * rsx);
        if (tk >= a.ntok) {      // unused token rows read as zero
            for (int k = lane * 8; k < K; k += 256) *reinterpret_cast<uint4*>(xrow + k) = make_uint4(0, 0, 0, 0);
            if (lane == 0) s_xscale[tk] = 0.f;
            continue;
        }
        const size_t row = (size_t)(a.tok0 + tk) * K;
        float m = 0.f;
        for (int k = lane; k < K; k += 32) m = fmaxf(m, fabsf(load_act(a.a, a.a_dtype, row + k)));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        // largest magnitude into [2^14, 2^15): exact power-of-two scaling into the f16 range
        const int e = (int)((__float_as_uint(m) >> 23) & 0xff);
        float inv = 1.0f, sc = 1.0f;
        if (e > 0 && e < 255) {
            inv = __uint_as_float((uint32_t)(127 + 14 - (e - 127)) << 23);
            sc = __uint_as_float((uint32_t)(127 - 14 + (e - 127)) << 23);
        }
        for (int k = lane * 2; k < K; k += 64) {
            const float v0 = load_act(a.a, a.a_dtype, row + k), v1 = load_act(a.a, a.a_dtype, row + k + 1);
            *reinterpret_cast<__half2*>(xrow + k) = __floats2half2_rn(v0 * inv, v1 * inv);
        }
        if (lane == 0) s_xscale[tk] = sc;
    }
    __syncthreads();

    const int tiles = (N + kDgTileRows - 1) / kDgTileRows;
    const int steps = K / (32 * a.splits);        // 32 k (four k-words) per step
    const long long items = (long long)tiles * a.splits;
    const long long stride = (long long)gridDim.x * kDgWarps;
    for (long long it = (long long)blockIdx.x * kDgWarps + warp; it < items; it += stride) {
        // items that run at the same time cover neighbouring rows of the same k-words: the bank is read in
        // wide contiguous stripes
        const int split = (int)(it / tiles), tile = (int)(it % tiles);
        const int n = tile * kDgTileRows + 4 * g8;           // this lane's four rows
        const bool live = n < N;                             // N is a multiple of 4: a quad is in or out
        const int kw0 = split * steps * 4 + t4;              // this lane's k-word of step 0
        const uint32_t* const pp = a.packed + (size_t)kw0 * N + n;
        const uint8_t* const sp = a.scale + (size_t)(kw0 >> 1) * N + n;
        uint4 wb[kDgPre];
        uint32_t sb[kDgPre];
        auto fetch = [&](int s, int sl) {
            if (live) {
                wb[sl] = ldg_stream128(pp + (size_t)s * 4 * N);
                sb[sl] = ldg_u32(sp + (size_t)s * 2 * N);     // k-word 4s + t4 lies in block 2s + (t4 >> 1)
            } else {
                wb[sl] = make_uint4(0, 0, 0, 0);
                sb[sl] = 0;
            }
        };
#pragma unroll
        for (int p = 0; p < kDgPre; p++)
            if (p < steps) fetch(p, p);
        float acc[NT][2][2][4];
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int pr = 0; pr < 2; pr++)
#pragma unroll
                for (int h = 0; h < 2; h++)
#pragma unroll
                    for (int r = 0; r < 4; r++) acc[nt][pr][h][r] = 0.f;
        const uint8_t* const xa = smem + (size_t)g8 * rsx + (size_t)kw0 * 16;
        for (int s0 = 0; s0 < steps; s0 += kDgPre) {
#pragma unroll
            for (int sl = 0; sl < kDgPre; sl++) {
                const int s = s0 + sl;
                if (s < steps) {
                    const uint4 w4 = wb[sl];
                    const uint32_t sc4 = sb[sl];
                    if (s + kDgPre < steps) fetch(s + kDgPre, sl);
                    // four rows' block scales -> f16x2 with the scale in both halves
                    uint32_t h01, h23;
                    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h01) : "h"((uint16_t)sc4));
                    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h23) : "h"((uint16_t)(sc4 >> 16)));
                    const uint32_t sr[4] = {__byte_perm(h01, h01, 0x1010), __byte_perm(h01, h01, 0x3232),
                                            __byte_perm(h23, h23, 0x1010), __byte_perm(h23, h23, 0x3232)};
                    const uint32_t wr[4] = {w4.x, w4.y, w4.z, w4.w};
                    uint32_t q[4][4];
#pragma unroll
                    for (int r = 0; r < 4; r++) {
                        e2m1x8_to_f16x2(wr[r], q[r]);
#pragma unroll
                        for (int e = 0; e < 4; e++) q[r][e] = hmul2_f16(q[r][e], sr[r]);
                    }
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        const uint4 xb = *reinterpret_cast<const uint4*>(xa + (size_t)nt * 8 * rsx + (size_t)s * 64);
#pragma unroll
                        for (int pr = 0; pr < 2; pr++) {
                            // k slots (2t, 2t+1 | 2t+8, 2t+9) <- the word's k (0,1 | 2,3), then (4,5 | 6,7)
                            mma_f16(acc[nt][pr][0], q[2 * pr][0], q[2 * pr + 1][0], q[2 * pr][1], q[2 * pr + 1][1], xb.x, xb.y);
                            mma_f16(acc[nt][pr][1], q[2 * pr][2], q[2 * pr + 1][2], q[2 * pr][3], q[2 * pr + 1][3], xb.z, xb.w);
                        }
                    }
                }
            }
        }
        // ---- epilogue: tile rows g8 / g8 + 8 are actual rows n + 2*pr / n + 2*pr + 1; tokens 2*t4, 2*t4 + 1 ----
        if (live) {
#pragma unroll
            for (int pr = 0; pr < 2; pr++) {
                const float g0 = f16_global_to_f32(a.global[n + 2 * pr]), g1 = f16_global_to_f32(a.global[n + 2 * pr + 1]);
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
#pragma unroll
                    for (int cc = 0; cc < 2; cc++) {
                        const int tok = nt * 8 + 2 * t4 + cc;
                        if (tok < a.ntok) {
                            const float ts = s_xscale[tok];
                            float* const dst = a.c + (size_t)(a.tok0 + tok) * N + n + 2 * pr;
                            const float v0 = ((acc[nt][pr][0][cc] + acc[nt][pr][1][cc]) * ts) * g0;
                            const float v1 = ((acc[nt][pr][0][2 + cc] + acc[nt][pr][1][2 + cc]) * ts) * g1;
                            if (a.splits > 1) {
                                atomicAdd(dst, v0);
                                atomicAdd(dst + 1, v1);
                            } else {
                                dst[0] = v0;
                                dst[1] = v1;
                            }
                        }
                    }
                }
            }
        }
    }
}


// ---- the same GEMV fed by TMA ------------------------------------------------------------------
// The register-streaming kernel above keeps few bytes in flight per SM for a bank whose k-word rows lie
// N * 4 bytes apart, and reaches a third of the HBM rate.  Here a CTA owns 672 consecutive rows and one half
// of K, and a producer warp brings, per stage of sixteen k-words, three boxes of [16 k-words x 232 rows] packed
// words and three boxes of [8 blocks x 224 rows] block scales into a ring of shared-memory stages (tiled TMA,
// one mbarrier per stage: six copy instructions per 50 KB; bulk copies of single 2 KB runs spent their time
// on the per-copy cost).  The 232-row box over-fetches eight rows so that its rows sit at a pitch of 928
// bytes, which puts the four k-words a quad reads into different banks.  Twenty-one consumer warps of 32 rows
// each read their fragments from there: the same lane -> (rows, k-word) map, the same conversions and MMAs
// as above.  The two K halves of a row meet in `c` by atomic add, as above (two partial sums commute).
constexpr int kTmBoxRows = 232;              // rows a weight box fetches
constexpr int kTmUseRows = 224;              // rows of it that are used: seven groups of 32
constexpr int kTmBoxes = 3;
constexpr int kTmTileRows = kTmBoxes * kTmUseRows;
constexpr int kTmWarps = kTmTileRows / 32;   // 21 consumer warps (the lm_head's 248 320 rows are 370 tiles: with the two
                                             // K halves 740 items, five for each of 148 CTAs)
constexpr int kTmKw = 16;                    // k-words per stage: four MMA steps
constexpr int kTmStages = 3;
constexpr int kTmWBoxBytes = kTmKw * kTmBoxRows * 4;
constexpr int kTmSBoxBytes = (kTmKw / 2) * kTmUseRows;
constexpr int kTmStageBytes = kTmBoxes * (kTmWBoxBytes + kTmSBoxBytes);
static_assert(kTmWBoxBytes % 128 == 0 && kTmSBoxBytes % 128 == 0, "TMA destinations are 128-byte aligned");

struct DenseMaps {
    CUtensorMap packed, scale;
};

template <int NT>
__global__ void __launch_bounds__((kTmWarps + 1) * 32, 1)
dense_gemv_tma_kernel(const __grid_constant__ DenseMaps maps, DenseArgs a) {
    using namespace umma;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* const smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~(uintptr_t)127);
    const int K = a.K, N = a.N;
    const int rsx = K * 2 + 64;
    uint8_t* const ring = smem;                                                    // [kTmStages][kTmStageBytes]
    uint8_t* const xrows = smem + (size_t)kTmStages * kTmStageBytes;               // [8 * NT][rsx]
    float* const s_xscale = reinterpret_cast<float*>(xrows + (size_t)8 * NT * rsx);
    uint64_t* const bars = reinterpret_cast<uint64_t*>(s_xscale + 8 * NT);         // full[stages], empty[stages]
    volatile int* const s_abort = reinterpret_cast<volatile int*>(bars + 2 * kTmStages);
    const uint32_t bar0 = smem_u32(bars);
    auto FULL = [&](int s) { return bar0 + 8u * s; };
    auto EMPTY = [&](int s) { return bar0 + 8u * (kTmStages + s); };
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int g8 = lane >> 2, t4 = lane & 3;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kTmStages; s++) {
            mbar_init(FULL(s), 1);
            mbar_init(EMPTY(s), kTmWarps);
        }
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();     // the barriers are initialised

    const int tiles = (N + kTmTileRows - 1) / kTmTileRows;
    const int stages_per_item = K / (8 * kTmKw * 2);      // half of K, sixteen k-words per stage
    const int items = tiles * 2;

    if (warp == kTmWarps) {
        // ===================== producer: one elected lane issues the four copies of a stage ===========
        uint32_t it = 0;
        for (int item = blockIdx.x; item < items && !*s_abort; item += gridDim.x) {
            const int split = item / tiles, n0 = (item % tiles) * kTmTileRows;
            bool ok = true;
            for (int s = 0; s < stages_per_item && ok; s++, it++) {
                const int st = it % kTmStages;
                ok = mbar_wait_warp(EMPTY(st), ((it / kTmStages) & 1) ^ 1, s_abort, a.err);
                if (!ok) break;
                if (elect_one()) {
                    const int kw = (split * stages_per_item + s) * kTmKw;
                    const uint32_t dst = smem_u32(ring + (size_t)st * kTmStageBytes);
                    // rows past N read as zero and count like the others
                    mbar_expect_tx(FULL(st), kTmStageBytes);
#pragma unroll
                    for (int b = 0; b < kTmBoxes; b++) {
                        tma_load_2d(dst + b * kTmWBoxBytes, &maps.packed, n0 + b * kTmUseRows, kw, FULL(st));
                        tma_load_2d(dst + kTmBoxes * kTmWBoxBytes + b * kTmSBoxBytes, &maps.scale, n0 + b * kTmUseRows, kw / 2, FULL(st));
                    }
                }
                __syncwarp();
            }
            if (!ok) break;
        }
        return;
    }

    // ===================== consumers: warp w owns rows 32 w .. 32 w + 31 of the tile ====================
    // ---- the activations (as in the kernel above): consumer warp w converts tokens w, w + 21, .. while the
    // producer already fills the ring ----
    for (int tk = warp; tk < 8 * NT; tk += kTmWarps) {
        __half* const xrow = reinterpret_cast<__half*>(xrows + (size_t)tk * rsx);
        if (tk >= a.ntok) {
            for (int k = lane * 8; k < K; k += 256) *reinterpret_cast<uint4*>(xrow + k) = make_uint4(0, 0, 0, 0);
            if (lane == 0) s_xscale[tk] = 0.f;
            continue;
        }
        const size_t row = (size_t)(a.tok0 + tk) * K;
        float m = 0.f;
#pragma unroll 16
        for (int k = lane; k < K; k += 32) m = fmaxf(m, fabsf(load_act(a.a, a.a_dtype, row + k)));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        const int e = (int)((__float_as_uint(m) >> 23) & 0xff);
        float inv = 1.0f, sc = 1.0f;
        if (e > 0 && e < 255) {
            inv = __uint_as_float((uint32_t)(127 + 14 - (e - 127)) << 23);
            sc = __uint_as_float((uint32_t)(127 - 14 + (e - 127)) << 23);
        }
#pragma unroll 8
        for (int k = lane * 2; k < K; k += 64) {
            const float v0 = load_act(a.a, a.a_dtype, row + k), v1 = load_act(a.a, a.a_dtype, row + k + 1);
            *reinterpret_cast<__half2*>(xrow + k) = __floats2half2_rn(v0 * inv, v1 * inv);
        }
        if (lane == 0) s_xscale[tk] = sc;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kTmWarps * 32) : "memory");     // the consumer warps only

    const int box = warp / 7, rbox = (warp % 7) * 32 + 4 * g8;     // this lane's four rows inside its box
    const uint32_t woff = box * kTmWBoxBytes + rbox * 4;
    const uint32_t soff = kTmBoxes * kTmWBoxBytes + box * kTmSBoxBytes + rbox;
    uint32_t it = 0;
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
        const int split = item / tiles, n0 = (item % tiles) * kTmTileRows;
        float acc[NT][2][2][4];      // [token tile][row pair][k half][fragment]
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int pr = 0; pr < 2; pr++)
#pragma unroll
                for (int h = 0; h < 2; h++)
#pragma unroll
                    for (int r = 0; r < 4; r++) acc[nt][pr][h][r] = 0.f;
        const uint8_t* const xa = xrows + (size_t)g8 * rsx + ((size_t)split * stages_per_item * kTmKw + t4) * 16;
        bool ok = true;
        for (int s = 0; s < stages_per_item; s++, it++) {
            const int st = it % kTmStages;
            ok = mbar_wait_warp(FULL(st), (it / kTmStages) & 1, s_abort, a.err);
            if (!ok) break;
            const uint8_t* const sp = ring + (size_t)st * kTmStageBytes;
#pragma unroll
            for (int j = 0; j < kTmKw / 4; j++) {
                const uint4 w4 = *reinterpret_cast<const uint4*>(sp + woff + (4 * j + t4) * (kTmBoxRows * 4));
                const uint32_t sc4 = *reinterpret_cast<const uint32_t*>(sp + soff + (2 * j + (t4 >> 1)) * kTmUseRows);
                uint32_t h01, h23;
                asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h01) : "h"((uint16_t)sc4));
                asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h23) : "h"((uint16_t)(sc4 >> 16)));
                const uint32_t sr[4] = {__byte_perm(h01, h01, 0x1010), __byte_perm(h01, h01, 0x3232),
                                        __byte_perm(h23, h23, 0x1010), __byte_perm(h23, h23, 0x3232)};
                const uint32_t wr[4] = {w4.x, w4.y, w4.z, w4.w};
                uint32_t q[4][4];
#pragma unroll
                for (int r = 0; r < 4; r++) {
                    e2m1x8_to_f16x2(wr[r], q[r]);
#pragma unroll
                    for (int e = 0; e < 4; e++) q[r][e] = hmul2_f16(q[r][e], sr[r]);
                }
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const uint4 xb = *reinterpret_cast<const uint4*>(xa + (size_t)nt * 8 * rsx + (size_t)(s * (kTmKw / 4) + j) * 64);
#pragma unroll
                    for (int pr = 0; pr < 2; pr++) {
                        mma_f16(acc[nt][pr][0], q[2 * pr][0], q[2 * pr + 1][0], q[2 * pr][1], q[2 * pr + 1][1], xb.x, xb.y);
                        mma_f16(acc[nt][pr][1], q[2 * pr][2], q[2 * pr + 1][2], q[2 * pr][3], q[2 * pr + 1][3], xb.z, xb.w);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(EMPTY(st));
        }
        if (!ok) break;
        // ---- epilogue: as above; rows past N of the last tile read as zero and are not stored ----
        const int n = n0 + box * kTmUseRows + rbox;
        if (n < N) {
#pragma unroll
            for (int pr = 0; pr < 2; pr++) {
                const float g0 = f16_global_to_f32(a.global[n + 2 * pr]), g1 = f16_global_to_f32(a.global[n + 2 * pr + 1]);
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
#pragma unroll
                    for (int cc = 0; cc < 2; cc++) {
                        const int tok = nt * 8 + 2 * t4 + cc;
                        if (tok < a.ntok) {
                            const float ts = s_xscale[tok];
                            float* const dst = a.c + (size_t)(a.tok0 + tok) * N + n + 2 * pr;
                            atomicAdd(dst, ((acc[nt][pr][0][cc] + acc[nt][pr][1][cc]) * ts) * g0);
                            atomicAdd(dst + 1, ((acc[nt][pr][0][2 + cc] + acc[nt][pr][1][2 + cc]) * ts) * g1);
                        }
                    }
                }
            }
        }
    }
}

template <int NT>
size_t tma_smem(int K) {
    return 128 + (size_t)kTmStages * kTmStageBytes + (size_t)8 * NT * (K * 2 + 64) + 8 * NT * sizeof(float) + 2 * kTmStages * 8 + 16;
}
template <int NT>
void launch_tma(const DenseMaps& maps, const DenseArgs& a, int sm_count, cudaStream_t s) {
    static PerDeviceOnce once;
    allow_dyn_smem(once, dense_gemv_tma_kernel<NT>, 222 * 1024);
    dense_gemv_tma_kernel<NT><<<sm_count, (kTmWarps + 1) * 32, tma_smem<NT>(a.K), s>>>(maps, a);
}

// [rows, inner] matrix of `esize`-byte elements, row-major, box = box_inner x box_rows, no swizzle
bool make_plain_map(CUtensorMap* map, CUtensorMapDataType type, int esize, const void* base, size_t inner, size_t rows,
                    int box_inner, int box_rows) {
    umma::EncodeTiledFn fn = umma::encode_tiled();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)inner * esize};
    cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, type, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int NT>
void launch_one(const DenseArgs& a, int sm_count, cudaStream_t s) {
    const size_t smem = (size_t)8 * NT * (a.K * 2 + 64) + 8 * NT * sizeof(float) + 16;
    static PerDeviceOnce once;
    allow_dyn_smem(once, dense_gemv_kernel<NT>, 100 * 1024);
    dense_gemv_kernel<NT><<<sm_count * 2, kDgWarps * 32, smem, s>>>(a);
}

}  // namespace

bool dense_gemv_supported(int N, int K) {
    // 16-byte loads of four rows, 32 k per step, the token rows of at most sixteen tokens in shared memory
    return N > 0 && K > 0 && N % 4 == 0 && K % 32 == 0 && (size_t)16 * (K * 2 + 64) + 256 <= 100 * 1024;
}

int launch_dense_gemv(const void* a, int a_dtype, const uint32_t* packed, const uint8_t* scale, const uint16_t* global,
                      int M, int N, int K, float* c, int sm_count, int32_t* err, const Ctx& ctx) {
    DenseArgs d{};
    d.a = a; d.a_dtype = a_dtype; d.packed = packed; d.scale = scale; d.global = global; d.c = c;
    d.M = M; d.N = N; d.K = K; d.err = err;
    // TMA wants the rows of both matrices 16-byte aligned (N % 16 for the scales) and whole stages per K half
    DenseMaps maps;
    const bool tma = N % 16 == 0 && K % 256 == 0 && N >= kTmTileRows && (reinterpret_cast<uintptr_t>(packed) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(scale) & 15) == 0 && tma_smem<2>(K) <= 222 * 1024 &&
                     make_plain_map(&maps.packed, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, packed, (size_t)N, (size_t)K / 8, kTmBoxRows, kTmKw) &&
                     make_plain_map(&maps.scale, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, scale, (size_t)N, (size_t)K / 16, kTmUseRows, kTmKw / 2);
    d.splits = (tma || K % 64 == 0) ? 2 : 1;
    int launches = 0;
    if (d.splits > 1) cudaMemsetAsync(c, 0, (size_t)M * N * sizeof(float), ctx.s);
    ctx.begin(K_DENSE_GEMV);
    // sixteen tokens per pass over the weights (the decode tail runs at one token per sequence)
    for (int t0 = 0; t0 < M; t0 += 16) {
        d.tok0 = t0;
        d.ntok = (M - t0 < 16) ? M - t0 : 16;
        if (tma) {
            if (d.ntok <= 8)
                launch_tma<1>(maps, d, sm_count, ctx.s);
            else
                launch_tma<2>(maps, d, sm_count, ctx.s);
        } else if (d.ntok <= 8) {
            launch_one<1>(d, sm_count, ctx.s);
        } else {
            launch_one<2>(d, sm_count, ctx.s);
        }
        launches++;
    }
    ctx.end();
    return launches;
}

}  // namespace ftm
