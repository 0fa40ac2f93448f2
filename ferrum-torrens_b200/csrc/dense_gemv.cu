// Dense NVFP4 GEMV for the decode tail (the lm_head): c[m, n] = global[n] * sum_k a[m, k] * W[n, k].
//
// Reference: python/ferrum_kernel/linear.py:41-150 (`_nvfp4_dense_gemv_kernel`, oracle
// `nvfp4_dense_gemv_reference`), launcher src/infrastructure/cuda_linear.rs:48-175 (`DenseGemv::gemv`).
// The weight is the engine's K-MAJOR resident bank, exactly as that launcher takes it:
//   packed [K/8, N] int32   word (w, n) holds the eight e2m1 codes k = 8w .. 8w+7 of row n, nibble j -> k = 8w + j
//   scale  [K/16, N] uint8  e4m3 block scale of block b of row n at (b, n)
//   global [N] f16
// 248 320 x 2048 is 254 MB of packed bytes and 32 MB of scales, streamed once per step: a pure
// HBM-bandwidth kernel, built like the register-streaming expert kernel of decode_mma.cu.
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

namespace ftm {

namespace {

constexpr int kDgWarps = 8;
constexpr int kDgPre = 4;        // steps in flight per warp
constexpr int kDgTileRows = 32;

struct DenseArgs {
    const void* a;           // [M, K] bf16 or f32
    int a_dtype;
    const uint32_t* packed;  // [K/8, N]
    const uint8_t* scale;    // [K/16, N]
    const uint16_t* global;  // [N]
    float* c;                // [M, N], cleared before the launch
    int M, N, K, tok0, ntok, splits;
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
                      int M, int N, int K, float* c, int sm_count, const Ctx& ctx) {
    DenseArgs d{};
    d.a = a; d.a_dtype = a_dtype; d.packed = packed; d.scale = scale; d.global = global; d.c = c;
    d.M = M; d.N = N; d.K = K;
    d.splits = (K % 64 == 0) ? 2 : 1;
    int launches = 0;
    if (d.splits > 1) cudaMemsetAsync(c, 0, (size_t)M * N * sizeof(float), ctx.s);
    ctx.begin(K_DENSE_GEMV);
    // sixteen tokens per pass over the weights (the decode tail runs at one token per sequence)
    for (int t0 = 0; t0 < M; t0 += 16) {
        d.tok0 = t0;
        d.ntok = (M - t0 < 16) ? M - t0 : 16;
        if (d.ntok <= 8)
            launch_one<1>(d, sm_count, ctx.s);
        else
            launch_one<2>(d, sm_count, ctx.s);
        launches++;
    }
    ctx.end();
    return launches;
}

}  // namespace ftm
