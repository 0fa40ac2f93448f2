// Shared expert for large batches: two dense bf16 GEMMs on the tcgen05 tensor cores.
//
// Reference behaviour (src/models/qwen3_6/forward.rs:684-714, src/infrastructure/cuda_linear.rs:391-450):
//   ic2    = silu(x . gate^T) * (x . up^T)            gate_up [2 * SI, H] bf16, f32 accumulate
//   shared = ic2 . down^T                             down [H, SI] bf16
//   se_gate = sigmoid(x . shared_gate)
// ic2 crosses between the GEMMs as a bf16 pair hi + lo (two planes [tokens, SI]; 16 significant bits),
// so the second GEMM runs over K = 2 * SI with the down rows read twice.
//
// One CTA per output tile D[128 tokens, 128 weight rows] (two CTAs share an SM, so one tile's epilogue
// overlaps the other's mainloop):
//   warp 0      TMA: activation tile [128 tokens x 64 k] and weight tile [128 rows x 64 k], 128-byte swizzle
//   warp 1      allocates 128 columns of tensor memory, issues tcgen05.mma (SS form, bf16 x bf16 -> f32)
//   warps 2..5  epilogue: tcgen05.ld, one thread per token row.  gate_up tiles hold 64 gate rows and the
//               64 matching up rows, so silu(gate) * up stays in one thread.
// Every mbarrier wait is bounded; a wait that gives up raises the error flag and the CTA drains.
#include "kernels.cuh"
#include "umma.cuh"

namespace ftm {

namespace {

using namespace umma;

constexpr int kTile = 128;                  // tokens per tile (M) and weight rows per tile (N)
constexpr int kStepK = 64;                  // one 128-byte swizzle atom of bf16
constexpr int kStages = 3;
constexpr int kOperandBytes = kTile * kStepK * 2;   // 16 KiB per operand tile
constexpr int kThreads = 192;
// bf16 x bf16 -> f32, both operands K-major, M = 128, N = 128
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kTile >> 3) << 17) | ((uint32_t)(kTile >> 4) << 24);

struct DenseArgs {
    int tokens;
    int k_steps;        // K / 64 of the activation matrix as the tensor map sees it
    int b_k_wrap;       // weight k coordinate = (step * 64) % b_k_wrap  (the hi and lo planes share the down rows)
    int a_row_plane;    // activation rows of the second plane start here (0: one plane)
    int k_steps_plane;  // steps per plane
    int up_row0;        // gate_up: first up row (SI); down: unused
    int out_ld;         // row stride of the output
    __nv_bfloat16* ic2b;    // gate_up out: planes hi, lo [tokens, SI]
    float* shared_out;      // down out [tokens, H] f32
    int32_t* err;
};

template <bool GATE_UP>
__global__ void __launch_bounds__(kThreads, 2)
dense_umma_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, DenseArgs a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* const a_tiles = smem;                                  // [kStages][16 KiB]
    uint8_t* const b_tiles = smem + kStages * kOperandBytes;        // [kStages][16 KiB]
    uint64_t* const bars = reinterpret_cast<uint64_t*>(b_tiles + kStages * kOperandBytes);
    uint32_t* const s_tmem = reinterpret_cast<uint32_t*>(bars + 8);
    volatile int* const s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
    const uint32_t bar0 = smem_u32(bars);
    auto FULL = [&](int s) { return bar0 + 8u * s; };
    auto EMPTY = [&](int s) { return bar0 + 8u * (3 + s); };
    const uint32_t ACC_FULL = bar0 + 8u * 6;

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; s++) {
            mbar_init(FULL(s), 1);
            mbar_init(EMPTY(s), 1);
        }
        mbar_init(ACC_FULL, 1);
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 128;" ::"r"(smem_u32(s_tmem)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *s_tmem;

    const int n_tile = blockIdx.x, t0 = blockIdx.y * kTile;

    if (warp == 0) {
        // TMA producer: the whole warp walks the loop, one elected lane issues
        bool ok = true;
        for (int ks = 0; ks < a.k_steps && ok; ks++) {
            const int st = ks % kStages;
            ok = mbar_wait_warp(EMPTY(st), ((ks / kStages) & 1) ^ 1, s_abort, a.err);
            if (!ok) break;
            if (elect_one()) {
                mbar_expect_tx(FULL(st), 2 * kOperandBytes);
                const int plane = ks / a.k_steps_plane;
                const int ka = (ks - plane * a.k_steps_plane) * kStepK;
                tma_load_2d(smem_u32(a_tiles + (size_t)st * kOperandBytes), &tmap_a, ka, plane * a.a_row_plane + t0, FULL(st));
                const int kb = (ks * kStepK) % a.b_k_wrap;
                const uint32_t bdst = smem_u32(b_tiles + (size_t)st * kOperandBytes);
                if (GATE_UP) {
                    // 64 gate rows, then the 64 matching up rows (the map's box is 64 rows)
                    tma_load_2d(bdst, &tmap_b, kb, n_tile * 64, FULL(st));
                    tma_load_2d(bdst + kOperandBytes / 2, &tmap_b, kb, a.up_row0 + n_tile * 64, FULL(st));
                } else {
                    tma_load_2d(bdst, &tmap_b, kb, n_tile * kTile, FULL(st));
                }
            }
            __syncwarp();
        }
    } else if (warp == 1) {
        // MMA issuer, same shape
        bool ok = true;
        for (int ks = 0; ks < a.k_steps && ok; ks++) {
            const int st = ks % kStages;
            ok = mbar_wait_warp(FULL(st), (ks / kStages) & 1, s_abort, a.err);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t adesc = umma_desc(smem_u32(a_tiles + (size_t)st * kOperandBytes));
            const uint64_t bdesc = umma_desc(smem_u32(b_tiles + (size_t)st * kOperandBytes));
            if (elect_one()) {
#pragma unroll
                for (int kk = 0; kk < 4; kk++) umma_f16_ss(tmem_base, adesc + kk * 2, bdesc + kk * 2, kIdesc, (ks > 0 || kk > 0) ? 1u : 0u);
                umma_commit(EMPTY(st));
            }
            __syncwarp();
        }
        if (ok && elect_one()) umma_commit(ACC_FULL);
        __syncwarp();
    } else {
        const int quarter = warp & 3;
        const int t = t0 + quarter * 32 + lane;
        const bool valid = t < a.tokens;
        if (mbar_wait(ACC_FULL, 0, s_abort, a.err)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
            if (GATE_UP) {
#pragma unroll 1
                for (int c0 = 0; c0 < 64; c0 += 16) {
                    float g[16], up[16];
                    tmem_ld16(taddr + c0, g);
                    tmem_ld16(taddr + 64 + c0, up);
                    tmem_ld_wait();
                    if (valid) {
                        uint32_t hi[8], lo[8];
#pragma unroll
                        for (int j = 0; j < 8; j++) {
                            const float v0 = (g[2 * j] / (1.0f + expf(-g[2 * j]))) * up[2 * j];
                            const float v1 = (g[2 * j + 1] / (1.0f + expf(-g[2 * j + 1]))) * up[2 * j + 1];
                            const __nv_bfloat162 h2 = __floats2bfloat162_rn(v0, v1);
                            const __nv_bfloat162 l2 = __floats2bfloat162_rn(v0 - __bfloat162float(h2.x), v1 - __bfloat162float(h2.y));
                            hi[j] = *reinterpret_cast<const uint32_t*>(&h2);
                            lo[j] = *reinterpret_cast<const uint32_t*>(&l2);
                        }
                        uint4* dh = reinterpret_cast<uint4*>(a.ic2b + (size_t)t * a.out_ld + n_tile * 64 + c0);
                        uint4* dl = reinterpret_cast<uint4*>(a.ic2b + (size_t)(a.tokens + t) * a.out_ld + n_tile * 64 + c0);
                        dh[0] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                        dh[1] = make_uint4(hi[4], hi[5], hi[6], hi[7]);
                        dl[0] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                        dl[1] = make_uint4(lo[4], lo[5], lo[6], lo[7]);
                    }
                }
            } else {
#pragma unroll 1
                for (int c0 = 0; c0 < kTile; c0 += 16) {
                    float v[16];
                    tmem_ld16(taddr + c0, v);
                    tmem_ld_wait();
                    if (valid) {
                        float4* dst = reinterpret_cast<float4*>(a.shared_out + (size_t)t * a.out_ld + n_tile * kTile + c0);
#pragma unroll
                        for (int j = 0; j < 4; j++) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 128;" ::"r"(tmem_base) : "memory");
    }
}

constexpr size_t kDenseSmem = 1024 + (size_t)2 * kStages * kOperandBytes + 8 * 8 + 64;

// bf16 matrix [rows, K] row-major, box = 64 k x box_rows, 128-byte swizzle
bool make_bf16_map(CUtensorMap* map, const void* base, size_t rows, int K, int box_rows) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)kStepK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// se_gate[t] = sigmoid(x[t] . shared_gate): one warp per token
__global__ void __launch_bounds__(256)
shared_gate_kernel(const __nv_bfloat16* __restrict__ x, int tokens, int H, const __nv_bfloat16* __restrict__ shared_gate,
                   float* __restrict__ se_gate) {
    const int t = blockIdx.x * 8 + threadIdx.x / 32, lane = threadIdx.x % 32;
    if (t >= tokens) return;
    float acc = 0.f;
    for (int k = lane * 8; k < H; k += 256) {
        const uint4 wv = *reinterpret_cast<const uint4*>(shared_gate + k);
        const uint4 xv = *reinterpret_cast<const uint4*>(x + (size_t)t * H + k);
        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w}, xx[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const float2 w2 = bf16x2_to_f32(ww[q]), x2 = bf16x2_to_f32(xx[q]);
            acc += w2.x * x2.x + w2.y * x2.y;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) se_gate[t] = 1.0f / (1.0f + expf(-acc));
}

}  // namespace

bool shared_umma_supported(int tokens, int hidden, int shared_inter) {
    return tokens >= 256 && hidden % 128 == 0 && shared_inter % 64 == 0 && shared_inter >= 64 && encode_tiled() != nullptr;
}

// ic2b: scratch of 2 * tokens * shared_inter bf16
int launch_shared_umma(const __nv_bfloat16* x, int tokens, int hidden, int shared_inter, const __nv_bfloat16* gate_up,
                       const __nv_bfloat16* down, const __nv_bfloat16* shared_gate, __nv_bfloat16* ic2b, float* shared_out,
                       float* se_gate, int32_t* err, const Ctx& c) {
    CUtensorMap map_x, map_gu, map_ic2, map_dn;
    if (!make_bf16_map(&map_x, x, (size_t)tokens, hidden, kTile) ||
        !make_bf16_map(&map_gu, gate_up, (size_t)2 * shared_inter, hidden, 64) ||
        !make_bf16_map(&map_ic2, ic2b, (size_t)2 * tokens, shared_inter, kTile) ||
        !make_bf16_map(&map_dn, down, (size_t)hidden, shared_inter, kTile))
        return -1;
    static PerDeviceOnce once_gu, once_dn;
    allow_dyn_smem(once_gu, dense_umma_kernel<true>, kDenseSmem);
    allow_dyn_smem(once_dn, dense_umma_kernel<false>, kDenseSmem);
    const int ttiles = (tokens + kTile - 1) / kTile;
    DenseArgs a{};
    a.tokens = tokens; a.err = err;
    // gate_up: K = hidden, one plane
    a.k_steps = hidden / kStepK; a.k_steps_plane = a.k_steps; a.b_k_wrap = hidden; a.a_row_plane = 0;
    a.up_row0 = shared_inter; a.out_ld = shared_inter; a.ic2b = ic2b;
    c.begin(K_SHARED_PHASE1);
    shared_gate_kernel<<<(tokens + 7) / 8, 256, 0, c.s>>>(x, tokens, hidden, shared_gate, se_gate);
    dense_umma_kernel<true><<<dim3(shared_inter / 64, ttiles), kThreads, kDenseSmem, c.s>>>(map_x, map_gu, a);
    c.end();
    // down: K = 2 * SI over the planes hi, lo; the down rows are read once per plane
    a.k_steps = 2 * shared_inter / kStepK; a.k_steps_plane = shared_inter / kStepK; a.b_k_wrap = shared_inter;
    a.a_row_plane = tokens; a.out_ld = hidden; a.shared_out = shared_out;
    c.begin(K_SHARED_PHASE2);
    dense_umma_kernel<false><<<dim3(hidden / kTile, ttiles), kThreads, kDenseSmem, c.s>>>(map_ic2, map_dn, a);
    c.end();
    return 3;
}

}  // namespace ftm
