// Shared device helpers of the NVFP4 MoE kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ftm_exact_math.h"

namespace ftm {

constexpr int kWarp = 32;

// ---- element decoders (src/domain/numerics.rs:6-68 of the reference) ----------------------

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t b16) { return __uint_as_float(b16 << 16); }

// two bf16 packed in a word -> two floats
__device__ __forceinline__ float2 bf16x2_to_f32(uint32_t w) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}

// e4m3fn code -> f32: normal codes rebias the exponent, subnormals are man * 2^-9, 0x7f/0xff are NaN
__device__ __forceinline__ float e4m3_to_f32(uint32_t c) {
    uint32_t sign = (c & 0x80u) << 24;
    uint32_t exp = (c >> 3) & 0xfu;
    uint32_t man = c & 7u;
    if (exp == 0) return __uint_as_float(sign | __float_as_uint((float)man * 0.001953125f));
    if (exp == 0xfu && man == 7u) return __uint_as_float(0x7fc00000u);
    return __uint_as_float(sign | ((exp + 120u) << 23) | (man << 20));
}

// f16 row global -> f32.  The reference's decoder returns man * 2^-24 for a subnormal
// whatever its sign bit says (src/domain/numerics.rs:19-22); kept so results are identical.
__device__ __forceinline__ float f16_global_to_f32(uint16_t bits) {
    if ((bits & 0x7c00u) == 0 && (bits & 0x3ffu) != 0) return (float)(bits & 0x3ffu) * 5.9604644775390625e-8f;
    return __half2float(__ushort_as_half(bits));
}

// e2m1 code (4 bits) -> f32, by arithmetic on the fields: s | ee | m
__device__ __forceinline__ float e2m1_to_f32(uint32_t c) {
    uint32_t sign = (c & 8u) << 28;
    uint32_t ee = (c >> 1) & 3u;
    uint32_t m = c & 1u;
    uint32_t mag = ee ? (((126u + ee) << 23) | (m << 22)) : (m ? 0x3f000000u : 0u);
    return __uint_as_float(sign | mag);
}

__device__ __forceinline__ float silu_f32(float v) { return v / (1.0f + __expf(-v)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// load / store one element of a boundary tensor given its dtype code (FTM_BF16 = 0, FTM_F32 = 1)
__device__ __forceinline__ float load_act(const void* p, int dtype, size_t i) {
    if (dtype == 0) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
    return reinterpret_cast<const float*>(p)[i];
}
__device__ __forceinline__ void store_act(void* p, int dtype, size_t i, float v) {
    if (dtype == 0)
        reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
    else
        reinterpret_cast<float*>(p)[i] = v;
}

// device view of the six banks plus the shapes the kernels index with
struct BankView {
    const uint8_t* gu_packed;  // [slots, 2I, H/2]
    const uint8_t* gu_scale;   // [slots, 2I, H/16]
    const uint16_t* gu_global; // [slots, 2I]
    const uint8_t* dn_packed;  // [slots, H, I/2]
    const uint8_t* dn_scale;   // [slots, H, I/16]
    const uint16_t* dn_global; // [slots, H]
    // the block scales once more, in the order the decode kernels' lanes consume them (see decode_mma.cu,
    // "fragment-ordered scales"); null when the adapter keeps no such copy
    const uint8_t* gu_scale_frag = nullptr;  // [slots, 2I * H / 16]
    const uint8_t* dn_scale_frag = nullptr;  // [slots, H * I / 16]
    int hidden, inter, slots;
};

}  // namespace ftm
