// Shared device helpers for the sm_100a decode kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace q3t {

constexpr int kWarp = 32;
constexpr float kRmsEps = 1.0e-6f;
constexpr float kRopeTheta = 1.0e6f;
constexpr int kPageTokens = 16;          // tokens per KV page
constexpr int kMaxRows = 64;             // lockstep batch capacity
constexpr int kMaxVocab = 3072;
constexpr int kPredictorVocab = 2048;
constexpr int kCodebooks = 16;

using bf16 = __nv_bfloat16;

__device__ __forceinline__ float bf2f(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ bf16 f2bf(float v) { return __float2bfloat16(v); }
__device__ __forceinline__ float rbf(float v) { return __bfloat162float(__float2bfloat16(v)); }

// low / high bf16 of a packed 32-bit word, widened to fp32 (exact)
__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

__device__ __forceinline__ float warp_sum_down(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max_xor(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ float warp_sum_xor(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// 128-bit streaming load that does not allocate in L1 (weights are read once).
__device__ __forceinline__ int4 ld_stream(const void* p) {
    int4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// Sum of 256 per-thread partials in the pairing order of a halving shared-memory tree
// (slot t += slot t+128, then +64, ... +1).  `partial` holds the 256 values in shared
// memory and must be visible (barrier before the call).  Every warp may call it; the
// result is valid in lane 0 and broadcast to all lanes.
__device__ __forceinline__ float tree_sum_256(const float* partial, int lane) {
    const float a = (partial[lane] + partial[lane + 128]) + (partial[lane + 64] + partial[lane + 192]);
    const float b = (partial[lane + 32] + partial[lane + 160]) + (partial[lane + 96] + partial[lane + 224]);
    float c = a + b;
    c = warp_sum_down(c);
    return __shfl_sync(0xffffffffu, c, 0);
}

// rotate-half RoPE of one (first, second) pair with the bf16 rounding chain:
// cos/sin rounded to bf16, each product rounded, sum and difference rounded.
__device__ __forceinline__ void rope_pair(float first, float second, float angle,
                                          float& out_first, float& out_second) {
    const float c = rbf(cosf(angle));
    const float s = rbf(sinf(angle));
    const float fc = rbf(first * c);
    const float ss = rbf(second * s);
    const float sc = rbf(second * c);
    const float fs = rbf(first * s);
    out_first = rbf(fc - ss);
    out_second = rbf(sc + fs);
}

// the same with cos and sin given (already rounded to bf16)
__device__ __forceinline__ void rope_pair_cs(float first, float second, float c, float s,
                                             float& out_first, float& out_second) {
    const float fc = rbf(first * c);
    const float ss = rbf(second * s);
    const float sc = rbf(second * c);
    const float fs = rbf(first * s);
    out_first = rbf(fc - ss);
    out_second = rbf(sc + fs);
}

__device__ __forceinline__ float rope_inv_freq(int d, int head_dim, float theta) {
    const float exponent = static_cast<float>(2 * d) / static_cast<float>(head_dim);
    return powf(theta, -exponent);
}

}  // namespace q3t
