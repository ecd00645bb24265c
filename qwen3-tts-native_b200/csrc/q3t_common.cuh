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

// ---- programmatic dependent launch --------------------------------------------------------
// A kernel launched with programmatic stream serialisation may start while its predecessor in
// the stream still runs.  pdl_wait() returns once the predecessor has completed and its writes
// are visible (at once when the launch was an ordinary one); nothing the predecessor wrote may
// be read before it.  pdl_trigger() lets the successor start its own preamble.
// Library-wide rule: a kernel calls pdl_trigger() only after its own pdl_wait() has returned (in
// the calling thread).  When a grid starts, every grid two or more launches upstream of it has
// therefore completed, and what those wrote may be read ahead of the wait; only the immediate
// predecessor's output has to wait.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- packed fp32 pairs (one instruction, two ordinary IEEE operations) -----------------------
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b,
                                                   unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

// Two weight vectors (16 int8 each) of one lane against their activations: returns the two vector
// sums, each the 16 sequential FMAs of the reference's dot product.
// xs4 points at this lane's first 16-byte group; groups of one pair are 32 * 16 bytes apart and
// hold {xA[i], xB[i], xA[i+1], xB[i+1]}.
__device__ __forceinline__ void dot16_pair(const int4& wa, const int4& wb, const float4* xs4, float& sum_a,
                                           float& sum_b) {
    const unsigned long long bias = pack2(-8388736.0f, -8388736.0f);
    unsigned long long sum = pack2(0.0f, 0.0f);
    const uint32_t a[4] = {(uint32_t)wa.x ^ 0x80808080u, (uint32_t)wa.y ^ 0x80808080u,
                           (uint32_t)wa.z ^ 0x80808080u, (uint32_t)wa.w ^ 0x80808080u};
    const uint32_t b[4] = {(uint32_t)wb.x ^ 0x80808080u, (uint32_t)wb.y ^ 0x80808080u,
                           (uint32_t)wb.z ^ 0x80808080u, (uint32_t)wb.w ^ 0x80808080u};
#pragma unroll
    for (int ip = 0; ip < 8; ++ip) {
        const float4 xx = xs4[ip * kWarp];
        const int q = ip >> 1;                 // word of the vector
        const int e0 = (ip & 1) * 2;           // byte of the word
        const unsigned long long w0 = add2(
            pack2(__uint_as_float(__byte_perm(a[q], 0x4B000000u, 0x7650 + e0)),
                  __uint_as_float(__byte_perm(b[q], 0x4B000000u, 0x7650 + e0))), bias);
        const unsigned long long w1 = add2(
            pack2(__uint_as_float(__byte_perm(a[q], 0x4B000000u, 0x7651 + e0)),
                  __uint_as_float(__byte_perm(b[q], 0x4B000000u, 0x7651 + e0))), bias);
        sum = fma2(w0, pack2(xx.x, xx.y), sum);
        sum = fma2(w1, pack2(xx.z, xx.w), sum);
    }
    unpack2(sum, sum_a, sum_b);
}


// Where element e of an activation row goes in the staged fp32 layout that dot16_pair reads:
// vector v = e / 16 belongs to lane v % 32, the lane's vectors j = v / 32 are paired (j, j + 1).
__device__ __forceinline__ int paired_index(int e) {
    const int vec = e >> 4, i = e & 15;
    const int l = vec & 31, j = vec >> 5;
    return ((((j >> 1) * 8 + (i >> 1)) * kWarp + l) << 2) + ((i & 1) << 1) + (j & 1);
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
