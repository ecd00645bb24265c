// Split-KV GQA decode attention over a bf16 KV cache, with the per-head RMSNorm, RoPE and
// KV append of the new token folded in.
//
// Semantics follow the reference's batch_causal_gqa_attention_fast_kernel
// (native/qwen3-tts-native/native/src/talker_kernels.cu:506-595): fp32 scores
// dot*rsqrtf(head_dim), expf, fp32 PV, out = bf16(acc * (1/sum)).  In fused mode the
// launch also does what the reference issues as six separate kernels before it: per-head
// RMSNorm of q and k (talker_kernels.cu:50-70), RoPE of q and k (:597-639) and the append
// of k/v at the row's position (:641-658).
//
// Grid (split, kv_head, row), 128 threads.  One CTA serves all query heads of its KV head
// (K/V are read once per group, not once per query head) for a chunk of kAttnChunk tokens;
// each warp owns 16 consecutive tokens = one KV page.  A token's head vector (head_dim
// bf16) is spread over head_dim/8 lanes as 16-byte loads.  Chunk results (max, sum,
// weighted V) go to scratch; the CTA that takes the last ticket of its (row, kv_head)
// merges the chunks in split order, so the result does not depend on scheduling.  The
// split count depends only on the row's own length, never on the batch around it.

#include "q3t_kernels.cuh"

namespace q3t {
namespace {

constexpr int kAttnThreads = 128;
constexpr int kAttnWarps = kAttnThreads / kWarp;
constexpr int kWarpTokens = kAttnChunk / kAttnWarps;   // 16 = one page
static_assert(kWarpTokens == kPageTokens, "a warp must cover exactly one KV page");

template <int HD, int G, bool PAGED>
__global__ void __launch_bounds__(kAttnThreads) decode_attention_kernel(const AttentionArgs a) {
    constexpr int LPT = HD / 8;            // lanes per token
    constexpr int TPI = kWarp / LPT;       // tokens per warp iteration
    constexpr int ITERS = kWarpTokens / TPI;

    const int kvh = blockIdx.y;
    const int row = blockIdx.z;
    const int pos = a.positions[row];
    const int len = pos + 1;
    const int nsplits = (len + kAttnChunk - 1) / kAttnChunk;
    // A CTA walks `units` consecutive 64-token splits.  Each split still produces its own
    // (max, sum, weighted V) partial, so the result does not depend on how many a CTA takes.
    const int units = a.units_per_cta > 0 ? a.units_per_cta : 1;
    const int split_first = blockIdx.x * units;
    if (split_first >= nsplits) return;
    const int split_end = min(nsplits, split_first + units);

    __shared__ float qs[G][HD];
    __shared__ float wm[kAttnWarps][G];
    __shared__ float wl[kAttnWarps][G];
    __shared__ __align__(16) float wacc[kAttnWarps][G][HD];
    __shared__ int is_last;

    const int tid = threadIdx.x;
    const int lane = tid % kWarp;
    const int warp = tid / kWarp;
    const int kvw = a.kv_heads * HD;
    const int qw = a.q_heads * HD;
    const int q_stride = a.q_stride > 0 ? a.q_stride : qw;
    const int kn_stride = a.kv_new_stride > 0 ? a.kv_new_stride : kvw;

    // ---- K/V row addressing ---------------------------------------------------------
    auto kv_row = [&](int token, bool value) -> bf16* {
        if (PAGED) {
            const int pid = a.kv.page_table[(size_t)row * a.kv.table_stride + token / kPageTokens];
            bf16* slab = a.kv.slabs[pid >> a.kv.slab_shift];
            const long long in_slab = (long long)(pid & ((1 << a.kv.slab_shift) - 1)) * a.kv.page_elems;
            return slab + in_slab + (value ? a.kv.v_offset : a.kv.k_offset)
                   + (size_t)(token % kPageTokens) * kvw + (size_t)kvh * HD;
        }
        bf16* base = value ? a.kv.v_bases[row] : a.kv.k_bases[row];
        return base + (size_t)token * kvw + (size_t)kvh * HD;
    };

    // ---- query heads (and, in fused mode, the new K/V row) ----------------------------
    if (a.fused) {
        if constexpr (HD >= 64) {
            constexpr int DPL = HD / 32;   // dims per lane: l, l+32, ...
            // warps 0..G-1: query heads; warp G%4: the new key (last split only)
            for (int job = warp; job <= G; job += kAttnWarps) {
                const bool is_key = job == G;
                if (is_key && split_end != nsplits) continue;
                const bf16* src = is_key ? a.k_new + (size_t)row * kn_stride + (size_t)kvh * HD
                                         : a.q + (size_t)row * q_stride + (size_t)(kvh * G + job) * HD;
                const bf16* nw = is_key ? a.k_norm_w : a.q_norm_w;
                float x[DPL];
                float sq[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int j = 0; j < DPL; ++j) {
                    x[j] = bf2f(src[lane + 32 * j]);
                    sq[j] = fmaf(x[j], x[j], 0.0f);
                }
                // pairing of the 256-slot halving tree with slots >= HD equal to zero
                float c = (sq[0] + sq[2]) + (sq[1] + sq[3]);
                c = warp_sum_down(c);
                c = __shfl_sync(0xffffffffu, c, 0);
                const float inv = rsqrtf(c / static_cast<float>(HD) + a.eps);
                float y[DPL];
#pragma unroll
                for (int j = 0; j < DPL; ++j) {
                    const float normalized = rbf(x[j] * inv);
                    y[j] = rbf(normalized * bf2f(nw[lane + 32 * j]));
                }
                // rotate-half pairs (d, d + HD/2): with dims l+32j per lane both members of a
                // pair sit in the same lane (j and j + DPL/2)
#pragma unroll
                for (int j = 0; j < DPL / 2; ++j) {
                    const int d = lane + 32 * j;
                    const float angle = static_cast<float>(pos) * rope_inv_freq(d, HD, a.theta);
                    float o1, o2;
                    rope_pair(y[j], y[j + DPL / 2], angle, o1, o2);
                    y[j] = o1;
                    y[j + DPL / 2] = o2;
                }
                if (is_key) {
                    bf16* kdst = kv_row(pos, false);
                    bf16* vdst = kv_row(pos, true);
                    const bf16* vsrc = a.v_new + (size_t)row * kn_stride + (size_t)kvh * HD;
#pragma unroll
                    for (int j = 0; j < DPL; ++j) {
                        kdst[lane + 32 * j] = f2bf(y[j]);
                        vdst[lane + 32 * j] = vsrc[lane + 32 * j];
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < DPL; ++j) qs[job][lane + 32 * j] = y[j];
                }
            }
        }
    } else {
        for (int i = tid; i < G * HD; i += kAttnThreads) {
            const int g = i / HD;
            const int d = i % HD;
            qs[g][d] = bf2f(a.q[(size_t)row * q_stride + (size_t)(kvh * G + g) * HD + d]);
        }
    }
    __syncthreads();   // qs ready; this CTA's K/V append is visible to its own loads

    const int sub = lane / LPT;
    const int j8 = (lane % LPT) * 8;
    const float scale = rsqrtf(static_cast<float>(HD));
    const size_t part_stride = HD + 2;
    float qreg[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int e = 0; e < 8; ++e) qreg[g][e] = qs[g][j8 + e];

    for (int split = split_first; split < split_end; ++split) {
    // ---- this warp's 16 tokens --------------------------------------------------------
    const int c1 = min(len, (split + 1) * kAttnChunk);
    const int w0 = split * kAttnChunk + warp * kWarpTokens;

    float m_w[G], l_w[G], acc[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m_w[g] = -INFINITY;
        l_w[g] = 0.0f;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[g][e] = 0.0f;
    }

    if (w0 < c1) {
        const bf16* kpage = kv_row(w0, false);   // the 16 tokens of a warp share one page
        const bf16* vpage = kv_row(w0, true);
        // keys and values of the page are requested together: one memory latency per page
        int4 raw[ITERS], rawv[ITERS];
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {
            const int t = it * TPI + sub;
            if (w0 + t < c1) raw[it] = *reinterpret_cast<const int4*>(kpage + (size_t)t * kvw + j8);
        }
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {
            const int t = it * TPI + sub;
            if (w0 + t < c1) rawv[it] = *reinterpret_cast<const int4*>(vpage + (size_t)t * kvw + j8);
        }

        float s[G][ITERS];
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {
            const bool valid = w0 + it * TPI + sub < c1;
            const uint32_t kw[4] = {(uint32_t)raw[it].x, (uint32_t)raw[it].y,
                                    (uint32_t)raw[it].z, (uint32_t)raw[it].w};
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float dot = 0.0f;
                if (valid) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        dot = fmaf(qreg[g][2 * e], bf_lo(kw[e]), dot);
                        dot = fmaf(qreg[g][2 * e + 1], bf_hi(kw[e]), dot);
                    }
                }
#pragma unroll
                for (int o = LPT / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
                s[g][it] = valid ? dot * scale : -INFINITY;
                m_w[g] = fmaxf(m_w[g], s[g][it]);
            }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
#pragma unroll
            for (int o = LPT; o < kWarp; o <<= 1)
                m_w[g] = fmaxf(m_w[g], __shfl_xor_sync(0xffffffffu, m_w[g], o));
        }
        // values
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {
            const bool valid = w0 + it * TPI + sub < c1;
            const uint32_t vw[4] = {(uint32_t)rawv[it].x, (uint32_t)rawv[it].y,
                                    (uint32_t)rawv[it].z, (uint32_t)rawv[it].w};
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float p = valid ? expf(s[g][it] - m_w[g]) : 0.0f;
                l_w[g] += p;
                if (valid) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        acc[g][2 * e] = fmaf(p, bf_lo(vw[e]), acc[g][2 * e]);
                        acc[g][2 * e + 1] = fmaf(p, bf_hi(vw[e]), acc[g][2 * e + 1]);
                    }
                }
            }
        }
        // fold the token sub-groups of the warp (lanes that hold the same dims)
#pragma unroll
        for (int g = 0; g < G; ++g) {
#pragma unroll
            for (int o = LPT; o < kWarp; o <<= 1) {
                l_w[g] += __shfl_xor_sync(0xffffffffu, l_w[g], o);
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[g][e] += __shfl_xor_sync(0xffffffffu, acc[g][e], o);
            }
        }
    }
    if (lane == 0) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
            wm[warp][g] = m_w[g];
            wl[warp][g] = l_w[g];
        }
    }
    if (sub == 0) {
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int e = 0; e < 8; ++e) wacc[warp][g][j8 + e] = acc[g][e];
    }
    __syncthreads();

    // ---- merge the four warps ------------------------------------------------------------
    for (int i = tid; i < G * HD; i += kAttnThreads) {
        const int g = i / HD;
        const int d = i % HD;
        float M = wm[0][g];
#pragma unroll
        for (int w = 1; w < kAttnWarps; ++w) M = fmaxf(M, wm[w][g]);
        float L = 0.0f, A = 0.0f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) {
            if (wl[w][g] > 0.0f) {
                const float f = expf(wm[w][g] - M);
                L = fmaf(wl[w][g], f, L);
                A = fmaf(wacc[w][g][d], f, A);
            }
        }
        const int head = kvh * G + g;
        if (nsplits == 1) {
            const float val = A * (1.0f / L);
            const size_t o = (size_t)row * qw + (size_t)head * HD + d;
            if (a.out32 != nullptr) a.out32[o] = val;
            a.out[o] = f2bf(val);
        } else {
            float* part = a.scratch
                + (((size_t)row * a.q_heads + head) * a.max_splits + split) * part_stride;
            if (d == 0) {
                part[0] = M;
                part[1] = L;
            }
            part[2 + d] = A;
        }
    }
    __syncthreads();   // the warp partials are reused by the next split
    }   // splits of this CTA
    if (nsplits == 1) return;

    // ---- last CTA of this (row, kv head) merges the splits in order -------------------------
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned int ticket = atomicAdd(&a.counters[row * a.kv_heads + kvh], 1u);
        is_last = ticket == static_cast<unsigned int>((nsplits + units - 1) / units - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (int i = tid; i < G * HD; i += kAttnThreads) {
        const int g = i / HD;
        const int d = i % HD;
        const int head = kvh * G + g;
        const float* base = a.scratch + ((size_t)row * a.q_heads + head) * a.max_splits * part_stride;
        float M = -INFINITY;
        for (int sp = 0; sp < nsplits; ++sp) M = fmaxf(M, __ldcg(base + sp * part_stride));
        float L = 0.0f, A = 0.0f;
        for (int sp = 0; sp < nsplits; ++sp) {
            const float f = expf(__ldcg(base + sp * part_stride) - M);
            L = fmaf(__ldcg(base + sp * part_stride + 1), f, L);
            A = fmaf(__ldcg(base + sp * part_stride + 2 + d), f, A);
        }
        const float val = A * (1.0f / L);
        const size_t o = (size_t)row * qw + (size_t)head * HD + d;
        if (a.out32 != nullptr) a.out32[o] = val;
        a.out[o] = f2bf(val);
    }
    if (tid == 0) a.counters[row * a.kv_heads + kvh] = 0u;   // ready for the next launch
}

template <int HD, int G>
cudaError_t launch_hd_g(const AttentionArgs& a, cudaStream_t stream) {
    const int units = a.units_per_cta > 0 ? a.units_per_cta : 1;
    const dim3 grid((a.max_splits + units - 1) / units, a.kv_heads, a.rows);
    if (a.kv.page_table != nullptr) {
        decode_attention_kernel<HD, G, true><<<grid, kAttnThreads, 0, stream>>>(a);
    } else {
        decode_attention_kernel<HD, G, false><<<grid, kAttnThreads, 0, stream>>>(a);
    }
    return cudaGetLastError();
}

template <int HD>
cudaError_t launch_hd(const AttentionArgs& a, cudaStream_t stream) {
    switch (a.q_heads / a.kv_heads) {
        case 1: return launch_hd_g<HD, 1>(a, stream);
        case 2: return launch_hd_g<HD, 2>(a, stream);
        case 4: return launch_hd_g<HD, 4>(a, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace

size_t attention_scratch_floats(int rows, int q_heads, int head_dim, int max_splits) {
    return (size_t)rows * q_heads * max_splits * (head_dim + 2);
}

cudaError_t launch_decode_attention(const AttentionArgs& a, cudaStream_t stream) {
    if (a.rows < 1 || a.q_heads < 1 || a.kv_heads < 1 || a.q_heads % a.kv_heads != 0
        || a.max_splits < 1 || a.q == nullptr || a.out == nullptr || a.positions == nullptr) {
        return cudaErrorInvalidValue;
    }
    if (a.kv.page_table == nullptr && (a.kv.k_bases == nullptr || a.kv.v_bases == nullptr)) {
        return cudaErrorInvalidValue;
    }
    if (a.kv.page_table != nullptr && a.kv.slabs == nullptr) return cudaErrorInvalidValue;
    if (a.max_splits > 1 && (a.scratch == nullptr || a.counters == nullptr)) {
        return cudaErrorInvalidValue;
    }
    if (a.fused && (a.k_new == nullptr || a.v_new == nullptr || a.q_norm_w == nullptr
                    || a.k_norm_w == nullptr || a.head_dim < 64)) {
        return cudaErrorInvalidValue;
    }
    AttentionArgs b = a;
    if (b.units_per_cta <= 0) {
        // many small CTAs pay the query prologue and the launch machinery once per 64 tokens:
        // with thousands of them, let each walk a few splits
        const long long ctas = (long long)a.rows * a.kv_heads * a.max_splits;
        b.units_per_cta = ctas >= 8192 ? 4 : (ctas >= 2048 ? 2 : 1);
    }
    switch (b.head_dim) {
        case 32: return launch_hd<32>(b, stream);
        case 64: return launch_hd<64>(b, stream);
        case 128: return launch_hd<128>(b, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace q3t
