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

#include <cstdlib>

namespace q3t {
namespace {

// Rows whose position lay outside [0, max_splits * kAttnChunk): the kernel clamps the length to what
// its scratch and grid were sized for, computes over that and counts the row here (and in the
// engine's host-mapped error word, if one is registered), so that the host can refuse the result.
__device__ unsigned int g_attention_range_errors = 0;
__device__ unsigned int* g_attention_error_sink = nullptr;

// chunks one CTA may walk (its shared-memory buffers are sized for it; 32 KB of partials at most)
__host__ __device__ constexpr int max_units_for(int) { return 4; }
constexpr int kAttnThreads = 128;
constexpr int kAttnWarps = kAttnThreads / kWarp;
constexpr int kWarpTokens = kAttnChunk / kAttnWarps;   // 16 = one page
static_assert(kWarpTokens == kPageTokens, "a warp must cover exactly one KV page");

// D += A (16 x 16, bf16, row-major) * B (16 x 8, bf16, column-major), fp32 accumulate.  Lane l
// holds, with g = l / 4 and t = l % 4:  a0 = A[g][2t, 2t+1], a1 = A[g+8][2t, 2t+1],
// a2 = A[g][2t+8, 2t+9], a3 = A[g+8][2t+8, 2t+9];  b0 = B[2t, 2t+1][g], b1 = B[2t+8, 2t+9][g];
// d0, d1 = D[g][2t, 2t+1], d2, d3 = D[g+8][2t, 2t+1].
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// (lo, hi) -> bf16x2 with lo in the low half
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// EARLY: the launcher has checked AttentionArgs::inputs_settled (plain decode step, head_dim 128,
// a grid that is resident at once); a separate instantiation, because holding the prefetched
// fragments across the query prologue costs registers.
template <int HD, int G, bool PAGED, bool EARLY>
__global__ void __launch_bounds__(kAttnThreads, EARLY ? 4 : 6) decode_attention_kernel(const AttentionArgs a) {
    constexpr int LPT = HD / 8;            // lanes per token
    constexpr int TPI = kWarp / LPT;       // tokens per warp iteration
    constexpr int ITERS = kWarpTokens / TPI;

    const int kvh = blockIdx.y;
    const int row = blockIdx.z;
    const int tid = threadIdx.x;
    const int lane = tid % kWarp;
    const int warp = tid / kWarp;
    const int kvw = a.kv_heads * HD;
    // elements between consecutive tokens of one KV head: pages are head-major ([kv head][16][HD], a
    // head's 16 tokens are one contiguous block), contiguous caches token-major
    const int tstride = PAGED ? HD : kvw;
    const int qw = a.q_heads * HD;
    const int q_stride = a.q_stride > 0 ? a.q_stride : qw;
    const int kn_stride = a.kv_new_stride > 0 ? a.kv_new_stride : kvw;
    const int units = a.units_per_cta > 0 ? a.units_per_cta : 1;
    const int split_first = blockIdx.x * units;
    const int gid = lane >> 2;
    const int tig = lane & 3;

    // ---- K/V row addressing ---------------------------------------------------------
    auto kv_row = [&](int token, bool value) -> bf16* {
        if (PAGED) {
            const int pid = a.kv.page_table[(size_t)row * a.kv.table_stride + token / kPageTokens];
            bf16* slab = a.kv.slabs[pid >> a.kv.slab_shift];
            const long long in_slab = (long long)(pid & ((1 << a.kv.slab_shift) - 1)) * a.kv.page_elems;
            return slab + in_slab + (value ? a.kv.v_offset : a.kv.k_offset)
                   + (size_t)kvh * (kPageTokens * HD) + (size_t)(token % kPageTokens) * HD;
        }
        bf16* base = value ? a.kv.v_bases[row] : a.kv.k_bases[row];
        return base + (size_t)token * kvw + (size_t)kvh * HD;
    };
    // head_dim 128: the K and V fragments of one warp's 16 tokens (the main loop explains the
    // layout); tokens at or past `bound` read as zero
    int4 kr[2][4];
    int4 vr[2][2][2];
    auto load_kv = [&](int w0, int bound) {
        const bf16* kpage = kv_row(w0, false);   // the 16 tokens of a warp share one page
        const bf16* vpage = kv_row(w0, true);
        const int4 zero4 = make_int4(0, 0, 0, 0);
        // K: token 8 nt + gid, dims 32 jj + 8 tig .. + 7
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const int t = 8 * nt + gid;
            const bool valid = w0 + t < bound;
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                kr[nt][jj] = valid ? *reinterpret_cast<const int4*>(kpage + (size_t)t * tstride + 32 * jj + 8 * tig)
                                   : zero4;
            }
        }
        // V: tokens 8 h + 2 tig + p, dims 64 jb + 8 gid .. + 7.  Tokens past the end read as
        // zero: their probability is zero, but 0 * (stale bits that decode as NaN) is not.
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int pp = 0; pp < 2; ++pp) {
                const int t = 8 * h + 2 * tig + pp;
                const bool valid = w0 + t < bound;
#pragma unroll
                for (int jb = 0; jb < 2; ++jb) {
                    vr[h][pp][jb] = valid ? *reinterpret_cast<const int4*>(vpage + (size_t)t * tstride + 64 * jb + 8 * gid)
                                          : zero4;
                }
            }
    };

    // ---- ahead of the dependency wait ---------------------------------------------------
    // Constants (the per-head norm weights) always; with inputs_settled also the position, its
    // cos/sin and the first split's K/V rows older than this step's token: what remains after the
    // wait is one round trip for q / k_new / v_new.
    constexpr int DPLN = HD >= 64 ? HD / 32 : 2;
    bf16 nwq[DPLN], nwk[DPLN];
    if (a.fused && HD >= 64) {
#pragma unroll
        for (int j = 0; j < DPLN; ++j) {
            nwq[j] = a.q_norm_w[lane + 32 * j];
            nwk[j] = a.k_norm_w[lane + 32 * j];
        }
    }
    constexpr bool early = EARLY && HD == 128;
    int pos = 0;
    uint32_t cs_pre[DPLN / 2];
    bool cs_ready = false;
    if (early) {
        pos = a.positions[row];
        if (a.rope_table != nullptr && pos < a.rope_positions) {
            cs_ready = true;
#pragma unroll
            for (int j = 0; j < DPLN / 2; ++j) cs_pre[j] = a.rope_table[(size_t)pos * (HD / 2) + lane + 32 * j];
        }
        const int w0e = split_first * kAttnChunk + warp * kWarpTokens;
        if (w0e < pos) {
            load_kv(w0e, pos);
        } else {
            const int4 zero4 = make_int4(0, 0, 0, 0);
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    kr[i][j] = zero4;
                    vr[i][j >> 1][j & 1] = zero4;
                }
        }
    }

    pdl_wait();        // q / k_new / v_new (and, unless settled, everything else) come from the kernel before
    pdl_trigger();
    if (!early) pos = a.positions[row];
    {
        // the position comes from device memory the caller filled; the grid, the scratch partials and
        // the ticket count were sized for max_splits chunks
        const int limit = a.max_splits * kAttnChunk - 1;
        if (pos < 0 || pos > limit) {
            if (tid == 0 && blockIdx.x == 0 && blockIdx.y == 0) {
                atomicAdd(&g_attention_range_errors, 1u);
                if (g_attention_error_sink != nullptr) atomicAdd_system(g_attention_error_sink, 1u);
            }
            pos = pos < 0 ? 0 : limit;
        }
    }
    const int len = pos + 1;
    const int nsplits = (len + kAttnChunk - 1) / kAttnChunk;
    // A CTA walks `units` consecutive 64-token splits.  Each split still produces its own
    // (max, sum, weighted V) partial, so the result does not depend on how many a CTA takes.
    if (split_first >= nsplits) return;
    const int split_end = min(nsplits, split_first + units);

    __shared__ float qs[G][HD];
    // per 64-token chunk of this CTA's range and per warp: (max, sum, weighted V) of the warp's page.
    // The warps walk the chunks without meeting; the chunks are merged after the last one.
    constexpr int kMaxUnits = max_units_for(G);
    __shared__ float wm[kMaxUnits][kAttnWarps][G];
    __shared__ float wl[kMaxUnits][kAttnWarps][G];
    __shared__ __align__(16) float wacc[kMaxUnits][kAttnWarps][G][HD];
    __shared__ int is_last;
    // this step's own K/V row, kept for the warp that attends to it (EARLY: saves re-reading
    // from global memory what this CTA has just written there)
    __shared__ __align__(16) bf16 knew[EARLY ? HD : 8];
    __shared__ __align__(16) bf16 vnew[EARLY ? HD : 8];

    // ---- query heads (and, in fused mode, the new K/V row) ----------------------------
    if (a.fused) {
        if constexpr (HD >= 64) {
            constexpr int DPL = HD / 32;   // dims per lane: l, l+32, ...
            // warps 0..G-1: query heads; warp G%4: the new key (last split only)
            for (int job = warp; job <= G; job += kAttnWarps) {
                const bool is_key = job == G;
                if (is_key && (split_end != nsplits || a.append_mode == 2)) continue;
                if (!is_key && a.append_mode == 1) continue;
                const bf16* src = is_key ? a.k_new + (size_t)row * kn_stride + (size_t)kvh * HD
                                         : a.q + (size_t)row * q_stride + (size_t)(kvh * G + job) * HD;
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
                    y[j] = rbf(normalized * bf2f(is_key ? nwk[j] : nwq[j]));
                }
                // rotate-half pairs (d, d + HD/2): with dims l+32j per lane both members of a
                // pair sit in the same lane (j and j + DPL/2)
#pragma unroll
                for (int j = 0; j < DPL / 2; ++j) {
                    const int d = lane + 32 * j;
                    float o1, o2;
                    if (a.rope_table != nullptr && pos < a.rope_positions) {
                        // cos | sin of this (position, pair) as two bf16, made by the same code below
                        const uint32_t cs = cs_ready ? cs_pre[j] : a.rope_table[(size_t)pos * (HD / 2) + d];
                        rope_pair_cs(y[j], y[j + DPL / 2], bf_lo(cs), bf_hi(cs), o1, o2);
                    } else {
                        const float angle = static_cast<float>(pos) * rope_inv_freq(d, HD, a.theta);
                        rope_pair(y[j], y[j + DPL / 2], angle, o1, o2);
                    }
                    y[j] = o1;
                    y[j + DPL / 2] = o2;
                }
                if (is_key) {
                    bf16* kdst = kv_row(pos, false);
                    bf16* vdst = kv_row(pos, true);
                    const bf16* vsrc = a.v_new + (size_t)row * kn_stride + (size_t)kvh * HD;
#pragma unroll
                    for (int j = 0; j < DPL; ++j) {
                        const bf16 kb = f2bf(y[j]);
                        const bf16 vb = vsrc[lane + 32 * j];
                        kdst[lane + 32 * j] = kb;
                        vdst[lane + 32 * j] = vb;
                        if constexpr (EARLY) {
                            knew[lane + 32 * j] = kb;
                            vnew[lane + 32 * j] = vb;
                        }
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
    if (a.fused && a.append_mode == 1) return;

    const int sub = lane / LPT;
    const int j8 = (lane % LPT) * 8;
    const float scale = rsqrtf(static_cast<float>(HD));
    const size_t part_stride = HD + 2;
    float qreg[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int e = 0; e < 8; ++e) qreg[g][e] = qs[g][j8 + e];

    // head_dim 128 runs on the tensor cores (mma.sync, 16 x 8 x 16): the G query heads are rows
    // 0..G-1 of the 16-row A operand, the other rows are zero.  A contraction may visit its
    // index in any order as long as both operands agree, so a lane loads 16 contiguous bytes of
    // K (8 dims of one token) and feeds them to two MMAs as they come; qa[] holds the query in
    // the matching order: MMA (jj, m) of lane (gid, tig) covers dims 32 jj + 8 tig + 4 m + 0..3.
    uint32_t qa[4][2][2];
    if constexpr (HD == 128) {
#pragma unroll
        for (int jj = 0; jj < 4; ++jj)
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                const int d = 32 * jj + 8 * tig + 4 * m;
                const bool real = gid < G;          // q is already bf16-valued: the pack is exact
                qa[jj][m][0] = real ? pack_bf16x2(qs[gid % G][d], qs[gid % G][d + 1]) : 0u;
                qa[jj][m][1] = real ? pack_bf16x2(qs[gid % G][d + 2], qs[gid % G][d + 3]) : 0u;
            }
    }

    for (int split = split_first; split < split_end; ++split) {
    const int unit = split - split_first;
    // ---- this warp's 16 tokens --------------------------------------------------------
    const int c1 = min(len, (split + 1) * kAttnChunk);
    const int w0 = split * kAttnChunk + warp * kWarpTokens;

    if constexpr (HD == 128) {
        float mx = -INFINITY, lsum = 0.0f;
        // out^T tile x: rows = dims (8 gid + x and 64 + 8 gid + x), columns = query heads
        float o[8][4];
#pragma unroll
        for (int x = 0; x < 8; ++x)
#pragma unroll
            for (int e = 0; e < 4; ++e) o[x][e] = 0.0f;
        if (w0 < c1) {
            if (early && split == split_first) {
                // fetched ahead of the wait, except this step's own token (appended above by the
                // CTA of the last split, visible since the barrier)
                const int t_new = pos - w0;
                if (t_new >= 0 && t_new < kWarpTokens) {
                    const bf16* krow = knew;     // written by the key warp before the barrier
                    const bf16* vrow = vnew;
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt)
                        if (8 * nt + gid == t_new) {
#pragma unroll
                            for (int jj = 0; jj < 4; ++jj)
                                kr[nt][jj] = *reinterpret_cast<const int4*>(krow + 32 * jj + 8 * tig);
                        }
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int pp = 0; pp < 2; ++pp)
                            if (8 * h + 2 * tig + pp == t_new) {
#pragma unroll
                                for (int jb = 0; jb < 2; ++jb)
                                    vr[h][pp][jb] = *reinterpret_cast<const int4*>(vrow + 64 * jb + 8 * gid);
                            }
                }
            } else {
                load_kv(w0, c1);
            }
            // scores: s[nt][0..1] = head gid, tokens 8 nt + 2 tig + {0, 1}
            float sc[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) sc[nt][e] = 0.0f;
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    mma_bf16_16816(sc[nt], qa[jj][0][0], 0u, qa[jj][0][1], 0u,
                                   (uint32_t)kr[nt][jj].x, (uint32_t)kr[nt][jj].y);
                    mma_bf16_16816(sc[nt], qa[jj][1][0], 0u, qa[jj][1][1], 0u,
                                   (uint32_t)kr[nt][jj].z, (uint32_t)kr[nt][jj].w);
                }
            }
            float pr[2][2];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const bool valid = w0 + 8 * nt + 2 * tig + e < c1;
                    pr[nt][e] = valid ? sc[nt][e] * scale : -INFINITY;
                    mx = fmaxf(mx, pr[nt][e]);
                }
            // the four lanes of a group hold the 16 tokens of one head
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    pr[nt][e] = pr[nt][e] == -INFINITY ? 0.0f : expf(pr[nt][e] - mx);
                    lsum += pr[nt][e];
                }
            lsum += __shfl_xor_sync(0xffffffffu, lsum, 1);
            lsum += __shfl_xor_sync(0xffffffffu, lsum, 2);
            // probabilities as the A operand of P V: the score fragment already has that layout.
            // bf16 holds 8 bits of a probability; hi + lo keeps 16, so the product stays within
            // 2^-16 of the fp32 one.
            uint32_t ph[2], pl[2];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                ph[nt] = pack_bf16x2(pr[nt][0], pr[nt][1]);
                const float r0 = pr[nt][0] - __uint_as_float(ph[nt] << 16);
                const float r1 = pr[nt][1] - __uint_as_float(ph[nt] & 0xffff0000u);
                pl[nt] = pack_bf16x2(r0, r1);
            }
            // out^T = V^T P^T: V^T is the 16 x 16 A operand (rows = dims, contraction = the warp's 16
            // tokens), P^T the 16 x 8 B operand, whose fragment is exactly what the score fragment holds
            // (lane (gid, tig): head gid, tokens 2 tig, 2 tig + 1 and 8 + 2 tig, 9 + 2 tig).  Row gid of
            // tile x is dim 8 gid + x, row gid + 8 is dim 64 + 8 gid + x, so that a lane builds its A
            // fragment (two tokens, one dim) from the 16 bytes it loaded per token: eight tiles cover
            // the 128 dims with half the MMAs and half the accumulators of the P V orientation.
            uint32_t tv[2][2][2][4];      // [token group][token of the pair][dim half][word]
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int pp = 0; pp < 2; ++pp)
#pragma unroll
                    for (int jb = 0; jb < 2; ++jb) {
                        tv[h][pp][jb][0] = (uint32_t)vr[h][pp][jb].x;
                        tv[h][pp][jb][1] = (uint32_t)vr[h][pp][jb].y;
                        tv[h][pp][jb][2] = (uint32_t)vr[h][pp][jb].z;
                        tv[h][pp][jb][3] = (uint32_t)vr[h][pp][jb].w;
                    }
#pragma unroll
            for (int x = 0; x < 8; ++x) {
                const uint32_t sel = (x & 1) ? 0x7632u : 0x5410u;
                const uint32_t a0 = __byte_perm(tv[0][0][0][x >> 1], tv[0][1][0][x >> 1], sel);
                const uint32_t a1 = __byte_perm(tv[0][0][1][x >> 1], tv[0][1][1][x >> 1], sel);
                const uint32_t a2 = __byte_perm(tv[1][0][0][x >> 1], tv[1][1][0][x >> 1], sel);
                const uint32_t a3 = __byte_perm(tv[1][0][1][x >> 1], tv[1][1][1][x >> 1], sel);
                mma_bf16_16816(o[x], a0, a1, a2, a3, ph[0], ph[1]);
                mma_bf16_16816(o[x], a0, a1, a2, a3, pl[0], pl[1]);
            }
        }
        if (len <= kWarpTokens) {
            // The whole row is this one page (the code predictor's caches): warp 0 holds everything,
            // the merges below would multiply by exp(0) = 1 and add zeros.  It writes the result from
            // its registers, the same value bit for bit, and nobody meets at a barrier again.
            if (warp == 0) {
                // 1 / sum of the heads in this lane's accumulator columns, from the lanes that hold them
                const float inv0 = 1.0f / __shfl_sync(0xffffffffu, lsum, (2 * tig) * 4 % kWarp);
                const float inv1 = 1.0f / __shfl_sync(0xffffffffu, lsum, (2 * tig + 1) * 4 % kWarp);
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int g = 2 * tig + c;
                    if (g < G) {
                        const float inv = c == 0 ? inv0 : inv1;
                        const size_t base = (size_t)row * qw + (size_t)(kvh * G + g) * HD;
#pragma unroll
                        for (int half = 0; half < 2; ++half) {     // dims 8 gid .. + 7 and 64 + 8 gid .. + 7
                            float v8[8];
#pragma unroll
                            for (int x = 0; x < 8; ++x) v8[x] = o[x][2 * half + c] * inv;
                            const size_t at = base + 64 * half + 8 * gid;
                            if (a.out32 != nullptr) {
#pragma unroll
                                for (int x = 0; x < 8; ++x) a.out32[at + x] = v8[x];
                            }
                            int4 packed;
                            packed.x = static_cast<int>(pack_bf16x2(v8[0], v8[1]));
                            packed.y = static_cast<int>(pack_bf16x2(v8[2], v8[3]));
                            packed.z = static_cast<int>(pack_bf16x2(v8[4], v8[5]));
                            packed.w = static_cast<int>(pack_bf16x2(v8[6], v8[7]));
                            *reinterpret_cast<int4*>(a.out + at) = packed;
                        }
                    }
                }
            }
            return;
        }
        if (gid < G && tig == 0) {
            wm[unit][warp][gid] = mx;
            wl[unit][warp][gid] = lsum;
        }
        // accumulator columns 2 tig and 2 tig + 1 are query heads; lanes past the group hold nothing
        if (2 * tig < G) {
#pragma unroll
            for (int x = 0; x < 8; ++x) {
                wacc[unit][warp][2 * tig][8 * gid + x] = o[x][0];
                wacc[unit][warp][2 * tig][64 + 8 * gid + x] = o[x][2];
            }
        }
        if (2 * tig + 1 < G) {
#pragma unroll
            for (int x = 0; x < 8; ++x) {
                wacc[unit][warp][(2 * tig + 1) % G][8 * gid + x] = o[x][1];
                wacc[unit][warp][(2 * tig + 1) % G][64 + 8 * gid + x] = o[x][3];
            }
        }
    } else {

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
            if (w0 + t < c1) raw[it] = *reinterpret_cast<const int4*>(kpage + (size_t)t * tstride + j8);
        }
#pragma unroll
        for (int it = 0; it < ITERS; ++it) {
            const int t = it * TPI + sub;
            if (w0 + t < c1) rawv[it] = *reinterpret_cast<const int4*>(vpage + (size_t)t * tstride + j8);
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
            wm[unit][warp][g] = m_w[g];
            wl[unit][warp][g] = l_w[g];
        }
    }
    if (sub == 0) {
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int e = 0; e < 8; ++e) wacc[unit][warp][g][j8 + e] = acc[g][e];
    }
    }   // head_dim other than 128
    }   // chunks of this CTA
    __syncthreads();

    // ---- merge the four warps, chunk by chunk ----------------------------------------------
    // The weight exp(max_w - max) of a warp's page is the same for every dimension: one thread per
    // (chunk, warp, head) evaluates it, everybody applies it.
    __shared__ float wf[kMaxUnits][kAttnWarps][G];
    __shared__ float wmax[kMaxUnits][G];
    {
        const int units_here = split_end - split_first;
        for (int i = tid; i < units_here * kAttnWarps * G; i += kAttnThreads) {
            const int g = i % G;
            const int w = (i / G) % kAttnWarps;
            const int unit = i / (G * kAttnWarps);
            float M = wm[unit][0][g];
#pragma unroll
            for (int ww = 1; ww < kAttnWarps; ++ww) M = fmaxf(M, wm[unit][ww][g]);
            wf[unit][w][g] = wl[unit][w][g] > 0.0f ? expf(wm[unit][w][g] - M) : 0.0f;
            if (w == 0) wmax[unit][g] = M;
        }
    }
    __syncthreads();
    for (int split = split_first; split < split_end; ++split) {
    const int unit = split - split_first;
    for (int i = tid; i < G * HD; i += kAttnThreads) {
        const int g = i / HD;
        const int d = i % HD;
        const float M = wmax[unit][g];
        float L = 0.0f, A = 0.0f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) {
            if (wl[unit][w][g] > 0.0f) {
                const float f = wf[unit][w][g];
                L = fmaf(wl[unit][w][g], f, L);
                A = fmaf(wacc[unit][w][g][d], f, A);
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
    }
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

int attention_sm_count() {
    static int cached[64] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 148;
    if (cached[device] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n < 1) n = 148;
        cached[device] = n;
    }
    return cached[device];
}

template <int HD, int G>
cudaError_t launch_hd_g(const AttentionArgs& a, cudaStream_t stream) {
    const int units = a.units_per_cta > 0 ? a.units_per_cta : 1;
    const dim3 grid((a.max_splits + units - 1) / units, a.kv_heads, a.rows);
    // fetching ahead of the dependency wait pays when every CTA is resident while the kernel before
    // this one still runs: one wave of 4 CTAs per SM
    const bool early = HD == 128 && a.inputs_settled != 0 && a.fused != 0 && a.append_mode == 0
                       && (size_t)grid.x * grid.y * grid.z <= (size_t)attention_sm_count() * 4;
    if (a.kv.page_table != nullptr) {
        if (early) return launch_pdl(decode_attention_kernel<HD, G, true, true>, grid, dim3(kAttnThreads), 0, stream, a);
        return launch_pdl(decode_attention_kernel<HD, G, true, false>, grid, dim3(kAttnThreads), 0, stream, a);
    }
    if (early) return launch_pdl(decode_attention_kernel<HD, G, false, true>, grid, dim3(kAttnThreads), 0, stream, a);
    return launch_pdl(decode_attention_kernel<HD, G, false, false>, grid, dim3(kAttnThreads), 0, stream, a);
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


// ---- the reference's order of summation ---------------------------------------------------
//
// Parity mode.  One CTA of 256 threads per (row, query head) that forms every fp32 sum in the
// order of the reference's batch_causal_gqa_attention_fast_kernel (talker_kernels.cu:506-595):
// a position's score is one thread's fmaf chain over the head's dimensions in ascending order;
// thread t exponentiates and adds up positions t, t + 256, ... and the 256 partial sums meet in a
// halving tree; a dimension's output is one thread's fmaf chain over the positions in ascending
// order, times the reciprocal of the sum.  The bf16 result is bit-identical to that kernel's, which
// the split-KV kernel above (tensor-core products, chunked sums) cannot promise.  In fused mode the
// query head gets its RMSNorm and rotation here, in the arithmetic of the kernel above; K and V of
// the new token are appended by that kernel beforehand (append_mode 1).  Slow by design: each
// thread walks whole rows of the cache.
constexpr int kOrderedThreads = 256;
constexpr int kOrderedMaxLength = 8192;     // scores of one head in shared memory

template <int HD>
__global__ void __launch_bounds__(kOrderedThreads) attention_reference_order_kernel(const AttentionArgs a) {
    __shared__ float scores[kOrderedMaxLength];
    __shared__ float reduction[kOrderedThreads];
    __shared__ float qs[HD];
    const int tid = threadIdx.x;
    const int lane = tid % kWarp;
    const int warp = tid / kWarp;
    const int row = blockIdx.x / a.q_heads;
    const int head = blockIdx.x % a.q_heads;
    const int kvh = head / (a.q_heads / a.kv_heads);
    const int kvw = a.kv_heads * HD;
    const int q_stride = a.q_stride > 0 ? a.q_stride : a.q_heads * HD;

    pdl_wait();
    pdl_trigger();
    int pos = a.positions[row];
    if (pos < 0 || pos >= kOrderedMaxLength) {
        if (tid == 0) {
            atomicAdd(&g_attention_range_errors, 1u);
            if (g_attention_error_sink != nullptr) atomicAdd_system(g_attention_error_sink, 1u);
        }
        pos = pos < 0 ? 0 : kOrderedMaxLength - 1;
    }
    const int len = pos + 1;

    auto kv_row = [&](int token, bool value) -> const bf16* {
        if (a.kv.page_table != nullptr) {
            const int pid = a.kv.page_table[(size_t)row * a.kv.table_stride + token / kPageTokens];
            const bf16* slab = a.kv.slabs[pid >> a.kv.slab_shift];
            const long long in_slab = (long long)(pid & ((1 << a.kv.slab_shift) - 1)) * a.kv.page_elems;
            return slab + in_slab + (value ? a.kv.v_offset : a.kv.k_offset)
                   + (size_t)kvh * (kPageTokens * HD) + (size_t)(token % kPageTokens) * HD;
        }
        const bf16* base = value ? a.kv.v_bases[row] : a.kv.k_bases[row];
        return base + (size_t)token * kvw + (size_t)kvh * HD;
    };

    // ---- the query head -------------------------------------------------------------------
    const bf16* qsrc = a.q + (size_t)row * q_stride + (size_t)head * HD;
    if (a.fused) {
        if (warp == 0) {
            constexpr int DPL = HD / 32;       // dims per lane: l, l + 32, ...
            float x[DPL];
            float sq[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int j = 0; j < DPL; ++j) {
                x[j] = bf2f(qsrc[lane + 32 * j]);
                sq[j] = fmaf(x[j], x[j], 0.0f);
            }
            float c = (sq[0] + sq[2]) + (sq[1] + sq[3]);      // the 256-slot halving tree, empty slots zero
            c = warp_sum_down(c);
            c = __shfl_sync(0xffffffffu, c, 0);
            const float inv = rsqrtf(c / static_cast<float>(HD) + a.eps);
            float y[DPL];
#pragma unroll
            for (int j = 0; j < DPL; ++j) y[j] = rbf(rbf(x[j] * inv) * bf2f(a.q_norm_w[lane + 32 * j]));
#pragma unroll
            for (int j = 0; j < DPL / 2; ++j) {
                const int d = lane + 32 * j;
                float o1, o2;
                if (a.rope_table != nullptr && pos < a.rope_positions) {
                    const uint32_t cs = a.rope_table[(size_t)pos * (HD / 2) + d];
                    rope_pair_cs(y[j], y[j + DPL / 2], bf_lo(cs), bf_hi(cs), o1, o2);
                } else {
                    rope_pair(y[j], y[j + DPL / 2], static_cast<float>(pos) * rope_inv_freq(d, HD, a.theta), o1, o2);
                }
                qs[d] = o1;
                qs[d + HD / 2] = o2;
            }
        }
    } else {
        for (int d = tid; d < HD; d += kOrderedThreads) qs[d] = bf2f(qsrc[d]);
    }
    __syncthreads();

    // ---- scores: one thread per position ----------------------------------------------------
    // The reference takes the head dimension as a kernel argument, so its scale is the hardware's
    // reciprocal square root evaluated at run time; a compile-time constant here would be folded to
    // the correctly rounded value, which can differ from it in the last bit.
    const float scale = rsqrtf(static_cast<float>(a.head_dim));
    float local_maximum = -__int_as_float(0x7f800000);
    for (int p = tid; p < len; p += kOrderedThreads) {
        const bf16* key = kv_row(p, false);
        float dot = 0.0f;
        for (int d = 0; d < HD; ++d) dot = fmaf(qs[d], bf2f(key[d]), dot);
        const float scored = dot * scale;
        scores[p] = scored;
        local_maximum = fmaxf(local_maximum, scored);
    }
    reduction[tid] = local_maximum;
    __syncthreads();
    for (int stride = kOrderedThreads / 2; stride > 0; stride /= 2) {
        if (tid < stride) reduction[tid] = fmaxf(reduction[tid], reduction[tid + stride]);
        __syncthreads();
    }
    const float maximum = reduction[0];
    __syncthreads();

    float local_sum = 0.0f;
    for (int p = tid; p < len; p += kOrderedThreads) {
        const float weight = expf(scores[p] - maximum);
        scores[p] = weight;
        local_sum += weight;
    }
    reduction[tid] = local_sum;
    __syncthreads();
    for (int stride = kOrderedThreads / 2; stride > 0; stride /= 2) {
        if (tid < stride) reduction[tid] += reduction[tid + stride];
        __syncthreads();
    }
    const float inverse = 1.0f / reduction[0];

    // ---- values: one thread per dimension ---------------------------------------------------
    for (int d = tid; d < HD; d += kOrderedThreads) {
        float accumulated = 0.0f;
        for (int p = 0; p < len; ++p) accumulated = fmaf(scores[p], bf2f(kv_row(p, true)[d]), accumulated);
        const size_t o = ((size_t)row * a.q_heads + head) * HD + d;
        const float value = accumulated * inverse;
        if (a.out32 != nullptr) a.out32[o] = value;
        a.out[o] = f2bf(value);
    }
}
}  // namespace

namespace {
__global__ void rope_table_kernel(uint32_t* table, int positions, int head_dim, float theta) {
    const int half = head_dim / 2;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= positions * half) return;
    const int pos = i / half;
    const int d = i % half;
    const float angle = static_cast<float>(pos) * rope_inv_freq(d, head_dim, theta);
    const uint32_t c = __bfloat16_as_ushort(f2bf(cosf(angle)));
    const uint32_t sn = __bfloat16_as_ushort(f2bf(sinf(angle)));
    table[i] = c | (sn << 16);
}
}  // namespace

cudaError_t launch_build_rope_table(uint32_t* table, int positions, int head_dim, float theta,
                                    cudaStream_t stream) {
    if (table == nullptr || positions < 1 || head_dim < 2 || head_dim % 2 != 0) return cudaErrorInvalidValue;
    const int total = positions * (head_dim / 2);
    rope_table_kernel<<<(total + 255) / 256, 256, 0, stream>>>(table, positions, head_dim, theta);
    return cudaGetLastError();
}

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
        static const int forced = [] {
            const char* v = std::getenv("QWEN3_TTS_ATTN_UNITS");
            return v != nullptr ? std::atoi(v) : 0;
        }();
        b.units_per_cta = forced > 0 ? forced : (ctas >= 8192 ? 4 : (ctas >= 2048 ? 2 : 1));
    }
    {
        const int most = max_units_for(b.q_heads / b.kv_heads);     // the kernel's buffers hold that many chunks
        if (b.units_per_cta > most) b.units_per_cta = most;
    }
    switch (b.head_dim) {
        case 32: return launch_hd<32>(b, stream);
        case 64: return launch_hd<64>(b, stream);
        case 128: return launch_hd<128>(b, stream);
        default: return cudaErrorInvalidValue;
    }
}

unsigned int attention_range_error_count() {
    unsigned int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_attention_range_errors, sizeof(v)) != cudaSuccess) return ~0u;
    return v;
}

cudaError_t set_attention_error_sink(unsigned int* device_visible_word) {
    return cudaMemcpyToSymbol(g_attention_error_sink, &device_visible_word, sizeof(device_visible_word));
}

namespace {
int g_attention_mode = 1;
}
// 1 (default): the split-KV kernel.  0: sums in the reference's order (parity mode).
int set_attention_mode(int mode) {
    const int before = g_attention_mode;
    g_attention_mode = mode == 0 ? 0 : 1;
    return before;
}
int attention_mode() { return g_attention_mode; }

// What the engine and the operator entry point call: append and attend in the mode in force.
cudaError_t launch_attention(const AttentionArgs& a, cudaStream_t stream) {
    if (g_attention_mode != 0) return launch_decode_attention(a, stream);
    if (a.fused && a.append_mode != 2) {
        AttentionArgs append = a;
        append.append_mode = 1;
        append.inputs_settled = 0;
        const cudaError_t e = launch_decode_attention(append, stream);
        if (e != cudaSuccess || a.append_mode == 1) return e;
    }
    return launch_attention_reference_order(a, stream);
}

cudaError_t launch_attention_reference_order(const AttentionArgs& a, cudaStream_t stream) {
    if (a.rows < 1 || a.q_heads < 1 || a.kv_heads < 1 || a.q_heads % a.kv_heads != 0 || a.q == nullptr
        || a.out == nullptr || a.positions == nullptr) {
        return cudaErrorInvalidValue;
    }
    if (a.kv.page_table == nullptr && (a.kv.k_bases == nullptr || a.kv.v_bases == nullptr)) return cudaErrorInvalidValue;
    if (a.kv.page_table != nullptr && a.kv.slabs == nullptr) return cudaErrorInvalidValue;
    if (a.fused && a.q_norm_w == nullptr) return cudaErrorInvalidValue;
    const dim3 grid(static_cast<unsigned int>(a.rows * a.q_heads));
    switch (a.head_dim) {
        case 64: return launch_pdl(attention_reference_order_kernel<64>, grid, dim3(kOrderedThreads), 0, stream, a);
        case 128: return launch_pdl(attention_reference_order_kernel<128>, grid, dim3(kOrderedThreads), 0, stream, a);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace q3t
