// Int8 weight-only GEMV / skinny GEMM for 1..8 activation rows: bulk copies ahead of the dependency
// wait, the arithmetic on the tensor cores.
//
// y[r][n] = epilogue( scale[n] * sum_k W[n][k] * x[r][k] ), W int8 [N][K] row-major, x bf16, fp32
// accumulate: the arithmetic of the reference's int8_dequant_gemm_kernel, its residual form and its
// gate/up/SiLU form (native/qwen3-tts-native/native/src/int8_gemv.cu:58-293) with the RMSNorm that
// precedes them (talker_kernels.cu:27-48) as an optional prologue.  What bounds a batch-1 GEMV on
// B200 is not the 12.6 MB it streams but what its CTAs still have to do once the launch before it
// has finished, so this kernel moves everything it can ahead of that point and keeps the rest short:
//
//   before the dependency wait    One CTA per SM owns a contiguous slice of the output channels.  Its
//                                 weights go to shared memory as tiles of 16 rows, one bulk
//                                 asynchronous copy per row (cp.async.bulk, completion counted on an
//                                 mbarrier per tile), rows 64 bytes further apart than their length so
//                                 that the fragment loads below hit every bank once.  Two CTAs fit on
//                                 an SM: under programmatic stream serialisation the slice of the next
//                                 GEMV in the stream is on its way while this one computes.  Scales,
//                                 biases, RMSNorm weights and (when the caller says they are settled)
//                                 the residual are requested here too.
//   after it                      Warp w owns an eighth of K.  Its lanes read their part of the
//                                 activation rows straight into registers, as the B fragments of
//                                 mma.sync.m16n8k16: row r of the batch is column r of B, so 1..8 rows
//                                 cost what one row costs and a row's result does not depend on the
//                                 rows beside it.  The weight tile is the A operand: a lane loads 16
//                                 bytes of rows g and g+8 and turns them into fp16 exactly (XOR to
//                                 unsigned, PRMT of two bytes beside the exponent byte of 1024, one
//                                 packed subtract of 1152): an eighth of the instructions that one FMA
//                                 per weight and lane needs.  Contraction index k is permuted the
//                                 same way on both operands, so 16 consecutive bytes feed four MMAs.
//   activations as fp16           bf16 has the range of fp32 and fp16 has not, so every warp scales
//                                 its part of a row by the power of two that puts the part's largest
//                                 magnitude in [2^14, 2^15) and removes the factor from its partial
//                                 sums again: exact for every element within 2^28 of the largest
//                                 (bf16 has 8 significant bits, fp16 11), below fp32 rounding noise
//                                 for the rest.  Products are exact, accumulation is fp32.
//   the end                       The eight warps' partial sums meet in shared memory and are added in
//                                 warp order (deterministic); the epilogues are the SIMT kernel's.
//
// The fp32 value differs from the SIMT kernel's only by the order of summation (the north-star
// tolerance is 1e-3 relative; this is ~1e-6).  Callers that need the reference's exact summation
// order select the SIMT kernel (set_gemv_mode).
// Every mbarrier wait is bounded; a wait that runs out bumps an error counter, lets the copies
// already issued land and ends the kernel.

#include "q3t_kernels.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace q3t {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / kWarp;
constexpr int kTileRows = 16;              // weight rows per tile = M of the MMA
constexpr int kMaxGroup = 3;               // tiles whose accumulators a warp keeps at once
constexpr int kMaxStages = 8;
constexpr int kSmemBudget = 110 * 1024;    // per CTA: two CTAs per SM
constexpr int kWaitLimit = 1 << 22;        // mbarrier try_wait attempts before giving up

__device__ unsigned int g_gemv_mma_errors = 0;
__device__ unsigned int* g_gemv_mma_error_sink = nullptr;   // host-mapped word of the engine, if any

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    for (int i = 0; i < kWaitLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    return false;
}
// global -> shared bulk copy of this GPU's own memory (no multicast); both addresses 16-byte
// aligned, size a multiple of 16
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// two bytes of a word of unsigned-biased weights (w + 128) as two fp16 weights, exactly:
// {byte, 0x64} is the fp16 1024 + byte = 1152 + w
template <int kSelector>
__device__ __forceinline__ uint32_t weights_f16x2(uint32_t biased_word) {
    const uint32_t carried = __byte_perm(biased_word, 0x64646464u, kSelector);
    uint32_t d;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(d) : "r"(carried), "r"(0x64806480u));   // - (1152, 1152)
    return d;
}

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct MmaParams {
    const int8_t* w;
    const float* scales;
    const bf16* x;
    bf16* y;
    float* y32;
    const bf16* norm_w;
    bf16* norm_out;
    const bf16* bias;
    bf16* resid;
    int K;
    int N;                  // output channels (GATEUP: the matrix has 2N rows, gate rows first)
    int rows;               // 1..8
    int epilogue;
    float eps;
    int chunks;             // K = chunks * 512 * J
    int stages;             // tiles resident in shared memory
    int group;              // tiles per accumulator group, 1..kMaxGroup
    int red_cols;           // columns kept per row in the exchange buffer: rows rounded up to even
    int residual_settled;
};

// Lane (g, t) = (lane / 4, lane % 4) of warp w owns, of chunk c of every activation and weight row,
// the 16 elements at c * KC + w * KW + 64 * j + 16 * t for j = 0..J-1.
template <int J, bool GATEUP, bool NORM>
__global__ void __launch_bounds__(kThreads, 2) gemv_mma_kernel(const MmaParams p) {
    constexpr int KC = 512 * J;                    // K elements per chunk
    constexpr int KW = 64 * J;                     // ... of which one warp owns these
    constexpr int kOut = GATEUP ? 8 : 16;          // output channels per tile
    constexpr uint32_t kFull = 0xffffffffu;

    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x;
    const int lane = tid % kWarp;
    const int warp = tid / kWarp;
    const int g = lane >> 2;
    const int t = lane & 3;
    const int N = p.N, K = p.K, R = p.rows, S = p.stages, C = p.chunks, RP = p.red_cols, Gf = p.group;

    const int stage_bytes = kTileRows * K;         // a tile: 16 weight rows, as they lie in global memory
    unsigned char* ring = smem;
    float* red = reinterpret_cast<float*>(smem + (size_t)S * stage_bytes);     // [warp][tile][16][RP]
    float* partial = red + kWarps * Gf * kTileRows * RP;                       // NORM: [rows][256]
    uint64_t* bars = reinterpret_cast<uint64_t*>(partial + (NORM ? R * kThreads : 0));
    unsigned int* done = reinterpret_cast<unsigned int*>(bars + S);

    // this CTA's output channels, in tiles of kOut
    const int c0 = static_cast<int>(static_cast<unsigned int>(N) * blockIdx.x / gridDim.x);        // N * grid < 2^32
    const int c1 = static_cast<int>(static_cast<unsigned int>(N) * (blockIdx.x + 1) / gridDim.x);
    const int T = (c1 - c0 + kOut - 1) / kOut;

    // One lane requests tile `tile` into its stage: the rows of a tile are consecutive in global
    // memory, so a tile is one bulk copy (two for gate and up rows); a copy costs the copy engine
    // about the same whatever its size, so fewer and larger ones arrive sooner.
    auto issue_tile = [&](int tile) {
        const int stage = tile % S;
        const int first = c0 + tile * kOut;
        const int valid = min(kOut, c1 - first);
        uint64_t* bar = &bars[stage];
        unsigned char* dst = ring + (size_t)stage * stage_bytes;
        const uint32_t bytes = static_cast<uint32_t>(valid) * K;
        mbar_expect_tx(bar, GATEUP ? 2 * bytes : bytes);
        bulk_load(dst, p.w + (size_t)first * K, bytes, bar);
        if (GATEUP) bulk_load(dst + 8 * (size_t)K, p.w + ((size_t)N + first) * K, bytes, bar);
    };

    // Warp w sets up the barrier of stage w and requests the unit that starts in it at once: nothing
    // here waits for another warp.  (The other warps meet these barriers only after the CTA-wide
    // barrier further down.)
    if (warp < S) {
        if (lane == 0) {
            mbar_init(&bars[warp], 1);
            done[warp] = 0;
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            if (warp < T) issue_tile(warp);
        }
    }

    // ---- constants of the epilogue, requested now ------------------------------------------------
    // Thread tid finishes outputs idx = tid and tid + 256 of a group: idx = (tile * 16 + row) * RP + col.
    const int first_group = min(Gf, T);
    float pre_scale[2] = {0.0f, 0.0f}, pre_scale_up[2] = {0.0f, 0.0f}, pre_bias[2] = {0.0f, 0.0f};
    float pre_base[2] = {0.0f, 0.0f};
    auto decode = [&](int idx, int group_base, int group_tiles, int& channel, int& col) -> bool {
        col = idx % RP;
        const int rest = idx / RP;
        const int row = rest & (kTileRows - 1);
        const int gt = rest >> 4;
        channel = c0 + (group_base + gt) * kOut + row;
        return gt < group_tiles && col < R && row < kOut && channel < c1;
    };
    const bool adds = p.epilogue == EPI_ADD || p.epilogue == EPI_BIAS_ADD;
    const bf16* base_src = p.epilogue == EPI_ADD ? p.y : p.resid;
    bool pre_ok[2];
    int pre_channel[2], pre_col[2];
#pragma unroll
    for (int q = 0; q < 2; ++q) {
        pre_ok[q] = decode(tid + q * kThreads, 0, first_group, pre_channel[q], pre_col[q]);
        if (pre_ok[q]) {
            pre_scale[q] = p.scales[pre_channel[q]];
            if (GATEUP) pre_scale_up[q] = p.scales[N + pre_channel[q]];
            if (p.epilogue == EPI_BIAS || p.epilogue == EPI_BIAS_SILU || p.epilogue == EPI_BIAS_ADD) {
                pre_bias[q] = bf2f(p.bias[pre_channel[q]]);
            }
            if (adds && p.residual_settled) pre_base[q] = bf2f(base_src[(size_t)pre_col[q] * N + pre_channel[q]]);
        }
    }
    // RMSNorm weights of this lane's K elements
    uint32_t nw[NORM ? 8 * J : 1];
    if (NORM) {
#pragma unroll
        for (int j = 0; j < J; ++j) {
            const int4* src = reinterpret_cast<const int4*>(p.norm_w + warp * KW + 64 * j + 16 * t);
            const int4 a = src[0], b = src[1];
            nw[NORM ? 8 * j + 0 : 0] = a.x; nw[NORM ? 8 * j + 1 : 0] = a.y;
            nw[NORM ? 8 * j + 2 : 0] = a.z; nw[NORM ? 8 * j + 3 : 0] = a.w;
            nw[NORM ? 8 * j + 4 : 0] = b.x; nw[NORM ? 8 * j + 5 : 0] = b.y;
            nw[NORM ? 8 * j + 6 : 0] = b.z; nw[NORM ? 8 * j + 7 : 0] = b.w;
        }
    }

    __syncthreads();     // the barriers set up above are visible to every warp

    // Everything above touched only constants of the model (and values the caller declared settled).
    pdl_wait();
    pdl_trigger();

    if (adds && !p.residual_settled) {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            if (pre_ok[q]) pre_base[q] = bf2f(base_src[(size_t)pre_col[q] * N + pre_channel[q]]);
        }
    }

    // ---- activations -----------------------------------------------------------------------------
    const bool has_row = g < R;
    const bf16* xrow = p.x + (size_t)(has_row ? g : 0) * K + warp * KW + 16 * t;
    uint32_t raw[8 * J];                    // packed bf16 pairs of the current (or next) chunk
    auto load_raw = [&](int chunk) {
#pragma unroll
        for (int j = 0; j < J; ++j) {
            int4 a = make_int4(0, 0, 0, 0), b = make_int4(0, 0, 0, 0);
            if (has_row) {
                const int4* src = reinterpret_cast<const int4*>(xrow + (size_t)chunk * KC + 64 * j);
                a = src[0];
                b = src[1];
            }
            raw[8 * j + 0] = a.x; raw[8 * j + 1] = a.y; raw[8 * j + 2] = a.z; raw[8 * j + 3] = a.w;
            raw[8 * j + 4] = b.x; raw[8 * j + 5] = b.y; raw[8 * j + 6] = b.z; raw[8 * j + 7] = b.w;
        }
    };
    load_raw(0);

    if (NORM) {
        // sum of squares in the order of the stand-alone RMSNorm (thread i takes elements i, i + 256,
        // ...; halving tree over the 256 partial sums), so that the normalised row is bit-identical
        for (int r = 0; r < R; ++r) {
            const bf16* xr = p.x + (size_t)r * K;
            float ss = 0.0f;
            for (int i = tid; i < K; i += kThreads) {
                const float v = bf2f(xr[i]);
                ss = fmaf(v, v, ss);
            }
            partial[r * kThreads + tid] = ss;
        }
        __syncthreads();
        float inv = 0.0f;
        for (int r = 0; r < R; ++r) {
            const float total = tree_sum_256(partial + r * kThreads, lane);
            const float v = rsqrtf(total / static_cast<float>(K) + p.eps);
            if (r == g) inv = v;
        }
#pragma unroll
        for (int m = 0; m < 8 * J; ++m) {
            const uint32_t wv = nw[NORM ? m : 0];
            const float lo = rbf(bf_lo(raw[m]) * inv) * bf_lo(wv);
            const float hi = rbf(bf_hi(raw[m]) * inv) * bf_hi(wv);
            const __nv_bfloat162 o = __floats2bfloat162_rn(lo, hi);
            raw[m] = *reinterpret_cast<const uint32_t*>(&o);
        }
        if (p.norm_out != nullptr && blockIdx.x == 0 && has_row) {
#pragma unroll
            for (int j = 0; j < J; ++j) {
                int4* dst = reinterpret_cast<int4*>(p.norm_out + (size_t)g * K + warp * KW + 64 * j + 16 * t);
                dst[0] = make_int4(raw[8 * j + 0], raw[8 * j + 1], raw[8 * j + 2], raw[8 * j + 3]);
                dst[1] = make_int4(raw[8 * j + 4], raw[8 * j + 5], raw[8 * j + 6], raw[8 * j + 7]);
            }
        }
    }

    // B fragments: the lane's elements of row g times 2^e, as fp16 pairs; `unscale` is 2^-e
    uint32_t xb[8 * J];
    float scale_now = 1.0f, unscale = 1.0f;
    auto convert = [&]() {
        __nv_bfloat162 m2 = __floats2bfloat162_rn(0.0f, 0.0f);
#pragma unroll
        for (int m = 0; m < 8 * J; ++m) {
            m2 = __hmax2(m2, __habs2(*reinterpret_cast<const __nv_bfloat162*>(&raw[m])));
        }
        const uint32_t mbits = *reinterpret_cast<const uint32_t*>(&m2);
        uint32_t top = max(mbits & 0xffffu, mbits >> 16);       // bits of the largest magnitude (bf16, sign clear)
        top = max(top, __shfl_xor_sync(kFull, top, 1));
        top = max(top, __shfl_xor_sync(kFull, top, 2));
        uint32_t eb = (top >> 7) & 0xffu;                        // its biased exponent
        eb = min(max(eb, 16u), 254u);
        scale_now = __uint_as_float((268u - eb) << 23);          // largest magnitude -> [2^14, 2^15)
        unscale = __uint_as_float((eb - 14u) << 23);
#pragma unroll
        for (int m = 0; m < 8 * J; ++m) {
            const __half2 h = __floats2half2_rn(bf_lo(raw[m]) * scale_now, bf_hi(raw[m]) * scale_now);
            xb[m] = *reinterpret_cast<const uint32_t*>(&h);
        }
    };

    // ---- tiles -----------------------------------------------------------------------------------
    // One tile at a time and one copy of the arithmetic (the loops over tiles and chunks are not
    // unrolled: the code stays in the instruction cache).  After up to Gf tiles the warps' partial
    // sums meet in shared memory.
    bool failed = false;
    int tile = 0;                            // tiles consumed so far (uniform over the CTA)
    bool converted = false;
    const unsigned char* my_rows = ring + (size_t)g * K + warp * KW + 16 * t;
    float* mine = red + (size_t)warp * Gf * kTileRows * RP;
    for (int group_base = 0; group_base < T && !failed; group_base += Gf) {
        const int G = min(Gf, T - group_base);
#pragma unroll 1
        for (int gt = 0; gt < G && !failed; ++gt) {
            // four accumulator sets, one per MMA of a 16-byte group: four independent chains instead of
            // one chain of dependent tensor-core instructions; they are added in a fixed order below
            float acc[4][4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                acc[i][0] = 0.0f; acc[i][1] = 0.0f; acc[i][2] = 0.0f; acc[i][3] = 0.0f;
            }
            const int stage = tile % S;
            const uint32_t parity = static_cast<uint32_t>(tile / S) & 1u;
            bool waited = false;
#pragma unroll 1
            for (int c = 0; c < C; ++c) {
                // activations of this chunk; with one chunk the first conversion serves every tile
                if (C > 1 || !converted) {
                    const float before = scale_now;
                    convert();
                    converted = true;
                    if (c > 0) {
                        // the accumulators carry the previous chunk's power of two: bring them to this one's
                        const float ratio = scale_now / before;
                        const float r0 = __shfl_sync(kFull, ratio, 8 * t);
                        const float r1 = __shfl_sync(kFull, ratio, 8 * t + 4);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            acc[i][0] *= r0; acc[i][1] *= r1; acc[i][2] *= r0; acc[i][3] *= r1;
                        }
                    }
                    // request the elements of the chunk after this one (of this tile or the next)
                    if (C > 1 && (c + 1 < C || tile + 1 < T)) load_raw((c + 1) % C);
                }
                if (!waited) {
                    waited = true;
                    if (!__all_sync(kFull, mbar_wait_bounded(&bars[stage], parity))) {
                        failed = true;
                        break;
                    }
                }
                const unsigned char* rows_lo = my_rows + (size_t)stage * stage_bytes + (size_t)c * KC;
                const unsigned char* rows_hi = rows_lo + 8 * (size_t)K;
                int4 wa = *reinterpret_cast<const int4*>(rows_lo);
                int4 wb = *reinterpret_cast<const int4*>(rows_hi);
#pragma unroll
                for (int j = 0; j < J; ++j) {
                    const uint32_t ua[4] = {(uint32_t)wa.x ^ 0x80808080u, (uint32_t)wa.y ^ 0x80808080u,
                                            (uint32_t)wa.z ^ 0x80808080u, (uint32_t)wa.w ^ 0x80808080u};
                    const uint32_t ub[4] = {(uint32_t)wb.x ^ 0x80808080u, (uint32_t)wb.y ^ 0x80808080u,
                                            (uint32_t)wb.z ^ 0x80808080u, (uint32_t)wb.w ^ 0x80808080u};
                    if (j + 1 < J) {      // the next group's bytes are on their way while this one is converted
                        wa = *reinterpret_cast<const int4*>(rows_lo + 64 * (j + 1));
                        wb = *reinterpret_cast<const int4*>(rows_hi + 64 * (j + 1));
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        mma_16816(acc[i], weights_f16x2<0x4140>(ua[i]), weights_f16x2<0x4140>(ub[i]),
                                  weights_f16x2<0x4342>(ua[i]), weights_f16x2<0x4342>(ub[i]),
                                  xb[8 * j + 2 * i], xb[8 * j + 2 * i + 1]);
                    }
                }
            }
            if (failed) break;
            __syncwarp();      // every lane has read the stage
            if (T > S) {
                // the last of the eight warps to leave a stage requests the tile that reuses it
                unsigned int before = 0;
                if (lane == 0) {
                    __threadfence_block();
                    before = atomicAdd(&done[stage], 1u);
                    if ((before & (kWarps - 1)) == kWarps - 1 && tile + S < T) {
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        issue_tile(tile + S);
                    }
                }
            }
            ++tile;
            // this warp's share of the tile, freed of its power of two
            const float i0 = __shfl_sync(kFull, unscale, 8 * t);
            const float i1 = __shfl_sync(kFull, unscale, 8 * t + 4);
            if (2 * t < RP) {
                float2* lo = reinterpret_cast<float2*>(mine + (gt * kTileRows + g) * RP + 2 * t);
                float2* hi = reinterpret_cast<float2*>(mine + (gt * kTileRows + g + 8) * RP + 2 * t);
                *lo = make_float2(((acc[0][0] + acc[1][0]) + (acc[2][0] + acc[3][0])) * i0,
                                  ((acc[0][1] + acc[1][1]) + (acc[2][1] + acc[3][1])) * i1);
                *hi = make_float2(((acc[0][2] + acc[1][2]) + (acc[2][2] + acc[3][2])) * i0,
                                  ((acc[0][3] + acc[1][3]) + (acc[2][3] + acc[3][3])) * i1);
            }
        }
        // ---- the warps' partial sums meet; epilogue ------------------------------------------------
        failed = __syncthreads_or(failed ? 1 : 0) != 0;      // every thread arrives here, whatever it saw
        if (failed) break;
        const int warp_stride = Gf * kTileRows * RP;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int idx = tid + q * kThreads;
            int channel = pre_channel[q], col = pre_col[q];
            if (group_base == 0 ? !pre_ok[q] : !decode(idx, group_base, G, channel, col)) continue;
            float sum = 0.0f, sum_up = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                sum += red[w * warp_stride + idx];
                if (GATEUP) sum_up += red[w * warp_stride + idx + 8 * RP];
            }
            const bool first = group_base == 0;
            const float scale = first ? pre_scale[q] : p.scales[channel];
            const size_t o = (size_t)col * N + channel;
            float val;
            if (GATEUP) {
                const float gate = sum * scale;
                const float up = sum_up * (first ? pre_scale_up[q] : p.scales[N + channel]);
                val = gate / (1.0f + expf(-gate)) * up;
            } else if (p.epilogue == EPI_PLAIN) {
                val = sum * scale;
            } else if (p.epilogue == EPI_ADD) {
                val = fmaf(sum, scale, first ? pre_base[q] : bf2f(p.y[o]));
            } else {
                const float b = first ? pre_bias[q] : bf2f(p.bias[channel]);
                val = rbf(sum * scale) + b;
                if (p.epilogue == EPI_BIAS_SILU) {
                    val *= 1.0f / (1.0f + expf(-val));
                } else if (p.epilogue == EPI_BIAS_ADD) {
                    val = (first ? pre_base[q] : bf2f(p.resid[o])) + rbf(val);
                    if (p.y32 != nullptr) p.y32[o] = val;
                    p.resid[o] = f2bf(val);
                    continue;
                }
            }
            if (p.y32 != nullptr) p.y32[o] = val;
            p.y[o] = f2bf(val);
        }
        if (group_base + Gf < T) __syncthreads();      // the exchange buffer is written again
    }

    if (failed) {
        if (tid == 0) {
            atomicAdd(&g_gemv_mma_errors, 1u);
            if (g_gemv_mma_error_sink != nullptr) atomicAdd_system(g_gemv_mma_error_sink, 1u);
        }
        // copies already requested must land before this CTA's shared memory is handed on
        for (int d = 0; d < S && tile + d < T; ++d) {
            mbar_wait_bounded(&bars[(tile + d) % S], static_cast<uint32_t>((tile + d) / S) & 1u);
        }
    }
}

int g_sm_count[64] = {};

int sm_count() {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 148;
    if (g_sm_count[device] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n < 1) n = 148;
        g_sm_count[device] = n;
    }
    return g_sm_count[device];
}

int lanes_of(int in_features) {       // J: 64-element groups per lane and chunk
    const int q = in_features / 512;
    if (in_features % 512 != 0 || q < 2) return 0;
    if (q % 4 == 0) return 4;
    if (q % 3 == 0) return 3;
    if (q % 2 == 0) return 2;
    return 0;
}

struct Plan {
    int j = 0, chunks = 0, grid = 0, stages = 0, group = 0, red_cols = 0;
    size_t smem = 0;
};

bool plan_for(const GemvArgs& a, int rows, Plan& plan) {
    const int j = lanes_of(a.in_features);
    if (j == 0 || rows < 1 || rows > 8 || a.out_features < 1) return false;
    const int chunks = a.in_features / (512 * j);
    if (chunks > 8 || (a.norm_w != nullptr && chunks != 1)) return false;
    const bool gateup = a.epilogue == EPI_GATE_UP_SILU;
    const int per_tile = gateup ? 8 : 16;
    int grid = sm_count();
    if (grid > a.out_features) grid = a.out_features;
    const int channels = (a.out_features + grid - 1) / grid;
    const int tiles = (channels + per_tile - 1) / per_tile;
    const int group = tiles < kMaxGroup ? tiles : kMaxGroup;
    const int red_cols = rows <= 2 ? 2 : (rows + 1) / 2 * 2;
    const size_t stage_bytes = (size_t)kTileRows * a.in_features;
    const size_t fixed = (size_t)kWarps * group * kTileRows * red_cols * sizeof(float)
        + (a.norm_w != nullptr ? (size_t)rows * kThreads * sizeof(float) : 0)
        + kMaxStages * (sizeof(uint64_t) + sizeof(unsigned int));
    if (fixed + stage_bytes > (size_t)kSmemBudget) return false;
    int stages = static_cast<int>(((size_t)kSmemBudget - fixed) / stage_bytes);
    if (stages > tiles) stages = tiles;
    if (stages > kMaxStages) stages = kMaxStages;
    plan.j = j; plan.chunks = chunks; plan.grid = grid; plan.stages = stages; plan.group = group;
    plan.red_cols = red_cols;
    plan.smem = fixed + (size_t)stages * stage_bytes;
    return true;
}

template <int J, bool GATEUP, bool NORM>
cudaError_t launch_kernel(const MmaParams& p, const Plan& plan, cudaStream_t stream) {
    return launch_pdl(gemv_mma_kernel<J, GATEUP, NORM>, dim3(static_cast<unsigned int>(plan.grid)), dim3(kThreads),
                      plan.smem, stream, p);
}

template <int J>
cudaError_t launch_flags(const MmaParams& p, const Plan& plan, bool gateup, bool norm, cudaStream_t stream) {
    if (gateup) {
        return norm ? launch_kernel<J, true, true>(p, plan, stream) : launch_kernel<J, true, false>(p, plan, stream);
    }
    return norm ? launch_kernel<J, false, true>(p, plan, stream) : launch_kernel<J, false, false>(p, plan, stream);
}

template <int J>
cudaError_t configure_j() {
    cudaError_t e = cudaFuncSetAttribute(gemv_mma_kernel<J, false, false>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_mma_kernel<J, false, true>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_mma_kernel<J, true, false>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_mma_kernel<J, true, true>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
    return e;
}

}  // namespace

cudaError_t configure_gemv_mma_kernels() {
    cudaError_t e = configure_j<2>();
    if (e == cudaSuccess) e = configure_j<3>();
    if (e == cudaSuccess) e = configure_j<4>();
    sm_count();
    return e;
}

bool gemv_mma_supports(const GemvArgs& a) {
    Plan plan;
    if (a.rows < 1 || a.rows > kMaxRows || !plan_for(a, a.rows < 8 ? a.rows : 8, plan)) return false;
    // bulk copies and 16-byte fragment loads need aligned sources; every row offset is a multiple of K
    if ((reinterpret_cast<uintptr_t>(a.w) & 15u) != 0 || (reinterpret_cast<uintptr_t>(a.x) & 15u) != 0) return false;
    if (a.norm_w != nullptr && (reinterpret_cast<uintptr_t>(a.norm_w) & 15u) != 0) return false;
    if (a.norm_out != nullptr && (reinterpret_cast<uintptr_t>(a.norm_out) & 15u) != 0) return false;
    return true;
}

// More than 8 rows: passes of 8 rows over the same weights, each row computed exactly as it would be alone.
cudaError_t launch_int8_gemv_mma(const GemvArgs& a, cudaStream_t stream) {
    if (!gemv_mma_supports(a) || a.w == nullptr || a.scales == nullptr || a.x == nullptr) {
        return cudaErrorInvalidValue;
    }
    const bool gateup = a.epilogue == EPI_GATE_UP_SILU;
    if (a.epilogue == EPI_BIAS_ADD ? (a.resid == nullptr) : (a.y == nullptr)) return cudaErrorInvalidValue;
    if ((a.epilogue == EPI_BIAS || a.epilogue == EPI_BIAS_SILU || a.epilogue == EPI_BIAS_ADD)
        && a.bias == nullptr) {
        return cudaErrorInvalidValue;
    }
    const bool norm = a.norm_w != nullptr;
    for (int r0 = 0; r0 < a.rows; r0 += 8) {
        const int rows = a.rows - r0 < 8 ? a.rows - r0 : 8;
        Plan plan;
        if (!plan_for(a, rows, plan)) return cudaErrorInvalidValue;
        MmaParams p;
        p.w = a.w; p.scales = a.scales; p.bias = a.bias; p.norm_w = a.norm_w;
        p.x = a.x + (size_t)r0 * a.in_features;
        p.y = a.y != nullptr ? a.y + (size_t)r0 * a.out_features : nullptr;
        p.y32 = a.y32 != nullptr ? a.y32 + (size_t)r0 * a.out_features : nullptr;
        p.norm_out = a.norm_out != nullptr ? a.norm_out + (size_t)r0 * a.in_features : nullptr;
        p.resid = a.resid != nullptr ? a.resid + (size_t)r0 * a.out_features : nullptr;
        p.K = a.in_features; p.N = a.out_features; p.rows = rows; p.epilogue = a.epilogue; p.eps = a.eps;
        p.chunks = plan.chunks; p.stages = plan.stages; p.group = plan.group; p.red_cols = plan.red_cols;
        p.residual_settled = a.residual_settled ? 1 : 0;
        cudaError_t e;
        switch (plan.j) {
            case 2: e = launch_flags<2>(p, plan, gateup, norm, stream); break;
            case 3: e = launch_flags<3>(p, plan, gateup, norm, stream); break;
            default: e = launch_flags<4>(p, plan, gateup, norm, stream); break;
        }
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

unsigned int gemv_mma_error_count() {
    unsigned int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemv_mma_errors, sizeof(v)) != cudaSuccess) return ~0u;
    return v;
}

cudaError_t set_gemv_mma_error_sink(unsigned int* device_visible_word) {
    return cudaMemcpyToSymbol(g_gemv_mma_error_sink, &device_visible_word, sizeof(device_visible_word));
}

}  // namespace q3t
