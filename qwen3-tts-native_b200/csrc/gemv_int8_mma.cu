// Int8 weight-only GEMV / skinny GEMM for 1..8 activation rows: bulk copies ahead of the dependency
// wait, integer tensor-core arithmetic on the raw weight bytes.
//
// y[r][n] = epilogue( scale[n] * sum_k W[n][k] * x[r][k] ), W int8 [N][K] row-major, x bf16: the
// operation of the reference's int8_dequant_gemm_kernel, its residual form and its gate/up/SiLU form
// (native/qwen3-tts-native/native/src/int8_gemv.cu:58-293) with the RMSNorm that precedes them
// (talker_kernels.cu:27-48) as an optional prologue.
//
// What bounds a batch-1 GEMV on B200 is not the 12.6 MB it streams but (a) when the copies are
// requested and (b) how many instructions each weight costs once the launch before it has finished:
// one FMA per weight and lane, or one byte permute per two weights to feed an fp16 MMA, both leave
// the kernel issue-bound at about half of the memory roofline.  So:
//
//   before the dependency wait    One CTA per SM owns a contiguous slice of the output channels, in
//                                 tiles of 16 rows.  The rows of a tile are consecutive in global
//                                 memory, so a tile is TWO bulk asynchronous copies of eight rows
//                                 into shared memory (cp.async.bulk, completion counted on an
//                                 mbarrier): the copy engine spends about as long on a 1 KB copy as on
//                                 a 16 KB one, and the 64 bytes between the two halves keep the
//                                 fragment loads below free of bank conflicts.  Two CTAs fit on an SM:
//                                 the slice of the next GEMV in the stream is on its way while this
//                                 one computes.  Scales, biases and RMSNorm weights are requested
//                                 here too.
//   after it, activations         Warp w owns an eighth of K.  Its 32 lanes fetch that part of every
//                                 activation row with coalesced loads and turn it into fixed point:
//                                 x * 2^e rounded to an integer of 22 bits, e chosen per row and warp
//                                 from the largest magnitude of the part.  Every element within 2^13
//                                 of that magnitude is represented exactly (bf16 has 8 significant
//                                 bits), the rest to 2^-21 of it: more than an fp32 accumulator keeps.
//                                 The integer plus 2^22 is written to shared memory as three unsigned
//                                 bytes ("limbs"), one row of bytes per limb.
//   after it, weights             mma.sync.m16n8k32 (s8 x u8 -> s32): the weight bytes are the A
//                                 operand exactly as they lie in memory, no conversion and no
//                                 instruction but the 16-byte shared-memory loads; the three limbs of
//                                 an activation row are three COLUMNS of B, a fourth column of ones
//                                 yields the row sums of W that the offset of 2^22 has to be corrected
//                                 by.  Products and sums are integers: exact, in any order.  A 16-byte
//                                 load of two weight rows feeds two MMAs; contraction index k is
//                                 permuted the same way on both operands.
//   the end                       Per warp: (limb2 - 64 * ones) * 65536 + limb1 * 256 + limb0, times
//                                 2^-e, in fp32.  The eight warps' values meet in shared memory and are
//                                 added in warp order; the epilogues are the SIMT kernel's.
//
// Against the SIMT kernel (the reference's summation order) the fp32 value differs at the 1e-6 level;
// the north-star tolerance is 1e-3 relative.  Because the arithmetic on the weights is exact, a row's
// result does not depend on the rows computed beside it, bit for bit.  Callers that need the
// reference's exact summation order select the SIMT kernel (set_gemv_mode).
//
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
constexpr int kMaxGroup = 3;               // tiles whose partial sums wait in shared memory at once
constexpr int kMaxStages = 8;
constexpr int kSmemBudget = 113 * 1024;    // per CTA: two CTAs per SM (228 KB, 1 KB of it reserved per CTA)
constexpr int kWaitLimit = 1 << 17;        // mbarrier try_wait attempts before giving up (a fraction of a second)
constexpr int kXsPad = 16;                 // bytes between limb rows in shared memory (bank spread)
constexpr int kLimbs = 3;
constexpr int kHalfPad = 64;               // bytes between the two halves of a weight tile (bank spread)

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

// D(16x8, s32) += A(16x32, s8, row) * B(32x8, u8, col)
__device__ __forceinline__ void imma_16832(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                           uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// byte `kByte` of four words, gathered into one word
template <int kByte>
__device__ __forceinline__ uint32_t gather_byte(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3) {
    const uint32_t lo = __byte_perm(w0, w1, ((4 + kByte) << 4) | kByte);
    const uint32_t hi = __byte_perm(w2, w3, ((4 + kByte) << 4) | kByte);
    return __byte_perm(lo, hi, 0x5410);
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
    int stages;             // tiles resident in shared memory
    int group;              // tiles per exchange of partial sums, 1..kMaxGroup
    int ring_bytes;         // shared memory of the weight stages (the last stage may be a short one)
};

// Q = K / 512: warp w owns the K elements [w * 64 Q, (w + 1) * 64 Q) of every row.  As MMA operand,
// lane (g, t) = (lane / 4, lane % 4) owns of that range the 16 elements at 64 j + 16 t, j = 0..Q-1; in
// the conversion of the activations lane l owns the 2 Q elements at 2 Q l.  Column c of the B operand
// of 8-column group q: limb c % 4 of activation row 2 q + c / 4, where "limb 3" is all ones.
// NTMAX: 8-column groups of B a launch may need: 1 serves one or two activation rows, 4 up to eight.
template <int Q, bool GATEUP, bool NORM, int NTMAX>
__global__ void __launch_bounds__(kThreads, NTMAX == 1 ? 2 : 1) gemv_mma_kernel(const MmaParams p) {
    constexpr int KW = 64 * Q;                     // K elements of one warp
    constexpr int kOut = GATEUP ? 8 : 16;          // output channels per tile
    constexpr uint32_t kFull = 0xffffffffu;
    constexpr int RB = (32 / Q) > 8 ? 8 : (32 / Q);   // activation rows fetched together (registers)

    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x;
    const int lane = tid % kWarp;
    const int warp = tid / kWarp;
    const int g = lane >> 2;
    const int t = lane & 3;
    const int N = p.N, K = p.K, R = p.rows, S = p.stages, Gf = p.group;
    const int xs_stride = K + kXsPad;              // bytes between limb rows
    const int NT = (R + 1) / 2;                    // MMAs per 32 k: two activation rows per 8 columns

    // A tile in shared memory: two halves of eight weight rows as they lie in global memory, the second
    // half 64 bytes further than the first ends.  MMA row m is row m / 2 of half m % 2, so the two
    // lanes of a quarter-warp that read the same 16-byte column of their rows hit different banks.
    const int half_bytes = 8 * K + kHalfPad;
    const int stage_bytes = 2 * half_bytes;
    unsigned char* ring = smem;
    unsigned char* xs = smem + p.ring_bytes;                                    // [R][limb][K + pad] bytes
    float* red = reinterpret_cast<float*>(xs + (size_t)R * kLimbs * xs_stride); // [warp][row of x][4][16]
    float* partial = red + kWarps * R * 64;                                      // NORM: [rows][256]
    uint64_t* bars = reinterpret_cast<uint64_t*>(partial + (NORM ? R * kThreads : 0));
    unsigned int* done = reinterpret_cast<unsigned int*>(bars + S);

    // this CTA's output channels, in tiles of kOut
    const int c0 = static_cast<int>(static_cast<unsigned int>(N) * blockIdx.x / gridDim.x);        // N * grid < 2^32
    const int c1 = static_cast<int>(static_cast<unsigned int>(N) * (blockIdx.x + 1) / gridDim.x);
    const int T = (c1 - c0 + kOut - 1) / kOut;

    // One lane requests tile `tile` into its stage: one bulk copy per half (gate rows and up rows, or
    // the first and the second eight channels).
    auto issue_tile = [&](int tile) {
        const int stage = tile % S;
        const int first = c0 + tile * kOut;
        const int valid = min(kOut, c1 - first);
        uint64_t* bar = &bars[stage];
        unsigned char* dst = ring + (size_t)stage * stage_bytes;
        if (GATEUP) {
            const uint32_t bytes = static_cast<uint32_t>(valid) * K;
            mbar_expect_tx(bar, 2 * bytes);
            bulk_load(dst, p.w + (size_t)first * K, bytes, bar);
            bulk_load(dst + half_bytes, p.w + ((size_t)N + first) * K, bytes, bar);
        } else {
            const int lower = min(valid, 8), upper = valid - lower;
            mbar_expect_tx(bar, static_cast<uint32_t>(valid) * K);
            bulk_load(dst, p.w + (size_t)first * K, static_cast<uint32_t>(lower) * K, bar);
            if (upper > 0) {
                bulk_load(dst + half_bytes, p.w + (size_t)(first + 8) * K, static_cast<uint32_t>(upper) * K, bar);
            }
        }
    };

    // Warp w sets up the barrier of stage w and requests the tile that starts in it at once: nothing
    // here waits for another warp.  (The other warps meet these barriers only after the CTA-wide
    // barrier further down.)
    if (warp < S && lane == 0) {
        mbar_init(&bars[warp], 1);
        done[warp] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        if (warp < T) issue_tile(warp);
    }

    // ---- constants of the epilogue, requested now ------------------------------------------------
    // Thread tid finishes outputs idx = tid and tid + 256 of a group: idx = col * 64 + tile * 16 + row.
    const int first_group = min(Gf, T);
    float pre_scale[2] = {0.0f, 0.0f}, pre_scale_up[2] = {0.0f, 0.0f}, pre_bias[2] = {0.0f, 0.0f};
    auto decode = [&](int idx, int group_base, int group_tiles, int& channel, int& col) -> bool {
        col = idx >> 6;
        const int gt = (idx >> 4) & 3;
        const int row = idx & (kTileRows - 1);
        channel = c0 + (group_base + gt) * kOut + row;
        return gt < group_tiles && col < R && row < kOut && channel < c1;
    };
    const bool adds = p.epilogue == EPI_ADD || p.epilogue == EPI_BIAS_ADD;
    const bool biased_epilogue = p.epilogue == EPI_BIAS || p.epilogue == EPI_BIAS_SILU || p.epilogue == EPI_BIAS_ADD;
    const bf16* base_src = p.epilogue == EPI_ADD ? p.y : p.resid;
    bool pre_ok[2];
    int pre_channel[2], pre_col[2];
#pragma unroll
    for (int q = 0; q < 2; ++q) {
        pre_ok[q] = decode(tid + q * kThreads, 0, first_group, pre_channel[q], pre_col[q]);
        if (pre_ok[q]) {
            pre_scale[q] = p.scales[pre_channel[q]];
            if (GATEUP) pre_scale_up[q] = p.scales[N + pre_channel[q]];
            if (biased_epilogue) pre_bias[q] = bf2f(p.bias[pre_channel[q]]);
        }
    }
    // RMSNorm weights of the elements this lane converts
    uint32_t nw[NORM ? Q : 1];
    if (NORM) {
        const uint32_t* src = reinterpret_cast<const uint32_t*>(p.norm_w + warp * KW + 2 * Q * lane);
#pragma unroll
        for (int m = 0; m < Q; ++m) nw[NORM ? m : 0] = src[m];
    }

    __syncthreads();     // the barriers set up above are visible to every warp

    // Everything above touched only constants of the model.
    pdl_wait();
    pdl_trigger();   // after the wait, as everywhere in the library.  (Triggering at kernel start was
                     // measured: the successor's bulk copies then collide with this kernel's fetch of
                     // its activations, which costs more than the earlier start of the copies gains.)

    // the value a residual epilogue adds to: requested now, needed at the very end
    float pre_base[2] = {0.0f, 0.0f};
    if (adds) {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            if (pre_ok[q]) pre_base[q] = bf2f(base_src[(size_t)pre_col[q] * N + pre_channel[q]]);
        }
    }

    // ---- activations: fetched by all lanes, converted, parked in shared memory as byte limbs -------
    // A lane's share of up to RB rows: 2 Q consecutive elements of each, in this warp's part of K.
    const size_t my_offset = (size_t)warp * KW + 2 * Q * lane;      // elements
    uint32_t raw[RB][Q];
    auto load_rows = [&](int r0) {
#pragma unroll
        for (int b = 0; b < RB; ++b) {
            if (r0 + b < R) {
                const bf16* src = p.x + (size_t)(r0 + b) * K + my_offset;
                if constexpr (Q % 4 == 0) {
#pragma unroll
                    for (int m = 0; m < Q / 4; ++m) {
                        const int4 v = reinterpret_cast<const int4*>(src)[m];
                        raw[b][4 * m + 0] = v.x; raw[b][4 * m + 1] = v.y;
                        raw[b][4 * m + 2] = v.z; raw[b][4 * m + 3] = v.w;
                    }
                } else if constexpr (Q % 2 == 0) {
#pragma unroll
                    for (int m = 0; m < Q / 2; ++m) {
                        const int2 v = reinterpret_cast<const int2*>(src)[m];
                        raw[b][2 * m + 0] = v.x; raw[b][2 * m + 1] = v.y;
                    }
                } else {
#pragma unroll
                    for (int m = 0; m < Q; ++m) raw[b][m] = reinterpret_cast<const uint32_t*>(src)[m];
                }
            }
        }
    };
    // With a norm prologue all rows fit one batch (RB = 8): request them now, so that they travel
    // together with the strided reads of the sum of squares instead of after its barrier.
    static_assert(!NORM || RB >= 8, "the norm prologue expects every row in the first batch");
    if (NORM) load_rows(0);

    float inv_mine = 0.0f;           // NORM: lane r keeps 1/rms of row r
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
        for (int r = 0; r < R; ++r) {
            const float total = tree_sum_256(partial + r * kThreads, lane);
            const float v = rsqrtf(total / static_cast<float>(K) + p.eps);
            if (r == lane) inv_mine = v;
        }
    }
    // Arrival of the tiles of a group (long there, in a chain of launches: the test costs its latency
    // only, which the first group hides behind the fetch of the activations).
    bool failed = false;
    int stage = 0;                           // (tiles waited for) % S and its phase, kept without divisions
    uint32_t parity = 0;
    int stage_of[kMaxGroup] = {};
    auto await_group = [&](int group_tiles) {
#pragma unroll
        for (int gt = 0; gt < kMaxGroup; ++gt) {
            if (gt < group_tiles && !failed) {
                bool ready = mbar_try_wait(&bars[stage], parity);
                if (!ready) ready = mbar_wait_bounded(&bars[stage], parity);
                if (!__all_sync(kFull, ready)) failed = true;
                stage_of[gt] = stage;
                if (++stage == S) {
                    stage = 0;
                    parity ^= 1u;
                }
            }
        }
    };

    float unscale_mine = 1.0f;       // lane r keeps 2^-e of row r in this warp's part
    {
#pragma unroll 1
        for (int r0 = 0; r0 < R; r0 += RB) {
            if (!NORM || r0 > 0) load_rows(r0);
            if (r0 == 0) await_group(min(Gf, T));      // the activations are in flight meanwhile
#pragma unroll
            for (int b = 0; b < RB; ++b) {
                const int r = r0 + b;
                if (r < R) {
                    if (NORM) {
                        const float inv = __shfl_sync(kFull, inv_mine, r);
#pragma unroll
                        for (int m = 0; m < Q; ++m) {
                            const uint32_t wv = nw[NORM ? m : 0];
                            const float lo = rbf(bf_lo(raw[b][m]) * inv) * bf_lo(wv);
                            const float hi = rbf(bf_hi(raw[b][m]) * inv) * bf_hi(wv);
                            const __nv_bfloat162 o = __floats2bfloat162_rn(lo, hi);
                            raw[b][m] = *reinterpret_cast<const uint32_t*>(&o);
                        }
                        if (p.norm_out != nullptr && blockIdx.x == 0) {
                            uint32_t* dst = reinterpret_cast<uint32_t*>(p.norm_out + (size_t)r * K + my_offset);
#pragma unroll
                            for (int m = 0; m < Q; ++m) dst[m] = raw[b][m];
                        }
                    }
                    // largest magnitude of the row in this warp's part -> its power of two
                    __nv_bfloat162 m2 = __habs2(*reinterpret_cast<const __nv_bfloat162*>(&raw[b][0]));
#pragma unroll
                    for (int m = 1; m < Q; ++m) {
                        m2 = __hmax2(m2, __habs2(*reinterpret_cast<const __nv_bfloat162*>(&raw[b][m])));
                    }
                    const uint32_t mbits = *reinterpret_cast<const uint32_t*>(&m2);
                    const uint32_t top = __reduce_max_sync(kFull, max(mbits & 0xffffu, mbits >> 16));
                    const uint32_t eb_raw = (top >> 7) & 0xffu;              // biased exponent of the largest magnitude
                    const uint32_t eb = min(max(eb_raw, 21u), 240u);
                    const float scale = __uint_as_float((274u - eb) << 23);  // largest magnitude -> [2^20, 2^21)
                    if (lane == r) {
                        // 1 / scale; an infinity or NaN among the activations makes the row's results NaN
                        unscale_mine = eb_raw == 255u ? __uint_as_float(0x7fc00000u) : __uint_as_float((eb - 20u) << 23);
                    }
                    // x * scale + 1.5 * 2^23 rounds to an integer in fp32 whose low 23 bits are the fixed-point
                    // value plus 2^22: bytes 0, 1, 2 of the float's bit pattern are the three limbs
                    uint32_t fixed[2 * Q];
#pragma unroll
                    for (int m = 0; m < Q; ++m) {
                        fixed[2 * m] = __float_as_uint(fmaf(bf_lo(raw[b][m]), scale, 12582912.0f));
                        fixed[2 * m + 1] = __float_as_uint(fmaf(bf_hi(raw[b][m]), scale, 12582912.0f));
                    }
                    unsigned char* dst = xs + (size_t)r * kLimbs * xs_stride + my_offset;
#pragma unroll
                    for (int m = 0; m < Q / 2; ++m) {
                        const uint32_t f0 = fixed[4 * m], f1 = fixed[4 * m + 1], f2 = fixed[4 * m + 2], f3 = fixed[4 * m + 3];
                        reinterpret_cast<uint32_t*>(dst)[m] = gather_byte<0>(f0, f1, f2, f3);
                        reinterpret_cast<uint32_t*>(dst + xs_stride)[m] = gather_byte<1>(f0, f1, f2, f3);
                        reinterpret_cast<uint32_t*>(dst + 2 * xs_stride)[m] = gather_byte<2>(f0, f1, f2, f3);
                    }
                }
            }
        }
    }
    __syncwarp();        // this warp's part of every row is in shared memory; no other warp reads it

    // ---- B fragments come from shared memory --------------------------------------------------------
    // Column g of 8-column group q, for activation rows 2q (g < 4) and 2q + 1 (g >= 4): limbs 0, 1, 2 and
    // a column of ones.  The accumulator lanes t = 0, 1 then hold {limb 0, limb 1} and {limb 2, ones} of
    // the even row, lanes t = 2, 3 the same of the odd row: a row's value is put together by two
    // neighbouring lanes.
    const int col_limb = g & 3;
    const unsigned char* my_x = xs + (size_t)col_limb * xs_stride + warp * KW + 16 * t;
    auto load_b = [&](int j, int q, uint32_t (&b)[4]) {
        const int row = 2 * q + (g >> 2);
        if (col_limb < 3 && row < R) {
            const int4 v = *reinterpret_cast<const int4*>(my_x + (size_t)row * kLimbs * xs_stride + 64 * j);
            b[0] = v.x; b[1] = v.y; b[2] = v.z; b[3] = v.w;
        } else {
            const uint32_t fill = col_limb == 3 ? 0x01010101u : 0u;
            b[0] = fill; b[1] = fill; b[2] = fill; b[3] = fill;
        }
    };

    // ---- tiles -----------------------------------------------------------------------------------
    // Up to kMaxGroup tiles run side by side: K is the outer loop, so a B fragment is fetched once for
    // all of them and a warp has several independent accumulator chains in flight.  After a group the
    // warps' values meet in shared memory.
    int tile = 0;                            // tiles consumed so far (uniform over the CTA)
    const unsigned char* my_rows = ring + (size_t)(g & 1) * half_bytes + (size_t)(g >> 1) * K + warp * KW + 16 * t;
    const int row_lo = 8 * (g & 1) + (g >> 1);      // where MMA rows g and g + 8 sit in the tile
    const int row_hi = row_lo + 4;
    float* mine = red + (size_t)warp * R * 64;
    constexpr int kChains = NTMAX == 1 ? 2 : 1;     // accumulator sets per tile and column group
    float unscale[NTMAX][2];                        // 2^-e of the activation rows 2q and 2q + 1
#pragma unroll
    for (int q = 0; q < NTMAX; ++q) {
        unscale[q][0] = __shfl_sync(kFull, unscale_mine, 2 * q);
        unscale[q][1] = __shfl_sync(kFull, unscale_mine, 2 * q + 1);
    }
    for (int group_base = 0; group_base < T; group_base += Gf) {      // left only after the CTA-wide vote below
        const int G = min(Gf, T - group_base);
        if (group_base > 0) await_group(G);
        const unsigned char* rows[kMaxGroup];
#pragma unroll
        for (int gt = 0; gt < kMaxGroup; ++gt) rows[gt] = my_rows + (size_t)stage_of[gt] * stage_bytes;
        if (!failed) {
            int acc[kMaxGroup][NTMAX][kChains][4];
#pragma unroll
            for (int gt = 0; gt < kMaxGroup; ++gt)
#pragma unroll
                for (int q = 0; q < NTMAX; ++q)
#pragma unroll
                    for (int h = 0; h < kChains; ++h)
#pragma unroll
                        for (int c = 0; c < 4; ++c) acc[gt][q][h][c] = 0;
#pragma unroll
            for (int j = 0; j < Q; ++j) {
                uint32_t b[NTMAX][4];
#pragma unroll
                for (int q = 0; q < NTMAX; ++q) {
                    if (q < NT) load_b(j, q, b[q]);
                }
#pragma unroll
                for (int gt = 0; gt < kMaxGroup; ++gt) {
                    if (gt < G) {
                        const int4 wa = *reinterpret_cast<const int4*>(rows[gt] + 64 * j);
                        const int4 wb = *reinterpret_cast<const int4*>(rows[gt] + 4 * (size_t)K + 64 * j);
#pragma unroll
                        for (int q = 0; q < NTMAX; ++q) {
                            if (q < NT) {
                                imma_16832(acc[gt][q][0], wa.x, wb.x, wa.y, wb.y, b[q][0], b[q][1]);
                                imma_16832(acc[gt][q][kChains - 1], wa.z, wb.z, wa.w, wb.w, b[q][2], b[q][3]);
                            }
                        }
                    }
                }
            }
            __syncwarp();      // every lane has read the stages
            if (T > S && lane == 0) {
                // the last of the eight warps to leave a stage requests the tile that reuses it
                __threadfence_block();
#pragma unroll
                for (int gt = 0; gt < kMaxGroup; ++gt) {
                    if (gt < G) {
                        const unsigned int before = atomicAdd(&done[stage_of[gt]], 1u);
                        if ((before & (kWarps - 1)) == kWarps - 1 && tile + gt + S < T) {
                            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                            issue_tile(tile + gt + S);
                        }
                    }
                }
            }
            tile += G;
            // This warp's share of the tiles.  Of a group of four lanes, t = 0 holds limbs 0 and 1 of the
            // even activation row and t = 1 its limb 2 and the row sum of W (t = 2, 3: the odd row).  The
            // three limb sums are exact integers below 2^25; their combination is done in fp32, high part
            // in the odd lane, low part in the even lane, one exchange.
#pragma unroll
            for (int gt = 0; gt < kMaxGroup; ++gt) {
                if (gt < G) {
#pragma unroll
                    for (int q = 0; q < NTMAX; ++q) {
                        if (q < NT) {
                            int d[4];
#pragma unroll
                            for (int c = 0; c < 4; ++c) d[c] = acc[gt][q][0][c] + (kChains == 2 ? acc[gt][q][kChains - 1][c] : 0);
                            float part[2];      // tile rows g, g + 8
#pragma unroll
                            for (int half = 0; half < 2; ++half) {
                                const int first = d[2 * half], second = d[2 * half + 1];
                                part[half] = (t & 1) ? static_cast<float>(first - 64 * second) * 65536.0f
                                                     : fmaf(static_cast<float>(second), 256.0f, static_cast<float>(first));
                                part[half] += __shfl_xor_sync(kFull, part[half], 1);
                            }
                            const int row = 2 * q + (t >> 1);
                            if ((t & 1) == 0 && row < R) {
                                const float u = unscale[q][t >> 1];
                                mine[row * 64 + gt * kTileRows + row_lo] = part[0] * u;
                                mine[row * 64 + gt * kTileRows + row_hi] = part[1] * u;
                            }
                        }
                    }
                }
            }
        }
        // ---- the warps' partial sums meet; epilogue ------------------------------------------------
        failed = __syncthreads_or(failed ? 1 : 0) != 0;      // every thread arrives here, whatever it saw
        if (failed) break;
        const int warp_stride = R * 64;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int idx = tid + q * kThreads;
            int channel = pre_channel[q], col = pre_col[q];
            if (group_base == 0 ? !pre_ok[q] : !decode(idx, group_base, G, channel, col)) continue;
            float sum = 0.0f, sum_up = 0.0f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                sum += red[w * warp_stride + idx];
                if (GATEUP) sum_up += red[w * warp_stride + idx + 8];
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

bool supported_q(int q, bool norm) {
    if (norm) return q == 2 || q == 4;                  // the fused RMSNorm is built for hidden sizes 1024 and 2048
    return q == 2 || q == 4 || q == 6 || q == 12;
}

struct Plan {
    int q = 0, grid = 0, stages = 0, group = 0;
    size_t ring = 0, smem = 0;
};

constexpr int kSmemBudgetAlone = 200 * 1024;   // one CTA per SM: launches of three or more activation rows

// Shared memory of a launch.  When every tile of a CTA can be resident at once, the last stage is
// only as long as the longest last tile needs (a CTA's channels rarely fill their last tile).
bool plan_with_budget(const GemvArgs& a, int rows, size_t budget, Plan& plan);

bool plan_for(const GemvArgs& a, int rows, Plan& plan) {
    // one or two rows: room for two CTAs per SM if the shape allows, else the SM to itself
    if (rows <= 2 && plan_with_budget(a, rows, kSmemBudget, plan)) return true;
    return plan_with_budget(a, rows, kSmemBudgetAlone, plan);
}

bool plan_with_budget(const GemvArgs& a, int rows, size_t budget, Plan& plan) {
    if (a.in_features % 512 != 0 || rows < 1 || rows > 8 || a.out_features < 1) return false;
    const int q = a.in_features / 512;
    if (!supported_q(q, a.norm_w != nullptr)) return false;
    const bool gateup = a.epilogue == EPI_GATE_UP_SILU;
    const int per_tile = gateup ? 8 : 16;
    const size_t K = a.in_features;
    int grid = sm_count();
    if (grid > a.out_features) grid = a.out_features;
    const int channels = (a.out_features + grid - 1) / grid;
    const int tiles = (channels + per_tile - 1) / per_tile;
    const size_t half_bytes = 8 * K + kHalfPad;
    const size_t stage_bytes = 2 * half_bytes;
    const int last_rows = channels - (tiles - 1) * per_tile;         // channels of the longest last tile
    const size_t last_bytes = gateup ? half_bytes + (size_t)last_rows * K
                                     : (last_rows > 8 ? half_bytes + (size_t)(last_rows - 8) * K : (size_t)last_rows * K);
    const size_t fixed = (size_t)rows * kLimbs * (K + kXsPad)
        + (size_t)kWarps * rows * 64 * sizeof(float)
        + (a.norm_w != nullptr ? (size_t)rows * kThreads * sizeof(float) : 0)
        + kMaxStages * (sizeof(uint64_t) + sizeof(unsigned int));
    const size_t all_resident = (size_t)(tiles - 1) * stage_bytes + last_bytes;
    int stages;
    size_t ring;
    // The tile loop reads all sixteen rows of a stage whatever was copied into it (rows past the
    // last channel feed accumulators nobody reads), so a short last stage must still lie inside the
    // allocation: what follows the ring has to cover the rows that were left out.
    if (tiles <= kMaxStages && fixed + all_resident <= budget && (size_t)tiles * stage_bytes <= budget) {
        stages = tiles;
        ring = (all_resident + 127) / 128 * 128;
        if (ring + fixed < (size_t)tiles * stage_bytes) ring = (size_t)tiles * stage_bytes - fixed / 128 * 128;
    } else {
        if (fixed + stage_bytes > budget) return false;
        stages = static_cast<int>((budget - fixed) / stage_bytes);
        if (stages > kMaxStages) stages = kMaxStages;
        if (stages >= tiles) stages = tiles;
        ring = (size_t)stages * stage_bytes;
    }
    int group = tiles < kMaxGroup ? tiles : kMaxGroup;
    if (group > stages) group = stages;         // a group's tiles are all resident before it starts
    plan.q = q; plan.grid = grid; plan.stages = stages; plan.group = group;
    plan.ring = ring;
    plan.smem = fixed + ring;
    return true;
}

// activation rows one launch can take for this shape (more rows run as several launches)
int rows_per_launch(const GemvArgs& a) {
    Plan plan;
    for (int rows = 8; rows >= 1; --rows) {
        if (plan_for(a, rows, plan)) return rows;
    }
    return 0;
}

template <int Q, bool GATEUP, bool NORM>
cudaError_t launch_rows(const MmaParams& p, const Plan& plan, cudaStream_t stream) {
    const dim3 grid(static_cast<unsigned int>(plan.grid));
    if (p.rows <= 2) return launch_pdl(gemv_mma_kernel<Q, GATEUP, NORM, 1>, grid, dim3(kThreads), plan.smem, stream, p);
    return launch_pdl(gemv_mma_kernel<Q, GATEUP, NORM, 4>, grid, dim3(kThreads), plan.smem, stream, p);
}

template <int Q>
cudaError_t launch_flags(const MmaParams& p, const Plan& plan, bool gateup, bool norm, cudaStream_t stream) {
    if constexpr (Q == 2 || Q == 4) {
        if (norm) {
            return gateup ? launch_rows<Q, true, true>(p, plan, stream) : launch_rows<Q, false, true>(p, plan, stream);
        }
    }
    return gateup ? launch_rows<Q, true, false>(p, plan, stream) : launch_rows<Q, false, false>(p, plan, stream);
}

template <int Q, bool GATEUP, bool NORM>
cudaError_t configure_one() {
    cudaError_t e = cudaFuncSetAttribute(gemv_mma_kernel<Q, GATEUP, NORM, 1>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudgetAlone);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_mma_kernel<Q, GATEUP, NORM, 4>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudgetAlone);
    return e;
}

template <int Q>
cudaError_t configure_q() {
    cudaError_t e = configure_one<Q, false, false>();
    if (e == cudaSuccess) e = configure_one<Q, true, false>();
    if constexpr (Q == 2 || Q == 4) {
        if (e == cudaSuccess) e = configure_one<Q, false, true>();
        if (e == cudaSuccess) e = configure_one<Q, true, true>();
    }
    return e;
}

}  // namespace

cudaError_t configure_gemv_mma_kernels() {
    cudaError_t e = configure_q<2>();
    if (e == cudaSuccess) e = configure_q<4>();
    if (e == cudaSuccess) e = configure_q<6>();
    if (e == cudaSuccess) e = configure_q<12>();
    sm_count();
    return e;
}

// Host-side planning only (no CUDA call beyond the cached SM count, 148 without a device): what one
// launch of `rows` activation rows would be given.  For tests of the plan arithmetic.
bool gemv_mma_plan(int in_features, int out_features, int rows, bool gate_up, bool norm, GemvMmaPlan* out) {
    if (out == nullptr) return false;
    GemvArgs a;
    a.in_features = in_features;
    a.out_features = out_features;
    a.rows = rows;
    a.epilogue = gate_up ? EPI_GATE_UP_SILU : EPI_PLAIN;
    static const bf16 some_weight = bf16();
    a.norm_w = norm ? &some_weight : nullptr;        // only its presence matters to the plan
    Plan plan;
    if (!plan_for(a, rows, plan)) return false;
    const int per_tile = gate_up ? 8 : 16;
    const int channels = (out_features + plan.grid - 1) / plan.grid;
    out->grid = plan.grid;
    out->stages = plan.stages;
    out->group = plan.group;
    out->tiles = (channels + per_tile - 1) / per_tile;
    out->stage_bytes = 2 * (8 * (long long)in_features + kHalfPad);
    out->ring_bytes = static_cast<long long>(plan.ring);
    out->shared_bytes = static_cast<long long>(plan.smem);
    out->rows_per_launch = rows_per_launch(a);
    return true;
}

bool gemv_mma_supports(const GemvArgs& a) {
    if (a.rows < 1 || a.rows > kMaxRows || rows_per_launch(a) == 0) return false;
    // bulk copies and vector loads need aligned sources; every row offset is a multiple of K
    if ((reinterpret_cast<uintptr_t>(a.w) & 15u) != 0 || (reinterpret_cast<uintptr_t>(a.x) & 15u) != 0) return false;
    if (a.norm_w != nullptr && (reinterpret_cast<uintptr_t>(a.norm_w) & 15u) != 0) return false;
    if (a.norm_out != nullptr && (reinterpret_cast<uintptr_t>(a.norm_out) & 15u) != 0) return false;
    return true;
}

// More rows than one launch takes (8, fewer for long rows): several launches over the same weights.
// The arithmetic on a row does not depend on the rows beside it, so the split is invisible.
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
    const int step = a.rows <= 2 ? a.rows : rows_per_launch(a);
    for (int r0 = 0; r0 < a.rows; r0 += step) {
        const int rows = a.rows - r0 < step ? a.rows - r0 : step;
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
        p.stages = plan.stages; p.group = plan.group; p.ring_bytes = static_cast<int>(plan.ring);
        cudaError_t e;
        switch (plan.q) {
            case 2: e = launch_flags<2>(p, plan, gateup, norm, stream); break;
            case 4: e = launch_flags<4>(p, plan, gateup, norm, stream); break;
            case 6: e = launch_flags<6>(p, plan, gateup, norm, stream); break;
            default: e = launch_flags<12>(p, plan, gateup, norm, stream); break;
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
