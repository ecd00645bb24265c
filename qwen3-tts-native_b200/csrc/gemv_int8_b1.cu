// Batch-1 int8 weight-only GEMV, the HBM-bound kernel of the decode step.
//
// Same arithmetic and fp32 summation order as gemv_rows_kernel<1,...> (and therefore as the
// reference's int8_dequant_gemm_kernel<1>, int8_gemv.cu:58-128: lane l owns the 16-byte vectors
// l, l+32, ... of a weight row, 16 sequential FMAs per vector, vector sums added to the lane
// accumulator in vector order, shuffle-down tree) -- what changes is when the bytes move and how
// they are converted:
//   * one CTA per SM owns a contiguous slice of the output channels, and two CTAs fit on an SM:
//     under programmatic stream serialisation the CTA of the next GEMV in the stream sits beside
//     the one that computes.  Every warp owns a private ring of shared-memory stages and fills it
//     with bulk asynchronous copies (cp.async.bulk global -> shared, completion counted on an
//     mbarrier) before the dependency wait: up to 96 KB per CTA, the whole slice of a 12.6 MB
//     matrix, is on its way while the predecessor still runs.  The row scales are fetched there
//     too.  No register is tied up by a load in flight;
//   * after the wait the activations go straight from global memory into registers, widened to
//     fp32 once and kept as pairs (x of vector 2j, x of vector 2j+1) for all rows of the slice
//     (rows of up to 2048 weights; longer rows keep packed bf16 and pair two rows instead);
//   * the FMA chains of two vectors run as one packed chain (fma.rn.f32x2: two ordinary IEEE
//     operations per instruction);
//   * int8 -> fp32 without the conversion pipe: bytes are biased to unsigned with one XOR per
//     word, dropped into the mantissa of 2^23 with PRMT and the bias 2^23+128 is subtracted
//     (exact), again two values per packed instruction;
//   * the pair loop is not unrolled (one copy of the arithmetic in the instruction cache), the
//     warp reductions of four consecutive row pairs run together, and their epilogues run side
//     by side on eight lanes.
// Every wait on an mbarrier is bounded; a wait that runs out records an error word that
// gemv_b1_error_count() returns, drains its own copies and lets the kernel finish.

#include "q3t_kernels.cuh"

namespace q3t {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / kWarp;
constexpr int kRingBudget = 96 * 1024;       // shared memory for the weight rings of one CTA
constexpr int kWaitLimit = 1 << 22;          // mbarrier try_wait attempts before giving up

__device__ unsigned int g_gemv_b1_errors = 0;

__device__ unsigned int* g_gemv_b1_error_sink = nullptr;   // host-mapped word of the engine, if any

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

// global -> shared bulk copy; both addresses 16-byte aligned, size a multiple of 16
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// byte `I` of a word of unsigned-biased weights as the float 2^23 + byte
template <int I>
__device__ __forceinline__ float biased_byte(uint32_t word) {
    return __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7650 + I));
}

struct B1Params {
    const int8_t* w;
    const float* scales;
    const bf16* x;
    bf16* y;
    float* y32;
    const bf16* norm_w;
    bf16* norm_out;
    const bf16* bias;
    bf16* resid;
    int out_features;
    int epilogue;
    float eps;
};

__device__ __forceinline__ void store_result(const B1Params& p, int channel, float acc, float scale) {
    float val;
    if (p.epilogue == EPI_PLAIN) {
        val = acc * scale;
    } else if (p.epilogue == EPI_ADD) {
        val = fmaf(acc, scale, bf2f(p.y[channel]));
    } else if (p.epilogue == EPI_BIAS) {
        val = rbf(acc * scale) + bf2f(p.bias[channel]);
    } else if (p.epilogue == EPI_BIAS_SILU) {
        val = rbf(acc * scale) + bf2f(p.bias[channel]);
        val *= 1.0f / (1.0f + expf(-val));
    } else {  // EPI_BIAS_ADD
        const float t = rbf(rbf(acc * scale) + bf2f(p.bias[channel]));
        val = bf2f(p.resid[channel]) + t;
        if (p.y32 != nullptr) p.y32[channel] = val;
        p.resid[channel] = f2bf(val);
        return;
    }
    if (p.y32 != nullptr) p.y32[channel] = val;
    p.y[channel] = f2bf(val);
}

template <int VPL>
struct Ring {
    static constexpr int kK = VPL * 512;
    static constexpr int kPairBytes = 2 * kK;
    static constexpr int kFit = kRingBudget / (kWarps * kPairBytes);
    static constexpr int kStages = kFit < 1 ? 1 : (kFit > 4 ? 4 : kFit);
    static constexpr size_t kRingBytes = (size_t)kWarps * kStages * kPairBytes;
    static constexpr size_t kSmemBytes =
        kRingBytes + (size_t)kK * sizeof(bf16) + kThreads * sizeof(float) + kWarps * kStages * sizeof(uint64_t);
};

template <int VPL, bool GATEUP, bool NORM>
__global__ void __launch_bounds__(kThreads, VPL <= 6 ? 2 : 1) gemv_b1_kernel(const B1Params p) {
    using R = Ring<VPL>;
    constexpr int K = R::kK;
    constexpr int STAGES = R::kStages;
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* ring = smem;
    bf16* xs = reinterpret_cast<bf16*>(smem + R::kRingBytes);
    float* partial = reinterpret_cast<float*>(smem + R::kRingBytes + (size_t)K * sizeof(bf16));
    uint64_t* bars = reinterpret_cast<uint64_t*>(partial + kThreads);

    const int tid = threadIdx.x;
    const int lane = tid % kWarp;
    const int warp = tid / kWarp;
    const int N = p.out_features;
    const long long pairs = GATEUP ? N : (N + 1) / 2;
    const int p0 = static_cast<int>(pairs * blockIdx.x / gridDim.x);
    const int p1 = static_cast<int>(pairs * (blockIdx.x + 1) / gridDim.x);

    unsigned char* my_ring = ring + (size_t)warp * STAGES * R::kPairBytes;
    uint64_t* my_bars = bars + warp * STAGES;

    // lane 0 of a warp is the producer of that warp's ring
    auto issue = [&](int stage, int pair) {
        unsigned char* dst = my_ring + (size_t)stage * R::kPairBytes;
        if (GATEUP) {
            mbar_expect_tx(&my_bars[stage], 2 * K);
            bulk_load(dst, p.w + (size_t)pair * K, K, &my_bars[stage]);
            bulk_load(dst + K, p.w + ((size_t)N + pair) * K, K, &my_bars[stage]);
        } else {
            const int c = 2 * pair;
            const uint32_t bytes = (c + 1 < N) ? 2 * K : K;
            mbar_expect_tx(&my_bars[stage], bytes);
            bulk_load(dst, p.w + (size_t)c * K, bytes, &my_bars[stage]);
        }
    };

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; ++s) mbar_init(&my_bars[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
#pragma unroll
        for (int s = 0; s < STAGES; ++s) {
            const int pair = p0 + warp + kWarps * s;
            if (pair < p1) issue(s, pair);
        }
    }
    __syncwarp();

    // The scales of this warp's rows are constants too: lane 2i (+1) fetches the scale of the
    // first (second) row of the warp's i-th pair now, so that no epilogue waits on memory.
    constexpr int kScaleSlots = kWarp / 2;
    float my_scale = 0.0f;
    {
        const int pr = p0 + warp + kWarps * (lane >> 1);
        if (pr < p1) {
            if (GATEUP) {
                my_scale = p.scales[(lane & 1) ? N + pr : pr];
            } else if (2 * pr + (lane & 1) < N) {
                my_scale = p.scales[2 * pr + (lane & 1)];
            }
        }
    }

    // Two of these CTAs fit on an SM, so under programmatic stream serialisation the next GEMV of
    // the stream is resident while this one computes: its weight slice is already in its rings
    // when this grid completes.  Only the weights and scales were touched so far; the activations
    // below are the predecessor's output.
    pdl_wait();
    pdl_trigger();   // after the wait, as everywhere in the library; the successor's CTAs move in as this
                     // grid's predecessors' CTAs leave and fetch their weights while this one computes

    // ---- the activations of this lane, as fp32 in registers ------------------------------
    // Lane l owns the 16-byte weight vectors l, l+32, ... of every row, so it needs the same
    // 16 * VPL activations for every row.  kVectorPairs: two vectors' FMA chains run as one
    // packed fp32x2 chain and the activations are kept as fp32 pairs (x of vector 2j, x of
    // vector 2j+1); otherwise (long rows, not enough registers) two rows share a packed chain and
    // the activations stay packed bf16.
    constexpr bool kVectorPairs = VPL <= 4;
    if (NORM) {
        float ss = 0.0f;
        for (int i = tid; i < K; i += kThreads) {
            const float v = bf2f(p.x[i]);
            ss = fmaf(v, v, ss);
        }
        partial[tid] = ss;
        __syncthreads();
        const float total = tree_sum_256(partial, lane);
        const float inv = rsqrtf(total / static_cast<float>(K) + p.eps);
        for (int i = tid; i < K; i += kThreads) {
            const float normalized = rbf(bf2f(p.x[i]) * inv);
            const bf16 o = f2bf(normalized * bf2f(p.norm_w[i]));
            xs[i] = o;
            if (p.norm_out != nullptr && blockIdx.x == 0) p.norm_out[i] = o;
        }
        __syncthreads();
    }
    const bf16* xsrc = NORM ? xs : p.x;          // shared or global: plain loads either way
    uint32_t xr[VPL][8];   // 16 activations per owned vector, packed bf16 pairs
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
        const int4* v4 = reinterpret_cast<const int4*>(xsrc + (size_t)(lane + 32 * j) * 16);
        const int4 a = v4[0];
        const int4 b = v4[1];
        xr[j][0] = a.x; xr[j][1] = a.y; xr[j][2] = a.z; xr[j][3] = a.w;
        xr[j][4] = b.x; xr[j][5] = b.y; xr[j][6] = b.z; xr[j][7] = b.w;
    }
    unsigned long long xp[kVectorPairs ? VPL / 2 : 1][16];
    if (kVectorPairs) {
#pragma unroll
        for (int jp = 0; jp < VPL / 2; ++jp) {
#pragma unroll
            for (int h = 0; h < 8; ++h) {
                xp[jp][2 * h] = pack2(bf_lo(xr[2 * jp][h]), bf_lo(xr[2 * jp + 1][h]));
                xp[jp][2 * h + 1] = pack2(bf_hi(xr[2 * jp][h]), bf_hi(xr[2 * jp + 1][h]));
            }
        }
    }

    const unsigned long long neg_bias = pack2(-8388736.0f, -8388736.0f);   // -(2^23 + 128)
    // The warp reductions of up to kGroup consecutive pairs run together (their shuffle chains
    // are independent, so a group pays the five-step latency once), and the group's results are
    // then spread over lanes 0..2*kGroup-1, which run the epilogue side by side.  The pair loop
    // itself is not unrolled: one copy of the arithmetic in the instruction cache.
    constexpr int kGroup = 4;
    bool failed = false;
    int it = 0;
    int pair = p0 + warp;
    while (pair < p1 && !failed) {
      const int base_pair = pair;
      const int base_it = it;
      int done = 0;
      float pa[kGroup], pb[kGroup];
#pragma unroll
      for (int gi = 0; gi < kGroup; ++gi) {
        pa[gi] = 0.0f;
        pb[gi] = 0.0f;
      }
#pragma unroll 1
      for (int gi = 0; gi < kGroup; ++gi) {
        if (pair >= p1) break;
        const int stage = it % STAGES;
        const uint32_t parity = (it / STAGES) & 1;
        if (!mbar_wait_bounded(&my_bars[stage], parity)) {
            failed = true;
            break;
        }
        const unsigned char* a = my_ring + (size_t)stage * R::kPairBytes;
        float ra, rb;
        if (kVectorPairs) {
            float row_acc[2] = {0.0f, 0.0f};
#pragma unroll
            for (int r = 0; r < 2; ++r) {
#pragma unroll
                for (int jp = 0; jp < VPL / 2; ++jp) {
                    const int4 w0 = *reinterpret_cast<const int4*>(a + (size_t)r * K + (size_t)(lane + 64 * jp) * 16);
                    const int4 w1 = *reinterpret_cast<const int4*>(a + (size_t)r * K + (size_t)(lane + 64 * jp + 32) * 16);
                    const uint32_t u0[4] = {(uint32_t)w0.x ^ 0x80808080u, (uint32_t)w0.y ^ 0x80808080u,
                                            (uint32_t)w0.z ^ 0x80808080u, (uint32_t)w0.w ^ 0x80808080u};
                    const uint32_t u1[4] = {(uint32_t)w1.x ^ 0x80808080u, (uint32_t)w1.y ^ 0x80808080u,
                                            (uint32_t)w1.z ^ 0x80808080u, (uint32_t)w1.w ^ 0x80808080u};
                    unsigned long long sum = pack2(0.0f, 0.0f);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        sum = fma2(add2(pack2(biased_byte<0>(u0[q]), biased_byte<0>(u1[q])), neg_bias),
                                   xp[jp][4 * q], sum);
                        sum = fma2(add2(pack2(biased_byte<1>(u0[q]), biased_byte<1>(u1[q])), neg_bias),
                                   xp[jp][4 * q + 1], sum);
                        sum = fma2(add2(pack2(biased_byte<2>(u0[q]), biased_byte<2>(u1[q])), neg_bias),
                                   xp[jp][4 * q + 2], sum);
                        sum = fma2(add2(pack2(biased_byte<3>(u0[q]), biased_byte<3>(u1[q])), neg_bias),
                                   xp[jp][4 * q + 3], sum);
                    }
                    float s0, s1;
                    unpack2(sum, s0, s1);
                    row_acc[r] += s0;      // vector sums join the lane accumulator in vector order
                    row_acc[r] += s1;
                }
            }
            ra = row_acc[0];
            rb = row_acc[1];
        } else {
            unsigned long long acc = pack2(0.0f, 0.0f);
#pragma unroll
            for (int j = 0; j < VPL; ++j) {
                const int4 wa = *reinterpret_cast<const int4*>(a + (size_t)(lane + 32 * j) * 16);
                const int4 wb = *reinterpret_cast<const int4*>(a + K + (size_t)(lane + 32 * j) * 16);
                const uint32_t ua[4] = {(uint32_t)wa.x ^ 0x80808080u, (uint32_t)wa.y ^ 0x80808080u,
                                        (uint32_t)wa.z ^ 0x80808080u, (uint32_t)wa.w ^ 0x80808080u};
                const uint32_t ub[4] = {(uint32_t)wb.x ^ 0x80808080u, (uint32_t)wb.y ^ 0x80808080u,
                                        (uint32_t)wb.z ^ 0x80808080u, (uint32_t)wb.w ^ 0x80808080u};
                unsigned long long sum = pack2(0.0f, 0.0f);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float x0 = bf_lo(xr[j][2 * q]);
                    const float x1 = bf_hi(xr[j][2 * q]);
                    const float x2 = bf_lo(xr[j][2 * q + 1]);
                    const float x3 = bf_hi(xr[j][2 * q + 1]);
                    sum = fma2(add2(pack2(biased_byte<0>(ua[q]), biased_byte<0>(ub[q])), neg_bias),
                               pack2(x0, x0), sum);
                    sum = fma2(add2(pack2(biased_byte<1>(ua[q]), biased_byte<1>(ub[q])), neg_bias),
                               pack2(x1, x1), sum);
                    sum = fma2(add2(pack2(biased_byte<2>(ua[q]), biased_byte<2>(ub[q])), neg_bias),
                               pack2(x2, x2), sum);
                    sum = fma2(add2(pack2(biased_byte<3>(ua[q]), biased_byte<3>(ub[q])), neg_bias),
                               pack2(x3, x3), sum);
                }
                acc = add2(acc, sum);
            }
            unpack2(acc, ra, rb);
        }
        __syncwarp();   // every lane has read the stage
        const int next = pair + kWarps * STAGES;
        if (lane == 0 && next < p1) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            issue(stage, next);
        }
#pragma unroll
        for (int k = 0; k < kGroup; ++k) {      // static indices keep the partials in registers
            if (gi == k) {
                pa[k] = ra;
                pb[k] = rb;
            }
        }
        pair += kWarps;
        ++it;
        done = gi + 1;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
        for (int gi = 0; gi < kGroup; ++gi) {
            pa[gi] += __shfl_down_sync(0xffffffffu, pa[gi], o);
            pb[gi] += __shfl_down_sync(0xffffffffu, pb[gi], o);
        }
      }
      // lane 2g takes the first row of the group's pair g, lane 2g+1 its second row
      float mine = 0.0f;
#pragma unroll
      for (int gi = 0; gi < kGroup; ++gi) {
        const float a0 = __shfl_sync(0xffffffffu, pa[gi], 0);
        const float b0 = __shfl_sync(0xffffffffu, pb[gi], 0);
        if (lane == 2 * gi) mine = a0;
        if (lane == 2 * gi + 1) mine = b0;
      }
      const int slot = 2 * base_it + lane;                 // which prefetched scale is this lane's
      float scale = __shfl_sync(0xffffffffu, my_scale, slot & 31);
      const bool active = lane < 2 * done;
      const int gpair = base_pair + kWarps * (lane >> 1);
      const int second = lane & 1;
      if (GATEUP) {
        if (active && slot >= 2 * kScaleSlots) scale = p.scales[second ? N + gpair : gpair];
        const float scaled = mine * scale;
        const float up = __shfl_down_sync(0xffffffffu, scaled, 1);
        if (active && !second) {
            const float gate = scaled;
            const float activated = gate / (1.0f + expf(-gate));
            const float val = activated * up;
            if (p.y32 != nullptr) p.y32[gpair] = val;
            p.y[gpair] = f2bf(val);
        }
      } else {
        const int c = 2 * gpair + second;
        if (active && c < N) {
            if (slot >= 2 * kScaleSlots) scale = p.scales[c];
            store_result(p, c, mine, scale);
        }
      }
    }
    if (failed) {
        // record, then give the copies already issued a bounded chance to land before leaving
        if (lane == 0) {
            atomicAdd(&g_gemv_b1_errors, 1u);
            if (g_gemv_b1_error_sink != nullptr) atomicAdd_system(g_gemv_b1_error_sink, 1u);
        }
        // (the stages after the failed one were filled or refilled earlier; none is issued now)
        for (int d = 1; d < STAGES; ++d) {
            pair += kWarps;
            ++it;
            if (pair < p1) mbar_wait_bounded(&my_bars[it % STAGES], (it / STAGES) & 1);
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

template <int VPL, bool GATEUP, bool NORM>
cudaError_t launch_vpl(const B1Params& p, cudaStream_t stream) {
    const long long pairs = GATEUP ? p.out_features : (p.out_features + 1) / 2;
    long long grid = sm_count();
    if (grid > pairs) grid = pairs;
    return launch_pdl(gemv_b1_kernel<VPL, GATEUP, NORM>, dim3(static_cast<unsigned int>(grid)), dim3(kThreads),
                      Ring<VPL>::kSmemBytes, stream, p);
}

template <int VPL>
cudaError_t launch_flags(const B1Params& p, bool gateup, bool norm, cudaStream_t stream) {
    if (gateup) {
        return norm ? launch_vpl<VPL, true, true>(p, stream) : launch_vpl<VPL, true, false>(p, stream);
    }
    return norm ? launch_vpl<VPL, false, true>(p, stream) : launch_vpl<VPL, false, false>(p, stream);
}

template <int VPL>
cudaError_t configure_vpl() {
    const int bytes = static_cast<int>(Ring<VPL>::kSmemBytes);
    cudaError_t e = cudaFuncSetAttribute(gemv_b1_kernel<VPL, false, false>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_b1_kernel<VPL, false, true>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_b1_kernel<VPL, true, false>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_b1_kernel<VPL, true, true>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    return e;
}

}  // namespace

cudaError_t configure_gemv_b1_kernels() {
    cudaError_t e = configure_vpl<2>();
    if (e == cudaSuccess) e = configure_vpl<4>();
    if (e == cudaSuccess) e = configure_vpl<6>();
    if (e == cudaSuccess) e = configure_vpl<12>();
    sm_count();
    return e;
}

bool gemv_b1_supports(const GemvArgs& a) {
    if (a.rows != 1) return false;
    const int k = a.in_features;
    if (k != 1024 && k != 2048 && k != 3072 && k != 6144) return false;
    // bulk copies need 16-byte aligned sources; every row offset is a multiple of K
    return (reinterpret_cast<uintptr_t>(a.w) & 15u) == 0 && (reinterpret_cast<uintptr_t>(a.x) & 15u) == 0;
}

cudaError_t launch_int8_gemv_b1(const GemvArgs& a, cudaStream_t stream) {
    if (!gemv_b1_supports(a) || a.out_features < 1 || a.w == nullptr || a.scales == nullptr
        || a.x == nullptr) {
        return cudaErrorInvalidValue;
    }
    const bool gateup = a.epilogue == EPI_GATE_UP_SILU;
    if (a.epilogue == EPI_BIAS_ADD ? (a.resid == nullptr) : (a.y == nullptr)) return cudaErrorInvalidValue;
    if ((a.epilogue == EPI_BIAS || a.epilogue == EPI_BIAS_SILU || a.epilogue == EPI_BIAS_ADD)
        && a.bias == nullptr) {
        return cudaErrorInvalidValue;
    }
    B1Params p;
    p.w = a.w; p.scales = a.scales; p.x = a.x; p.y = a.y; p.y32 = a.y32;
    p.norm_w = a.norm_w; p.norm_out = a.norm_out; p.bias = a.bias; p.resid = a.resid;
    p.out_features = a.out_features; p.epilogue = a.epilogue; p.eps = a.eps;
    const bool norm = a.norm_w != nullptr;
    switch (a.in_features / 512) {
        case 2: return launch_flags<2>(p, gateup, norm, stream);
        case 4: return launch_flags<4>(p, gateup, norm, stream);
        case 6: return launch_flags<6>(p, gateup, norm, stream);
        default: return launch_flags<12>(p, gateup, norm, stream);
    }
}

unsigned int gemv_b1_error_count() {
    unsigned int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemv_b1_errors, sizeof(v)) != cudaSuccess) return ~0u;
    return v;
}

cudaError_t set_gemv_b1_error_sink(unsigned int* device_visible_word) {
    return cudaMemcpyToSymbol(g_gemv_b1_error_sink, &device_visible_word, sizeof(device_visible_word));
}

}  // namespace q3t
