// Weight-only int8 GEMV / skinny GEMM for 1..8 activation rows (SIMT path).
//
// y[r][n] = epilogue( scale[n] * sum_k W[n][k] * x[r][k] ), W int8 [N][K] row-major,
// x bf16, fp32 accumulate.  Replaces the reference's int8_dequant_gemm_kernel,
// int8_dequant_gemm_add_kernel and int8_dequant_gate_up_silu_kernel
// (native/qwen3-tts-native/native/src/int8_gemv.cu:58-293) and folds the RMSNorm that
// precedes q/k/v, gate/up and the vocabulary heads (talker_kernels.cu:27-48) and the bias
// / SiLU / residual glue that follows the small projections (talker_kernels.cu:660-678,
// 359-371) into the same launch.
//
// Layout of one launch: a CTA of 8 warps first issues the 128-bit streaming loads of its
// first weight vectors, then stages the activation rows in shared memory (normalising
// them if asked), and then every warp owns one output channel at a time: lane l
// multiplies the 16-byte vectors l, l+32, ... of the weight row with the staged
// activations (16 sequential FMAs per vector, vector sums added to a lane accumulator),
// the 32 lane accumulators are folded with a shuffle-down tree and lane 0 applies the
// epilogue.  That is the summation order of the reference kernel, so the fp32 value
// before the epilogue is bit-identical to it.

#include "q3t_kernels.cuh"

#include <cstdlib>
#include <cstring>

namespace q3t {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / kWarp;
constexpr int kVecBytes = 16;

__device__ __forceinline__ float s8_to_f32(int v) { return static_cast<float>(v); }

// 16 sequential FMAs: weights (one int4 = 16 int8) against 16 bf16 activations (2 int4).
__device__ __forceinline__ float dot16(const int4& w, const int4& xa, const int4& xb) {
    float sum = 0.0f;
    const int wi[4] = {w.x, w.y, w.z, w.w};
    const uint32_t xi[8] = {(uint32_t)xa.x, (uint32_t)xa.y, (uint32_t)xa.z, (uint32_t)xa.w,
                            (uint32_t)xb.x, (uint32_t)xb.y, (uint32_t)xb.z, (uint32_t)xb.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int word = wi[q];
        const float w0 = s8_to_f32(static_cast<int8_t>(word));
        const float w1 = s8_to_f32(static_cast<int8_t>(word >> 8));
        const float w2 = s8_to_f32(static_cast<int8_t>(word >> 16));
        const float w3 = s8_to_f32(word >> 24);
        sum = fmaf(w0, bf_lo(xi[2 * q]), sum);
        sum = fmaf(w1, bf_hi(xi[2 * q]), sum);
        sum = fmaf(w2, bf_lo(xi[2 * q + 1]), sum);
        sum = fmaf(w3, bf_hi(xi[2 * q + 1]), sum);
    }
    return sum;
}

// KPRE = weight vectors a lane has in flight at once (and requests before the activations are
// staged): 4 covers a whole row up to K = 2048; the long rows of the batch-1 down projection use
// 12 so that a row is one round trip to memory instead of three.
template <int ROWS, bool GATEUP, bool NORM, int KPRE = 4>
__global__ void __launch_bounds__(kThreads)
gemv_rows_kernel(const int8_t* __restrict__ weight, const float* __restrict__ scales,
                 const bf16* __restrict__ input, bf16* __restrict__ output,
                 float* __restrict__ output32, const bf16* __restrict__ norm_w,
                 bf16* __restrict__ norm_out, const bf16* __restrict__ bias,
                 bf16* __restrict__ resid, int in_features, int out_features, int epilogue,
                 float eps, int residual_settled) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* xs = reinterpret_cast<bf16*>(smem_raw);                  // [ROWS][K]
    __shared__ float partial[NORM ? ROWS * kThreads : 1];

    const int tid = threadIdx.x;
    const int lane = tid % kWarp;
    const int warp = tid / kWarp;
    const int vectors = in_features / kVecBytes;
    const int total_warps = gridDim.x * kWarps;
    const int first_channel = blockIdx.x * kWarps + warp;

    // Weight loads of the first channel go out before the activations are staged.
    constexpr int kPre = KPRE;
    int4 pre[GATEUP ? 2 : 1][kPre];
    if (first_channel < out_features) {
        const int4* row0 = reinterpret_cast<const int4*>(weight + (size_t)first_channel * in_features);
#pragma unroll
        for (int u = 0; u < kPre; ++u) {
            const int v = lane + u * kWarp;
            if (v < vectors) pre[0][u] = ld_stream(row0 + v);
        }
        if (GATEUP) {
            const int4* row1 = reinterpret_cast<const int4*>(
                weight + ((size_t)out_features + first_channel) * in_features);
#pragma unroll
            for (int u = 0; u < kPre; ++u) {
                const int v = lane + u * kWarp;
                if (v < vectors) pre[GATEUP ? 1 : 0][u] = ld_stream(row1 + v);
            }
        }
    }

    // ... and so do its scales, so that the epilogue of the first channel does not wait on memory.
    float pre_scale = 0.0f, pre_scale_up = 0.0f;
    if (first_channel < out_features) {
        pre_scale = scales[first_channel];
        if (GATEUP) pre_scale_up = scales[out_features + first_channel];
    }

    // The RMSNorm weights of the elements this thread normalises (constants, like the weights).
    constexpr int kNormPre = 8;                       // covers K <= 2048
    bf16 nw_pre[NORM ? kNormPre : 1];
    const bool nw_ready = NORM && in_features <= kNormPre * kThreads;
    if (NORM && nw_ready) {
#pragma unroll
        for (int u = 0; u < kNormPre; ++u) {
            const int i = tid + u * kThreads;
            if (i < in_features) nw_pre[u] = norm_w[i];
        }
    }
    // The value a residual epilogue adds to, when its writer is known to be long done.
    float pre_resid[ROWS];
    const bool resid_ready = !GATEUP && residual_settled != 0 && lane == 0 && first_channel < out_features
                             && (epilogue == EPI_ADD || epilogue == EPI_BIAS_ADD);
    if (resid_ready) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const size_t o = (size_t)r * out_features + first_channel;
            pre_resid[r] = bf2f(epilogue == EPI_ADD ? output[o] : resid[o]);
        }
    }

    // Launched with programmatic stream serialisation: this grid may start while the one before
    // it in the stream is still running.  Everything above touches only the weights; from here on
    // the previous grid's output is read, so wait for it to complete (a no-op when the launch
    // was an ordinary one), and let the grid after this one start its own weight loads.
    pdl_wait();
    pdl_trigger();

    // ---- stage activations --------------------------------------------------------
    if (NORM) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const bf16* xr = input + (size_t)r * in_features;
            float ss = 0.0f;
            for (int i = tid; i < in_features; i += kThreads) {
                const float v = bf2f(xr[i]);
                ss = fmaf(v, v, ss);
            }
            partial[r * kThreads + tid] = ss;
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const float total = tree_sum_256(partial + r * kThreads, lane);
            const float inv = rsqrtf(total / static_cast<float>(in_features) + eps);
            const bf16* xr = input + (size_t)r * in_features;
            for (int i = tid, u = 0; i < in_features; i += kThreads, ++u) {
                const float normalized = rbf(bf2f(xr[i]) * inv);
                bf16 nw;
                if (nw_ready) {
                    nw = nw_pre[0];
#pragma unroll
                    for (int k = 1; k < kNormPre; ++k) nw = (u == k) ? nw_pre[NORM ? k : 0] : nw;
                } else {
                    nw = norm_w[i];
                }
                const bf16 o = f2bf(normalized * bf2f(nw));
                xs[(size_t)r * in_features + i] = o;
                if (norm_out != nullptr && blockIdx.x == 0) norm_out[(size_t)r * in_features + i] = o;
            }
        }
    } else {
        const int4* src = reinterpret_cast<const int4*>(input);
        int4* dst = reinterpret_cast<int4*>(xs);
        const int count = ROWS * in_features / 8;
        for (int i = tid; i < count; i += kThreads) dst[i] = src[i];
    }
    __syncthreads();

    const int4* xs4 = reinterpret_cast<const int4*>(xs);
    const int row_vec = in_features / 8;   // int4 per activation row

    for (int channel = first_channel; channel < out_features; channel += total_warps) {
        const int4* wrow = reinterpret_cast<const int4*>(weight + (size_t)channel * in_features);
        const int4* urow = reinterpret_cast<const int4*>(
            weight + ((size_t)out_features + channel) * in_features);
        float acc[ROWS];
        float acc_up[GATEUP ? ROWS : 1];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            acc[r] = 0.0f;
            if (GATEUP) acc_up[r] = 0.0f;
        }
        for (int v0 = lane; v0 < vectors; v0 += kPre * kWarp) {
            int4 wv[GATEUP ? 2 : 1][kPre];
            const bool use_pre = (channel == first_channel) && (v0 == lane);
#pragma unroll
            for (int u = 0; u < kPre; ++u) {
                const int v = v0 + u * kWarp;
                if (v < vectors) {
                    if (use_pre) {
                        wv[0][u] = pre[0][u];
                        if (GATEUP) wv[GATEUP ? 1 : 0][u] = pre[GATEUP ? 1 : 0][u];
                    } else {
                        wv[0][u] = ld_stream(wrow + v);
                        if (GATEUP) wv[GATEUP ? 1 : 0][u] = ld_stream(urow + v);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < kPre; ++u) {
                const int v = v0 + u * kWarp;
                if (v < vectors) {
#pragma unroll
                    for (int r = 0; r < ROWS; ++r) {
                        const int4 xa = xs4[r * row_vec + 2 * v];
                        const int4 xb = xs4[r * row_vec + 2 * v + 1];
                        acc[r] += dot16(wv[0][u], xa, xb);
                        if (GATEUP) acc_up[r] += dot16(wv[GATEUP ? 1 : 0][u], xa, xb);
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const float a = warp_sum_down(acc[r]);
            float b = 0.0f;
            if (GATEUP) b = warp_sum_down(acc_up[r]);
            if (lane == 0) {
                const size_t o = (size_t)r * out_features + channel;
                const bool first = channel == first_channel;
                const float scale = first ? pre_scale : scales[channel];
                if (GATEUP) {
                    const float gate = a * scale;
                    const float up = b * (first ? pre_scale_up : scales[out_features + channel]);
                    const float activated = gate / (1.0f + expf(-gate));
                    const float val = activated * up;
                    if (output32 != nullptr) output32[o] = val;
                    output[o] = f2bf(val);
                } else if (epilogue == EPI_PLAIN) {
                    const float val = a * scale;
                    if (output32 != nullptr) output32[o] = val;
                    output[o] = f2bf(val);
                } else if (epilogue == EPI_ADD) {
                    const float base = (first && resid_ready) ? pre_resid[r] : bf2f(output[o]);
                    const float val = fmaf(a, scale, base);
                    if (output32 != nullptr) output32[o] = val;
                    output[o] = f2bf(val);
                } else if (epilogue == EPI_BIAS) {
                    const float val = rbf(a * scale) + bf2f(bias[channel]);
                    if (output32 != nullptr) output32[o] = val;
                    output[o] = f2bf(val);
                } else if (epilogue == EPI_BIAS_SILU) {
                    float val = rbf(a * scale) + bf2f(bias[channel]);
                    val *= 1.0f / (1.0f + expf(-val));
                    if (output32 != nullptr) output32[o] = val;
                    output[o] = f2bf(val);
                } else {  // EPI_BIAS_ADD
                    const float t = rbf(rbf(a * scale) + bf2f(bias[channel]));
                    const float val = ((first && resid_ready) ? pre_resid[r] : bf2f(resid[o])) + t;
                    if (output32 != nullptr) output32[o] = val;
                    resid[o] = f2bf(val);
                }
            }
        }
    }
}

constexpr int kMaxInFeatures = 8192;   // 8 rows x 8192 x bf16 = 128 KB of staged activations

template <int ROWS, bool GATEUP, bool NORM>
cudaError_t configure_one() {
    cudaError_t e = cudaFuncSetAttribute(gemv_rows_kernel<ROWS, GATEUP, NORM>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         ROWS * kMaxInFeatures * static_cast<int>(sizeof(bf16)));
    if constexpr (ROWS == 1 && !GATEUP) {
        if (e == cudaSuccess) {
            e = cudaFuncSetAttribute(gemv_rows_kernel<ROWS, GATEUP, NORM, 12>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     ROWS * kMaxInFeatures * static_cast<int>(sizeof(bf16)));
        }
    }
    return e;
}

template <bool GATEUP, bool NORM>
cudaError_t configure_rows() {
    cudaError_t e = configure_one<1, GATEUP, NORM>();
    if (e == cudaSuccess) e = configure_one<2, GATEUP, NORM>();
    if (e == cudaSuccess) e = configure_one<3, GATEUP, NORM>();
    if (e == cudaSuccess) e = configure_one<4, GATEUP, NORM>();
    if (e == cudaSuccess) e = configure_one<5, GATEUP, NORM>();
    if (e == cudaSuccess) e = configure_one<6, GATEUP, NORM>();
    if (e == cudaSuccess) e = configure_one<7, GATEUP, NORM>();
    if (e == cudaSuccess) e = configure_one<8, GATEUP, NORM>();
    return e;
}

template <int ROWS, bool GATEUP, bool NORM, int KPRE = 4>
cudaError_t launch_one(const GemvArgs& a, const bf16* x, bf16* y, float* y32, bf16* norm_out,
                       bf16* resid, cudaStream_t stream) {
    if constexpr (ROWS == 1 && !GATEUP && KPRE == 4) {
        if (a.in_features > 2048) {
            return launch_one<ROWS, GATEUP, NORM, 12>(a, x, y, y32, norm_out, resid, stream);
        }
    }
    const size_t smem = (size_t)ROWS * a.in_features * sizeof(bf16);
    auto kernel = gemv_rows_kernel<ROWS, GATEUP, NORM, KPRE>;
    int grid = (a.out_features + kWarps - 1) / kWarps;
    const int cap = 148 * 8;
    if (grid > cap) grid = cap;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, a.w, a.scales, x, y, y32, a.norm_w, norm_out, a.bias, resid,
                              a.in_features, a.out_features, a.epilogue, a.eps, a.residual_settled ? 1 : 0);
}

template <bool GATEUP, bool NORM>
cudaError_t launch_rows(const GemvArgs& a, int rows, const bf16* x, bf16* y, float* y32,
                        bf16* norm_out, bf16* resid, cudaStream_t s) {
    switch (rows) {
        case 1: return launch_one<1, GATEUP, NORM>(a, x, y, y32, norm_out, resid, s);
        case 2: return launch_one<2, GATEUP, NORM>(a, x, y, y32, norm_out, resid, s);
        case 3: return launch_one<3, GATEUP, NORM>(a, x, y, y32, norm_out, resid, s);
        case 4: return launch_one<4, GATEUP, NORM>(a, x, y, y32, norm_out, resid, s);
        case 5: return launch_one<5, GATEUP, NORM>(a, x, y, y32, norm_out, resid, s);
        case 6: return launch_one<6, GATEUP, NORM>(a, x, y, y32, norm_out, resid, s);
        case 7: return launch_one<7, GATEUP, NORM>(a, x, y, y32, norm_out, resid, s);
        default: return launch_one<8, GATEUP, NORM>(a, x, y, y32, norm_out, resid, s);
    }
}

}  // namespace

// Raises the dynamic shared-memory ceiling of every instantiation on the current device.
// Done once per device up front (never inside a stream capture).
cudaError_t configure_gemv_kernels() {
    cudaError_t e = configure_rows<false, false>();
    if (e == cudaSuccess) e = configure_rows<false, true>();
    if (e == cudaSuccess) e = configure_rows<true, false>();
    if (e == cudaSuccess) e = configure_rows<true, true>();
    return e;
}

// overlap of a kernel's preamble with the tail of the kernel before it
bool pdl_enabled() {
    static const bool on = [] {
        const char* v = std::getenv("QWEN3_TTS_PDL");
        return v == nullptr || *v != '0';
    }();
    return on;
}

namespace {
// 0: SIMT only, 1: int8 tensor-core GEMV where it applies (default)
int g_gemv_mode = [] {
    const char* v = std::getenv("QWEN3_TTS_B1_GEMV");
    if (v != nullptr && std::strcmp(v, "simt") == 0) return 0;
    return 1;
}();
}  // namespace

int set_gemv_mode(int mode) {
    const int before = g_gemv_mode;
    if (mode == 0 || mode == 1) g_gemv_mode = mode;
    return before;
}
int gemv_mode() { return g_gemv_mode; }

// Which kernel takes a projection:
//   9..64 rows, K a multiple of 128     tcgen05 kernel (gemm_int8_tc.cu)
//   1..8 rows, K = 512 * {2,4,6,12}     int8 mma.sync kernel (gemv_int8_mma.cu): weights bulk-copied ahead of
//                                       the dependency wait, exact integer sums, 1e-7-level agreement with fp64
//   everything else, or gemv mode 0     SIMT kernel below, which keeps the reference's summation order
//                                       bit for bit (mode 0 is for callers that need exactly that)
cudaError_t launch_int8_gemm(const GemvArgs& a, cudaStream_t stream) {
    if (gemm_tc_supports(a)) return launch_int8_gemm_tc(a, stream);
    if (g_gemv_mode == 1 && gemv_mma_supports(a)) return launch_int8_gemv_mma(a, stream);
    return launch_int8_gemm_simt(a, stream);
}

cudaError_t launch_int8_gemm_simt(const GemvArgs& a, cudaStream_t stream) {
    if (a.in_features <= 0 || a.in_features % kVecBytes != 0 || a.in_features > kMaxInFeatures
        || a.out_features <= 0 || a.rows < 1
        || a.rows > kMaxRows || a.w == nullptr || a.scales == nullptr || a.x == nullptr) {
        return cudaErrorInvalidValue;
    }
    const bool gateup = a.epilogue == EPI_GATE_UP_SILU;
    const bool norm = a.norm_w != nullptr;
    if (a.epilogue == EPI_BIAS_ADD ? (a.resid == nullptr) : (a.y == nullptr)) return cudaErrorInvalidValue;
    if ((a.epilogue == EPI_BIAS || a.epilogue == EPI_BIAS_SILU || a.epilogue == EPI_BIAS_ADD)
        && a.bias == nullptr) {
        return cudaErrorInvalidValue;
    }
    // More than 8 rows: passes of 8 rows each over the same weights.
    for (int r0 = 0; r0 < a.rows; r0 += 8) {
        const int rows = a.rows - r0 < 8 ? a.rows - r0 : 8;
        const bf16* x = a.x + (size_t)r0 * a.in_features;
        bf16* y = a.y ? a.y + (size_t)r0 * a.out_features : nullptr;
        float* y32 = a.y32 ? a.y32 + (size_t)r0 * a.out_features : nullptr;
        bf16* no = a.norm_out ? a.norm_out + (size_t)r0 * a.in_features : nullptr;
        bf16* rs = a.resid ? a.resid + (size_t)r0 * a.out_features : nullptr;
        cudaError_t e;
        if (gateup) {
            e = norm ? launch_rows<true, true>(a, rows, x, y, y32, no, rs, stream)
                     : launch_rows<true, false>(a, rows, x, y, y32, no, rs, stream);
        } else {
            e = norm ? launch_rows<false, true>(a, rows, x, y, y32, no, rs, stream)
                     : launch_rows<false, false>(a, rows, x, y, y32, no, rs, stream);
        }
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

// ------------------------------------------------------------------ load-time quantizer
// Per-output-channel symmetric int8 quantization of a bf16 weight row, the arithmetic of the
// reference's quantize_weight_rows_kernel (int8_gemv.cu:20-52): scale = absmax/127 (1 for an
// all-zero row), q = lrintf(clamp(w * (1/scale), -127, 127)).  max is exact in any order.
namespace {
__global__ void __launch_bounds__(kThreads)
quantize_rows_kernel(const bf16* __restrict__ weight, int8_t* __restrict__ q,
                     float* __restrict__ scales, int in_features) {
    __shared__ float warp_max[kWarps];
    const size_t off = (size_t)blockIdx.x * in_features;
    const bf16* row = weight + off;
    float m = 0.0f;
    for (int i = threadIdx.x; i < in_features; i += kThreads) m = fmaxf(m, fabsf(bf2f(row[i])));
    m = warp_max_xor(m);
    if (threadIdx.x % kWarp == 0) warp_max[threadIdx.x / kWarp] = m;
    __syncthreads();
    float total = warp_max[0];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) total = fmaxf(total, warp_max[w]);
    const float scale = total > 0.0f ? total / 127.0f : 1.0f;
    const float inverse = 1.0f / scale;
    if (threadIdx.x == 0) scales[blockIdx.x] = scale;
    for (int i = threadIdx.x; i < in_features; i += kThreads) {
        const float v = bf2f(row[i]) * inverse;
        const float c = fminf(fmaxf(v, -127.0f), 127.0f);
        q[off + i] = static_cast<int8_t>(lrintf(c));
    }
}
}  // namespace

cudaError_t launch_quantize_weight_rows(const bf16* weight, int8_t* quantized, float* scales,
                                        int in_features, int out_features, cudaStream_t stream) {
    if (in_features % kVecBytes != 0 || in_features <= 0 || out_features <= 0) {
        return cudaErrorInvalidValue;
    }
    quantize_rows_kernel<<<out_features, kThreads, 0, stream>>>(weight, quantized, scales,
                                                                in_features);
    return cudaGetLastError();
}

}  // namespace q3t
