// A chain of dependent batch-1 int8 GEMVs in one persistent, cooperative launch.
//
// A decode step at batch 1 is a string of small matrix-vector products (attention output, gate/up,
// down, the next layer's q/k/v ...), each reading the vector the previous one wrote.  As separate
// launches every one of them pays the launch, an empty memory pipe at its start and a drained one
// at its end.  Here one grid (as many CTAs as the device holds at once) walks the whole chain:
//
//   for each op:   request the first weight vectors of my channels      (weights never depend
//                                                                          on the previous op)
//                  grid barrier: the previous op's output is complete
//                  stage the activation row in shared memory (RMSNorm if asked), as fp32 pairs
//                  every warp: one output channel at a time, weight vectors through a register
//                  ring that is refilled across channel boundaries
//
// so the weight stream of op i+1 is already in flight while op i finishes and the barrier runs.
//
// Arithmetic is that of the single-launch SIMT kernel (gemv_int8.cu), which is the reference's
// (int8_gemv.cu:58-293): lane l owns the 16-byte vectors l, l+32, ... of a weight row, 16
// sequential FMAs per vector, vector sums added to the lane accumulator in vector order, a
// shuffle-down tree, the same epilogues; so results are bit-identical to it.  What differs is how
// the FMAs are issued: two vectors of a lane advance together in one fma.rn.f32x2 (each half is an
// ordinary fp32 FMA), int8 -> fp32 goes through PRMT into the mantissa of 2^23 and a packed
// subtract (exact) instead of integer-to-float conversions, and the activations are staged
// already widened and interleaved for that pairing.
//
// The grid barrier is a counter in global memory; every wait on it is bounded (about a second),
// after which the kernel records an error and carries on to its end without waiting again.

#include "q3t_kernels.cuh"

#include <mutex>

namespace q3t {
namespace {

constexpr int kChainThreads = 512;
constexpr int kChainWarps = kChainThreads / kWarp;
constexpr int kMaxChainK = 6144;
constexpr int kRing = 4;                     // weight units in flight per warp
constexpr long long kBarrierBudgetCycles = 2000000000ll;   // ~1 s at 2 GHz

struct ChainOp {
    const int8_t* w;
    const float* scales;
    const bf16* x;
    bf16* y;
    float* y32;
    const bf16* norm_w;
    bf16* norm_out;
    const bf16* bias;
    bf16* resid;
    int in_features;
    int out_features;
    int epilogue;
    float eps;
};

struct ChainParams {
    ChainOp ops[kMaxChainOps];
    int count;
    unsigned int* sync;      // [0] barrier arrivals, [1] exit tickets, [2] errors
};

__device__ __forceinline__ unsigned int ld_acquire(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// All CTAs of the grid meet; `target` = arrivals expected so far.  Returns false once the budget
// has run out anywhere (the caller stops waiting for the rest of the kernel).
__device__ __forceinline__ bool grid_barrier(unsigned int* sync, unsigned int target, int* gave_up) {
    __syncthreads();
    if (threadIdx.x == 0) {
        if (*gave_up == 0) {
            __threadfence();
            atomicAdd(&sync[0], 1u);
            const long long start = clock64();
            while (ld_acquire(&sync[0]) < target) {
                if (clock64() - start > kBarrierBudgetCycles) {
                    atomicAdd(&sync[2], 1u);
                    *gave_up = 1;
                    break;
                }
            }
            __threadfence();
        }
    }
    __syncthreads();
    return *gave_up == 0;
}

__global__ void __launch_bounds__(kChainThreads, 1)
gemv_chain_kernel(const __grid_constant__ ChainParams p) {
    __shared__ __align__(16) float xs[kMaxChainK];      // staged activations, paired layout
    __shared__ __align__(16) bf16 raw[kMaxChainK];      // the row as it is in memory
    __shared__ float partial[256];
    __shared__ int gave_up;

    const int tid = threadIdx.x;
    const int lane = tid % kWarp;
    const int warp = tid / kWarp;
    const int total_warps = gridDim.x * kChainWarps;
    const int first_channel = blockIdx.x * kChainWarps + warp;
    if (tid == 0) gave_up = 0;
    __syncthreads();

    for (int op_index = 0; op_index < p.count; ++op_index) {
        const ChainOp& op = p.ops[op_index];
        const int K = op.in_features;
        const int N = op.out_features;
        const bool gateup = op.epilogue == EPI_GATE_UP_SILU;
        // a unit = two vectors per lane of one weight row; a gate/up channel is two rows (gate, then up)
        const int units_per_row = K / 1024;
        const int units_per_channel = gateup ? 2 * units_per_row : units_per_row;
        const int my_channels = first_channel < N ? (N - first_channel + total_warps - 1) / total_warps : 0;
        const int total_units = my_channels * units_per_channel;
        const size_t row_vectors = (size_t)K / 16;

        // weight address of unit u of this warp: vectors lane + 64 jp and lane + 64 jp + 32
        auto unit_ptr = [&](int u) -> const int4* {
            const int ci = u / units_per_channel;
            int jp = u - ci * units_per_channel;
            size_t row = (size_t)first_channel + (size_t)ci * total_warps;
            if (jp >= units_per_row) {
                jp -= units_per_row;
                row += (size_t)N;
            }
            return reinterpret_cast<const int4*>(op.w) + row * row_vectors + 64 * jp + lane;
        };

        // ---- the first units go out before anything that depends on the previous op ----------
        int4 ring[kRing][2];
#pragma unroll
        for (int d = 0; d < kRing; ++d) {
            if (d < total_units) {
                const int4* src = unit_ptr(d);
                ring[d][0] = ld_stream(src);
                ring[d][1] = ld_stream(src + 32);
            }
        }

        if (op_index > 0) grid_barrier(p.sync, (unsigned int)op_index * gridDim.x, &gave_up);

        // ---- stage the activation row: one trip to L2 for the raw bf16 row, then fp32,
        // interleaved for the vector pairing ------------------------------------------------------
        {
            const int4* src = reinterpret_cast<const int4*>(op.x);
            int4* dst = reinterpret_cast<int4*>(raw);
            for (int i = tid; i < K / 8; i += kChainThreads) dst[i] = __ldcg(src + i);
        }
        __syncthreads();
        float inv = 1.0f;
        if (op.norm_w != nullptr) {
            // the reference's sum of squares: 256 strided partials, then a halving tree
            if (tid < 256) {
                float ss = 0.0f;
                for (int i = tid; i < K; i += 256) {
                    const float v = bf2f(raw[i]);
                    ss = fmaf(v, v, ss);
                }
                partial[tid] = ss;
            }
            __syncthreads();
            const float total = tree_sum_256(partial, lane);
            inv = rsqrtf(total / static_cast<float>(K) + op.eps);
        }
        for (int e = tid; e < K; e += kChainThreads) {
            float v = bf2f(raw[e]);
            if (op.norm_w != nullptr) {
                const float normalized = rbf(v * inv);
                const bf16 o = f2bf(normalized * bf2f(op.norm_w[e]));
                if (op.norm_out != nullptr && blockIdx.x == 0) op.norm_out[e] = o;
                v = bf2f(o);
            }
            xs[paired_index(e)] = v;
        }
        __syncthreads();

        // ---- channels ---------------------------------------------------------------------------
        const float4* xs4 = reinterpret_cast<const float4*>(xs) + lane;
        float acc = 0.0f, gate_sum = 0.0f;
        int jp = 0;
        int channel = first_channel;
        for (int u0 = 0; u0 < total_units; u0 += kRing) {
#pragma unroll
            for (int d = 0; d < kRing; ++d) {
                const int u = u0 + d;
                if (u < total_units) {
                    const int4 wa = ring[d][0], wb = ring[d][1];
                    if (u + kRing < total_units) {
                        const int4* src = unit_ptr(u + kRing);
                        ring[d][0] = ld_stream(src);
                        ring[d][1] = ld_stream(src + 32);
                    }
                    const int jx = jp >= units_per_row ? jp - units_per_row : jp;
                    float sa, sb;
                    dot16_pair(wa, wb, xs4 + jx * 8 * kWarp, sa, sb);
                    acc += sa;
                    acc += sb;
                    ++jp;
                    if (gateup && jp == units_per_row) {
                        gate_sum = warp_sum_down(acc);      // the gate row is complete; the up row follows
                        acc = 0.0f;
                    }
                    if (jp == units_per_channel) {
                        // ---- channel complete: fold the lanes, epilogue on lane 0 ----------------
                        const float folded = warp_sum_down(acc);
                        const float a = gateup ? gate_sum : folded;
                        const float b = folded;
                        if (lane == 0) {
                            const size_t o = (size_t)channel;
                            float val;
                            if (gateup) {
                                const float gate = a * op.scales[channel];
                                const float up = b * op.scales[N + channel];
                                const float activated = gate / (1.0f + expf(-gate));
                                val = activated * up;
                                op.y[o] = f2bf(val);
                            } else if (op.epilogue == EPI_PLAIN) {
                                val = a * op.scales[channel];
                                op.y[o] = f2bf(val);
                            } else if (op.epilogue == EPI_ADD) {
                                val = fmaf(a, op.scales[channel], bf2f(op.y[o]));
                                op.y[o] = f2bf(val);
                            } else if (op.epilogue == EPI_BIAS) {
                                val = rbf(a * op.scales[channel]) + bf2f(op.bias[channel]);
                                op.y[o] = f2bf(val);
                            } else if (op.epilogue == EPI_BIAS_SILU) {
                                val = rbf(a * op.scales[channel]) + bf2f(op.bias[channel]);
                                val *= 1.0f / (1.0f + expf(-val));
                                op.y[o] = f2bf(val);
                            } else {  // EPI_BIAS_ADD
                                const float t = rbf(rbf(a * op.scales[channel]) + bf2f(op.bias[channel]));
                                val = bf2f(op.resid[o]) + t;
                                op.resid[o] = f2bf(val);
                            }
                            if (op.y32 != nullptr) op.y32[o] = val;
                        }
                        acc = 0.0f;
                        jp = 0;
                        channel += total_warps;
                    }
                }
            }
        }
        __syncthreads();     // the staged row is rewritten by the next op
    }

    // ---- leave the counters at zero for the next launch: the last CTA out resets them ----------
    if (tid == 0) {
        __threadfence();
        const unsigned int ticket = atomicAdd(&p.sync[1], 1u);
        if (ticket == gridDim.x - 1) {
            p.sync[0] = 0u;
            p.sync[1] = 0u;
            __threadfence();
        }
    }
}

struct ChainDevice {
    unsigned int* sync = nullptr;     // default counters of the operator-level entry point
    int grid = 0;
    bool ready = false;
};
ChainDevice g_chain[64];
std::mutex g_chain_guard;

ChainDevice* chain_for_current_device() {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return nullptr;
    return g_chain[device].ready ? &g_chain[device] : nullptr;
}

}  // namespace

cudaError_t configure_gemv_chain_kernels() {
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_chain_guard);
    ChainDevice& c = g_chain[device];
    if (c.ready) return cudaSuccess;
    int per_sm = 0, sms = 0, cooperative = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemv_chain_kernel, kChainThreads, 0);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&cooperative, cudaDevAttrCooperativeLaunch, device);
    if (e != cudaSuccess) return e;
    if (per_sm < 1 || sms < 1 || cooperative == 0) return cudaErrorNotSupported;
    e = cudaMalloc(&c.sync, kChainSyncWords * sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMemset(c.sync, 0, kChainSyncWords * sizeof(unsigned int));
    if (e != cudaSuccess) return e;
    c.grid = per_sm * sms;
    c.ready = true;
    return cudaSuccess;
}

bool gemv_chain_supports(const GemvArgs& a) {
    if (a.rows != 1 || a.in_features < 1024 || a.in_features > kMaxChainK || a.in_features % 1024 != 0) return false;
    if (a.out_features < 1 || a.w == nullptr || a.scales == nullptr || a.x == nullptr) return false;
    if ((reinterpret_cast<uintptr_t>(a.w) & 15u) != 0) return false;
    if (a.epilogue == EPI_BIAS_ADD ? a.resid == nullptr : a.y == nullptr) return false;
    if ((a.epilogue == EPI_BIAS || a.epilogue == EPI_BIAS_SILU || a.epilogue == EPI_BIAS_ADD) && a.bias == nullptr) return false;
    return chain_for_current_device() != nullptr;
}

cudaError_t launch_gemv_chain(const GemvArgs* ops, int count, unsigned int* sync, cudaStream_t stream) {
    ChainDevice* dev = chain_for_current_device();
    if (dev == nullptr || ops == nullptr || count < 1 || count > kMaxChainOps) return cudaErrorInvalidValue;
    ChainParams p;
    for (int i = 0; i < count; ++i) {
        if (!gemv_chain_supports(ops[i])) return cudaErrorInvalidValue;
        ChainOp& o = p.ops[i];
        o.w = ops[i].w; o.scales = ops[i].scales; o.x = ops[i].x; o.y = ops[i].y; o.y32 = ops[i].y32;
        o.norm_w = ops[i].norm_w; o.norm_out = ops[i].norm_out; o.bias = ops[i].bias; o.resid = ops[i].resid;
        o.in_features = ops[i].in_features; o.out_features = ops[i].out_features;
        o.epilogue = ops[i].epilogue; o.eps = ops[i].eps;
    }
    p.count = count;
    p.sync = sync != nullptr ? sync : dev->sync;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)dev->grid, 1, 1);
    cfg.blockDim = dim3(kChainThreads, 1, 1);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;      // all CTAs resident: the barrier needs it
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gemv_chain_kernel, p);
}

unsigned int gemv_chain_error_count() {
    ChainDevice* dev = chain_for_current_device();
    if (dev == nullptr) return 0u;
    unsigned int v = 0;
    if (cudaMemcpy(&v, dev->sync + 2, sizeof(v), cudaMemcpyDeviceToHost) != cudaSuccess) return ~0u;
    return v;
}

}  // namespace q3t
