// Stand-alone forms of the small row operators of the decode step.  The frame engine
// runs their fused forms (inside the GEMV prologue/epilogue and the attention kernel);
// these launchers exist so that every operator of the reference's
// native/qwen3-tts-native/native/src/talker_kernels.cu decode path has a directly
// testable counterpart built from the same device functions.

#include "q3t_kernels.cuh"

namespace q3t {
namespace {

constexpr int kThreads = 256;

// talker_kernels.cu:27-48 -- same per-thread strided fmaf sums and the same tree pairing
__global__ void __launch_bounds__(kThreads)
rms_norm_rows_kernel(const bf16* __restrict__ input, const bf16* __restrict__ weight,
                     bf16* __restrict__ output, int width, float eps) {
    // the norm weights are constants: requested before the wait for the rows' producer
    constexpr int kPre = 8;                              // widths up to 2048 stay in registers
    const bool in_registers = width <= kPre * kThreads;
    bf16 wpre[kPre];
    if (in_registers) {
#pragma unroll
        for (int u = 0; u < kPre; ++u) {
            const int i = threadIdx.x + u * kThreads;
            if (i < width) wpre[u] = weight[i];
        }
    }
    pdl_wait();
    pdl_trigger();
    __shared__ float partial[kThreads];
    const bf16* xr = input + (size_t)blockIdx.x * width;
    bf16* yr = output + (size_t)blockIdx.x * width;
    float ss = 0.0f;
    float xpre[kPre];
    if (in_registers) {
#pragma unroll
        for (int u = 0; u < kPre; ++u) {
            const int i = threadIdx.x + u * kThreads;
            xpre[u] = i < width ? bf2f(xr[i]) : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < kPre; ++u) {
            if (threadIdx.x + u * kThreads < width) ss = fmaf(xpre[u], xpre[u], ss);
        }
    } else {
        for (int i = threadIdx.x; i < width; i += kThreads) {
            const float v = bf2f(xr[i]);
            ss = fmaf(v, v, ss);
        }
    }
    partial[threadIdx.x] = ss;
    __syncthreads();
    const float total = tree_sum_256(partial, threadIdx.x % kWarp);
    const float inv = rsqrtf(total / static_cast<float>(width) + eps);
    if (in_registers) {
#pragma unroll
        for (int u = 0; u < kPre; ++u) {
            const int i = threadIdx.x + u * kThreads;
            if (i < width) {
                const float normalized = rbf(xpre[u] * inv);
                yr[i] = f2bf(normalized * bf2f(wpre[u]));
            }
        }
    } else {
        for (int i = threadIdx.x; i < width; i += kThreads) {
            const float normalized = rbf(bf2f(xr[i]) * inv);
            yr[i] = f2bf(normalized * bf2f(weight[i]));
        }
    }
}

// talker_kernels.cu:50-70, one warp per (row, head); head_dim in {32, 64, 128, 256}
__global__ void __launch_bounds__(kThreads)
head_rms_norm_kernel(bf16* __restrict__ values, const bf16* __restrict__ weight, int heads_total,
                     int head_dim, float eps) {
    const int lane = threadIdx.x % kWarp;
    const int head = blockIdx.x * (kThreads / kWarp) + threadIdx.x / kWarp;
    if (head >= heads_total) return;
    bf16* h = values + (size_t)head * head_dim;
    float x[8];
    float sq[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int d = lane + 32 * j;
        x[j] = d < head_dim ? bf2f(h[d]) : 0.0f;
        sq[j] = fmaf(x[j], x[j], 0.0f);
    }
    // slots d, d+128 | d+64, d+192 | d+32, d+160 | d+96, d+224 of the 256-slot tree
    const float a = (sq[0] + sq[4]) + (sq[2] + sq[6]);
    const float b = (sq[1] + sq[5]) + (sq[3] + sq[7]);
    float c = a + b;
    c = warp_sum_down(c);
    c = __shfl_sync(0xffffffffu, c, 0);
    const float inv = rsqrtf(c / static_cast<float>(head_dim) + eps);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int d = lane + 32 * j;
        if (d < head_dim) {
            const float normalized = rbf(x[j] * inv);
            h[d] = f2bf(normalized * bf2f(weight[d]));
        }
    }
}

// talker_kernels.cu:597-639
__global__ void rope_rows_at_kernel(bf16* __restrict__ values, int rows, int heads, int head_dim,
                                    const int* __restrict__ positions, float theta) {
    const int half = head_dim / 2;
    const int pair = blockIdx.x * blockDim.x + threadIdx.x;
    const int row_pairs = heads * half;
    if (pair >= rows * row_pairs) return;
    const int row = pair / row_pairs;
    const int head = (pair % row_pairs) / half;
    const int d = pair % half;
    bf16* base = values + ((size_t)row * heads + head) * head_dim;
    const float angle = static_cast<float>(positions[row]) * rope_inv_freq(d, head_dim, theta);
    float o1, o2;
    rope_pair(bf2f(base[d]), bf2f(base[d + half]), angle, o1, o2);
    base[d] = f2bf(o1);
    base[d + half] = f2bf(o2);
}

// talker_kernels.cu:641-658
__global__ void kv_scatter_rows_kernel(const bf16* __restrict__ rows_data, bf16* const* cache_bases,
                                       const int* __restrict__ positions, int rows, int width) {
    const int index = blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= rows * width) return;
    const int row = index / width;
    const int col = index % width;
    cache_bases[row][(size_t)positions[row] * width + col] = rows_data[(size_t)row * width + col];
}

// talker_kernels.cu:660-678
__global__ void bias_activation_rows_kernel(bf16* __restrict__ values, const bf16* __restrict__ bias,
                                            int total, int width, bool silu) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += blockDim.x * gridDim.x) {
        float v = bf2f(values[i]) + bf2f(bias[i % width]);
        if (silu) v *= 1.0f / (1.0f + expf(-v));
        values[i] = f2bf(v);
    }
}

// talker_kernels.cu:359-371
__global__ void add_in_place_kernel(bf16* __restrict__ dst, const bf16* __restrict__ src, int count) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += blockDim.x * gridDim.x) {
        dst[i] = f2bf(bf2f(dst[i]) + bf2f(src[i]));
    }
}

// talker_kernels.cu:405-421 (unfused form: silu(g) is rounded to bf16 before the product)
__global__ void silu_gate_kernel(bf16* __restrict__ gate, const bf16* __restrict__ up, int count) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += blockDim.x * gridDim.x) {
        const float g = bf2f(gate[i]);
        const float activated = rbf(g / (1.0f + expf(-g)));
        gate[i] = f2bf(activated * bf2f(up[i]));
    }
}

// talker_kernels.cu:680-709
__global__ void gather_embedding_rows_kernel(const bf16* __restrict__ table, int vocabulary,
                                             int width, const int* const* tokens, int token_offset,
                                             bf16* __restrict__ output, int rows, bool add) {
    const int total = rows * width;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += blockDim.x * gridDim.x) {
        const int row = i / width;
        const int col = i % width;
        const int token = tokens[row][token_offset];
        if (token < 0 || token >= vocabulary) continue;
        const bf16 v = table[(size_t)token * width + col];
        output[i] = add ? f2bf(bf2f(output[i]) + bf2f(v)) : v;
    }
}

// sampling_kernels.cu:421-426
__global__ void pack_frame_codes_rows_kernel(const int* const* tokens,
                                             unsigned short* const* codes, int rows) {
    const int row = blockIdx.x;
    if (row < rows && threadIdx.x < kCodebooks) {
        codes[row][threadIdx.x] = static_cast<unsigned short>(tokens[row][threadIdx.x]);
    }
}

int blocks_for(int n) {
    int b = (n + kThreads - 1) / kThreads;
    return b < 1 ? 1 : (b > 4096 ? 4096 : b);
}

}  // namespace

cudaError_t launch_rms_norm_rows(const bf16* input, const bf16* weight, bf16* output, int rows,
                                 int width, float eps, cudaStream_t stream) {
    if (rows < 1 || width < 1) return cudaErrorInvalidValue;
    return launch_pdl(rms_norm_rows_kernel, dim3(rows), dim3(kThreads), 0, stream, input, weight, output, width,
                      eps);
}

cudaError_t launch_head_rms_norm_rows(bf16* values, const bf16* weight, int rows, int heads,
                                      int head_dim, float eps, cudaStream_t stream) {
    if (rows < 1 || heads < 1 || head_dim < 1 || head_dim > 256) return cudaErrorInvalidValue;
    const int total = rows * heads;
    const int per_block = kThreads / kWarp;
    head_rms_norm_kernel<<<(total + per_block - 1) / per_block, kThreads, 0, stream>>>(
        values, weight, total, head_dim, eps);
    return cudaGetLastError();
}

cudaError_t launch_rope_rows_at(bf16* values, int rows, int heads, int head_dim,
                                const int* positions, float theta, cudaStream_t stream) {
    if (rows < 1 || heads < 1 || head_dim < 2 || head_dim % 2 != 0) return cudaErrorInvalidValue;
    const int pairs = rows * heads * (head_dim / 2);
    rope_rows_at_kernel<<<(pairs + kThreads - 1) / kThreads, kThreads, 0, stream>>>(
        values, rows, heads, head_dim, positions, theta);
    return cudaGetLastError();
}

cudaError_t launch_kv_scatter_rows(const bf16* rows_data, bf16* const* cache_bases,
                                   const int* positions, int rows, int width, cudaStream_t stream) {
    if (rows < 1 || width < 1) return cudaErrorInvalidValue;
    const int total = rows * width;
    kv_scatter_rows_kernel<<<(total + kThreads - 1) / kThreads, kThreads, 0, stream>>>(
        rows_data, cache_bases, positions, rows, width);
    return cudaGetLastError();
}

cudaError_t launch_bias_activation_rows(bf16* values, const bf16* bias, int rows, int width,
                                        bool silu, cudaStream_t stream) {
    if (rows < 1 || width < 1) return cudaErrorInvalidValue;
    bias_activation_rows_kernel<<<blocks_for(rows * width), kThreads, 0, stream>>>(
        values, bias, rows * width, width, silu);
    return cudaGetLastError();
}

cudaError_t launch_add_in_place(bf16* destination, const bf16* source, int count,
                                cudaStream_t stream) {
    if (count < 1) return cudaErrorInvalidValue;
    add_in_place_kernel<<<blocks_for(count), kThreads, 0, stream>>>(destination, source, count);
    return cudaGetLastError();
}

cudaError_t launch_silu_gate(bf16* gate, const bf16* up, int count, cudaStream_t stream) {
    if (count < 1) return cudaErrorInvalidValue;
    silu_gate_kernel<<<blocks_for(count), kThreads, 0, stream>>>(gate, up, count);
    return cudaGetLastError();
}

cudaError_t launch_gather_embedding_rows(const bf16* table, int vocabulary, int width,
                                         const int* const* tokens, int token_offset, bf16* output,
                                         int rows, bool add, cudaStream_t stream) {
    if (rows < 1 || width < 1) return cudaErrorInvalidValue;
    gather_embedding_rows_kernel<<<blocks_for(rows * width), kThreads, 0, stream>>>(
        table, vocabulary, width, tokens, token_offset, output, rows, add);
    return cudaGetLastError();
}

cudaError_t launch_pack_frame_codes_rows(const int* const* tokens, unsigned short* const* codes,
                                         int rows, cudaStream_t stream) {
    if (rows < 1) return cudaErrorInvalidValue;
    pack_frame_codes_rows_kernel<<<rows, 32, 0, stream>>>(tokens, codes, rows);
    return cudaGetLastError();
}

}  // namespace q3t
