// The entry points of the reference ABI that only its command-line tools use: the weight-upload
// arena and two bf16 microbenchmarks.  None of them is on the decode path; they are here so that
// the library resolves every symbol the reference's host looks up.
//
//   qwen3_tts_device_buffer_*          native/qwen3-tts-native/native/src/weights.cu:98-340
//   qwen3_tts_benchmark_bf16_argmax    runtime.cu:127-255
//   qwen3_tts_benchmark_bf16_gemv      gemv.cu:88-270 (cuBLAS there; an own kernel here)
//
// The arena differs from the reference in one respect: staging memory is used as two halves, so
// that the host copy of chunk i + 1 overlaps the transfer of chunk i.

#include "q3t_common.cuh"
#include "../../include/qwen3_tts_native.h"

#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <limits>
#include <new>
#include <vector>

struct Qwen3TtsDeviceBuffer {
    int device_index = 0;
    unsigned char* device_data = nullptr;
    unsigned char* staging = nullptr;       // pinned, two halves
    uint64_t capacity_bytes = 0;
    uint64_t staging_bytes = 0;
    uint64_t uploaded_bytes = 0;
    uint64_t upload_calls = 0;
    uint64_t free_before = 0, free_after = 0;
    double allocation_us = 0.0, upload_us = 0.0;
    cudaStream_t stream = nullptr;
    cudaEvent_t half_free[2] = {nullptr, nullptr};
};

namespace {

using q3t::bf16;

constexpr uint64_t kMaximumStagingBytes = 256ull << 20;

void say(char* error, size_t capacity, const char* message) {
    if (error == nullptr || capacity == 0) return;
    std::snprintf(error, capacity, "%s", message);
}

int32_t cuda_failure(cudaError_t status, const char* what, char* error, size_t capacity) {
    if (error != nullptr && capacity > 0) {
        std::snprintf(error, capacity, "%s failed: %s", what, cudaGetErrorString(status));
    }
    return static_cast<int32_t>(status);
}

void fill_metrics(const Qwen3TtsDeviceBuffer& b, Qwen3TtsWeightUploadMetrics* m) {
    std::memset(m, 0, sizeof(*m));
    m->device_index = b.device_index;
    m->allocation_bytes = b.capacity_bytes;
    m->pinned_staging_bytes = b.staging_bytes;
    m->uploaded_bytes = b.uploaded_bytes;
    m->upload_calls = b.upload_calls;
    m->free_before_bytes = b.free_before;
    m->free_after_allocation_bytes = b.free_after;
    m->allocation_microseconds = static_cast<float>(b.allocation_us);
    m->upload_microseconds = static_cast<float>(b.upload_us);
}

void release(Qwen3TtsDeviceBuffer* b) {
    if (b == nullptr) return;
    cudaSetDevice(b->device_index);
    if (b->stream != nullptr) cudaStreamSynchronize(b->stream);
    for (cudaEvent_t e : b->half_free) if (e != nullptr) cudaEventDestroy(e);
    if (b->staging != nullptr) cudaFreeHost(b->staging);
    if (b->device_data != nullptr) cudaFree(b->device_data);
    if (b->stream != nullptr) cudaStreamDestroy(b->stream);
    delete b;
}

// one block: largest logit, ties to the lower index
__global__ void __launch_bounds__(256) bf16_argmax_kernel(const bf16* logits, int count, int* selected) {
    __shared__ float best_value[8];
    __shared__ int best_index[8];
    float v = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < count; i += 256) {
        const float x = q3t::bf2f(logits[i]);
        if (x > v || (x == v && i < idx)) {
            v = x;
            idx = i;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) {
            v = ov;
            idx = oi;
        }
    }
    if (threadIdx.x % 32 == 0) {
        best_value[threadIdx.x / 32] = v;
        best_index[threadIdx.x / 32] = idx;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) {
            if (best_value[w] > v || (best_value[w] == v && best_index[w] < idx)) {
                v = best_value[w];
                idx = best_index[w];
            }
        }
        *selected = idx;
    }
}

// y[n] = sum_k W[n][k] x[k], bf16 operands, fp32 accumulate, one warp per output
__global__ void __launch_bounds__(256)
bf16_gemv_kernel(const bf16* __restrict__ w, const bf16* __restrict__ x, bf16* __restrict__ y, int in_features,
                 int out_features) {
    const int lane = threadIdx.x % 32;
    const int row = blockIdx.x * 8 + threadIdx.x / 32;
    if (row >= out_features) return;
    const bf16* wr = w + (size_t)row * in_features;
    float acc = 0.0f;
    if (in_features % 8 == 0) {
        const int4* w4 = reinterpret_cast<const int4*>(wr);
        const int4* x4 = reinterpret_cast<const int4*>(x);
        for (int v = lane; v < in_features / 8; v += 32) {
            const int4 a = q3t::ld_stream(w4 + v);
            const int4 b = x4[v];
            const uint32_t aw[4] = {(uint32_t)a.x, (uint32_t)a.y, (uint32_t)a.z, (uint32_t)a.w};
            const uint32_t bw[4] = {(uint32_t)b.x, (uint32_t)b.y, (uint32_t)b.z, (uint32_t)b.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                acc = fmaf(q3t::bf_lo(aw[q]), q3t::bf_lo(bw[q]), acc);
                acc = fmaf(q3t::bf_hi(aw[q]), q3t::bf_hi(bw[q]), acc);
            }
        }
    } else {
        for (int k = lane; k < in_features; k += 32) acc = fmaf(q3t::bf2f(wr[k]), q3t::bf2f(x[k]), acc);
    }
    acc = q3t::warp_sum_xor(acc);
    if (lane == 0) y[row] = q3t::f2bf(acc);
}

struct Scoped {
    void* p = nullptr;
    ~Scoped() { if (p != nullptr) cudaFree(p); }
};

}  // namespace

extern "C" {

int32_t qwen3_tts_device_buffer_create(int32_t device_index, uint64_t capacity_bytes, uint64_t staging_bytes,
                                       Qwen3TtsDeviceBuffer** output, Qwen3TtsWeightUploadMetrics* metrics,
                                       char* error, size_t error_capacity) {
    if (output == nullptr || metrics == nullptr) {
        say(error, error_capacity, "output buffer or metrics pointer is null");
        return -1;
    }
    *output = nullptr;
    std::memset(metrics, 0, sizeof(*metrics));
    if (capacity_bytes == 0 || capacity_bytes > static_cast<uint64_t>(std::numeric_limits<size_t>::max())) {
        say(error, error_capacity, "device capacity is zero or exceeds size_t");
        return -2;
    }
    if (staging_bytes == 0 || staging_bytes > kMaximumStagingBytes) {
        say(error, error_capacity, "staging capacity must be in [1, 256 MiB] and fit size_t");
        return -3;
    }
    cudaError_t status = cudaSetDevice(device_index);
    if (status != cudaSuccess) return cuda_failure(status, "cudaSetDevice", error, error_capacity);
    size_t free_bytes = 0, total_bytes = 0;
    status = cudaMemGetInfo(&free_bytes, &total_bytes);
    if (status != cudaSuccess) return cuda_failure(status, "cudaMemGetInfo(before)", error, error_capacity);
    Qwen3TtsDeviceBuffer* b = new (std::nothrow) Qwen3TtsDeviceBuffer();
    if (b == nullptr) {
        say(error, error_capacity, "failed to allocate device-buffer metadata");
        return -4;
    }
    b->device_index = device_index;
    b->capacity_bytes = capacity_bytes;
    b->staging_bytes = staging_bytes;
    b->free_before = free_bytes;
    const auto started = std::chrono::steady_clock::now();
    const char* what = "cudaStreamCreateWithFlags";
    status = cudaStreamCreateWithFlags(&b->stream, cudaStreamNonBlocking);
    if (status == cudaSuccess) {
        what = "cudaMalloc(weight arena)";
        status = cudaMalloc(reinterpret_cast<void**>(&b->device_data), static_cast<size_t>(capacity_bytes));
    }
    if (status == cudaSuccess) {
        what = "cudaHostAlloc(staging)";
        status = cudaHostAlloc(reinterpret_cast<void**>(&b->staging), static_cast<size_t>(staging_bytes),
                               cudaHostAllocDefault);
    }
    for (int h = 0; h < 2 && status == cudaSuccess; ++h) {
        what = "cudaEventCreate";
        status = cudaEventCreateWithFlags(&b->half_free[h], cudaEventDisableTiming);
    }
    if (status == cudaSuccess) {
        what = "cudaMemGetInfo(after)";
        status = cudaMemGetInfo(&free_bytes, &total_bytes);
    }
    if (status != cudaSuccess) {
        release(b);
        return cuda_failure(status, what, error, error_capacity);
    }
    b->free_after = free_bytes;
    b->allocation_us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - started).count();
    fill_metrics(*b, metrics);
    *output = b;
    say(error, error_capacity, "");
    return 0;
}

int32_t qwen3_tts_device_buffer_upload(Qwen3TtsDeviceBuffer* buffer, uint64_t offset_bytes, const void* source,
                                       uint64_t bytes, char* error, size_t error_capacity) {
    if (buffer == nullptr) {
        say(error, error_capacity, "device buffer is null");
        return -1;
    }
    if (bytes != 0 && source == nullptr) {
        say(error, error_capacity, "upload source is null");
        return -2;
    }
    if (offset_bytes != buffer->uploaded_bytes) {
        say(error, error_capacity, "uploads must be contiguous and sequential");
        return -3;
    }
    if (bytes > buffer->capacity_bytes - offset_bytes) {
        say(error, error_capacity, "upload exceeds device-buffer capacity");
        return -4;
    }
    cudaError_t status = cudaSetDevice(buffer->device_index);
    if (status != cudaSuccess) return cuda_failure(status, "cudaSetDevice", error, error_capacity);
    const auto started = std::chrono::steady_clock::now();
    const unsigned char* input = static_cast<const unsigned char*>(source);
    // two halves of the staging memory take turns: while one is in flight the other is filled
    const uint64_t half = buffer->staging_bytes >= 2 ? buffer->staging_bytes / 2 : buffer->staging_bytes;
    const int halves = buffer->staging_bytes >= 2 ? 2 : 1;
    uint64_t copied = 0;
    int turn = 0;
    bool used[2] = {false, false};
    while (copied < bytes) {
        const uint64_t chunk = std::min(half, bytes - copied);
        unsigned char* slot = buffer->staging + (size_t)turn * half;
        if (used[turn]) {
            status = cudaEventSynchronize(buffer->half_free[turn]);
            if (status != cudaSuccess) return cuda_failure(status, "cudaEventSynchronize(staging)", error, error_capacity);
        }
        std::memcpy(slot, input + copied, static_cast<size_t>(chunk));
        status = cudaMemcpyAsync(buffer->device_data + offset_bytes + copied, slot, static_cast<size_t>(chunk),
                                 cudaMemcpyHostToDevice, buffer->stream);
        if (status == cudaSuccess) status = cudaEventRecord(buffer->half_free[turn], buffer->stream);
        if (status != cudaSuccess) return cuda_failure(status, "cudaMemcpyAsync(weight chunk)", error, error_capacity);
        used[turn] = true;
        turn = (turn + 1) % halves;
        copied += chunk;
        buffer->upload_calls += 1;
    }
    status = cudaStreamSynchronize(buffer->stream);
    if (status != cudaSuccess) return cuda_failure(status, "cudaStreamSynchronize(upload)", error, error_capacity);
    buffer->upload_us += std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - started).count();
    buffer->uploaded_bytes += bytes;
    say(error, error_capacity, "");
    return 0;
}

int32_t qwen3_tts_device_buffer_finish(Qwen3TtsDeviceBuffer* buffer, Qwen3TtsWeightUploadMetrics* metrics,
                                       char* error, size_t error_capacity) {
    if (buffer == nullptr || metrics == nullptr) {
        say(error, error_capacity, "device buffer or metrics pointer is null");
        return -1;
    }
    if (buffer->uploaded_bytes != buffer->capacity_bytes) {
        say(error, error_capacity, "device buffer is not completely uploaded");
        return -2;
    }
    cudaSetDevice(buffer->device_index);
    const cudaError_t status = cudaStreamSynchronize(buffer->stream);
    if (status != cudaSuccess) return cuda_failure(status, "cudaStreamSynchronize(finish)", error, error_capacity);
    fill_metrics(*buffer, metrics);
    say(error, error_capacity, "");
    return 0;
}

int32_t qwen3_tts_device_buffer_read(Qwen3TtsDeviceBuffer* buffer, uint64_t offset_bytes, void* destination,
                                     uint64_t bytes, char* error, size_t error_capacity) {
    if (buffer == nullptr || (bytes != 0 && destination == nullptr)) {
        say(error, error_capacity, "device buffer or read destination is null");
        return -1;
    }
    if (offset_bytes > buffer->uploaded_bytes || bytes > buffer->uploaded_bytes - offset_bytes) {
        say(error, error_capacity, "read exceeds uploaded device-buffer range");
        return -2;
    }
    cudaError_t status = cudaSetDevice(buffer->device_index);
    if (status != cudaSuccess) return cuda_failure(status, "cudaSetDevice", error, error_capacity);
    unsigned char* out = static_cast<unsigned char*>(destination);
    uint64_t copied = 0;
    while (copied < bytes) {
        const uint64_t chunk = std::min(buffer->staging_bytes, bytes - copied);
        status = cudaMemcpyAsync(buffer->staging, buffer->device_data + offset_bytes + copied,
                                 static_cast<size_t>(chunk), cudaMemcpyDeviceToHost, buffer->stream);
        if (status == cudaSuccess) status = cudaStreamSynchronize(buffer->stream);
        if (status != cudaSuccess) return cuda_failure(status, "cudaMemcpyAsync(readback chunk)", error, error_capacity);
        std::memcpy(out + copied, buffer->staging, static_cast<size_t>(chunk));
        copied += chunk;
    }
    say(error, error_capacity, "");
    return 0;
}

const void* qwen3_tts_device_buffer_data(const Qwen3TtsDeviceBuffer* buffer) {
    return buffer == nullptr ? nullptr : buffer->device_data;
}

void qwen3_tts_device_buffer_destroy(Qwen3TtsDeviceBuffer* buffer) { release(buffer); }

int32_t qwen3_tts_benchmark_bf16_argmax(int32_t device_index, int32_t vocabulary_size, int32_t iterations,
                                        Qwen3TtsArgmaxBenchmark* output, char* error, size_t error_capacity) {
    if (output == nullptr) {
        say(error, error_capacity, "output benchmark pointer is null");
        return -1;
    }
    if (vocabulary_size <= 0 || vocabulary_size > 65536) {
        say(error, error_capacity, "vocabulary size must be in [1, 65536]");
        return -2;
    }
    if (iterations <= 0) {
        say(error, error_capacity, "iterations must be positive");
        return -3;
    }
    cudaError_t status = cudaSetDevice(device_index);
    if (status != cudaSuccess) return cuda_failure(status, "cudaSetDevice", error, error_capacity);
    const int expected = std::min(1729, vocabulary_size - 1);
    std::vector<bf16> host(static_cast<size_t>(vocabulary_size));
    for (int i = 0; i < vocabulary_size; ++i) host[i] = __float2bfloat16(static_cast<float>((i * 37) % 211) * 0.05f - 5.0f);
    host[expected] = __float2bfloat16(19.0f);
    Scoped logits, token;
    status = cudaMalloc(&logits.p, host.size() * sizeof(bf16));
    if (status == cudaSuccess) status = cudaMalloc(&token.p, sizeof(int));
    if (status == cudaSuccess) {
        status = cudaMemcpy(logits.p, host.data(), host.size() * sizeof(bf16), cudaMemcpyHostToDevice);
    }
    if (status != cudaSuccess) return cuda_failure(status, "argmax benchmark set-up", error, error_capacity);
    cudaEvent_t a = nullptr, b = nullptr;
    cudaEventCreate(&a);
    cudaEventCreate(&b);
    float cold_ms = 0.0f, total_ms = 0.0f;
    auto launch = [&] {
        bf16_argmax_kernel<<<1, 256>>>(static_cast<const bf16*>(logits.p), vocabulary_size, static_cast<int*>(token.p));
    };
    cudaEventRecord(a);
    launch();
    cudaEventRecord(b);
    status = cudaEventSynchronize(b);
    if (status == cudaSuccess) status = cudaEventElapsedTime(&cold_ms, a, b);
    if (status == cudaSuccess) {
        for (int i = 0; i < 8; ++i) launch();
        cudaEventRecord(a);
        for (int i = 0; i < iterations; ++i) launch();
        cudaEventRecord(b);
        status = cudaEventSynchronize(b);
    }
    if (status == cudaSuccess) status = cudaEventElapsedTime(&total_ms, a, b);
    int selected = -1;
    if (status == cudaSuccess) status = cudaMemcpy(&selected, token.p, sizeof(int), cudaMemcpyDeviceToHost);
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    if (status != cudaSuccess) return cuda_failure(status, "argmax benchmark", error, error_capacity);
    if (selected != expected) {
        say(error, error_capacity, "argmax kernel selected the wrong token");
        return -4;
    }
    output->vocabulary_size = vocabulary_size;
    output->iterations = iterations;
    output->selected_token = selected;
    output->expected_token = expected;
    output->cold_launch_microseconds = cold_ms * 1000.0f;
    output->mean_launch_microseconds = total_ms * 1000.0f / static_cast<float>(iterations);
    say(error, error_capacity, "");
    return 0;
}

int32_t qwen3_tts_benchmark_bf16_gemv(int32_t device_index, int32_t input_features, int32_t output_features,
                                      int32_t iterations, Qwen3TtsGemvBenchmark* output, char* error,
                                      size_t error_capacity) {
    if (output == nullptr) {
        say(error, error_capacity, "output benchmark pointer is null");
        return -1;
    }
    if (input_features <= 0 || input_features > 65536 || output_features <= 0 || output_features > 65536) {
        say(error, error_capacity, "feature sizes must be in [1, 65536]");
        return -2;
    }
    if (iterations <= 0) {
        say(error, error_capacity, "iterations must be positive");
        return -3;
    }
    cudaError_t status = cudaSetDevice(device_index);
    if (status != cudaSuccess) return cuda_failure(status, "cudaSetDevice", error, error_capacity);
    const uint64_t elements = static_cast<uint64_t>(input_features) * static_cast<uint64_t>(output_features);
    const uint64_t weight_bytes = elements * sizeof(bf16);
    Scoped w, x, y;
    status = cudaMalloc(&w.p, static_cast<size_t>(weight_bytes));
    if (status == cudaSuccess) status = cudaMalloc(&x.p, (size_t)input_features * sizeof(bf16));
    if (status == cudaSuccess) status = cudaMalloc(&y.p, (size_t)output_features * sizeof(bf16));
    if (status == cudaSuccess) status = cudaMemset(w.p, 0, static_cast<size_t>(weight_bytes));
    if (status == cudaSuccess) status = cudaMemset(x.p, 0, (size_t)input_features * sizeof(bf16));
    if (status == cudaSuccess) status = cudaMemset(y.p, 0xff, (size_t)output_features * sizeof(bf16));
    if (status != cudaSuccess) return cuda_failure(status, "bf16 GEMV benchmark set-up", error, error_capacity);
    cudaEvent_t a = nullptr, b = nullptr;
    cudaEventCreate(&a);
    cudaEventCreate(&b);
    auto launch = [&] {
        bf16_gemv_kernel<<<(output_features + 7) / 8, 256>>>(static_cast<const bf16*>(w.p), static_cast<const bf16*>(x.p),
                                                            static_cast<bf16*>(y.p), input_features, output_features);
    };
    float cold_ms = 0.0f, total_ms = 0.0f;
    cudaEventRecord(a);
    launch();
    cudaEventRecord(b);
    status = cudaEventSynchronize(b);
    if (status == cudaSuccess) status = cudaEventElapsedTime(&cold_ms, a, b);
    if (status == cudaSuccess) {
        for (int i = 0; i < 8; ++i) launch();
        cudaEventRecord(a);
        for (int i = 0; i < iterations; ++i) launch();
        cudaEventRecord(b);
        status = cudaEventSynchronize(b);
    }
    if (status == cudaSuccess) status = cudaEventElapsedTime(&total_ms, a, b);
    std::vector<uint16_t> host(static_cast<size_t>(output_features), 1);
    if (status == cudaSuccess) {
        status = cudaMemcpy(host.data(), y.p, host.size() * sizeof(uint16_t), cudaMemcpyDeviceToHost);
    }
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    if (status != cudaSuccess) return cuda_failure(status, "bf16 GEMV benchmark", error, error_capacity);
    for (uint16_t v : host) {
        if ((v & 0x7fffu) != 0) {
            say(error, error_capacity, "zero GEMV correctness check failed");
            return -4;
        }
    }
    const float mean_us = total_ms * 1000.0f / static_cast<float>(iterations);
    output->input_features = input_features;
    output->output_features = output_features;
    output->iterations = iterations;
    output->reserved = 0;
    output->weight_bytes = weight_bytes;
    output->cold_launch_microseconds = cold_ms * 1000.0f;
    output->mean_launch_microseconds = mean_us;
    output->tera_operations_per_second = static_cast<float>(2.0 * static_cast<double>(elements) / (mean_us * 1.0e-6) / 1.0e12);
    say(error, error_capacity, "");
    return 0;
}

}  // extern "C"
