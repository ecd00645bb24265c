// Decode attention for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc where they call the attention operator:
// a real-time audio thread that may not block in the driver, a process whose memory budget was
// carved up at start-up and is policed afterwards, or a plugin that is handed streams and
// buffers but no right to create device memory.  The regular entry point
// (q3t_launch_batch_causal_gqa_attention_fast) asks such a caller to bring a scratch buffer,
// which only moves the allocation to them.  This variant brings its own: the split-KV partials
// and ticket counters live in a fixed array inside the library's device image.
//
// Cost and limits.  Every GPU that loads the library holds kStaticScratchBytes (4 MiB) until the
// process exits, used or not.  A call whose shape needs more scratch than that is rejected with
// an error message, never truncated.  All calls on one device share the one array, and it keeps
// whatever the previous call left in it: the counters that must start at zero are cleared at the
// head of every call (a memset on the caller's stream, no allocation), the partials are always
// written before they are read.  Two calls that overlap on the GPU (different streams, no
// ordering between them) would race on the array; callers must order them.
//
// Set-up.  The array's name is, in host code, only a handle of the host-side runtime, not a
// device address, so the first call on each device asks the runtime for the real address
// (cudaGetSymbolAddress) with that device current, checks the result and keeps it.  That first
// call should therefore happen before any stream capture is begun on the thread.

#include "q3t_kernels.cuh"
#include "q3t_ops.h"

#include <cstdio>
#include <atomic>

namespace {

constexpr size_t kStaticScratchBytes = 4u << 20;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_attention_scratch[kStaticScratchBytes];

// resolved once per device; a first call racing another resolves the same address twice, harmlessly
std::atomic<void*> g_scratch_address[kMaxDevices] = {};

void message(char* error, size_t capacity, const char* text) {
    if (error != nullptr && capacity != 0) std::snprintf(error, capacity, "%s", text);
}

// device address of the array on the current device, resolved once per device
cudaError_t scratch_for_current_device(void** out) {
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
    void* address = g_scratch_address[device].load(std::memory_order_acquire);
    if (address == nullptr) {
        e = cudaGetSymbolAddress(&address, g_attention_scratch);
        if (e != cudaSuccess) return e;
        if (address == nullptr) return cudaErrorInvalidSymbol;
        g_scratch_address[device].store(address, std::memory_order_release);
    }
    *out = address;
    return cudaSuccess;
}

}  // namespace

extern "C" size_t q3t_attention_static_scratch_capacity(void) { return kStaticScratchBytes; }

extern "C" int32_t q3t_launch_batch_causal_gqa_attention_fast_noalloc(
    const uint16_t* query, uint16_t* const* key_bases, uint16_t* const* value_bases,
    const int32_t* positions, uint16_t* output, int32_t rows, int32_t query_heads,
    int32_t key_value_heads, int32_t head_dimension, int32_t max_sequence_length, void* stream,
    char* error, size_t error_capacity) {
    using namespace q3t;
    if (query == nullptr || key_bases == nullptr || value_bases == nullptr || positions == nullptr
        || output == nullptr || rows < 1 || rows > kMaxRows || query_heads < 1
        || key_value_heads < 1 || max_sequence_length < 1) {
        message(error, error_capacity, "attention arguments are null or out of range");
        return QWEN3_TTS_TALKER_STATUS_INVALID_ARGUMENT;
    }
    const size_t need = q3t_attention_scratch_bytes(rows, query_heads, key_value_heads,
                                                    head_dimension, max_sequence_length);
    if (need == 0 || need > kStaticScratchBytes) {
        char text[200];
        std::snprintf(text, sizeof(text),
                      "this shape needs %zu bytes of attention scratch; the built-in array holds %zu "
                      "(use q3t_launch_batch_causal_gqa_attention_fast with your own buffer)",
                      need, kStaticScratchBytes);
        message(error, error_capacity, text);
        return QWEN3_TTS_TALKER_STATUS_INVALID_ARGUMENT;
    }
    void* scratch = nullptr;
    cudaError_t e = scratch_for_current_device(&scratch);
    if (e != cudaSuccess) {
        message(error, error_capacity, cudaGetErrorString(e));
        return QWEN3_TTS_TALKER_STATUS_CUDA;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int splits = attention_splits_for(max_sequence_length);
    const size_t counter_bytes = attention_counters_bytes(rows, key_value_heads);
    AttentionArgs a;
    a.q = reinterpret_cast<const bf16*>(query);
    a.positions = positions;
    a.out = reinterpret_cast<bf16*>(output);
    a.kv.k_bases = reinterpret_cast<bf16* const*>(key_bases);
    a.kv.v_bases = reinterpret_cast<bf16* const*>(value_bases);
    a.rows = rows;
    a.q_heads = query_heads;
    a.kv_heads = key_value_heads;
    a.head_dim = head_dimension;
    a.max_splits = splits;
    a.counters = static_cast<unsigned int*>(scratch);
    a.scratch = reinterpret_cast<float*>(static_cast<char*>(scratch) + counter_bytes);
    // the array holds the last call's contents: the ticket counters have to start at zero
    e = cudaMemsetAsync(scratch, 0, counter_bytes, s);
    if (e == cudaSuccess) e = launch_decode_attention(a, s);
    if (e != cudaSuccess) {
        message(error, error_capacity, cudaGetErrorString(e));
        return e == cudaErrorInvalidValue ? QWEN3_TTS_TALKER_STATUS_INVALID_ARGUMENT
                                          : QWEN3_TTS_TALKER_STATUS_CUDA;
    }
    message(error, error_capacity, "");
    return QWEN3_TTS_TALKER_STATUS_OK;
}
