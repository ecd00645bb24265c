// extern "C" surface of libqwen3_tts_cuda.so: the native talker ABI v3
// (include/qwen3_tts_native.h) and the operator-level additions (include/q3t_ops.h).

#include "engine.hpp"
#include "q3t_ops.h"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>

using namespace q3t;

static_assert(sizeof(Qwen3TtsSamplingConfig) == 20, "ABI layout");
static_assert(sizeof(Qwen3TtsTalkerPrefillResult) == 12, "ABI layout");
static_assert(sizeof(Qwen3TtsCodecFrameInfo) == 16, "ABI layout");
static_assert(sizeof(Qwen3TtsModelMemory) == 16, "ABI layout");
static_assert(sizeof(Qwen3TtsSessionMemory) == 32, "ABI layout");
static_assert(sizeof(Qwen3TtsTalkerStateInfo) == 40, "ABI layout");
static_assert(sizeof(Qwen3TtsDeviceFrameViewV2) == 40 && alignof(Qwen3TtsDeviceFrameViewV2) == 8,
              "ABI layout");
static_assert(sizeof(SamplingParams) == sizeof(Qwen3TtsSamplingConfig), "sampling layout");
static_assert(QWEN3_TTS_MAX_BATCH_SESSIONS == kMaxRows && Q3T_MAX_ROWS == kMaxRows, "batch limit");
static_assert(Q3T_KV_PAGE_TOKENS == kPageTokens && Q3T_ATTENTION_CHUNK == kAttnChunk, "constants");

namespace q3t {
cudaError_t set_gemv_mma_error_sink(unsigned int* device_visible_word);
cudaError_t set_tc_error_sink(unsigned int* device_visible_word);

namespace {
std::atomic<unsigned int*> g_error_words[64];
}

volatile unsigned int* device_error_word(int device) {
    return device >= 0 && device < 64 ? g_error_words[device].load(std::memory_order_acquire) : nullptr;
}

cudaError_t configure_device() {
    static std::mutex guard;
    static bool done[64] = {};
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> lock(guard);
    if (device >= 0 && device < 64 && done[device]) return cudaSuccess;
    e = configure_gemv_kernels();
    if (e == cudaSuccess) e = configure_tc_kernels();
    if (e == cudaSuccess) e = configure_gemv_mma_kernels();
    if (e == cudaSuccess) e = configure_sampler_kernels();
    if (e == cudaSuccess && device >= 0 && device < 64 && g_error_words[device].load() == nullptr) {
        // the word the kernels' bounded waits bump when they give up; pinned and device-mapped, so
        // the host reads it at its synchronisation points without a copy
        unsigned int* word = nullptr;
        e = cudaHostAlloc(reinterpret_cast<void**>(&word), sizeof(unsigned int), cudaHostAllocMapped);
        if (e == cudaSuccess) {
            *word = 0;
            e = set_gemv_mma_error_sink(word);
            if (e == cudaSuccess) e = set_tc_error_sink(word);
            if (e == cudaSuccess) e = set_attention_error_sink(word);
            if (e == cudaSuccess) g_error_words[device].store(word, std::memory_order_release);
        }
    }
    if (e == cudaSuccess && device >= 0 && device < 64) done[device] = true;
    return e;
}
}  // namespace q3t

namespace {

using ModelBox = std::shared_ptr<Model>;

void write_error(char* destination, size_t capacity, const char* message) {
    if (destination != nullptr && capacity != 0) std::snprintf(destination, capacity, "%s", message);
}

ModelBox& model_of(Qwen3TtsModelHandle handle) {
    if (handle == nullptr) throw std::runtime_error("model handle is null");
    return *static_cast<ModelBox*>(handle);
}

Session* session_of(Qwen3TtsSessionHandle handle) {
    if (handle == nullptr) throw std::runtime_error("session handle is null");
    return static_cast<Session*>(handle);
}

// talker.cu:3790-3811
template <class Operation>
int32_t protect(Operation&& operation, int32_t failure_status, char* error, size_t capacity) {
    try {
        operation();
        write_error(error, capacity, "");
        return QWEN3_TTS_TALKER_STATUS_OK;
    } catch (const CudaFailure& e) {
        write_error(error, capacity, e.what());
        return QWEN3_TTS_TALKER_STATUS_CUDA;
    } catch (const std::bad_alloc& e) {
        write_error(error, capacity, e.what());
        return QWEN3_TTS_TALKER_STATUS_ALLOCATION;
    } catch (const std::exception& e) {
        write_error(error, capacity, e.what());
        return failure_status;
    }
}

SamplingParams params_of(const Qwen3TtsSamplingConfig& c) {
    return SamplingParams{c.do_sample, c.top_k, c.top_p, c.temperature, c.repetition_penalty};
}

void fill_view(Qwen3TtsDeviceFrameViewV2* out, const FrameView& v) {
    Qwen3TtsDeviceFrameViewV2 view{};
    view.struct_size = sizeof(Qwen3TtsDeviceFrameViewV2);
    view.code_count = kCodebooks;
    view.device_codes = v.device_codes;
    view.ready_event = reinterpret_cast<Qwen3TtsCudaEventHandle>(v.ready_event);
    view.lease_id = v.lease_id;
    view.device_index = v.device;
    *out = view;
}

const bf16* B(const uint16_t* p) { return reinterpret_cast<const bf16*>(p); }
bf16* B(uint16_t* p) { return reinterpret_cast<bf16*>(p); }
cudaStream_t S(void* s) { return static_cast<cudaStream_t>(s); }

int32_t ready() {
    const cudaError_t e = configure_device();
    return static_cast<int32_t>(e);
}

size_t counters_bytes(int rows, int kv_heads) { return attention_counters_bytes(rows, kv_heads); }
int splits_for(int max_sequence_length) { return attention_splits_for(max_sequence_length); }

}  // namespace

// =====================================================================================
// native talker ABI v3
// =====================================================================================

extern "C" {

uint32_t qwen3_tts_talker_abi_version(void) { return QWEN3_TTS_TALKER_ABI_VERSION; }

int32_t qwen3_tts_probe_device(int32_t device_index, Qwen3TtsDeviceInfo* output, char* error,
                               size_t error_capacity) {
    if (output == nullptr) {
        write_error(error, error_capacity, "device info output pointer is null");
        return QWEN3_TTS_TALKER_STATUS_INVALID_ARGUMENT;
    }
    return protect([&] {
        check_cuda(cudaSetDevice(device_index), "cudaSetDevice");
        cudaDeviceProp prop{};
        check_cuda(cudaGetDeviceProperties(&prop, device_index), "cudaGetDeviceProperties");
        size_t free_bytes = 0, total_bytes = 0;
        check_cuda(cudaMemGetInfo(&free_bytes, &total_bytes), "cudaMemGetInfo");
        Qwen3TtsDeviceInfo info{};
        info.device_index = device_index;
        info.compute_major = prop.major;
        info.compute_minor = prop.minor;
        info.total_global_memory_bytes = prop.totalGlobalMem;
        info.runtime_free_memory_bytes = free_bytes;
        info.runtime_total_memory_bytes = total_bytes;
        std::snprintf(info.device_name, sizeof(info.device_name), "%s", prop.name);
        *output = info;
    }, QWEN3_TTS_TALKER_STATUS_CUDA, error, error_capacity);
}

int32_t qwen3_tts_model_create(int32_t device_index, Qwen3TtsModelHandle* output, char* error,
                               size_t error_capacity) {
    if (output == nullptr) {
        write_error(error, error_capacity, "model output handle pointer is null");
        return QWEN3_TTS_TALKER_STATUS_INVALID_ARGUMENT;
    }
    return protect([&] {
        check_cuda(cudaSetDevice(device_index), "cudaSetDevice(model)");
        check_cuda(configure_device(), "configure kernels");
        *output = new ModelBox(std::make_shared<Model>(device_index));
    }, QWEN3_TTS_TALKER_STATUS_MODEL, error, error_capacity);
}

void qwen3_tts_model_destroy(Qwen3TtsModelHandle handle) { delete static_cast<ModelBox*>(handle); }

int32_t qwen3_tts_model_upload_tensor(Qwen3TtsModelHandle handle, const char* name,
                                      const void* bf16_data, uint64_t byte_size, int32_t rank,
                                      const uint64_t* shape, char* error, size_t error_capacity) {
    return protect([&] {
        model_of(handle)->upload_tensor(name, bf16_data, byte_size, rank, shape);
    }, QWEN3_TTS_TALKER_STATUS_MODEL, error, error_capacity);
}

int32_t q3t_model_tensor_image(Qwen3TtsModelHandle handle, const char* name, Q3tTensorImage* image,
                               char* error, size_t error_capacity) {
    if (image == nullptr || image->struct_size != sizeof(Q3tTensorImage)) {
        write_error(error, error_capacity, "tensor image output is null or has the wrong struct_size");
        return QWEN3_TTS_TALKER_STATUS_INVALID_ARGUMENT;
    }
    return protect([&] {
        const Model::TensorImage t = model_of(handle)->tensor_image(name);
        image->data = t.data;
        image->data_bytes = t.data_bytes;
        image->scales = t.scales;
        image->scales_bytes = t.scales_bytes;
        image->quantized = t.quantized ? 1 : 0;
        image->loaded = t.loaded ? 1 : 0;
        image->device_index = model_of(handle)->device();
    }, QWEN3_TTS_TALKER_STATUS_MODEL, error, error_capacity);
}

int32_t q3t_model_adopt_tensor(Qwen3TtsModelHandle handle, const char* name, char* error,
                               size_t error_capacity) {
    return protect([&] { model_of(handle)->adopt_tensor(name); }, QWEN3_TTS_TALKER_STATUS_MODEL, error,
                   error_capacity);
}

int32_t qwen3_tts_model_finalize(Qwen3TtsModelHandle handle, Qwen3TtsModelMemory* memory,
                                 char* error, size_t error_capacity) {
    if (memory == nullptr) {
        write_error(error, error_capacity, "talker memory output pointer is null");
        return QWEN3_TTS_TALKER_STATUS_INVALID_ARGUMENT;
    }
    return protect([&] {
        Qwen3TtsModelMemory m{};
        model_of(handle)->finalize(&m.shared_weight_bytes, &m.tensor_count);
        m.device_index = model_of(handle)->device();
        *memory = m;
    }, QWEN3_TTS_TALKER_STATUS_MODEL, error, error_capacity);
}

int32_t qwen3_tts_session_create(Qwen3TtsModelHandle model_handle, int32_t max_sequence_length,
                                 uint64_t random_seed, Qwen3TtsSessionHandle* output,
                                 Qwen3TtsSessionMemory* memory, char* error, size_t error_capacity) {
    if (output == nullptr || memory == nullptr) {
        write_error(error, error_capacity, "session output or memory pointer is null");
        return QWEN3_TTS_TALKER_STATUS_INVALID_ARGUMENT;
    }
    return protect([&] {
        std::unique_ptr<Session> created(
            new Session(model_of(model_handle), max_sequence_length, random_seed));
        Qwen3TtsSessionMemory m{};
        m.talker_kv_bytes = created->talker_kv_bytes;
        m.predictor_kv_bytes = created->predictor_kv_bytes;
        m.workspace_bytes = created->workspace_bytes;
        m.max_sequence_length = static_cast<uint32_t>(created->max_sequence_length());
        *memory = m;
        *output = created.release();
    }, QWEN3_TTS_TALKER_STATUS_STATE, error, error_capacity);
}

void qwen3_tts_session_destroy(Qwen3TtsSessionHandle handle) { delete static_cast<Session*>(handle); }

int32_t qwen3_tts_session_reset(Qwen3TtsSessionHandle handle, uint64_t random_seed, char* error,
                                size_t error_capacity) {
    return protect([&] { session_of(handle)->reset(random_seed); },
                   QWEN3_TTS_TALKER_STATUS_STATE, error, error_capacity);
}

int32_t qwen3_tts_session_prefill(Qwen3TtsSessionHandle handle, const int32_t* text_token_ids,
                                  const int32_t* codec_token_ids, int32_t token_count,
                                  Qwen3TtsSamplingConfig sampling,
                                  Qwen3TtsTalkerPrefillResult* output, char* error,
                                  size_t error_capacity) {
    if (output == nullptr) {
        write_error(error, error_capacity, "prefill output pointer is null");
        return QWEN3_TTS_TALKER_STATUS_INVALID_ARGUMENT;
    }
    return protect([&] {
        Qwen3TtsTalkerPrefillResult r{};
        session_of(handle)->prefill(text_token_ids, codec_token_ids, token_count,
                                    params_of(sampling), &r.first_semantic_token,
                                    &r.talker_gpu_milliseconds);
        r.prompt_tokens = static_cast<uint32_t>(token_count);
        *output = r;
    }, QWEN3_TTS_TALKER_STATUS_STATE, error, error_capacity);
}

int32_t qwen3_tts_session_next_frame(Qwen3TtsSessionHandle handle, uint16_t semantic_token,
                                     int32_t trailing_text_token_id,
                                     Qwen3TtsSamplingConfig talker_sampling,
                                     Qwen3TtsSamplingConfig predictor_sampling,
                                     uint16_t* output_codes, size_t output_code_capacity,
                                     uint16_t* next_semantic_token,
                                     Qwen3TtsCodecFrameInfo* frame_info, char* error,
                                     size_t error_capacity) {
    if (output_codes == nullptr || output_code_capacity < kCodebooks
        || next_semantic_token == nullptr || frame_info == nullptr) {
        write_error(error, error_capacity, "codec-frame outputs are null or undersized");
        return QWEN3_TTS_TALKER_STATUS_INVALID_ARGUMENT;
    }
    return protect([&] {
        Session* s = session_of(handle);
        const FrameView view = s->begin_frame(semantic_token, trailing_text_token_id,
                                              params_of(talker_sampling),
                                              params_of(predictor_sampling), true);
        const FrameResult r = s->finish_frame(view.lease_id, nullptr);
        std::copy_n(r.codes, kCodebooks, output_codes);
        *next_semantic_token = r.next_semantic;
        frame_info->talker_position = r.talker_position;
        frame_info->ended_by_eos = r.ended;
        frame_info->predictor_gpu_milliseconds = r.predictor_ms;
        frame_info->talker_gpu_milliseconds = r.talker_ms;
    }, QWEN3_TTS_TALKER_STATUS_STATE, error, error_capacity);
}

int32_t qwen3_tts_session_next_frame_begin_v2(Qwen3TtsSessionHandle handle,
                                              int32_t trailing_text_token_id,
                                              Qwen3TtsSamplingConfig talker_sampling,
                                              Qwen3TtsSamplingConfig predictor_sampling,
                                              Qwen3TtsDeviceFrameViewV2* output, char* error,
                                              size_t error_capacity) {
    if (output == nullptr) {
        write_error(error, error_capacity, "device-frame output is null");
        return QWEN3_TTS_TALKER_STATUS_INVALID_ARGUMENT;
    }
    if (output->struct_size != sizeof(Qwen3TtsDeviceFrameViewV2) || output->reserved != 0) {
        write_error(error, error_capacity,
                    "device-frame output has an unsupported size or nonzero reserved field");
        return QWEN3_TTS_TALKER_STATUS_INVALID_ARGUMENT;
    }
    return protect([&] {
        Session* s = session_of(handle);
        fill_view(output, s->begin_frame(s->current_token(), trailing_text_token_id,
                                         params_of(talker_sampling),
                                         params_of(predictor_sampling), false));
    }, QWEN3_TTS_TALKER_STATUS_STATE, error, error_capacity);
}

int32_t qwen3_tts_session_next_frame_finish_v2(Qwen3TtsSessionHandle handle, uint64_t lease_id,
                                               Qwen3TtsCudaEventHandle consumer_done_event,
                                               uint16_t* next_semantic_token,
                                               Qwen3TtsCodecFrameInfo* frame_info, char* error,
                                               size_t error_capacity) {
    if (next_semantic_token == nullptr || frame_info == nullptr) {
        write_error(error, error_capacity, "device-frame finish outputs are null");
        return QWEN3_TTS_TALKER_STATUS_INVALID_ARGUMENT;
    }
    return protect([&] {
        const FrameResult r = session_of(handle)->finish_frame(
            lease_id, reinterpret_cast<cudaEvent_t>(consumer_done_event));
        *next_semantic_token = r.next_semantic;
        frame_info->talker_position = r.talker_position;
        frame_info->ended_by_eos = r.ended;
        frame_info->predictor_gpu_milliseconds = r.predictor_ms;
        frame_info->talker_gpu_milliseconds = r.talker_ms;
    }, QWEN3_TTS_TALKER_STATUS_STATE, error, error_capacity);
}

int32_t qwen3_tts_model_batch_next_frame_begin_v2(
    Qwen3TtsModelHandle model_handle, Qwen3TtsSessionHandle* sessions, int32_t session_count,
    const int32_t* trailing_text_token_ids, const Qwen3TtsSamplingConfig* talker_sampling,
    const Qwen3TtsSamplingConfig* predictor_sampling, Qwen3TtsDeviceFrameViewV2* outputs,
    char* error, size_t error_capacity) {
    if (sessions == nullptr || session_count <= 0 || session_count > QWEN3_TTS_MAX_BATCH_SESSIONS
        || trailing_text_token_ids == nullptr || talker_sampling == nullptr
        || predictor_sampling == nullptr || outputs == nullptr) {
        write_error(error, error_capacity, "batch frame arguments are null or out of range");
        return QWEN3_TTS_TALKER_STATUS_INVALID_ARGUMENT;
    }
    for (int32_t i = 0; i < session_count; ++i) {
        if (sessions[i] == nullptr || outputs[i].struct_size != sizeof(Qwen3TtsDeviceFrameViewV2)
            || outputs[i].reserved != 0) {
            write_error(error, error_capacity,
                        "batch frame outputs have an unsupported size or nonzero reserved field");
            return QWEN3_TTS_TALKER_STATUS_INVALID_ARGUMENT;
        }
    }
    return protect([&] {
        Session* contexts[QWEN3_TTS_MAX_BATCH_SESSIONS];
        int trailing[QWEN3_TTS_MAX_BATCH_SESSIONS];
        SamplingParams talker[QWEN3_TTS_MAX_BATCH_SESSIONS];
        SamplingParams predictor[QWEN3_TTS_MAX_BATCH_SESSIONS];
        FrameView views[QWEN3_TTS_MAX_BATCH_SESSIONS];
        for (int32_t i = 0; i < session_count; ++i) {
            contexts[i] = session_of(sessions[i]);
            trailing[i] = trailing_text_token_ids[i];
            talker[i] = params_of(talker_sampling[i]);
            predictor[i] = params_of(predictor_sampling[i]);
        }
        Session::batch_begin(model_of(model_handle).get(), contexts, session_count, trailing, talker,
                             predictor, views);
        for (int32_t i = 0; i < session_count; ++i) fill_view(&outputs[i], views[i]);
    }, QWEN3_TTS_TALKER_STATUS_STATE, error, error_capacity);
}

int32_t qwen3_tts_session_state_info(Qwen3TtsSessionHandle handle, Qwen3TtsTalkerStateInfo* output,
                                     char* error, size_t error_capacity) {
    if (output == nullptr) {
        write_error(error, error_capacity, "session state output pointer is null");
        return QWEN3_TTS_TALKER_STATUS_INVALID_ARGUMENT;
    }
    return protect([&] {
        const Session* s = session_of(handle);
        Qwen3TtsTalkerStateInfo info{};
        info.abi_version = QWEN3_TTS_TALKER_ABI_VERSION;
        info.phase = s->phase();
        info.talker_position = s->position();
        info.semantic_history_count = s->history_count();
        info.frames_generated = s->frames_generated;
        info.device_sample_count = s->device_sample_count;
        info.host_sync_count = s->host_sync_count;
        *output = info;
    }, QWEN3_TTS_TALKER_STATUS_STATE, error, error_capacity);
}

// -------------------------------------------------------------------------------------
// Known-answer check of the row operators against host fp32 formulas, the shapes and inputs
// of the reference's primitive_parity.cu:115-324 (RMSNorm W=128; RoPE 2x128 at position 37;
// attention 4 query / 2 KV heads x 32, 7 positions; SiLU gate W=257).
// -------------------------------------------------------------------------------------

}  // extern "C"

namespace {

struct Scratch {
    std::vector<DeviceBuffer> buffers;
    template <class T> T* upload(const std::vector<T>& host) {
        buffers.emplace_back(host.size() * sizeof(T));
        check_cuda(cudaMemcpy(buffers.back().as<void>(), host.data(), host.size() * sizeof(T),
                              cudaMemcpyHostToDevice), "cudaMemcpy(H2D)");
        return buffers.back().as<T>();
    }
    template <class T> T* zeros(size_t count) {
        buffers.emplace_back(count * sizeof(T));
        check_cuda(cudaMemset(buffers.back().as<void>(), 0, count * sizeof(T)), "cudaMemset");
        return buffers.back().as<T>();
    }
};

std::vector<bf16> to_bf16(const std::vector<float>& v) {
    std::vector<bf16> o(v.size());
    for (size_t i = 0; i < v.size(); ++i) o[i] = __float2bfloat16(v[i]);
    return o;
}

std::vector<float> rounded(const std::vector<bf16>& v) {
    std::vector<float> o(v.size());
    for (size_t i = 0; i < v.size(); ++i) o[i] = __bfloat162float(v[i]);
    return o;
}

float max_error(const bf16* device, const std::vector<float>& expected) {
    std::vector<bf16> host(expected.size());
    check_cuda(cudaMemcpy(host.data(), device, host.size() * sizeof(bf16), cudaMemcpyDeviceToHost),
               "cudaMemcpy(D2H)");
    float worst = 0.0f;
    for (size_t i = 0; i < host.size(); ++i) {
        worst = std::max(worst, std::fabs(__bfloat162float(host[i]) - expected[i]));
    }
    return worst;
}

float rb(float v) { return __bfloat162float(__float2bfloat16(v)); }

}  // namespace

extern "C" {

int32_t qwen3_tts_validate_transformer_primitives(int32_t device_index,
                                                  Qwen3TtsPrimitiveParity* output, char* error,
                                                  size_t error_capacity) {
    if (output == nullptr) {
        write_error(error, error_capacity, "primitive parity output pointer is null");
        return QWEN3_TTS_TALKER_STATUS_INVALID_ARGUMENT;
    }
    return protect([&] {
        check_cuda(cudaSetDevice(device_index), "cudaSetDevice");
        check_cuda(configure_device(), "configure kernels");
        Scratch mem;
        Qwen3TtsPrimitiveParity result{};
        {   // RMSNorm
            const int width = 128;
            std::vector<float> x(width), w(width);
            for (int i = 0; i < width; ++i) {
                x[i] = std::sin(i * 0.071f) * 1.7f;
                w[i] = 0.75f + std::cos(i * 0.037f) * 0.2f;
            }
            const auto xb = to_bf16(x), wb = to_bf16(w);
            x = rounded(xb);
            w = rounded(wb);
            float ss = 0.0f;
            for (float v : x) ss += v * v;
            const float inv = 1.0f / std::sqrt(ss / width + 1.0e-6f);
            std::vector<float> expected(width);
            for (int i = 0; i < width; ++i) expected[i] = rb(x[i] * inv * w[i]);
            bf16* dy = mem.zeros<bf16>(width);
            check_cuda(launch_rms_norm_rows(mem.upload(xb), mem.upload(wb), dy, 1, width, 1.0e-6f, 0),
                       "rms norm");
            check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
            result.rms_norm_max_absolute_error = max_error(dy, expected);
        }
        {   // RoPE
            const int heads = 2, dim = 128, half = 64, position = 37;
            const float theta = 1.0e6f;
            std::vector<float> v(heads * dim);
            for (size_t i = 0; i < v.size(); ++i) v[i] = std::sin(static_cast<float>(i) * 0.019f);
            const auto vb = to_bf16(v);
            v = rounded(vb);
            std::vector<float> expected(v.size());
            for (int h = 0; h < heads; ++h) {
                for (int i = 0; i < half; ++i) {
                    const float angle = position * std::pow(theta, -static_cast<float>(2 * i) / dim);
                    const float a = v[h * dim + i], b = v[h * dim + i + half];
                    expected[h * dim + i] = rb(a * std::cos(angle) - b * std::sin(angle));
                    expected[h * dim + i + half] = rb(b * std::cos(angle) + a * std::sin(angle));
                }
            }
            bf16* dv = mem.upload(vb);
            const std::vector<int> pos{position};
            check_cuda(launch_rope_rows_at(dv, 1, heads, dim, mem.upload(pos), theta, 0), "rope");
            check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
            result.rope_max_absolute_error = max_error(dv, expected);
        }
        {   // attention
            const int qh = 4, kvh = 2, dim = 32, seq = 7;
            std::vector<float> q(qh * dim), k(seq * kvh * dim), v(seq * kvh * dim);
            for (size_t i = 0; i < q.size(); ++i) q[i] = std::sin(static_cast<float>(i) * 0.031f) * 0.4f;
            for (size_t i = 0; i < k.size(); ++i) {
                k[i] = std::cos(static_cast<float>(i) * 0.023f) * 0.3f;
                v[i] = std::sin(static_cast<float>(i) * 0.017f) * 0.5f;
            }
            const auto qb = to_bf16(q), kb = to_bf16(k), vb = to_bf16(v);
            q = rounded(qb);
            k = rounded(kb);
            v = rounded(vb);
            std::vector<float> expected(q.size()), scores(seq);
            for (int h = 0; h < qh; ++h) {
                const int g = h / (qh / kvh);
                float maximum = -INFINITY;
                for (int p = 0; p < seq; ++p) {
                    float dot = 0.0f;
                    for (int i = 0; i < dim; ++i) dot += q[h * dim + i] * k[(p * kvh + g) * dim + i];
                    scores[p] = dot / std::sqrt(static_cast<float>(dim));
                    maximum = std::max(maximum, scores[p]);
                }
                float den = 0.0f;
                for (float& s : scores) {
                    s = std::exp(s - maximum);
                    den += s;
                }
                for (int i = 0; i < dim; ++i) {
                    float acc = 0.0f;
                    for (int p = 0; p < seq; ++p) acc += scores[p] / den * v[(p * kvh + g) * dim + i];
                    expected[h * dim + i] = rb(acc);
                }
            }
            bf16* dk = mem.upload(kb);
            bf16* dv = mem.upload(vb);
            const std::vector<bf16*> kbase{dk}, vbase{dv};
            const std::vector<int> pos{seq - 1};
            AttentionArgs a;
            a.q = mem.upload(qb);
            a.positions = mem.upload(pos);
            a.out = mem.zeros<bf16>(qh * dim);
            a.kv.k_bases = mem.upload(kbase);
            a.kv.v_bases = mem.upload(vbase);
            a.rows = 1; a.q_heads = qh; a.kv_heads = kvh; a.head_dim = dim; a.max_splits = 1;
            check_cuda(launch_decode_attention(a, 0), "attention");
            check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
            result.attention_max_absolute_error = max_error(a.out, expected);
        }
        {   // SiLU gate
            const int width = 257;
            std::vector<float> g(width), u(width);
            for (int i = 0; i < width; ++i) {
                g[i] = std::sin(i * 0.043f) * 2.0f;
                u[i] = std::cos(i * 0.029f);
            }
            const auto gb = to_bf16(g), ub = to_bf16(u);
            g = rounded(gb);
            u = rounded(ub);
            std::vector<float> expected(width);
            for (int i = 0; i < width; ++i) expected[i] = rb(g[i] / (1.0f + std::exp(-g[i])) * u[i]);
            bf16* dg = mem.upload(gb);
            check_cuda(launch_silu_gate(dg, mem.upload(ub), width, 0), "silu gate");
            check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
            result.silu_gate_max_absolute_error = max_error(dg, expected);
        }
        *output = result;
    }, QWEN3_TTS_TALKER_STATUS_CUDA, error, error_capacity);
}

// =====================================================================================
// operator-level ABI
// =====================================================================================

static int32_t gemm_rows(const int8_t* w, const float* s, const uint16_t* x, uint16_t* y, int in,
                         int out, int rows, int epilogue, void* stream) {
    if (const int32_t e = ready()) return e;
    GemvArgs a;
    a.w = w; a.scales = s; a.x = B(x); a.y = B(y);
    a.in_features = in; a.out_features = out; a.rows = rows; a.epilogue = epilogue;
    return static_cast<int32_t>(launch_int8_gemm(a, S(stream)));
}

int32_t q3t_launch_int8_gemm_rows(const int8_t* weight, const float* scales, const uint16_t* input,
                                  uint16_t* output, int32_t in_features, int32_t out_features,
                                  int32_t rows, void* stream) {
    return gemm_rows(weight, scales, input, output, in_features, out_features, rows, EPI_PLAIN, stream);
}

int32_t q3t_launch_int8_gemm_rows_add(const int8_t* weight, const float* scales,
                                      const uint16_t* input, uint16_t* output, int32_t in_features,
                                      int32_t out_features, int32_t rows, void* stream) {
    return gemm_rows(weight, scales, input, output, in_features, out_features, rows, EPI_ADD, stream);
}

int32_t q3t_launch_int8_gate_up_silu_rows(const int8_t* weight, const float* scales,
                                          const uint16_t* input, uint16_t* output,
                                          int32_t in_features, int32_t out_features, int32_t rows,
                                          void* stream) {
    return gemm_rows(weight, scales, input, output, in_features, out_features, rows,
                     EPI_GATE_UP_SILU, stream);
}

int32_t q3t_launch_int8_gemm_ex(const Q3tGemmDesc* d, void* stream) {
    if (d == nullptr || d->struct_size != sizeof(Q3tGemmDesc)) return cudaErrorInvalidValue;
    if (d->epilogue < Q3T_EPI_PLAIN || d->epilogue > Q3T_EPI_GATE_UP_SILU) return cudaErrorInvalidValue;
    if (const int32_t e = ready()) return e;
    GemvArgs a;
    a.w = d->weight; a.scales = d->scales; a.x = B(d->input); a.y = B(d->output);
    a.y32 = d->output_f32; a.norm_w = B(d->norm_weight); a.norm_out = B(d->norm_output);
    a.bias = B(d->bias); a.resid = B(d->residual);
    a.in_features = d->in_features; a.out_features = d->out_features; a.rows = d->rows;
    a.epilogue = d->epilogue;
    a.eps = d->epsilon > 0.0f ? d->epsilon : kRmsEps;
    return static_cast<int32_t>(launch_int8_gemm(a, S(stream)));
}

int32_t q3t_launch_quantize_weight_rows(const uint16_t* weight, int8_t* quantized, float* scales,
                                        int32_t in_features, int32_t out_features, void* stream) {
    return static_cast<int32_t>(launch_quantize_weight_rows(B(weight), quantized, scales, in_features,
                                                            out_features, S(stream)));
}

}  // extern "C"

extern "C" {

int32_t q3t_benchmark_int8_gemv(int32_t device_index, int32_t input_features,
                                int32_t output_features, int32_t rows, int32_t buffers,
                                int32_t iterations, Qwen3TtsGemvBenchmark* output, char* error,
                                size_t error_capacity) {
    if (output == nullptr || input_features <= 0 || input_features % 16 != 0 || output_features <= 0
        || rows < 1 || rows > kMaxRows || buffers < 1 || iterations < 1) {
        write_error(error, error_capacity, "int8 GEMV benchmark arguments are out of range");
        return QWEN3_TTS_TALKER_STATUS_INVALID_ARGUMENT;
    }
    return protect([&] {
        check_cuda(cudaSetDevice(device_index), "cudaSetDevice");
        check_cuda(configure_device(), "configure kernels");
        const size_t wbytes = (size_t)input_features * output_features;
        DeviceBuffer w(wbytes * buffers), s((size_t)output_features * sizeof(float));
        DeviceBuffer x((size_t)rows * input_features * sizeof(bf16));
        DeviceBuffer y((size_t)rows * output_features * sizeof(bf16));
        cudaStream_t stream = nullptr;
        cudaEvent_t t0 = nullptr, t1 = nullptr;
        check_cuda(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking), "cudaStreamCreate");
        // seeded pseudo-random weights, scales and activations (a constant fill would understate the
        // switching activity of the memory system and of the arithmetic)
        check_cuda(launch_fill_bytes(w.as<unsigned char>(), w.bytes(), 0x51ed27u, stream), "fill weights");
        check_cuda(launch_fill_normal(x.as<bf16>(), (size_t)rows * input_features, 17, stream), "fill activations");
        {
            std::vector<float> scales(output_features);
            for (int i = 0; i < output_features; ++i) scales[i] = (0.5f + (i % 97) / 97.0f) / 127.0f;
            check_cuda(cudaMemcpyAsync(s.as<void>(), scales.data(), s.bytes(), cudaMemcpyHostToDevice, stream),
                       "upload scales");
            check_cuda(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
        }
        check_cuda(cudaEventCreate(&t0), "cudaEventCreate");
        check_cuda(cudaEventCreate(&t1), "cudaEventCreate");
        auto run = [&](int i) {
            GemvArgs a;
            a.scales = s.as<float>(); a.x = x.as<bf16>(); a.y = y.as<bf16>();
            a.in_features = input_features; a.out_features = output_features; a.rows = rows;
            a.w = w.as<int8_t>() + (size_t)(i % buffers) * wbytes;
            check_cuda(launch_int8_gemm(a, stream), "int8 GEMV");
        };
        float cold_ms = 0.0f, total_ms = 0.0f;
        try {
            check_cuda(cudaEventRecord(t0, stream), "cudaEventRecord");
            run(0);
            check_cuda(cudaEventRecord(t1, stream), "cudaEventRecord");
            check_cuda(cudaEventSynchronize(t1), "cudaEventSynchronize");
            check_cuda(cudaEventElapsedTime(&cold_ms, t0, t1), "cudaEventElapsedTime");
            // The timed launches replay a captured graph (4 passes over the weight images), so
            // that the figure is the kernel's and not the host's launch rate.
            const int per_graph = buffers * 4;
            cudaGraph_t graph = nullptr;
            check_cuda(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal),
                       "cudaStreamBeginCapture");
            try {
                for (int i = 0; i < per_graph; ++i) run(i);
            } catch (...) {
                cudaStreamEndCapture(stream, &graph);
                if (graph != nullptr) cudaGraphDestroy(graph);
                throw;
            }
            check_cuda(cudaStreamEndCapture(stream, &graph), "cudaStreamEndCapture");
            cudaGraphExec_t exec = nullptr;
            const cudaError_t ie = cudaGraphInstantiate(&exec, graph, 0);
            cudaGraphDestroy(graph);
            check_cuda(ie, "cudaGraphInstantiate");
            const int replays = (iterations + per_graph - 1) / per_graph;
            cudaError_t le = cudaGraphLaunch(exec, stream);
            if (le == cudaSuccess) le = cudaStreamSynchronize(stream);
            if (le == cudaSuccess) le = cudaEventRecord(t0, stream);
            for (int i = 0; i < replays && le == cudaSuccess; ++i) le = cudaGraphLaunch(exec, stream);
            if (le == cudaSuccess) le = cudaEventRecord(t1, stream);
            if (le == cudaSuccess) le = cudaEventSynchronize(t1);
            if (le == cudaSuccess) le = cudaEventElapsedTime(&total_ms, t0, t1);
            cudaGraphExecDestroy(exec);
            check_cuda(le, "timed GEMV graph replays");
            iterations = replays * per_graph;
        } catch (...) {
            cudaEventDestroy(t0); cudaEventDestroy(t1); cudaStreamDestroy(stream);
            throw;
        }
        cudaEventDestroy(t0); cudaEventDestroy(t1); cudaStreamDestroy(stream);
        Qwen3TtsGemvBenchmark b{};
        b.input_features = input_features;
        b.output_features = output_features;
        b.iterations = iterations;
        b.weight_bytes = wbytes;
        b.cold_launch_microseconds = cold_ms * 1000.0f;
        b.mean_launch_microseconds = total_ms * 1000.0f / iterations;
        b.tera_operations_per_second = static_cast<float>(
            2.0 * input_features * output_features * rows / (b.mean_launch_microseconds * 1.0e-6) / 1.0e12);
        *output = b;
    }, QWEN3_TTS_TALKER_STATUS_CUDA, error, error_capacity);
}

// Operator-level attention case: `rows` sessions with KV lengths drawn uniformly from
// [min_length, max_length] (seeded), 16 query / 8 KV heads of 128, paged bf16 caches (16-token
// head-major pages in one slab) filled with N(0,1); `iterations` launches of the decode attention in the mode in force, timed with
// events.  One launch reads every row's K and V once: *kv_bytes.
int32_t q3t_benchmark_decode_attention(int32_t device_index, int32_t rows, int32_t min_length,
                                       int32_t max_length, uint64_t seed, int32_t iterations,
                                       float* mean_launch_microseconds, uint64_t* kv_bytes, char* error,
                                       size_t error_capacity) {
    if (rows < 1 || rows > kMaxRows || min_length < 1 || max_length < min_length || max_length > 8192
        || iterations < 1 || mean_launch_microseconds == nullptr || kv_bytes == nullptr) {
        write_error(error, error_capacity, "attention benchmark arguments are out of range");
        return QWEN3_TTS_TALKER_STATUS_INVALID_ARGUMENT;
    }
    return protect([&] {
        check_cuda(cudaSetDevice(device_index), "cudaSetDevice");
        check_cuda(configure_device(), "configure kernels");
        constexpr int kQHeads = 16, kKvHeads = 8, kHeadDim = 128, kKvWidth = kKvHeads * kHeadDim;
        std::vector<int> positions(rows);
        uint64_t state = seed * 0x9e3779b97f4a7c15ull + 0x2545f4914f6cdd1dull;
        size_t tokens = 0;
        const int stride = (max_length + kPageTokens - 1) / kPageTokens;      // page-table entries per row
        std::vector<int> table((size_t)rows * stride, 0);
        int pages = 0;
        for (int r = 0; r < rows; ++r) {
            state ^= state >> 12; state ^= state << 25; state ^= state >> 27;
            const int length = min_length + static_cast<int>((state * 0x2545f4914f6cdd1dull >> 33)
                                                             % static_cast<uint64_t>(max_length - min_length + 1));
            positions[r] = length - 1;
            tokens += static_cast<size_t>(length);
            for (int p = 0; p < (length + kPageTokens - 1) / kPageTokens; ++p) table[(size_t)r * stride + p] = pages++;
        }
        // one slab: the K planes of all pages, then the V planes (pages are head-major, see q3t_ops.h)
        const size_t page_elems = (size_t)kPageTokens * kKvWidth;
        DeviceBuffer slab((size_t)pages * page_elems * 2 * sizeof(bf16));
        DeviceBuffer q((size_t)rows * kQHeads * kHeadDim * sizeof(bf16)), out((size_t)rows * kQHeads * kHeadDim * sizeof(bf16));
        DeviceBuffer dpos((size_t)rows * sizeof(int)), dtable(table.size() * sizeof(int)), dslabs(sizeof(bf16*));
        const int splits = splits_for(max_length);
        DeviceBuffer scratch(attention_scratch_floats(rows, kQHeads, kHeadDim, splits) * sizeof(float));
        DeviceBuffer counters(counters_bytes(rows, kKvHeads));
        cudaStream_t stream = nullptr;
        cudaEvent_t t0 = nullptr, t1 = nullptr;
        check_cuda(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking), "cudaStreamCreate");
        float total_ms = 0.0f;
        try {
            check_cuda(cudaEventCreate(&t0), "cudaEventCreate");
            check_cuda(cudaEventCreate(&t1), "cudaEventCreate");
            check_cuda(launch_fill_normal(slab.as<bf16>(), (size_t)pages * page_elems * 2, seed * 3 + 1, stream), "fill K and V");
            check_cuda(launch_fill_normal(q.as<bf16>(), (size_t)rows * kQHeads * kHeadDim, seed * 3 + 3, stream), "fill q");
            check_cuda(cudaMemsetAsync(counters.as<void>(), 0, counters.bytes(), stream), "cudaMemsetAsync");
            check_cuda(cudaMemcpyAsync(dpos.as<void>(), positions.data(), dpos.bytes(), cudaMemcpyHostToDevice, stream), "upload positions");
            check_cuda(cudaMemcpyAsync(dtable.as<void>(), table.data(), dtable.bytes(), cudaMemcpyHostToDevice, stream), "upload page table");
            bf16* slab_base = slab.as<bf16>();
            check_cuda(cudaMemcpyAsync(dslabs.as<void>(), &slab_base, sizeof(slab_base), cudaMemcpyHostToDevice, stream), "upload slab table");
            check_cuda(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
            AttentionArgs a;
            a.q = q.as<bf16>(); a.out = out.as<bf16>(); a.positions = dpos.as<int>();
            a.kv.page_table = dtable.as<int>(); a.kv.table_stride = stride;
            a.kv.slabs = dslabs.as<bf16*>(); a.kv.slab_shift = 30;
            a.kv.page_elems = static_cast<long long>(page_elems);
            a.kv.k_offset = 0; a.kv.v_offset = static_cast<long long>((size_t)pages * page_elems);
            a.rows = rows; a.q_heads = kQHeads; a.kv_heads = kKvHeads; a.head_dim = kHeadDim;
            a.max_splits = splits;
            a.scratch = scratch.as<float>(); a.counters = counters.as<unsigned int>();
            for (int i = 0; i < 3; ++i) check_cuda(launch_attention(a, stream), "decode attention");
            check_cuda(cudaEventRecord(t0, stream), "cudaEventRecord");
            for (int i = 0; i < iterations; ++i) check_cuda(launch_attention(a, stream), "decode attention");
            check_cuda(cudaEventRecord(t1, stream), "cudaEventRecord");
            check_cuda(cudaEventSynchronize(t1), "cudaEventSynchronize");
            check_cuda(cudaEventElapsedTime(&total_ms, t0, t1), "cudaEventElapsedTime");
        } catch (...) {
            if (t0 != nullptr) cudaEventDestroy(t0);
            if (t1 != nullptr) cudaEventDestroy(t1);
            cudaStreamSynchronize(stream);
            cudaStreamDestroy(stream);
            throw;
        }
        cudaEventDestroy(t0); cudaEventDestroy(t1); cudaStreamDestroy(stream);
        *mean_launch_microseconds = total_ms * 1000.0f / iterations;
        *kv_bytes = static_cast<uint64_t>(tokens) * kKvWidth * sizeof(bf16) * 2;
    }, QWEN3_TTS_TALKER_STATUS_CUDA, error, error_capacity);
}

}  // extern "C"

extern "C" {

int32_t q3t_launch_rms_norm_rows(const uint16_t* input, const uint16_t* weight, uint16_t* output,
                                 int32_t rows, int32_t width, float epsilon, void* stream) {
    return static_cast<int32_t>(launch_rms_norm_rows(B(input), B(weight), B(output), rows, width,
                                                     epsilon, S(stream)));
}

int32_t q3t_launch_head_rms_norm_rows(uint16_t* values, const uint16_t* weight, int32_t rows,
                                      int32_t heads, int32_t head_dimension, float epsilon,
                                      void* stream) {
    return static_cast<int32_t>(launch_head_rms_norm_rows(B(values), B(weight), rows, heads,
                                                          head_dimension, epsilon, S(stream)));
}

int32_t q3t_launch_rope_rows_at(uint16_t* values, int32_t rows, int32_t heads, int32_t head_dimension,
                                const int32_t* positions, float theta, void* stream) {
    return static_cast<int32_t>(launch_rope_rows_at(B(values), rows, heads, head_dimension, positions,
                                                    theta, S(stream)));
}

int32_t q3t_launch_kv_scatter_rows(const uint16_t* rows_data, uint16_t* const* cache_bases,
                                   const int32_t* positions, int32_t rows, int32_t width,
                                   void* stream) {
    return static_cast<int32_t>(launch_kv_scatter_rows(
        B(rows_data), reinterpret_cast<bf16* const*>(cache_bases), positions, rows, width, S(stream)));
}

int32_t q3t_launch_bias_activation_rows(uint16_t* values, const uint16_t* bias, int32_t rows,
                                        int32_t width, int32_t silu, void* stream) {
    return static_cast<int32_t>(launch_bias_activation_rows(B(values), B(bias), rows, width, silu != 0,
                                                            S(stream)));
}

int32_t q3t_launch_add_in_place(uint16_t* destination, const uint16_t* source, int32_t width,
                                void* stream) {
    return static_cast<int32_t>(launch_add_in_place(B(destination), B(source), width, S(stream)));
}

int32_t q3t_launch_silu_gate(uint16_t* gate, const uint16_t* up, int32_t width, void* stream) {
    return static_cast<int32_t>(launch_silu_gate(B(gate), B(up), width, S(stream)));
}

int32_t q3t_launch_gather_embedding_rows(const uint16_t* table, int32_t vocabulary, int32_t width,
                                         const int32_t* const* tokens, int32_t token_offset,
                                         uint16_t* output, int32_t rows, void* stream) {
    return static_cast<int32_t>(launch_gather_embedding_rows(B(table), vocabulary, width, tokens,
                                                             token_offset, B(output), rows, false,
                                                             S(stream)));
}

int32_t q3t_launch_add_embedding_rows(const uint16_t* table, int32_t vocabulary, int32_t width,
                                      const int32_t* const* tokens, int32_t token_offset,
                                      uint16_t* output, int32_t rows, void* stream) {
    return static_cast<int32_t>(launch_gather_embedding_rows(B(table), vocabulary, width, tokens,
                                                             token_offset, B(output), rows, true,
                                                             S(stream)));
}

size_t q3t_attention_scratch_bytes(int32_t rows, int32_t query_heads, int32_t key_value_heads,
                                   int32_t head_dimension, int32_t max_sequence_length) {
    if (rows < 1 || query_heads < 1 || key_value_heads < 1 || head_dimension < 1
        || max_sequence_length < 1) {
        return 0;
    }
    return counters_bytes(rows, key_value_heads)
        + attention_scratch_floats(rows, query_heads, head_dimension, splits_for(max_sequence_length))
              * sizeof(float);
}

static int32_t attention_common(AttentionArgs& a, int max_sequence_length, void* scratch,
                                size_t scratch_bytes, cudaStream_t stream) {
    a.max_splits = splits_for(max_sequence_length);
    const size_t need = q3t_attention_scratch_bytes(a.rows, a.q_heads, a.kv_heads, a.head_dim,
                                                    max_sequence_length);
    if (a.max_splits > 1) {
        if (scratch == nullptr || need == 0 || scratch_bytes < need) return cudaErrorInvalidValue;
        const size_t cb = counters_bytes(a.rows, a.kv_heads);
        a.counters = static_cast<unsigned int*>(scratch);
        a.scratch = reinterpret_cast<float*>(static_cast<char*>(scratch) + cb);
        const cudaError_t e = cudaMemsetAsync(scratch, 0, cb, stream);
        if (e != cudaSuccess) return static_cast<int32_t>(e);
    }
    return static_cast<int32_t>(launch_attention(a, stream));
}

int32_t q3t_launch_batch_causal_gqa_attention_fast(
    const uint16_t* query, uint16_t* const* key_bases, uint16_t* const* value_bases,
    const int32_t* positions, uint16_t* output, int32_t rows, int32_t query_heads,
    int32_t key_value_heads, int32_t head_dimension, int32_t max_sequence_length, void* scratch,
    size_t scratch_bytes, void* stream) {
    if (rows < 1 || max_sequence_length < 1) return cudaErrorInvalidValue;
    AttentionArgs a;
    a.q = B(query);
    a.positions = positions;
    a.out = B(output);
    a.kv.k_bases = reinterpret_cast<bf16* const*>(key_bases);
    a.kv.v_bases = reinterpret_cast<bf16* const*>(value_bases);
    a.rows = rows; a.q_heads = query_heads; a.kv_heads = key_value_heads; a.head_dim = head_dimension;
    return attention_common(a, max_sequence_length, scratch, scratch_bytes, S(stream));
}

int32_t q3t_launch_decode_attention_ex(const Q3tAttentionDesc* d, void* stream) {
    if (d == nullptr || d->struct_size != sizeof(Q3tAttentionDesc) || d->rows < 1
        || d->max_sequence_length < 1) {
        return cudaErrorInvalidValue;
    }
    AttentionArgs a;
    a.q = B(d->query); a.k_new = B(d->key_new); a.v_new = B(d->value_new);
    a.q_norm_w = B(d->query_norm_weight); a.k_norm_w = B(d->key_norm_weight);
    a.positions = d->positions;
    a.out = B(d->output); a.out32 = d->output_f32;
    a.kv.k_bases = reinterpret_cast<bf16* const*>(d->key_bases);
    a.kv.v_bases = reinterpret_cast<bf16* const*>(d->value_bases);
    a.kv.page_table = d->page_table;
    a.kv.table_stride = d->page_table_stride;
    a.kv.slabs = reinterpret_cast<bf16* const*>(d->slabs);
    a.kv.slab_shift = d->slab_shift;
    a.kv.page_elems = d->page_elements;
    a.kv.k_offset = d->key_offset;
    a.kv.v_offset = d->value_offset;
    a.q_stride = d->query_stride; a.kv_new_stride = d->new_stride;
    a.rows = d->rows; a.q_heads = d->query_heads; a.kv_heads = d->key_value_heads;
    a.head_dim = d->head_dimension; a.fused = d->fused;
    a.eps = d->epsilon > 0.0f ? d->epsilon : kRmsEps;
    a.theta = d->theta > 0.0f ? d->theta : kRopeTheta;
    return attention_common(a, d->max_sequence_length, d->scratch, d->scratch_bytes, S(stream));
}

static int32_t sample_common(const uint16_t* logits, int vocabulary, int suppress, int eos,
                             const int* history, const int* count_ptr, int count_value, int do_sample,
                             int top_k, float top_p, float temperature, float penalty,
                             uint64_t* rng, int* selected, void* stream) {
    if (vocabulary <= 0 || vocabulary > kMaxVocab) return cudaErrorInvalidValue;
    if (const int32_t e = ready()) return e;
    SamplerRow r{};
    r.logits = B(logits);
    r.history = history;
    r.history_count = count_ptr;
    r.history_count_value = count_value;
    r.rng = reinterpret_cast<unsigned long long*>(rng);
    r.selected = selected;
    r.vocabulary = vocabulary;
    r.suppress = suppress != 0;
    r.eos = eos;
    r.do_sample = do_sample;
    r.top_k = top_k;
    r.top_p = top_p;
    r.temperature = temperature;
    r.penalty = penalty;
    return static_cast<int32_t>(launch_sample_value(r, S(stream)));
}

int32_t q3t_launch_sample_logits(const uint16_t* logits, int32_t vocabulary,
                                 int32_t suppress_talker_reserved, int32_t codec_eos_token,
                                 const int32_t* semantic_history, int32_t semantic_history_count,
                                 int32_t do_sample, int32_t top_k, float top_p, float temperature,
                                 float repetition_penalty, uint64_t* random_state,
                                 int32_t* selected_token, void* stream) {
    return sample_common(logits, vocabulary, suppress_talker_reserved, codec_eos_token,
                         semantic_history, nullptr, semantic_history_count, do_sample, top_k, top_p,
                         temperature, repetition_penalty, random_state, selected_token, stream);
}

int32_t q3t_launch_sample_logits_at(const uint16_t* logits, int32_t vocabulary,
                                    int32_t suppress_talker_reserved, int32_t codec_eos_token,
                                    const int32_t* semantic_history,
                                    const int32_t* semantic_history_count, int32_t do_sample,
                                    int32_t top_k, float top_p, float temperature,
                                    float repetition_penalty, uint64_t* random_state,
                                    int32_t* selected_token, void* stream) {
    return sample_common(logits, vocabulary, suppress_talker_reserved, codec_eos_token,
                         semantic_history, semantic_history_count, 0, do_sample, top_k, top_p,
                         temperature, repetition_penalty, random_state, selected_token, stream);
}

int32_t q3t_model_set_option(Qwen3TtsModelHandle model, const char* key, int32_t value, char* error,
                             size_t error_capacity) {
    if (key == nullptr) {
        write_error(error, error_capacity, "option key is null");
        return QWEN3_TTS_TALKER_STATUS_INVALID_ARGUMENT;
    }
    return protect([&] {
        Model* m = model_of(model).get();
        if (std::strcmp(key, "mask_eos") == 0) {
            m->mask_eos = value != 0;
        } else if (std::strcmp(key, "use_graphs") == 0) {
            m->use_graphs = value != 0;
        } else if (std::strcmp(key, "batch_host_codes") == 0) {
            m->batch_host_codes = value != 0;
        } else if (std::strcmp(key, "prefill_chunk") == 0) {
            m->prefill_chunk = value < 1 ? 1 : (value > kMaxRows ? kMaxRows : value);
        } else if (std::strcmp(key, "tc_min_rows") == 0) {
            set_tc_min_rows(value);     // process-wide: rows at or above this use the tensor cores
        } else if (std::strcmp(key, "gemv_mode") == 0) {
            if (value < 0 || value > 1) throw std::runtime_error("gemv_mode must be 0 or 1");
            set_gemv_mode(value);       // process-wide: kernel for projections of 1..8 rows
        } else if (std::strcmp(key, "attention_mode") == 0) {
            if (value < 0 || value > 1) throw std::runtime_error("attention_mode must be 0 or 1");
            set_attention_mode(value);  // process-wide: 0 sums in the reference's order (parity, slow)
        } else {
            throw std::runtime_error(std::string("unknown model option: ") + key);
        }
        // captured graphs bake the option in
        std::lock_guard<std::mutex> one_batch(m->batch_mutex);
        if (Workspace* w = m->batch_workspace_if_any()) {
            check_cuda(cudaStreamSynchronize(w->stream), "cudaStreamSynchronize");
            w->destroy_graphs();
        }
        ++m->option_epoch;
    }, QWEN3_TTS_TALKER_STATUS_INVALID_ARGUMENT, error, error_capacity);
}

int32_t q3t_model_run_frames(Qwen3TtsModelHandle model, Qwen3TtsSessionHandle* sessions,
                             int32_t session_count, int32_t frames, int32_t trailing_text_token_id,
                             Qwen3TtsSamplingConfig talker_sampling,
                             Qwen3TtsSamplingConfig predictor_sampling, float* frame_milliseconds,
                             float* total_milliseconds, char* error, size_t error_capacity) {
    if (sessions == nullptr || session_count <= 0 || session_count > QWEN3_TTS_MAX_BATCH_SESSIONS
        || frames <= 0) {
        write_error(error, error_capacity, "frame-loop arguments are null or out of range");
        return QWEN3_TTS_TALKER_STATUS_INVALID_ARGUMENT;
    }
    return protect([&] {
        Session* contexts[QWEN3_TTS_MAX_BATCH_SESSIONS];
        for (int32_t i = 0; i < session_count; ++i) contexts[i] = session_of(sessions[i]);
        Session::run_frames(model_of(model).get(), contexts, session_count, frames,
                            trailing_text_token_id, params_of(talker_sampling),
                            params_of(predictor_sampling), frame_milliseconds, total_milliseconds);
    }, QWEN3_TTS_TALKER_STATUS_STATE, error, error_capacity);
}

int32_t q3t_session_synthetic_prefill(Qwen3TtsSessionHandle session, int32_t position, uint64_t seed,
                                      char* error, size_t error_capacity) {
    return protect([&] { session_of(session)->synthetic_prefill(position, seed); },
                   QWEN3_TTS_TALKER_STATUS_STATE, error, error_capacity);
}

int32_t q3t_set_gemv_mode(int32_t mode) { return set_gemv_mode(mode); }

int32_t q3t_test_gemv_plan(int32_t in_features, int32_t out_features, int32_t rows, int32_t gate_up,
                           int32_t norm, int64_t* fields) {
    GemvMmaPlan plan{};
    if (fields == nullptr || !gemv_mma_plan(in_features, out_features, rows, gate_up != 0, norm != 0, &plan)) return 0;
    fields[0] = plan.grid; fields[1] = plan.stages; fields[2] = plan.group; fields[3] = plan.tiles;
    fields[4] = plan.rows_per_launch; fields[5] = plan.stage_bytes; fields[6] = plan.ring_bytes;
    fields[7] = plan.shared_bytes;
    return 1;
}
int32_t q3t_set_attention_mode(int32_t mode) { return set_attention_mode(mode); }

void q3t_test_fail_launch_after(int32_t launches) { fail_launch_after(launches); }
void q3t_test_fail_allocation_after(int32_t allocations) { fail_allocation_after(allocations); }
int32_t q3t_test_report_device_wait_failure(int32_t device_index) {
    volatile unsigned int* word = device_error_word(device_index);
    if (word == nullptr) return QWEN3_TTS_TALKER_STATUS_STATE;
    *word = *word + 1;
    return QWEN3_TTS_TALKER_STATUS_OK;
}

uint32_t q3t_kernel_error_count(void) {
    return gemm_tc_error_count() + gemv_mma_error_count();
}

uint32_t q3t_attention_range_error_count(void) { return attention_range_error_count(); }

int32_t q3t_session_current_token(Qwen3TtsSessionHandle session, uint16_t* token, char* error,
                                  size_t error_capacity) {
    if (token == nullptr) {
        write_error(error, error_capacity, "token output pointer is null");
        return QWEN3_TTS_TALKER_STATUS_INVALID_ARGUMENT;
    }
    return protect([&] { *token = session_of(session)->current_token(); },
                   QWEN3_TTS_TALKER_STATUS_STATE, error, error_capacity);
}

int32_t q3t_model_kernel_launches(Qwen3TtsModelHandle model, uint64_t* launches, char* error,
                                  size_t error_capacity) {
    if (launches == nullptr) {
        write_error(error, error_capacity, "launch counter output pointer is null");
        return QWEN3_TTS_TALKER_STATUS_INVALID_ARGUMENT;
    }
    return protect([&] { *launches = model_of(model)->kernel_launches.load(); },
                   QWEN3_TTS_TALKER_STATUS_STATE, error, error_capacity);
}

int32_t q3t_session_read_state(Qwen3TtsSessionHandle session, uint16_t* last_hidden,
                               int32_t* frame_tokens, uint64_t* random_state, char* error,
                               size_t error_capacity) {
    return protect([&] {
        session_of(session)->read_state(last_hidden, frame_tokens,
                                        reinterpret_cast<unsigned long long*>(random_state));
    }, QWEN3_TTS_TALKER_STATUS_STATE, error, error_capacity);
}

int32_t q3t_session_read_kv(Qwen3TtsSessionHandle session, int32_t layer, int32_t first_position,
                            int32_t count, uint16_t* keys, uint16_t* values, char* error,
                            size_t error_capacity) {
    return protect([&] { session_of(session)->read_kv(layer, first_position, count, keys, values); },
                   QWEN3_TTS_TALKER_STATUS_STATE, error, error_capacity);
}

}  // extern "C"
