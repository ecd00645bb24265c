/*
 * Native talker C ABI, version 3 -- the drop-in boundary of libqwen3_tts_cuda.so.
 *
 * This header restates, symbol for symbol and field for field, the interface that the
 * reference project (luka-loehr/qwen3-tts-native) declares in
 * native/qwen3-tts-native/native/include/qwen3_tts_native.h and that its Rust host crate
 * resolves by name at run time (native/qwen3-tts-native/src/native_talker.rs:776-821).
 * A library that exports these symbols with these layouts can be put in the place of the
 * reference's libqwen3_tts_cuda.so without rebuilding the host.
 *
 * Differences, all additive:
 *   - QWEN3_TTS_MAX_BATCH_SESSIONS is 64 here (the reference stops at 8);
 *   - decode always runs the int8 weight-only path (the reference needs
 *     QWEN3_TTS_INT8_DECODE=1 for it);
 *   - extra entry points live in q3t_ops.h.
 *
 * Conventions shared by every call that returns int32_t: 0 on success, a negative
 * QWEN3_TTS_TALKER_STATUS_* otherwise; `error` (capacity `error_capacity`, may be NULL/0)
 * receives a NUL-terminated message, "" on success; no C++ exception crosses the boundary.
 */
#ifndef QWEN3_TTS_NATIVE_H_
#define QWEN3_TTS_NATIVE_H_

#include <stddef.h>
#include <stdint.h>

#define QWEN3_TTS_API __attribute__((visibility("default")))

#ifdef __cplusplus
extern "C" {
#endif

#define QWEN3_TTS_TALKER_ABI_VERSION 3U
#define QWEN3_TTS_MAX_BATCH_SESSIONS 64          /* reference header :17 has 8 */
#define QWEN3_TTS_CODEC_CODEBOOKS 16U

/* reference header :20-27 */
enum {
    QWEN3_TTS_TALKER_STATUS_OK = 0,
    QWEN3_TTS_TALKER_STATUS_INVALID_ARGUMENT = -1,
    QWEN3_TTS_TALKER_STATUS_CUDA = -2,
    QWEN3_TTS_TALKER_STATUS_STATE = -3,
    QWEN3_TTS_TALKER_STATUS_ALLOCATION = -4,
    QWEN3_TTS_TALKER_STATUS_MODEL = -5
};

/* reference header :29-37 */
typedef struct Qwen3TtsDeviceInfo {
    int32_t device_index;
    int32_t compute_major;
    int32_t compute_minor;
    uint64_t total_global_memory_bytes;
    uint64_t runtime_free_memory_bytes;
    uint64_t runtime_total_memory_bytes;
    char device_name[256];
} Qwen3TtsDeviceInfo;

/* reference header :48-57; filled by qwen3_tts_benchmark_bf16_gemv and, for the int8
 * kernel, by q3t_benchmark_int8_gemv (q3t_ops.h) */
typedef struct Qwen3TtsGemvBenchmark {
    int32_t input_features;
    int32_t output_features;
    int32_t iterations;
    int32_t reserved;
    uint64_t weight_bytes;
    float cold_launch_microseconds;
    float mean_launch_microseconds;
    float tera_operations_per_second;
} Qwen3TtsGemvBenchmark;

/* reference header :39-46; filled by qwen3_tts_benchmark_bf16_argmax */
typedef struct Qwen3TtsArgmaxBenchmark {
    int32_t vocabulary_size;
    int32_t iterations;
    int32_t selected_token;
    int32_t expected_token;
    float cold_launch_microseconds;
    float mean_launch_microseconds;
} Qwen3TtsArgmaxBenchmark;

/* reference header :59 and :61-72: a device arena filled by sequential uploads through pinned
 * staging memory (the host's weight loader, src/device_weights.rs) */
typedef struct Qwen3TtsDeviceBuffer Qwen3TtsDeviceBuffer;
typedef struct Qwen3TtsWeightUploadMetrics {
    int32_t device_index;
    int32_t reserved;
    uint64_t allocation_bytes;
    uint64_t pinned_staging_bytes;
    uint64_t uploaded_bytes;
    uint64_t upload_calls;
    uint64_t free_before_bytes;
    uint64_t free_after_allocation_bytes;
    float allocation_microseconds;
    float upload_microseconds;
} Qwen3TtsWeightUploadMetrics;

/* reference header :74-79 */
typedef struct Qwen3TtsPrimitiveParity {
    float rms_norm_max_absolute_error;
    float rope_max_absolute_error;
    float attention_max_absolute_error;
    float silu_gate_max_absolute_error;
} Qwen3TtsPrimitiveParity;

/* reference header :81-87; 20 bytes, passed BY VALUE */
typedef struct Qwen3TtsSamplingConfig {
    int32_t do_sample;
    int32_t top_k;
    float top_p;
    float temperature;
    float repetition_penalty;
} Qwen3TtsSamplingConfig;

/* reference header :89-94; 12 bytes */
typedef struct Qwen3TtsTalkerPrefillResult {
    uint16_t first_semantic_token;
    uint16_t reserved;
    uint32_t prompt_tokens;
    float talker_gpu_milliseconds;
} Qwen3TtsTalkerPrefillResult;

/* reference header :105-110; 16 bytes */
typedef struct Qwen3TtsCodecFrameInfo {
    uint32_t talker_position;
    uint32_t ended_by_eos;
    float predictor_gpu_milliseconds;
    float talker_gpu_milliseconds;
} Qwen3TtsCodecFrameInfo;

/* Borrowed cudaEvent_t: wait on it, never record or destroy it (reference header :112-114). */
typedef void* Qwen3TtsCudaEventHandle;

/* reference header :116-128; 40 bytes, align 8.  The caller sets struct_size and reserved
 * (0) before a begin call; device_codes and ready_event stay valid until the matching
 * finish; one lease per session at a time. */
typedef struct Qwen3TtsDeviceFrameViewV2 {
    uint32_t struct_size;
    uint32_t code_count;
    const uint16_t* device_codes;
    Qwen3TtsCudaEventHandle ready_event;
    uint64_t lease_id;
    int32_t device_index;
    uint32_t reserved;
} Qwen3TtsDeviceFrameViewV2;

/* reference header :130-135 */
typedef enum Qwen3TtsTalkerPhase {
    QWEN3_TTS_TALKER_CREATED = 0,
    QWEN3_TTS_TALKER_READY = 1,
    QWEN3_TTS_TALKER_PREFILLED = 2,
    QWEN3_TTS_TALKER_ENDED = 3
} Qwen3TtsTalkerPhase;

/* reference header :137-145; 40 bytes */
typedef struct Qwen3TtsTalkerStateInfo {
    uint32_t abi_version;
    uint32_t phase;
    uint32_t talker_position;
    uint32_t semantic_history_count;
    uint64_t frames_generated;
    uint64_t device_sample_count;
    uint64_t host_sync_count;
} Qwen3TtsTalkerStateInfo;

/* reference header :147-151; 16 bytes */
typedef struct Qwen3TtsModelMemory {
    uint64_t shared_weight_bytes;
    uint32_t tensor_count;
    int32_t device_index;
} Qwen3TtsModelMemory;

/* reference header :153-159; 32 bytes */
typedef struct Qwen3TtsSessionMemory {
    uint64_t talker_kv_bytes;
    uint64_t predictor_kv_bytes;
    uint64_t workspace_bytes;
    uint32_t max_sequence_length;
    uint32_t reserved;
} Qwen3TtsSessionMemory;

typedef void* Qwen3TtsModelHandle;
typedef void* Qwen3TtsSessionHandle;

/* reference header :164 (talker.cu:3815) */
QWEN3_TTS_API uint32_t qwen3_tts_talker_abi_version(void);

/* reference header :166-171 (runtime.cu) */
QWEN3_TTS_API int32_t qwen3_tts_probe_device(int32_t device_index, Qwen3TtsDeviceInfo* output,
                                             char* error, size_t error_capacity);

/* reference header :173-180 (runtime.cu:127-255): one-block argmax over a bf16 logit vector whose
 * maximum is planted at token min(1729, V - 1); fails if another token comes back.  CLI only. */
QWEN3_TTS_API int32_t qwen3_tts_benchmark_bf16_argmax(int32_t device_index, int32_t vocabulary_size,
                                                      int32_t iterations,
                                                      Qwen3TtsArgmaxBenchmark* output, char* error,
                                                      size_t error_capacity);

/* reference header :182-190 (gemv.cu:88-270, cuBLAS there): bf16 matrix-vector product on zero-filled
 * operands with a zero-output check, here on this library's own kernel.  CLI only; the int8
 * figure of the decode path is q3t_benchmark_int8_gemv. */
QWEN3_TTS_API int32_t qwen3_tts_benchmark_bf16_gemv(int32_t device_index, int32_t input_features,
                                                    int32_t output_features, int32_t iterations,
                                                    Qwen3TtsGemvBenchmark* output, char* error,
                                                    size_t error_capacity);

/* reference header :192-240 (weights.cu:98-340).  Return codes are the reference's: 0, or -1..-4
 * for the argument checks in the order they are made, or the CUDA error number. */
QWEN3_TTS_API int32_t qwen3_tts_device_buffer_create(int32_t device_index, uint64_t capacity_bytes,
                                                     uint64_t staging_bytes,
                                                     Qwen3TtsDeviceBuffer** output,
                                                     Qwen3TtsWeightUploadMetrics* metrics,
                                                     char* error, size_t error_capacity);
QWEN3_TTS_API int32_t qwen3_tts_device_buffer_upload(Qwen3TtsDeviceBuffer* buffer,
                                                     uint64_t offset_bytes, const void* source,
                                                     uint64_t bytes, char* error,
                                                     size_t error_capacity);
QWEN3_TTS_API int32_t qwen3_tts_device_buffer_finish(Qwen3TtsDeviceBuffer* buffer,
                                                     Qwen3TtsWeightUploadMetrics* metrics,
                                                     char* error, size_t error_capacity);
QWEN3_TTS_API int32_t qwen3_tts_device_buffer_read(Qwen3TtsDeviceBuffer* buffer,
                                                   uint64_t offset_bytes, void* destination,
                                                   uint64_t bytes, char* error,
                                                   size_t error_capacity);
QWEN3_TTS_API const void* qwen3_tts_device_buffer_data(const Qwen3TtsDeviceBuffer* buffer);
QWEN3_TTS_API void qwen3_tts_device_buffer_destroy(Qwen3TtsDeviceBuffer* buffer);

/* reference header :202-207 (primitive_parity.cu:328): runs the four closed-form known-answer
 * cases (RMSNorm, RoPE, attention, SiLU gate) through this library's kernels */
QWEN3_TTS_API int32_t qwen3_tts_validate_transformer_primitives(int32_t device_index,
                                                                Qwen3TtsPrimitiveParity* output,
                                                                char* error, size_t error_capacity);

/* reference header :242-249 (talker.cu:3819-3836) */
QWEN3_TTS_API int32_t qwen3_tts_model_create(int32_t device_index, Qwen3TtsModelHandle* output,
                                             char* error, size_t error_capacity);
QWEN3_TTS_API void qwen3_tts_model_destroy(Qwen3TtsModelHandle handle);

/* reference header :251-260 (talker.cu:434-482): one of the 404 named bf16 tensors.  Decode
 * matrices are quantized to int8 on arrival; the bf16 original is not kept. */
QWEN3_TTS_API int32_t qwen3_tts_model_upload_tensor(Qwen3TtsModelHandle handle, const char* name,
                                                    const void* bf16_data, uint64_t byte_size,
                                                    int32_t rank, const uint64_t* shape,
                                                    char* error, size_t error_capacity);

/* reference header :262-267 (talker.cu:484-680) */
QWEN3_TTS_API int32_t qwen3_tts_model_finalize(Qwen3TtsModelHandle handle,
                                               Qwen3TtsModelMemory* memory, char* error,
                                               size_t error_capacity);

/* reference header :269-286 (talker.cu:792-1034); max_sequence_length in [16, 8192] */
QWEN3_TTS_API int32_t qwen3_tts_session_create(Qwen3TtsModelHandle model,
                                               int32_t max_sequence_length, uint64_t random_seed,
                                               Qwen3TtsSessionHandle* output,
                                               Qwen3TtsSessionMemory* memory, char* error,
                                               size_t error_capacity);
QWEN3_TTS_API void qwen3_tts_session_destroy(Qwen3TtsSessionHandle handle);
QWEN3_TTS_API int32_t qwen3_tts_session_reset(Qwen3TtsSessionHandle handle, uint64_t random_seed,
                                              char* error, size_t error_capacity);

/* reference header :288-297 (talker.cu:1036-1093).  Here the prompt runs through the same
 * int8 decode kernels, one position per step (the reference uses bf16 cuBLAS GEMMs). */
QWEN3_TTS_API int32_t qwen3_tts_session_prefill(Qwen3TtsSessionHandle handle,
                                                const int32_t* text_token_ids,
                                                const int32_t* codec_token_ids,
                                                int32_t token_count,
                                                Qwen3TtsSamplingConfig sampling,
                                                Qwen3TtsTalkerPrefillResult* output, char* error,
                                                size_t error_capacity);

/* reference header :299-311 (talker.cu:1326-1340, 3931-3963) */
QWEN3_TTS_API int32_t qwen3_tts_session_next_frame(
    Qwen3TtsSessionHandle handle, uint16_t semantic_token, int32_t trailing_text_token_id,
    Qwen3TtsSamplingConfig talker_sampling, Qwen3TtsSamplingConfig predictor_sampling,
    uint16_t* output_codes, size_t output_code_capacity, uint16_t* next_semantic_token,
    Qwen3TtsCodecFrameInfo* frame_info, char* error, size_t error_capacity);

/* reference header :313-328 (talker.cu:1095-1262, 3965-3997) */
QWEN3_TTS_API int32_t qwen3_tts_session_next_frame_begin_v2(
    Qwen3TtsSessionHandle handle, int32_t trailing_text_token_id,
    Qwen3TtsSamplingConfig talker_sampling, Qwen3TtsSamplingConfig predictor_sampling,
    Qwen3TtsDeviceFrameViewV2* output, char* error, size_t error_capacity);

/* reference header :330-343 (talker.cu:1264-1324, 3999-4023) */
QWEN3_TTS_API int32_t qwen3_tts_session_next_frame_finish_v2(
    Qwen3TtsSessionHandle handle, uint64_t lease_id, Qwen3TtsCudaEventHandle consumer_done_event,
    uint16_t* next_semantic_token, Qwen3TtsCodecFrameInfo* frame_info, char* error,
    size_t error_capacity);

/* reference header :345-364 (talker.cu:1352-1969, 4025-4072); up to
 * QWEN3_TTS_MAX_BATCH_SESSIONS sessions per call */
QWEN3_TTS_API int32_t qwen3_tts_model_batch_next_frame_begin_v2(
    Qwen3TtsModelHandle model_handle, Qwen3TtsSessionHandle* sessions, int32_t session_count,
    const int32_t* trailing_text_token_ids, const Qwen3TtsSamplingConfig* talker_sampling,
    const Qwen3TtsSamplingConfig* predictor_sampling, Qwen3TtsDeviceFrameViewV2* outputs,
    char* error, size_t error_capacity);

/* reference header :366-371 (talker.cu:3657-3667, 4074-4087) */
QWEN3_TTS_API int32_t qwen3_tts_session_state_info(Qwen3TtsSessionHandle handle,
                                                   Qwen3TtsTalkerStateInfo* output, char* error,
                                                   size_t error_capacity);

#ifdef __cplusplus
}
#endif

#endif /* QWEN3_TTS_NATIVE_H_ */
