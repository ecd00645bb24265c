/*
 * Operator-level C ABI of libqwen3_tts_cuda.so (additive to qwen3_tts_native.h).
 *
 * The reference keeps its kernel launchers C++-internal (namespace qwen3_tts,
 * native/qwen3-tts-native/native/src/talker_internal.cuh); these entry points expose the
 * sm_100a replacements one by one with the same names, argument order and meaning, so that
 * each operator can be driven, checked and timed on its own.  Differences from the
 * reference's launchers: C linkage and a q3t_ prefix; bf16 tensors are passed as
 * uint16_t bit patterns; `stream` is a cudaStream_t passed as void*; `rows` may go up to
 * Q3T_MAX_ROWS (the reference stops at 8); the return value is the cudaError_t of the
 * launch as int32_t (0 = cudaSuccess, 1 = cudaErrorInvalidValue for rejected arguments).
 * All pointers are DEVICE pointers unless the name says host.  Nothing here allocates
 * device memory except q3t_benchmark_int8_gemv.
 */
#ifndef Q3T_OPS_H_
#define Q3T_OPS_H_

#include "qwen3_tts_native.h"

#ifdef __cplusplus
extern "C" {
#endif

#define Q3T_MAX_ROWS 64
#define Q3T_KV_PAGE_TOKENS 16
#define Q3T_ATTENTION_CHUNK 64

/* ---- int8 weight-only GEMV / skinny GEMM --------------------------------------------- */

/* talker_internal.cuh launch_int8_gemm_rows (int8_gemv.cu:319-368):
 * y[r][n] = bf16(scales[n] * sum_k w[n][k] * x[r][k]); w int8 [out][in] row-major. */
QWEN3_TTS_API int32_t q3t_launch_int8_gemm_rows(const int8_t* weight, const float* scales,
                                                const uint16_t* input, uint16_t* output,
                                                int32_t in_features, int32_t out_features,
                                                int32_t rows, void* stream);

/* launch_int8_gemm_rows_add (int8_gemv.cu:370-395): output += result (residual epilogue) */
QWEN3_TTS_API int32_t q3t_launch_int8_gemm_rows_add(const int8_t* weight, const float* scales,
                                                    const uint16_t* input, uint16_t* output,
                                                    int32_t in_features, int32_t out_features,
                                                    int32_t rows, void* stream);

/* launch_int8_gate_up_silu_rows (int8_gemv.cu:397-422): weight [2*out][in], gate rows first;
 * output = bf16(silu(gate) * up) */
QWEN3_TTS_API int32_t q3t_launch_int8_gate_up_silu_rows(const int8_t* weight, const float* scales,
                                                        const uint16_t* input, uint16_t* output,
                                                        int32_t in_features, int32_t out_features,
                                                        int32_t rows, void* stream);

/* Fused form used by the frame engine.  No counterpart in the reference, which launches the
 * RMSNorm (talker_kernels.cu:27-48), the GEMM and the bias/activation/add kernels
 * (talker_kernels.cu:660-678, 359-371) separately. */
enum {
    Q3T_EPI_PLAIN = 0,
    Q3T_EPI_ADD = 1,
    Q3T_EPI_BIAS = 2,        /* y = bf16(bf16(acc*scale) + bias) */
    Q3T_EPI_BIAS_SILU = 3,   /* v = bf16(acc*scale) + bias; y = bf16(v * 1/(1+exp(-v))) */
    Q3T_EPI_BIAS_ADD = 4,    /* t = bf16(bf16(acc*scale) + bias); residual = bf16(residual + t) */
    Q3T_EPI_GATE_UP_SILU = 5
};
typedef struct Q3tGemmDesc {
    uint32_t struct_size;        /* sizeof(Q3tGemmDesc) */
    int32_t epilogue;
    const int8_t* weight;
    const float* scales;
    const uint16_t* input;       /* [rows][in_features] */
    uint16_t* output;            /* [rows][out_features] */
    float* output_f32;           /* optional: the fp32 value before the last bf16 round */
    const uint16_t* norm_weight; /* optional: RMSNorm(input) * norm_weight feeds the GEMM */
    uint16_t* norm_output;       /* optional: the normalized rows */
    const uint16_t* bias;        /* bias epilogues */
    uint16_t* residual;          /* Q3T_EPI_BIAS_ADD */
    int32_t in_features;
    int32_t out_features;
    int32_t rows;
    float epsilon;
} Q3tGemmDesc;
QWEN3_TTS_API int32_t q3t_launch_int8_gemm_ex(const Q3tGemmDesc* desc, void* stream);

/* launch_quantize_weight_rows (int8_gemv.cu:302-317) */
QWEN3_TTS_API int32_t q3t_launch_quantize_weight_rows(const uint16_t* weight, int8_t* quantized,
                                                      float* scales, int32_t in_features,
                                                      int32_t out_features, void* stream);

/* Mirrors qwen3_tts_benchmark_bf16_gemv (gemv.cu) for the int8 kernel: `buffers` distinct
 * weight images (choose buffers*in*out > L2) are streamed round-robin for `iterations`
 * launches; tera_operations_per_second counts 2*in*out*rows per launch. */
QWEN3_TTS_API int32_t q3t_benchmark_int8_gemv(int32_t device_index, int32_t input_features,
                                              int32_t output_features, int32_t rows,
                                              int32_t buffers, int32_t iterations,
                                              Qwen3TtsGemvBenchmark* output, char* error,
                                              size_t error_capacity);

/* The reference host's per-frame call sequence as a compiled loop, for end-to-end timing without
 * an interpreter between the calls: qwen3_tts_model_batch_next_frame_begin_v2 + one
 * qwen3_tts_session_next_frame_finish_v2 per session (native_talker.rs:314-380), or
 * qwen3_tts_session_next_frame when session_count is 1.  Uses only exported functions.
 * wall_milliseconds: host clock around the loop; last_tokens: [session_count] next semantic tokens. */
QWEN3_TTS_API int32_t q3t_host_pump_frames(Qwen3TtsModelHandle model, Qwen3TtsSessionHandle* sessions,
                                           int32_t session_count, int32_t frames,
                                           int32_t trailing_text_token_id,
                                           Qwen3TtsSamplingConfig talker_sampling,
                                           Qwen3TtsSamplingConfig predictor_sampling,
                                           uint16_t* last_tokens, double* wall_milliseconds,
                                           char* error, size_t error_capacity);

/* The host's lockstep rendezvous (BatchFramePump, native_talker.rs:267-401) in C++, for up to 64
 * sessions: owner threads call q3t_pump_begin_frame; a worker thread gathers the requests of the
 * registered (decoding) sessions, up to max_batch or until gather_window_microseconds after the
 * first one (the reference waits 2 ms), and begins them with one
 * qwen3_tts_model_batch_next_frame_begin_v2.  Each owner finishes its own lease with
 * qwen3_tts_session_next_frame_finish_v2.  frames_emitted == 0 bypasses the rendezvous
 * (native_talker.rs:1426-1431): the first frame is begun on the caller's thread. */
typedef struct Q3tFramePump Q3tFramePump;
QWEN3_TTS_API int32_t q3t_pump_create(Qwen3TtsModelHandle model, int32_t max_batch,
                                      int32_t gather_window_microseconds, Q3tFramePump** output,
                                      char* error, size_t error_capacity);
QWEN3_TTS_API void q3t_pump_destroy(Q3tFramePump* pump);
QWEN3_TTS_API void q3t_pump_register(Q3tFramePump* pump);
QWEN3_TTS_API void q3t_pump_unregister(Q3tFramePump* pump);
QWEN3_TTS_API int32_t q3t_pump_begin_frame(Q3tFramePump* pump, Qwen3TtsSessionHandle session,
                                           int32_t frames_emitted, int32_t trailing_text_token_id,
                                           Qwen3TtsSamplingConfig talker_sampling,
                                           Qwen3TtsSamplingConfig predictor_sampling,
                                           Qwen3TtsDeviceFrameViewV2* output, char* error,
                                           size_t error_capacity);
QWEN3_TTS_API int32_t q3t_pump_statistics(Q3tFramePump* pump, uint64_t* batches, uint64_t* frames);
/* Placement of a new session over the GPUs of one host: fewest active sessions, lowest index
 * first (sessions are pinned for life, docs/ARCHITECTURE.md:285 of the reference). */
QWEN3_TTS_API int32_t q3t_pick_device(const int32_t* active_sessions_per_device, int32_t devices);

/* ---- hand-over of finished frames to the codec ------------------------------------------------
 * The reference host's CudaPacketStager (native/qwen3-tts-runtime/src/cuda_packet_stager.rs:167-340)
 * as a C object: one per session, on the session's GPU.  stage_frame copies the 16 codes of a frame
 * begun with *_next_frame_begin_v2 from the talker's device buffer into the next slot of a 128-byte
 * packet (up to 4 frames), ordered behind the frame's ready event, and returns the event to pass to
 * qwen3_tts_session_next_frame_finish_v2 as consumer_done_event.  packet_view is what the codec
 * reads (after ready_event); release_after_consumer orders the next packet behind the codec's own
 * event and empties the packet.  Return codes: 0 ok, 1 refused (message says why; same refusals as
 * the reference), 2 a CUDA call failed (the stager is poisoned and refuses everything after). */
typedef struct Q3tPacketStager Q3tPacketStager;
typedef struct Q3tStagedPacketView {
    const uint16_t* device_codes;   /* [frame_count][16] */
    uint64_t frame_count;
    void* ready_event;              /* cudaEvent_t */
} Q3tStagedPacketView;
QWEN3_TTS_API Q3tPacketStager* q3t_packet_stager_create(int32_t device_index, char* error, size_t error_capacity);
QWEN3_TTS_API void q3t_packet_stager_destroy(Q3tPacketStager* stager);
QWEN3_TTS_API uint64_t q3t_packet_stager_device_bytes(const Q3tPacketStager* stager);
QWEN3_TTS_API int32_t q3t_packet_stager_staged_frames(const Q3tPacketStager* stager);
QWEN3_TTS_API int32_t q3t_packet_stager_stage_frame(Q3tPacketStager* stager, const uint16_t* device_codes,
                                                    size_t code_count, void* producer_ready_event,
                                                    int32_t source_device, void** copied_event, char* error,
                                                    size_t error_capacity);
QWEN3_TTS_API int32_t q3t_packet_stager_packet_view(const Q3tPacketStager* stager, Q3tStagedPacketView* view,
                                                    char* error, size_t error_capacity);
QWEN3_TTS_API int32_t q3t_packet_stager_release_after_consumer(Q3tPacketStager* stager,
                                                               void* consumer_done_event, char* error,
                                                               size_t error_capacity);

/* ---- weight image -------------------------------------------------------------------------
 * The reference quantizes every decode matrix on every GPU while the checkpoint is uploaded
 * (talker.cu:564-668, int8_gemv.cu:20-52).  With one replica per GPU the work can be done once:
 * the rank that received the bf16 checkpoint through qwen3_tts_model_upload_tensor exposes where
 * each tensor lives on its device in decode form (int8 rows + fp32 row scales for the projection
 * matrices, bf16 for norms, biases and embeddings); the other ranks ask their own, still empty,
 * model for the same tensor's storage, fill it (ncclBroadcast, a peer copy, a file read) and
 * declare it loaded.  qwen3_tts_model_finalize then accepts the model as if every tensor had been
 * uploaded.  Stacked matrices (q/k/v, gate/up) are addressed by their checkpoint names; each
 * name is a contiguous row range of the stacked storage. */
typedef struct Q3tTensorImage {
    uint32_t struct_size;      /* sizeof(Q3tTensorImage), set by the caller */
    int32_t device_index;
    void* data;                /* device pointer */
    uint64_t data_bytes;
    float* scales;             /* device pointer, null unless quantized */
    uint64_t scales_bytes;
    int32_t quantized;         /* 1: data is int8 [rows][cols], scales is fp32 [rows] */
    int32_t loaded;            /* 1: uploaded or adopted already */
} Q3tTensorImage;
QWEN3_TTS_API int32_t q3t_model_tensor_image(Qwen3TtsModelHandle model, const char* name,
                                             Q3tTensorImage* image, char* error, size_t error_capacity);
/* Declares the tensor's device storage filled by the caller; counts like an upload (a second
 * upload or adoption of the same name is an error, as in the reference's upload path). */
QWEN3_TTS_API int32_t q3t_model_adopt_tensor(Qwen3TtsModelHandle model, const char* name, char* error,
                                             size_t error_capacity);

/* Which kernel takes projections of 1..8 rows (process-wide; returns the previous mode):
 *   0  the SIMT kernel only: the summation order of the reference's int8_dequant_gemm_kernel
 *      (int8_gemv.cu:58-128), outputs bit-identical to it;
 *   1  (default) the int8 tensor-core kernel where the shape allows (K = 512 * {2, 4, 6, 12}; with a
 *      fused RMSNorm K = 512 * {2, 4}): activations as three byte limbs of a per-row fixed-point
 *      value, exact integer products and sums (agreement ~1e-7 relative, a row's result bitwise
 *      independent of the rows beside it), weights bulk-copied ahead of the launch dependency;
 * Also reachable as model option "gemv_mode" and as QWEN3_TTS_B1_GEMV=simt at load time.
 * No reference counterpart (one kernel there). */
QWEN3_TTS_API int32_t q3t_set_gemv_mode(int32_t mode);

/* Test hook, host arithmetic only (works without a GPU): the shared-memory plan the mode-1 kernel
 * would give one launch of `rows` rows of this shape.  Returns 1 and fills fields[0..7] = grid, stages,
 * tile group, tiles per CTA, rows one launch takes for this shape, bytes of a full stage, bytes of the
 * weight ring, dynamic shared memory of the launch; returns 0 when the kernel does not take the shape. */
QWEN3_TTS_API int32_t q3t_test_gemv_plan(int32_t in_features, int32_t out_features, int32_t rows,
                                         int32_t gate_up, int32_t norm, int64_t* fields);

/* Which kernel computes decode attention (process-wide; returns the previous mode):
 *   1  (default) the split-KV kernel: tensor-core products, chunked fp32 sums; within 1e-3 of the
 *      reference's batch_causal_gqa_attention_fast_kernel (talker_kernels.cu:506-595) on the fp32 value;
 *   0  parity mode: every fp32 sum in that kernel's order, bf16 output bit-identical to it; one
 *      thread walks a whole cache row, so it is slow.  Positions must be below 8192.
 * With gemv mode 0 and "tc_min_rows" 65 every operator of a frame is then bit-identical to the
 * reference's.  Also reachable as model option "attention_mode". */
QWEN3_TTS_API int32_t q3t_set_attention_mode(int32_t mode);

/* Operator-level attention case for profiling: `rows` sessions with KV lengths uniform in
 * [min_length, max_length] (seeded), 16 query / 8 KV heads of 128, paged bf16 caches of N(0,1);
 * `iterations` launches in the attention mode in force, timed with CUDA events on their stream.
 * *kv_bytes = the K and V bytes one launch reads (the algorithmic traffic). */
QWEN3_TTS_API int32_t q3t_benchmark_decode_attention(int32_t device_index, int32_t rows, int32_t min_length,
                                                     int32_t max_length, uint64_t seed, int32_t iterations,
                                                     float* mean_launch_microseconds, uint64_t* kv_bytes,
                                                     char* error, size_t error_capacity);

/* ---- norms, RoPE, KV append, glue (talker_kernels.cu) --------------------------------- */

QWEN3_TTS_API int32_t q3t_launch_rms_norm_rows(const uint16_t* input, const uint16_t* weight,
                                               uint16_t* output, int32_t rows, int32_t width,
                                               float epsilon, void* stream);              /* :27-48 */
QWEN3_TTS_API int32_t q3t_launch_head_rms_norm_rows(uint16_t* values, const uint16_t* weight,
                                                    int32_t rows, int32_t heads,
                                                    int32_t head_dimension, float epsilon,
                                                    void* stream);                          /* :50-70 */
QWEN3_TTS_API int32_t q3t_launch_rope_rows_at(uint16_t* values, int32_t rows, int32_t heads,
                                              int32_t head_dimension, const int32_t* positions,
                                              float theta, void* stream);                  /* :597-639 */
QWEN3_TTS_API int32_t q3t_launch_kv_scatter_rows(const uint16_t* rows_data,
                                                 uint16_t* const* cache_bases,
                                                 const int32_t* positions, int32_t rows,
                                                 int32_t width, void* stream);             /* :641-658 */
QWEN3_TTS_API int32_t q3t_launch_bias_activation_rows(uint16_t* values, const uint16_t* bias,
                                                      int32_t rows, int32_t width, int32_t silu,
                                                      void* stream);                       /* :660-678 */
QWEN3_TTS_API int32_t q3t_launch_add_in_place(uint16_t* destination, const uint16_t* source,
                                              int32_t width, void* stream);                /* :359-371 */
QWEN3_TTS_API int32_t q3t_launch_silu_gate(uint16_t* gate, const uint16_t* up, int32_t width,
                                           void* stream);                                  /* :405-421 */
QWEN3_TTS_API int32_t q3t_launch_gather_embedding_rows(const uint16_t* table, int32_t vocabulary,
                                                       int32_t width, const int32_t* const* tokens,
                                                       int32_t token_offset, uint16_t* output,
                                                       int32_t rows, void* stream);        /* :680-709 */
QWEN3_TTS_API int32_t q3t_launch_add_embedding_rows(const uint16_t* table, int32_t vocabulary,
                                                    int32_t width, const int32_t* const* tokens,
                                                    int32_t token_offset, uint16_t* output,
                                                    int32_t rows, void* stream);           /* :680-709 */

/* ---- decode attention ------------------------------------------------------------------ */

/* Bytes of scratch a decode-attention launch needs for rows whose lengths do not exceed
 * max_sequence_length (ticket counters followed by split-KV partials). */
QWEN3_TTS_API size_t q3t_attention_scratch_bytes(int32_t rows, int32_t query_heads,
                                                 int32_t key_value_heads, int32_t head_dimension,
                                                 int32_t max_sequence_length);

/* launch_batch_causal_gqa_attention_fast (talker_kernels.cu:506-595, 1024-1044): per-row
 * contiguous caches [position][kv_heads][head_dim]; row r attends positions 0..positions[r].
 * Extra arguments: the scratch buffer above (the reference kernel needs none). */
QWEN3_TTS_API int32_t q3t_launch_batch_causal_gqa_attention_fast(
    const uint16_t* query, uint16_t* const* key_bases, uint16_t* const* value_bases,
    const int32_t* positions, uint16_t* output, int32_t rows, int32_t query_heads,
    int32_t key_value_heads, int32_t head_dimension, int32_t max_sequence_length, void* scratch,
    size_t scratch_bytes, void* stream);

/* Positions are read from the caller's device memory and must lie in [0, max_sequence_length) (the
 * scratch, the grid and the per-row ticket counts are sized from max_sequence_length).  A row whose
 * position lies outside is computed over the clamped length instead of running past them, and is
 * counted (process-wide) in q3t_attention_range_error_count(): a caller that cannot vouch for its
 * positions compares that counter before and after. */
QWEN3_TTS_API uint32_t q3t_attention_range_error_count(void);

/* No counterpart in the reference.  The same operator for hosts that may not allocate device
 * memory where they run it (a real-time audio thread, a process with a fixed, policed memory
 * budget, a plugin that is lent streams and buffers only): the scratch lives in a 4 MiB array
 * built into the library's device image, so the caller passes inputs and outputs and nothing
 * else, and the call itself allocates nothing.  Shapes that need more scratch than the array holds
 * (see q3t_attention_scratch_bytes) are rejected with STATUS_INVALID_ARGUMENT and a message.
 * The first call on a device resolves the array's device address; make it before any stream
 * capture.  All calls on a device share the array: calls that overlap on the GPU race.
 * Returns a QWEN3_TTS_TALKER_STATUS_* code; `error` follows the convention of qwen3_tts_native.h. */
QWEN3_TTS_API int32_t q3t_launch_batch_causal_gqa_attention_fast_noalloc(
    const uint16_t* query, uint16_t* const* key_bases, uint16_t* const* value_bases,
    const int32_t* positions, uint16_t* output, int32_t rows, int32_t query_heads,
    int32_t key_value_heads, int32_t head_dimension, int32_t max_sequence_length, void* stream,
    char* error, size_t error_capacity);

/* Bytes of the built-in scratch array used by the _noalloc entry point. */
QWEN3_TTS_API size_t q3t_attention_static_scratch_capacity(void);

/* Full form: paged KV and/or the fused per-head RMSNorm + RoPE + KV append, which the reference
 * issues as launch_head_rms_norm_rows x2, launch_rope_rows_at x2, launch_kv_scatter_rows x2
 * (talker.cu:2101-2175) before the attention launch.
 * Paged caches: a page holds Q3T_KV_PAGE_TOKENS tokens of one plane (K or V) of one layer as
 * [key_value_heads][Q3T_KV_PAGE_TOKENS][head_dimension] bf16, i.e. head-major: the tokens of one KV
 * head are contiguous.  (The reference's caches are contiguous per session, [position][kv width];
 * the paged layout has no counterpart there.) */
typedef struct Q3tAttentionDesc {
    uint32_t struct_size;        /* sizeof(Q3tAttentionDesc) */
    int32_t fused;               /* 1: q/key_new are raw projections; normalize, rotate, append */
    const uint16_t* query;       /* [rows][query_stride] */
    const uint16_t* key_new;     /* fused: [rows][new_stride] */
    const uint16_t* value_new;
    const uint16_t* query_norm_weight;   /* fused: [head_dimension] */
    const uint16_t* key_norm_weight;
    const int32_t* positions;    /* [rows] */
    uint16_t* output;            /* [rows][query_heads*head_dimension] */
    float* output_f32;           /* optional fp32 value before the last bf16 round */
    uint16_t* const* key_bases;  /* contiguous caches, or NULL when paged */
    uint16_t* const* value_bases;
    const int32_t* page_table;   /* paged: [rows][page_table_stride] page ids */
    uint16_t* const* slabs;      /* paged: slab base pointers */
    int64_t page_elements;       /* paged: elements between consecutive pages of a plane */
    int64_t key_offset;          /* paged: element offset of the K plane inside a slab */
    int64_t value_offset;
    int32_t page_table_stride;
    int32_t slab_shift;          /* paged: page id >> slab_shift selects the slab */
    int32_t query_stride;        /* 0: query_heads*head_dimension */
    int32_t new_stride;          /* 0: key_value_heads*head_dimension */
    int32_t rows;
    int32_t query_heads;
    int32_t key_value_heads;
    int32_t head_dimension;      /* 32 (not fused), 64, 128 */
    int32_t max_sequence_length;
    float epsilon;
    float theta;
    void* scratch;
    size_t scratch_bytes;
} Q3tAttentionDesc;
QWEN3_TTS_API int32_t q3t_launch_decode_attention_ex(const Q3tAttentionDesc* desc, void* stream);

/* ---- sampler (sampling_kernels.cu) ------------------------------------------------------- */

/* launch_sample_logits (sampling_kernels.cu:460-498) */
QWEN3_TTS_API int32_t q3t_launch_sample_logits(
    const uint16_t* logits, int32_t vocabulary, int32_t suppress_talker_reserved,
    int32_t codec_eos_token, const int32_t* semantic_history, int32_t semantic_history_count,
    int32_t do_sample, int32_t top_k, float top_p, float temperature, float repetition_penalty,
    uint64_t* random_state, int32_t* selected_token, void* stream);

/* launch_sample_logits_at (sampling_kernels.cu:500-538): the history count is read from device */
QWEN3_TTS_API int32_t q3t_launch_sample_logits_at(
    const uint16_t* logits, int32_t vocabulary, int32_t suppress_talker_reserved,
    int32_t codec_eos_token, const int32_t* semantic_history, const int32_t* semantic_history_count,
    int32_t do_sample, int32_t top_k, float top_p, float temperature, float repetition_penalty,
    uint64_t* random_state, int32_t* selected_token, void* stream);

/* ---- engine extras --------------------------------------------------------------------- */

/* Options: "mask_eos" (1: the talker sampler also masks EOS, for synthetic weights whose
 * logits would otherwise end a run at random), "use_graphs" (0: launch kernels one by one),
 * "batch_host_codes" (1: lockstep batches also mirror each frame's 16 codes to host memory),
 * "gemv_mode" (process-wide, see q3t_set_gemv_mode),
 * "attention_mode" (process-wide, see q3t_set_attention_mode),
 * "tc_min_rows" (process-wide: projections with at least this many rows run on the tensor
 * cores, default 9; 65 keeps every row count on the SIMT kernels, whose results do not depend on
 * the batch size), "prefill_chunk" (prompt positions per decoder pass, 1..64, default 64: a
 * prompt runs as the rows of skinny GEMMs instead of position by position (talker.cu:2750-3249
 * is the reference's prompt path); 1 restores the position-by-position path). */
QWEN3_TTS_API int32_t q3t_model_set_option(Qwen3TtsModelHandle model, const char* key,
                                           int32_t value, char* error, size_t error_capacity);

/* Frame loop without a host round trip per frame: `frames` codec frames for each of the
 * `session_count` prefilled sessions, enqueued back to back; returns after the last one.
 * frame_milliseconds (host, [frames], optional) receives each frame's GPU time,
 * total_milliseconds (host, optional) the whole loop's.  Session state afterwards is as if
 * begin/finish had been called `frames` times (an EOS inside the loop is not acted on). */
QWEN3_TTS_API int32_t q3t_model_run_frames(Qwen3TtsModelHandle model,
                                           Qwen3TtsSessionHandle* sessions, int32_t session_count,
                                           int32_t frames, int32_t trailing_text_token_id,
                                           Qwen3TtsSamplingConfig talker_sampling,
                                           Qwen3TtsSamplingConfig predictor_sampling,
                                           float* frame_milliseconds, float* total_milliseconds,
                                           char* error, size_t error_capacity);

/* Benchmark harness: puts a READY session into the PREFILLED phase at `position` without a
 * prompt.  KV rows [0, position) and the last hidden state get seeded pseudo-random N(0,1)
 * values, the semantic history one token (the benchmark configurations ask for a KV cache
 * "pre-filled with N(0,1) values"; values do not influence timing). */
QWEN3_TTS_API int32_t q3t_session_synthetic_prefill(Qwen3TtsSessionHandle session, int32_t position,
                                                    uint64_t seed, char* error,
                                                    size_t error_capacity);

/* The semantic token the next frame of the session will expand (what the reference's host
 * tracks from the prefill result and each finished frame; needed after q3t_model_run_frames). */
QWEN3_TTS_API int32_t q3t_session_current_token(Qwen3TtsSessionHandle session, uint16_t* token,
                                                char* error, size_t error_capacity);

/* Health counter: how many bounded device-side waits (mbarrier waits of the bulk-copy GEMVs and
 * of the tensor-core GEMM)
 * have run out since the library was loaded.  0 on a healthy run; kernels never spin forever. */
QWEN3_TTS_API uint32_t q3t_kernel_error_count(void);

/* Host-side fault injection for tests of the failure paths (a failed enqueue poisons the session,
 * talker.cu:1245-1252; in a lockstep batch every session of it, talker.cu:1946-1956; a failed
 * allocation is STATUS_ALLOCATION).  Nothing here makes a GPU fault: the engine is told that a call
 * failed.  fail_launch_after(n): the n-th kernel launch the engine enqueues from now on reports a
 * launch failure (n = 1: the next one; 0 disarms).  fail_allocation_after(n): likewise for device
 * allocations.  report_device_wait_failure(device): bumps, from the host, the word that a bounded
 * device-side wait bumps when it runs out; the calls in flight on that device then end with
 * STATUS_CUDA and poisoned sessions.  Process-wide, for single-threaded tests. */
QWEN3_TTS_API void q3t_test_fail_launch_after(int32_t launches);
QWEN3_TTS_API void q3t_test_fail_allocation_after(int32_t allocations);
QWEN3_TTS_API int32_t q3t_test_report_device_wait_failure(int32_t device_index);

/* Number of this library's kernels launched so far through frame graphs of the model. */
QWEN3_TTS_API int32_t q3t_model_kernel_launches(Qwen3TtsModelHandle model, uint64_t* launches,
                                                char* error, size_t error_capacity);

/* Test hook: host copies of a session's device state (any pointer may be NULL):
 * last_hidden [2048] bf16, frame_tokens [16], random_state [1]. */
QWEN3_TTS_API int32_t q3t_session_read_state(Qwen3TtsSessionHandle session, uint16_t* last_hidden,
                                             int32_t* frame_tokens, uint64_t* random_state,
                                             char* error, size_t error_capacity);

/* Test hook: the talker K and V rows of positions [first_position, first_position + count) of one
 * layer as the session's cache holds them (K after its head norm and rotation), copied to host
 * memory as [count][1024] bf16 each; either pointer may be NULL. */
QWEN3_TTS_API int32_t q3t_session_read_kv(Qwen3TtsSessionHandle session, int32_t layer,
                                          int32_t first_position, int32_t count, uint16_t* keys,
                                          uint16_t* values, char* error, size_t error_capacity);

#ifdef __cplusplus
}
#endif

#endif /* Q3T_OPS_H_ */
