// TEST INFRASTRUCTURE ONLY -- not part of the shipped library.
//
// The reference project's talker.cu, compiled where it lies and unmodified, plus two
// extern "C" functions that let a test see and seed the state a session holds after its
// prompt.  The reference's ABI has no call that imports or exports session state, and its
// prompt path (bf16 cuBLAS) differs in rounding from this library's (int8 decode kernels),
// so the only way to hand both libraries the SAME state before the first frame is to write
// it into the reference's session: K/V rows of the prompt, the last hidden row, the first
// semantic token and the sampler's random state.  After that every frame of the reference's
// fused int8 decode path must produce the same 16 codes and next token as this library.
//
// The classes of talker.cu live in an anonymous namespace of that translation unit, so this
// file includes the source itself (resolved through -I<checkout>/native/qwen3-tts-native/
// native/src by build_ref.sh; nothing is copied) with member access opened up by the
// preprocessor.  Every standard, CUDA and cuBLAS header talker.cu uses is included first, so
// the macro reaches the reference's own code only.  Access specifiers do not change layout
// or behaviour.  Linked with the reference's seven other .cu files into
// oracle/_ref/libqwen3_tts_cuda_ref_state.so.
//
// Nothing in the product library links against or loads this file.

#include <cublas_v2.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <array>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <memory>
#include <mutex>
#include <new>
#include <numeric>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "qwen3_tts_native.h"
#include "talker_internal.cuh"

#define private public
#include "talker.cu"
#undef private

extern "C" {

// Device pointers and host scalars of one session, valid until the session is destroyed.
struct Q3tRefSessionState {
    void* keys[28];             // per talker layer: [max_sequence_length][1024] bf16
    void* values[28];
    void* last_hidden;          // [2048] bf16
    void* semantic_history;     // int32 per generated semantic token
    void* random_state;         // uint64
    void* sampled_token;        // int32: the semantic token the next frame starts from
    int32_t position;
    int32_t history_count;
    int32_t max_sequence_length;
    uint32_t current_token;
    uint32_t phase;
};

QWEN3_TTS_API int32_t q3t_ref_session_state(Qwen3TtsSessionHandle handle, Q3tRefSessionState* out) {
    if (handle == nullptr || out == nullptr) return -1;
    TalkerContext* s = static_cast<TalkerContext*>(handle);
    if (s->talker_cache_.size() != 28) return -2;
    for (int layer = 0; layer < 28; ++layer) {
        out->keys[layer] = s->talker_cache_[layer].key.as<void>();
        out->values[layer] = s->talker_cache_[layer].value.as<void>();
    }
    out->last_hidden = s->last_hidden_.as<void>();
    out->semantic_history = s->semantic_history_.as<void>();
    out->random_state = s->random_state_.as<void>();
    out->sampled_token = s->sampled_token_.as<void>();
    out->position = s->position_;
    out->history_count = s->generated_semantic_count_;
    out->max_sequence_length = s->max_sequence_length_;
    out->current_token = s->current_semantic_token_;
    out->phase = static_cast<uint32_t>(s->phase_);
    return 0;
}

// The token the next frame has to be begun with (the caller also writes it to
// semantic_history[history_count - 1] and to sampled_token on the device).
QWEN3_TTS_API int32_t q3t_ref_session_set_current_token(Qwen3TtsSessionHandle handle, uint32_t token) {
    if (handle == nullptr || token >= 3072u || token == 2150u) return -1;
    TalkerContext* s = static_cast<TalkerContext*>(handle);
    s->current_semantic_token_ = static_cast<uint16_t>(token);
    s->phase_ = QWEN3_TTS_TALKER_PREFILLED;
    return 0;
}

}  // extern "C"
