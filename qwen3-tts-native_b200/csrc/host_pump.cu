// A compiled host loop over the public frame ABI, for measuring the library the way the
// reference's host drives it.
//
// The reference's host is compiled Rust: per frame its runtime calls
// qwen3_tts_model_batch_next_frame_begin_v2 once for the lockstep batch and
// qwen3_tts_session_next_frame_finish_v2 once per session
// (native/qwen3-tts-native/src/native_talker.rs:314-380, session_bench.rs:180-260), or
// qwen3_tts_session_next_frame for a single session.  This file is that loop in C++, calling the
// same exported functions and nothing else, so that an end-to-end figure does not carry the cost
// of an interpreter between the calls.  It is not part of the decode path.

#include "../../include/q3t_ops.h"

#include <chrono>
#include <cstdio>
#include <cstring>
#include <vector>

extern "C" int32_t q3t_host_pump_frames(Qwen3TtsModelHandle model, Qwen3TtsSessionHandle* sessions,
                                        int32_t session_count, int32_t frames,
                                        int32_t trailing_text_token_id,
                                        Qwen3TtsSamplingConfig talker_sampling,
                                        Qwen3TtsSamplingConfig predictor_sampling,
                                        uint16_t* last_tokens, double* wall_milliseconds,
                                        char* error, size_t error_capacity) {
    if (model == nullptr || sessions == nullptr || session_count < 1
        || session_count > QWEN3_TTS_MAX_BATCH_SESSIONS || frames < 1) {
        if (error != nullptr && error_capacity > 0) {
            std::snprintf(error, error_capacity, "host pump arguments are null or out of range");
        }
        return QWEN3_TTS_TALKER_STATUS_INVALID_ARGUMENT;
    }
    const int n = session_count;
    std::vector<int32_t> trailing(n, trailing_text_token_id);
    std::vector<Qwen3TtsSamplingConfig> talker(n, talker_sampling), predictor(n, predictor_sampling);
    std::vector<Qwen3TtsDeviceFrameViewV2> views(n);
    std::vector<uint16_t> tokens(n, 0);
    if (n == 1) {
        const int32_t rc = q3t_session_current_token(sessions[0], &tokens[0], error, error_capacity);
        if (rc != QWEN3_TTS_TALKER_STATUS_OK) return rc;
    }
    const auto start = std::chrono::steady_clock::now();
    for (int f = 0; f < frames; ++f) {
        if (n == 1) {
            uint16_t codes[16];
            uint16_t next = 0;
            Qwen3TtsCodecFrameInfo info;
            const int32_t rc = qwen3_tts_session_next_frame(sessions[0], tokens[0], trailing_text_token_id,
                                                            talker_sampling, predictor_sampling, codes, 16,
                                                            &next, &info, error, error_capacity);
            if (rc != QWEN3_TTS_TALKER_STATUS_OK) return rc;
            tokens[0] = next;
            continue;
        }
        for (int i = 0; i < n; ++i) {
            std::memset(&views[i], 0, sizeof(views[i]));
            views[i].struct_size = sizeof(Qwen3TtsDeviceFrameViewV2);
        }
        int32_t rc = qwen3_tts_model_batch_next_frame_begin_v2(model, sessions, n, trailing.data(), talker.data(),
                                                               predictor.data(), views.data(), error,
                                                               error_capacity);
        if (rc != QWEN3_TTS_TALKER_STATUS_OK) return rc;
        for (int i = 0; i < n; ++i) {
            Qwen3TtsCodecFrameInfo info;
            rc = qwen3_tts_session_next_frame_finish_v2(sessions[i], views[i].lease_id, nullptr, &tokens[i], &info,
                                                        error, error_capacity);
            if (rc != QWEN3_TTS_TALKER_STATUS_OK) return rc;
        }
    }
    const auto stop = std::chrono::steady_clock::now();
    if (wall_milliseconds != nullptr) {
        *wall_milliseconds = std::chrono::duration<double, std::milli>(stop - start).count();
    }
    if (last_tokens != nullptr) std::memcpy(last_tokens, tokens.data(), sizeof(uint16_t) * n);
    return QWEN3_TTS_TALKER_STATUS_OK;
}
