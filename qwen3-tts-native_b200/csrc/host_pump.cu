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

#include <algorithm>
#include <chrono>
#include <new>
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

// ---------------------------------------------------------------------------------------------
// The lockstep rendezvous of the reference's host (BatchFramePump, native_talker.rs:267-401) in C++:
// session-owner threads ask for their next frame; a worker thread gathers the requests of the
// sessions that are decoding (registered), up to the batch limit or until a gather window has
// passed since the first one, and begins them as one lockstep batch.  Each owner then finishes its
// own lease as usual.  A session's first frame does not wait for the others (native_talker.rs:
// 1426-1431): it is begun on the caller's thread through the single-session entry point.

#include <atomic>
#include <condition_variable>
#include <deque>
#include <mutex>
#include <string>
#include <thread>

namespace {

struct PumpRequest {
    Qwen3TtsSessionHandle session = nullptr;
    int32_t trailing = 0;
    Qwen3TtsSamplingConfig talker{}, predictor{};
    Qwen3TtsDeviceFrameViewV2 view{};
    int32_t status = 0;
    std::string message;
    bool done = false;
    std::condition_variable ready;
};

}  // namespace

struct Q3tFramePump {
    Qwen3TtsModelHandle model = nullptr;
    int max_batch = 8;
    std::chrono::microseconds window{2000};
    std::atomic<int> registered{0};
    std::mutex lock;
    std::condition_variable arrived;
    std::deque<PumpRequest*> queue;
    bool closing = false;
    std::thread worker;
    uint64_t batches = 0, frames = 0;

    void run() {
        std::unique_lock<std::mutex> hold(lock);
        for (;;) {
            arrived.wait(hold, [&] { return closing || !queue.empty(); });
            if (queue.empty()) return;      // closing and drained
            const auto deadline = std::chrono::steady_clock::now() + window;
            for (;;) {
                const int expected = std::min(std::max(registered.load(std::memory_order_relaxed), 1), max_batch);
                if (static_cast<int>(queue.size()) >= expected || closing) break;
                if (arrived.wait_until(hold, deadline) == std::cv_status::timeout) break;
            }
            std::vector<PumpRequest*> batch;
            while (!queue.empty() && static_cast<int>(batch.size()) < max_batch) {
                batch.push_back(queue.front());
                queue.pop_front();
            }
            hold.unlock();
            begin(batch);
            hold.lock();
            ++batches;
            frames += batch.size();
            for (PumpRequest* r : batch) {
                r->done = true;
                r->ready.notify_one();
            }
        }
    }

    void begin(std::vector<PumpRequest*>& batch) {
        const int n = static_cast<int>(batch.size());
        std::vector<Qwen3TtsSessionHandle> sessions(n);
        std::vector<int32_t> trailing(n);
        std::vector<Qwen3TtsSamplingConfig> talker(n), predictor(n);
        std::vector<Qwen3TtsDeviceFrameViewV2> views(n);
        for (int i = 0; i < n; ++i) {
            sessions[i] = batch[i]->session;
            trailing[i] = batch[i]->trailing;
            talker[i] = batch[i]->talker;
            predictor[i] = batch[i]->predictor;
            std::memset(&views[i], 0, sizeof(views[i]));
            views[i].struct_size = sizeof(Qwen3TtsDeviceFrameViewV2);
        }
        char error[512];
        error[0] = 0;
        const int32_t rc = qwen3_tts_model_batch_next_frame_begin_v2(model, sessions.data(), n, trailing.data(),
                                                                     talker.data(), predictor.data(), views.data(),
                                                                     error, sizeof(error));
        for (int i = 0; i < n; ++i) {
            batch[i]->status = rc;
            batch[i]->view = views[i];
            if (rc != QWEN3_TTS_TALKER_STATUS_OK) batch[i]->message = error;
        }
    }
};

extern "C" {

int32_t q3t_pump_create(Qwen3TtsModelHandle model, int32_t max_batch, int32_t gather_window_microseconds,
                        Q3tFramePump** output, char* error, size_t error_capacity) {
    if (model == nullptr || output == nullptr || max_batch < 1 || max_batch > QWEN3_TTS_MAX_BATCH_SESSIONS
        || gather_window_microseconds < 0) {
        if (error != nullptr && error_capacity > 0) std::snprintf(error, error_capacity, "frame pump arguments are out of range");
        return QWEN3_TTS_TALKER_STATUS_INVALID_ARGUMENT;
    }
    Q3tFramePump* pump = new (std::nothrow) Q3tFramePump();
    if (pump == nullptr) {
        if (error != nullptr && error_capacity > 0) std::snprintf(error, error_capacity, "out of memory");
        return QWEN3_TTS_TALKER_STATUS_ALLOCATION;
    }
    pump->model = model;
    pump->max_batch = max_batch;
    pump->window = std::chrono::microseconds(gather_window_microseconds);
    try {
        pump->worker = std::thread([pump] { pump->run(); });
    } catch (...) {
        delete pump;
        if (error != nullptr && error_capacity > 0) std::snprintf(error, error_capacity, "could not start the pump thread");
        return QWEN3_TTS_TALKER_STATUS_STATE;
    }
    *output = pump;
    if (error != nullptr && error_capacity > 0) error[0] = 0;
    return QWEN3_TTS_TALKER_STATUS_OK;
}

void q3t_pump_destroy(Q3tFramePump* pump) {
    if (pump == nullptr) return;
    {
        std::lock_guard<std::mutex> hold(pump->lock);
        pump->closing = true;
    }
    pump->arrived.notify_all();
    if (pump->worker.joinable()) pump->worker.join();
    delete pump;
}

/* A session that is decoding registers, so that the pump knows how many requests make a full
 * batch; it unregisters when it ends or pauses. */
void q3t_pump_register(Q3tFramePump* pump) {
    if (pump != nullptr) pump->registered.fetch_add(1, std::memory_order_relaxed);
}
void q3t_pump_unregister(Q3tFramePump* pump) {
    if (pump != nullptr) pump->registered.fetch_sub(1, std::memory_order_relaxed);
}

int32_t q3t_pump_begin_frame(Q3tFramePump* pump, Qwen3TtsSessionHandle session, int32_t frames_emitted,
                             int32_t trailing_text_token_id, Qwen3TtsSamplingConfig talker_sampling,
                             Qwen3TtsSamplingConfig predictor_sampling, Qwen3TtsDeviceFrameViewV2* output,
                             char* error, size_t error_capacity) {
    if (pump == nullptr || session == nullptr || output == nullptr) {
        if (error != nullptr && error_capacity > 0) std::snprintf(error, error_capacity, "pump, session or output is null");
        return QWEN3_TTS_TALKER_STATUS_INVALID_ARGUMENT;
    }
    if (frames_emitted == 0) {
        // first audio does not wait for the rendezvous
        return qwen3_tts_session_next_frame_begin_v2(session, trailing_text_token_id, talker_sampling,
                                                     predictor_sampling, output, error, error_capacity);
    }
    PumpRequest request;
    request.session = session;
    request.trailing = trailing_text_token_id;
    request.talker = talker_sampling;
    request.predictor = predictor_sampling;
    {
        std::unique_lock<std::mutex> hold(pump->lock);
        if (pump->closing) {
            if (error != nullptr && error_capacity > 0) std::snprintf(error, error_capacity, "the frame pump has shut down");
            return QWEN3_TTS_TALKER_STATUS_STATE;
        }
        pump->queue.push_back(&request);
        pump->arrived.notify_all();
        request.ready.wait(hold, [&] { return request.done; });
    }
    if (request.status == QWEN3_TTS_TALKER_STATUS_OK) {
        const uint32_t caller_size = output->struct_size;
        *output = request.view;
        if (caller_size != 0) output->struct_size = caller_size;
        if (error != nullptr && error_capacity > 0) error[0] = 0;
    } else if (error != nullptr && error_capacity > 0) {
        std::snprintf(error, error_capacity, "%s", request.message.c_str());
    }
    return request.status;
}

int32_t q3t_pump_statistics(Q3tFramePump* pump, uint64_t* batches, uint64_t* frames) {
    if (pump == nullptr) return QWEN3_TTS_TALKER_STATUS_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> hold(pump->lock);
    if (batches != nullptr) *batches = pump->batches;
    if (frames != nullptr) *frames = pump->frames;
    return QWEN3_TTS_TALKER_STATUS_OK;
}

/* Where a new session goes when one process drives several GPUs: the device with the fewest
 * active sessions (the lowest index among equals); sessions stay where they were created. */
int32_t q3t_pick_device(const int32_t* active_sessions_per_device, int32_t devices) {
    if (active_sessions_per_device == nullptr || devices < 1) return -1;
    int32_t best = 0;
    for (int32_t d = 1; d < devices; ++d) {
        if (active_sessions_per_device[d] < active_sessions_per_device[best]) best = d;
    }
    return best;
}

}  // extern "C"
