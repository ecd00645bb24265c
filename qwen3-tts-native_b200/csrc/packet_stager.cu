// Device-to-device hand-over of finished code frames to the consumer of the path (the codec).
//
// Follows the reference host's CudaPacketStager (native/qwen3-tts-runtime/src/
// cuda_packet_stager.rs:167-340): a session owns one 128-byte device buffer of up to four
// frames of 16 uint16 codes, a non-blocking stream and one event without timing.  Staging a
// frame makes that stream wait for the talker's ready event, copies the 32 bytes behind the
// frames already staged, records the event and returns it: it is what the host hands to
// qwen3_tts_session_next_frame_finish_v2 as the consumer-done event of the frame's lease.  The
// codec reads the packet once the event has fired; release_after_consumer orders the next
// packet's copies behind the codec's own event.  No host copy of a code is involved.
// The same refusals as the reference, in the same order; a CUDA failure poisons the stager.

#include "q3t_ops.h"

#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <new>
#include <string>

namespace {

constexpr int kCodebooks = 16;
constexpr int kMaxPacketFrames = 4;
constexpr size_t kFrameBytes = kCodebooks * sizeof(uint16_t);
constexpr size_t kPacketBytes = kFrameBytes * kMaxPacketFrames;

void write_message(char* error, size_t capacity, const std::string& message) {
    if (error == nullptr || capacity == 0) return;
    std::snprintf(error, capacity, "%s", message.c_str());
}

}  // namespace

struct Q3tPacketStager {
    int device = 0;
    uint16_t* codes = nullptr;
    cudaStream_t stream = nullptr;
    cudaEvent_t copied = nullptr;
    int staged = 0;
    bool poisoned = false;

    // false (and poisoned) when a CUDA call failed
    bool check(const char* what, cudaError_t status, char* error, size_t capacity, bool poison = true) {
        if (status == cudaSuccess) return true;
        if (poison) poisoned = true;
        write_message(error, capacity, std::string(what) + " failed: " + cudaGetErrorString(status));
        return false;
    }
};

extern "C" {

Q3tPacketStager* q3t_packet_stager_create(int32_t device_index, char* error, size_t error_capacity) {
    Q3tPacketStager* s = new (std::nothrow) Q3tPacketStager();
    if (s == nullptr) {
        write_message(error, error_capacity, "out of host memory");
        return nullptr;
    }
    s->device = device_index;
    bool ok = s->check("select CUDA device", cudaSetDevice(device_index), error, error_capacity);
    ok = ok && s->check("allocate CUDA packet staging buffer",
                        cudaMalloc(reinterpret_cast<void**>(&s->codes), kPacketBytes), error, error_capacity);
    ok = ok && s->check("create CUDA packet staging stream",
                        cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking), error, error_capacity);
    ok = ok && s->check("create CUDA packet staging event",
                        cudaEventCreateWithFlags(&s->copied, cudaEventDisableTiming), error, error_capacity);
    if (!ok) {
        q3t_packet_stager_destroy(s);
        return nullptr;
    }
    return s;
}

void q3t_packet_stager_destroy(Q3tPacketStager* s) {
    if (s == nullptr) return;
    cudaSetDevice(s->device);
    if (s->stream != nullptr) cudaStreamSynchronize(s->stream);
    if (s->copied != nullptr) cudaEventDestroy(s->copied);
    if (s->stream != nullptr) cudaStreamDestroy(s->stream);
    if (s->codes != nullptr) cudaFree(s->codes);
    delete s;
}

uint64_t q3t_packet_stager_device_bytes(const Q3tPacketStager*) { return kPacketBytes; }

int32_t q3t_packet_stager_staged_frames(const Q3tPacketStager* s) { return s == nullptr ? 0 : s->staged; }

int32_t q3t_packet_stager_stage_frame(Q3tPacketStager* s, const uint16_t* device_codes, size_t code_count,
                                      void* producer_ready_event, int32_t source_device,
                                      void** copied_event, char* error, size_t error_capacity) {
    if (s == nullptr || copied_event == nullptr) {
        write_message(error, error_capacity, "packet stager or output pointer is null");
        return 1;
    }
    if (s->poisoned) {
        write_message(error, error_capacity, "CUDA packet stager is poisoned");
        return 1;
    }
    if (source_device != s->device) {
        write_message(error, error_capacity, "Talker device " + std::to_string(source_device)
                                             + " does not match stager device " + std::to_string(s->device));
        return 1;
    }
    if (device_codes == nullptr || producer_ready_event == nullptr) {
        write_message(error, error_capacity, "Talker device codes and ready event are required");
        return 1;
    }
    if (code_count != static_cast<size_t>(kCodebooks)) {
        write_message(error, error_capacity, "Talker returned " + std::to_string(code_count)
                                             + " codes; expected " + std::to_string(kCodebooks));
        return 1;
    }
    if (s->staged >= kMaxPacketFrames) {
        write_message(error, error_capacity, "CUDA packet staging buffer is full");
        return 1;
    }
    if (!s->check("select CUDA device", cudaSetDevice(s->device), error, error_capacity, false)) return 2;
    if (!s->check("wait for Talker frame",
                  cudaStreamWaitEvent(s->stream, static_cast<cudaEvent_t>(producer_ready_event), 0), error,
                  error_capacity)) {
        return 2;
    }
    uint16_t* destination = s->codes + static_cast<size_t>(s->staged) * kCodebooks;
    if (!s->check("stage Talker codec frame",
                  cudaMemcpyAsync(destination, device_codes, kFrameBytes, cudaMemcpyDeviceToDevice, s->stream),
                  error, error_capacity)) {
        return 2;
    }
    if (!s->check("record staged Talker frame", cudaEventRecord(s->copied, s->stream), error, error_capacity)) {
        return 2;
    }
    ++s->staged;
    *copied_event = s->copied;
    return 0;
}

int32_t q3t_packet_stager_packet_view(const Q3tPacketStager* s, Q3tStagedPacketView* view, char* error,
                                      size_t error_capacity) {
    if (s == nullptr || view == nullptr) {
        write_message(error, error_capacity, "packet stager or output pointer is null");
        return 1;
    }
    if (s->poisoned) {
        write_message(error, error_capacity, "CUDA packet stager is poisoned");
        return 1;
    }
    if (s->staged == 0) {
        write_message(error, error_capacity, "CUDA packet staging buffer is empty");
        return 1;
    }
    view->device_codes = s->codes;
    view->frame_count = static_cast<uint64_t>(s->staged);
    view->ready_event = s->copied;
    return 0;
}

int32_t q3t_packet_stager_release_after_consumer(Q3tPacketStager* s, void* consumer_done_event, char* error,
                                                 size_t error_capacity) {
    if (s == nullptr) {
        write_message(error, error_capacity, "packet stager is null");
        return 1;
    }
    if (s->poisoned) {
        write_message(error, error_capacity, "CUDA packet stager is poisoned");
        return 1;
    }
    if (s->staged == 0) {
        write_message(error, error_capacity, "no staged packet is awaiting a consumer");
        return 1;
    }
    if (consumer_done_event == nullptr) {
        write_message(error, error_capacity, "Codec consume event is required");
        return 1;
    }
    if (!s->check("select CUDA device", cudaSetDevice(s->device), error, error_capacity, false)) return 2;
    if (!s->check("wait for Codec packet snapshot",
                  cudaStreamWaitEvent(s->stream, static_cast<cudaEvent_t>(consumer_done_event), 0), error,
                  error_capacity)) {
        return 2;
    }
    s->staged = 0;
    return 0;
}

}  // extern "C"
