// Model / session / frame engine behind the native talker C ABI.
//
// Host-side counterpart of the reference's TalkerModel, TalkerContext and BatchWorkspace
// (native/qwen3-tts-native/native/src/talker.cu:213-411, 413-788, 790-3772), rebuilt around
// three ideas:
//   * decode weights exist only as one int8 image per model (quantized as tensors arrive),
//     with q/k/v and gate/up stored as single fused matrices;
//   * KV lives in a per-model pool of 16-token pages, sessions hold page lists;
//   * a frame is two captured CUDA graphs (predictor, talker) whose kernels read every
//     per-session value through a device-resident FrameTable, so one graph serves any
//     set of sessions of the same count.
#pragma once

#include "q3t_kernels.cuh"

#include <cuda_runtime.h>

#include <array>
#include <atomic>
#include <cstdint>
#include <map>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace q3t {

class CudaFailure final : public std::runtime_error {
public:
    using std::runtime_error::runtime_error;
};

void check_cuda(cudaError_t status, const char* what);
// check_cuda for the kernel launches of a frame or prompt: the host-side fault injector below can
// make the n-th of them report a failure without any CUDA call failing
void check_launch(cudaError_t status, const char* what);

// Host-side fault injection for tests (nothing here makes a GPU fault).  fail_launch_after(n): the
// n-th kernel launch the engine enqueues from now on reports cudaErrorLaunchOutOfResources (n = 1: the
// next one; 0 disarms).  fail_allocation_after(n): the n-th device allocation of the engine from now
// on throws std::bad_alloc.  Both disarm themselves after firing.
void fail_launch_after(int n);
void fail_allocation_after(int n);

// One host-mapped word per device that the kernels' bounded waits bump when they run out, so that
// the host sees it at its next synchronisation point without a copy.  Null before configure_device().
volatile unsigned int* device_error_word(int device);

class DeviceBuffer {
public:
    DeviceBuffer() = default;
    explicit DeviceBuffer(size_t bytes);
    DeviceBuffer(const DeviceBuffer&) = delete;
    DeviceBuffer& operator=(const DeviceBuffer&) = delete;
    DeviceBuffer(DeviceBuffer&& o) noexcept;
    DeviceBuffer& operator=(DeviceBuffer&& o) noexcept;
    ~DeviceBuffer();
    template <class T> T* as() const { return static_cast<T*>(ptr_); }
    size_t bytes() const { return bytes_; }
private:
    void* ptr_ = nullptr;
    size_t bytes_ = 0;
};

struct ModelDims {
    int hidden, intermediate, q_heads, kv_heads, head_dim, q_width, kv_width, layers;
};

struct Quantized {
    const int8_t* data = nullptr;
    const float* scales = nullptr;
};

// int8 image of one decoder layer; q/k/v rows are one [q_width + 2*kv_width][hidden]
// matrix, gate/up one [2*intermediate][hidden] matrix (gate rows first)
struct LayerWeights {
    const bf16* input_norm = nullptr;
    const bf16* q_norm = nullptr;
    const bf16* k_norm = nullptr;
    const bf16* post_norm = nullptr;
    Quantized qkv, o, gate_up, down;
};

// Pool of 16-token KV pages.  A slab holds, for every layer, a K plane and a V plane of
// `pages_per_slab` pages: slab[layer][k|v][page][kv_head][16][head_dim] (head-major pages).
class KvPool {
public:
    KvPool(int layers, int kv_width, int slab_shift);
    int allocate();                 // page id; grows by one slab when empty
    void release(int page);
    KvLayout layout(int layer, const int* page_table, int table_stride) const;
    uint64_t page_bytes() const;    // K+V bytes of one page over all layers
    bf16* const* slab_table() const { return slab_table_.as<bf16*>(); }
    int slab_shift() const { return slab_shift_; }
    int layers() const { return layers_; }
    long long page_elems() const { return page_elems_; }
    long long plane_elems() const { return plane_elems_; }
    // device address of token 0 of `page` in the K (value = false) or V plane of `layer`
    const bf16* page_rows(int page, int layer, bool value) const;
    static constexpr int kMaxSlabs = 512;
private:
    void add_slab();
    int layers_, kv_width_, slab_shift_;
    long long page_elems_, plane_elems_;
    std::vector<DeviceBuffer> slabs_;
    DeviceBuffer slab_table_;       // device array of slab base pointers
    std::vector<int> free_;
};

class Session;

// Activation buffers, frame table and captured graphs for up to `capacity` lockstep rows.
struct Workspace {
    Workspace(int capacity, int device);
    ~Workspace();
    Workspace(const Workspace&) = delete;
    Workspace& operator=(const Workspace&) = delete;

    void ensure_scratch(int splits);
    void destroy_graphs() noexcept;
    void release() noexcept;
    uint64_t bytes() const;

    int capacity;
    int device;
    cudaStream_t stream = nullptr;
    DeviceBuffer hidden, qkv, attention, gate, logits, x_in, projection, normalized;
    DeviceBuffer table;              // FrameTable
    FrameTable* host_table = nullptr;   // pinned mirror
    DeviceBuffer talker_pages;       // [capacity][kMaxPagesPerRow]
    DeviceBuffer predictor_pages;    // [capacity][1]
    int* host_pages = nullptr;       // pinned staging for the two page tables
    DeviceBuffer predictor_positions;   // [16][kMaxRows], slot p filled with p
    DeviceBuffer prompt_positions;      // [kMaxRows], positions of the rows of a prompt chunk
    DeviceBuffer scratch;
    DeviceBuffer counters;
    int scratch_splits = 0;
    int option_epoch = 0;            // Model::option_epoch the captured graphs were built under
    std::vector<uint64_t> bound;     // ids of the sessions whose page lists are resident (ids are never reused)
    struct Graphs {
        cudaGraphExec_t predictor = nullptr;
        cudaGraphExec_t talker = nullptr;
        int predictor_kernels = 0;   // kernel nodes in each graph
        int talker_kernels = 0;
    };
    std::map<std::pair<int, int>, Graphs> graphs;   // (rows, talker splits) -> graphs
    cudaEvent_t predictor_start = nullptr, predictor_stop = nullptr;
    // frames launched on this workspace, and the GPU times of the frame `timed_frame` (every
    // session of a lockstep frame reports the same two numbers: they are read from the events once)
    uint64_t frame_serial = 0, timed_frame = 0;
    float timed_predictor_ms = 0.0f, timed_talker_ms = 0.0f;
    cudaEvent_t talker_start = nullptr, talker_stop = nullptr;
    cudaEvent_t table_uploaded = nullptr;   // the pinned host table may be rewritten after this
    std::array<cudaEvent_t, kMaxRows> join_events{};
    static constexpr int kMaxPagesPerRow = 8192 / kPageTokens;
};

class Model {
public:
    explicit Model(int device);
    ~Model();
    Model(const Model&) = delete;
    Model& operator=(const Model&) = delete;

    // Where a checkpoint tensor lives on the device in the form the decode step reads (int8 rows
    // + fp32 row scales for the projection matrices, bf16 otherwise), and a way to declare such
    // storage filled by other means than upload_tensor (a broadcast from the rank that quantized).
    struct TensorImage {
        void* data = nullptr;
        uint64_t data_bytes = 0;
        float* scales = nullptr;
        uint64_t scales_bytes = 0;
        bool quantized = false;
        bool loaded = false;
    };
    TensorImage tensor_image(const char* name) const;
    void adopt_tensor(const char* name);
    void upload_tensor(const char* name, const void* data, uint64_t bytes, int rank,
                       const uint64_t* shape);
    void finalize(uint64_t* weight_bytes, uint32_t* tensor_count);
    bool finalized() const { return finalized_; }
    int device() const { return device_; }
    Workspace& batch_workspace();
    Workspace& prefill_workspace();     // rows of a prompt chunk; one prompt at a time (prefill_mutex)
    std::mutex prefill_mutex;
    // serialises every use of the lockstep workspace (its page tables, captured graphs and stream):
    // batch_begin, run_frames with more than one session, option changes
    std::mutex batch_mutex;
    // How many bounded device-side waits have run out on this device so far.  A session notes the
    // count when it enqueues work and compares at the host synchronisation point that follows: a
    // frame or prompt during which it advanced cannot be trusted (check_device_errors throws).
    unsigned int device_errors() const;
    void check_device_errors(unsigned int count_at_enqueue) const;
    int prefill_chunk = kMaxRows;       // prompt positions per pass (1: one position at a time)
    Workspace* batch_workspace_if_any() {
        std::lock_guard<std::mutex> lock(mutex);
        return batch_.get();
    }

    ModelDims talker{}, predictor{};
    std::vector<LayerWeights> talker_layers, predictor_layers;
    Quantized codec_head, small_to_mtp, text_fc1, text_fc2;
    std::array<Quantized, 15> predictor_heads{};
    const bf16 *codec_embedding = nullptr, *text_embedding = nullptr, *text_fc1_bias = nullptr,
               *text_fc2_bias = nullptr, *talker_norm = nullptr, *small_to_mtp_bias = nullptr,
               *predictor_norm = nullptr;
    std::array<const bf16*, 15> predictor_embeddings{};
    const bf16* const* predictor_embedding_table = nullptr;   // device copy of the 15 pointers
    std::unique_ptr<KvPool> talker_pool, predictor_pool;
    // bf16 cos | sin of every (position, rotary pair), one table per head_dim in use
    static constexpr int kRopePositions = 8192;
    const uint32_t* talker_rope = nullptr;
    const uint32_t* predictor_rope = nullptr;
    std::mutex mutex;               // pools, workspaces
    int mask_eos = 0;
    int use_graphs = 1;
    int option_epoch = 0;           // bumped when an option that captured graphs bake in changes
    int batch_host_codes = 0;       // lockstep batches also mirror the 16 codes to pinned host memory
    std::atomic<uint64_t> kernel_launches{0};   // kernels of this library launched through frame graphs

private:
    struct Spec {
        std::vector<uint64_t> shape;
        bool quantize = false;
        void* destination = nullptr;    // bf16 tensor, or int8 rows
        float* scales = nullptr;
        bool seen = false;
    };
    void add_keep(const std::string& name, std::vector<uint64_t> shape, const bf16** slot);
    void add_quant_rows(const std::string& name, uint64_t rows, uint64_t cols, int8_t* data,
                        float* scales);
    Quantized allocate_quantized(uint64_t rows, uint64_t cols);
    Quantized add_quant_matrix(const std::string& name, uint64_t rows, uint64_t cols);
    void plan_layers(const std::string& prefix, const ModelDims& d, std::vector<LayerWeights>& out);

    int device_;
    bool finalized_ = false;
    uint64_t weight_bytes_ = 0;
    uint32_t tensor_count_ = 0;
    cudaStream_t upload_stream_ = nullptr;
    std::unordered_map<std::string, Spec> specs_;
    std::vector<DeviceBuffer> storage_;   // every resident tensor (int8 rows, scales, bf16)
    DeviceBuffer staging_, embedding_ptrs_, talker_rope_, predictor_rope_;
    size_t staging_bytes_ = 0;
    std::unique_ptr<Workspace> batch_, prefill_;
};

struct FrameResult {
    uint16_t codes[16];
    uint16_t next_semantic;
    uint32_t ended;
    uint32_t talker_position;
    float predictor_ms, talker_ms;
};

struct FrameView {
    const uint16_t* device_codes;
    cudaEvent_t ready_event;
    uint64_t lease_id;
    int device;
};

class Session {
public:
    Session(std::shared_ptr<Model> model, int max_sequence_length, uint64_t seed);
    ~Session();
    Session(const Session&) = delete;
    Session& operator=(const Session&) = delete;

    void reset(uint64_t seed);
    void prefill(const int32_t* text_ids, const int32_t* codec_ids, int count,
                 const SamplingParams& sampling, uint16_t* first_token, float* gpu_ms);
    FrameView begin_frame(uint16_t semantic_token, int trailing_text, const SamplingParams& talker,
                          const SamplingParams& predictor, bool host_codes);
    FrameResult finish_frame(uint64_t lease_id, cudaEvent_t consumer_done);
    static void batch_begin(Model* model, Session** sessions, int n, const int* trailing_text,
                            const SamplingParams* talker, const SamplingParams* predictor,
                            FrameView* views);
    // Benchmark path: `frames` frames back to back for the given sessions with no host round
    // trip in between; per-frame GPU milliseconds are written to frame_ms when non-null.
    static void run_frames(Model* model, Session** sessions, int n, int frames, int trailing_text,
                           const SamplingParams& talker, const SamplingParams& predictor,
                           float* frame_ms, float* total_ms);

    uint16_t current_token() const { return current_token_; }
    Model* model() const { return model_.get(); }

    // state_info / session_memory
    uint32_t phase() const { return phase_; }
    uint32_t position() const { return static_cast<uint32_t>(position_); }
    uint32_t history_count() const { return static_cast<uint32_t>(generated_); }
    uint64_t frames_generated = 0, device_sample_count = 0, host_sync_count = 0;
    uint64_t talker_kv_bytes = 0, predictor_kv_bytes = 0, workspace_bytes = 0;
    int max_sequence_length() const { return max_seq_; }

    // parity-test hook: copies of the device-side state (any pointer may be null)
    void read_state(uint16_t* last_hidden, int* frame_tokens, unsigned long long* rng) const;
    // parity-test hook: the talker's K and V rows of positions [first, first + count) of one layer,
    // as stored (K after its head norm and rotation), copied to host memory, [count][kv width] each
    void read_kv(int layer, int first, int count, uint16_t* keys, uint16_t* values) const;
    // Benchmark harness: puts the session in the PREFILLED phase at `position` without running a
    // prompt: KV rows [0, position) and last_hidden are filled with seeded pseudo-random
    // N(0,1) values, the semantic history gets one token.
    void synthetic_prefill(int position, uint64_t seed);

private:
    friend struct Workspace;
    void validate_begin(int semantic_token, int trailing_text, const SamplingParams& talker,
                        const SamplingParams& predictor) const;
    void release() noexcept;
    uint64_t take_lease(Workspace* w, bool host_codes);
    void drop_lease_poisoned() noexcept;
    void fill_row(FrameTable& t, int row, int trailing_text, const SamplingParams& talker,
                  const SamplingParams& predictor, bool host_codes) const;
    static void bind_rows(Workspace& w, Session** s, int n);
    static Workspace::Graphs& frame_graphs(Workspace& w, Model& m, int n, int splits);
    static void launch_frame(Workspace& w, Model& m, Session** s, int n, bool upload_table,
                             bool record_session_events);

    std::shared_ptr<Model> model_;
    const uint64_t id_;             // unique for the life of the process
    int device_;
    int max_seq_;
    int position_ = 0;
    int generated_ = 0;
    uint16_t current_token_ = 0;
    uint32_t phase_ = 0;
    bool frame_in_flight_ = false;
    bool poisoned_ = false;
    bool pending_host_codes_ = false;
    uint64_t next_lease_ = 1;
    uint64_t pending_lease_ = 0;
    uint32_t pending_position_ = 0;
    Workspace* pending_workspace_ = nullptr;   // whose timing events belong to the pending frame
    uint64_t pending_frame_serial_ = 0;
    unsigned int pending_errors_ = 0;           // Model::device_errors() when the pending frame was enqueued
    // true while this session's own stream may hold work a lockstep frame has to be ordered after
    // (prompt, solo frame, reset, a consumer's event); lockstep frames themselves leave it false
    bool own_stream_busy_ = true;
    cudaStream_t stream_ = nullptr;
    cudaEvent_t codes_ready_ = nullptr, semantic_ready_ = nullptr;
    std::unique_ptr<Workspace> solo_;
    std::vector<int> talker_pages_;
    int predictor_page_ = -1;
    DeviceBuffer state_;            // frame_tokens | frame_codes | sampled | rng | last_hidden | history
    int* d_frame_tokens_ = nullptr;
    unsigned short* d_frame_codes_ = nullptr;
    int* d_sampled_ = nullptr;
    unsigned long long* d_rng_ = nullptr;
    bf16* d_last_hidden_ = nullptr;
    int* d_history_ = nullptr;
    int* h_token_ = nullptr;            // pinned
    unsigned short* h_codes_ = nullptr; // pinned
};

}  // namespace q3t
