// Model / session / frame engine (see engine.hpp).

#include "engine.hpp"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstddef>
#include <cstdlib>
#include <cstdio>
#include <cstring>
#include <functional>
#include <limits>
#include <numeric>

namespace q3t {

namespace {
constexpr int kTalkerLayers = 28;
constexpr int kPredictorLayers = 5;
constexpr int kResidualCodebooks = 15;
constexpr int kTalkerVocab = 3072;
constexpr int kTextVocab = 151936;
constexpr int kPredictorSequence = 16;
constexpr int kEos = 2150;
constexpr uint32_t kPhaseCreated = 0, kPhaseReady = 1, kPhasePrefilled = 2, kPhaseEnded = 3;

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int env_int(const char* name, int fallback) {
    const char* v = std::getenv(name);
    return v != nullptr && *v != '\0' ? std::atoi(v) : fallback;
}
}  // namespace

void check_cuda(cudaError_t status, const char* what) {
    if (status != cudaSuccess) {
        throw CudaFailure(std::string(what) + " failed: " + cudaGetErrorString(status));
    }
}

namespace {
std::atomic<int> g_fail_launch{0}, g_fail_allocation{0};
std::atomic<uint64_t> g_next_session_id{1};

// true exactly once, when an armed countdown reaches zero
bool countdown_fires(std::atomic<int>& countdown) {
    int left = countdown.load(std::memory_order_relaxed);
    while (left > 0) {
        if (countdown.compare_exchange_weak(left, left - 1, std::memory_order_relaxed)) return left == 1;
    }
    return false;
}
}  // namespace

void fail_launch_after(int n) { g_fail_launch.store(n > 0 ? n : 0); }
void fail_allocation_after(int n) { g_fail_allocation.store(n > 0 ? n : 0); }

void check_launch(cudaError_t status, const char* what) {
    if (status == cudaSuccess && countdown_fires(g_fail_launch)) status = cudaErrorLaunchOutOfResources;
    check_cuda(status, what);
}

// ------------------------------------------------------------------ DeviceBuffer

DeviceBuffer::DeviceBuffer(size_t bytes) : bytes_(bytes) {
    if (bytes == 0) return;
    if (countdown_fires(g_fail_allocation)) throw std::bad_alloc();
    const cudaError_t e = cudaMalloc(&ptr_, bytes);
    if (e == cudaErrorMemoryAllocation) {
        cudaGetLastError();
        throw std::bad_alloc();
    }
    check_cuda(e, "cudaMalloc");
}
DeviceBuffer::DeviceBuffer(DeviceBuffer&& o) noexcept : ptr_(o.ptr_), bytes_(o.bytes_) {
    o.ptr_ = nullptr;
    o.bytes_ = 0;
}
DeviceBuffer& DeviceBuffer::operator=(DeviceBuffer&& o) noexcept {
    if (this != &o) {
        if (ptr_ != nullptr) cudaFree(ptr_);
        ptr_ = o.ptr_;
        bytes_ = o.bytes_;
        o.ptr_ = nullptr;
        o.bytes_ = 0;
    }
    return *this;
}
DeviceBuffer::~DeviceBuffer() {
    if (ptr_ != nullptr) cudaFree(ptr_);
}

// ------------------------------------------------------------------ KvPool

KvPool::KvPool(int layers, int kv_width, int slab_shift)
    : layers_(layers), kv_width_(kv_width), slab_shift_(slab_shift),
      page_elems_((long long)kPageTokens * kv_width),
      plane_elems_(((long long)1 << slab_shift) * kPageTokens * kv_width),
      slab_table_(kMaxSlabs * sizeof(bf16*)) {
    check_cuda(cudaMemset(slab_table_.as<void>(), 0, kMaxSlabs * sizeof(bf16*)), "cudaMemset(slab table)");
}

void KvPool::add_slab() {
    if (static_cast<int>(slabs_.size()) >= kMaxSlabs) throw std::bad_alloc();
    const size_t bytes = (size_t)layers_ * 2 * plane_elems_ * sizeof(bf16);
    DeviceBuffer slab(bytes);
    bf16* base = slab.as<bf16>();
    const int index = static_cast<int>(slabs_.size());
    check_cuda(cudaMemcpy(slab_table_.as<bf16*>() + index, &base, sizeof(base), cudaMemcpyHostToDevice),
               "cudaMemcpy(slab table)");
    slabs_.push_back(std::move(slab));
    const int per = 1 << slab_shift_;
    for (int i = per - 1; i >= 0; --i) free_.push_back(index * per + i);
}

int KvPool::allocate() {
    if (free_.empty()) add_slab();
    const int page = free_.back();
    free_.pop_back();
    return page;
}

void KvPool::release(int page) { free_.push_back(page); }

KvLayout KvPool::layout(int layer, const int* page_table, int table_stride) const {
    KvLayout l;
    l.page_table = page_table;
    l.table_stride = table_stride;
    l.slabs = slab_table_.as<bf16*>();
    l.slab_shift = slab_shift_;
    l.page_elems = page_elems_;
    l.k_offset = (long long)(layer * 2) * plane_elems_;
    l.v_offset = (long long)(layer * 2 + 1) * plane_elems_;
    return l;
}

const bf16* KvPool::page_rows(int page, int layer, bool value) const {
    const int slab = page >> slab_shift_;
    if (page < 0 || slab >= static_cast<int>(slabs_.size()) || layer < 0 || layer >= layers_) {
        throw std::runtime_error("KV page or layer out of range");
    }
    return slabs_[slab].as<bf16>() + (long long)(page & ((1 << slab_shift_) - 1)) * page_elems_
           + (long long)(layer * 2 + (value ? 1 : 0)) * plane_elems_;
}

uint64_t KvPool::page_bytes() const { return (uint64_t)layers_ * 2 * page_elems_ * sizeof(bf16); }

// ------------------------------------------------------------------ Workspace

Workspace::Workspace(int capacity_, int device_) : capacity(capacity_), device(device_) {
    check_cuda(cudaSetDevice(device), "cudaSetDevice(workspace)");
    const size_t e = sizeof(bf16);
    const size_t c = capacity;
    hidden = DeviceBuffer(c * 2048 * e);
    qkv = DeviceBuffer(c * 4096 * e);
    attention = DeviceBuffer(c * 2048 * e);
    gate = DeviceBuffer(c * 6144 * e);
    logits = DeviceBuffer(c * kTalkerVocab * e);
    x_in = DeviceBuffer(c * 2048 * e);
    projection = DeviceBuffer(c * 2048 * e);
    normalized = DeviceBuffer(c * 2048 * e);
    table = DeviceBuffer(sizeof(FrameTable));
    talker_pages = DeviceBuffer(c * kMaxPagesPerRow * sizeof(int));
    predictor_pages = DeviceBuffer(c * sizeof(int));
    predictor_positions = DeviceBuffer((size_t)kPredictorSequence * kMaxRows * sizeof(int));
    prompt_positions = DeviceBuffer((size_t)kMaxRows * sizeof(int));
    counters = DeviceBuffer(c * 16 * sizeof(unsigned int));
    try {
        check_cuda(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking), "cudaStreamCreate");
        check_cuda(cudaHostAlloc(reinterpret_cast<void**>(&host_table), sizeof(FrameTable),
                                 cudaHostAllocDefault), "cudaHostAlloc(frame table)");
        std::memset(host_table, 0, sizeof(FrameTable));
        check_cuda(cudaHostAlloc(reinterpret_cast<void**>(&host_pages),
                                 c * (kMaxPagesPerRow + 1) * sizeof(int), cudaHostAllocDefault),
                   "cudaHostAlloc(page tables)");
        check_cuda(cudaMemset(table.as<void>(), 0, sizeof(FrameTable)), "cudaMemset(frame table)");
        check_cuda(cudaMemset(counters.as<void>(), 0, counters.bytes()), "cudaMemset(counters)");
        std::vector<int> positions((size_t)kPredictorSequence * kMaxRows);
        for (int p = 0; p < kPredictorSequence; ++p)
            for (int r = 0; r < kMaxRows; ++r) positions[(size_t)p * kMaxRows + r] = p;
        check_cuda(cudaMemcpy(predictor_positions.as<void>(), positions.data(),
                              positions.size() * sizeof(int), cudaMemcpyHostToDevice),
                   "cudaMemcpy(predictor positions)");
        check_cuda(cudaEventCreate(&predictor_start), "cudaEventCreate");
        check_cuda(cudaEventCreate(&predictor_stop), "cudaEventCreate");
        check_cuda(cudaEventCreate(&talker_start), "cudaEventCreate");
        check_cuda(cudaEventCreate(&talker_stop), "cudaEventCreate");
        check_cuda(cudaEventCreateWithFlags(&table_uploaded, cudaEventDisableTiming), "cudaEventCreate");
        for (int i = 0; i < capacity && i < kMaxRows; ++i) {
            check_cuda(cudaEventCreateWithFlags(&join_events[i], cudaEventDisableTiming),
                       "cudaEventCreate(join)");
        }
    } catch (...) {
        release();
        throw;
    }
}

void Workspace::release() noexcept {
    destroy_graphs();
    for (cudaEvent_t& ev : join_events) {
        if (ev != nullptr) cudaEventDestroy(ev);
        ev = nullptr;
    }
    for (cudaEvent_t* ev : {&predictor_start, &predictor_stop, &talker_start, &talker_stop,
                            &table_uploaded}) {
        if (*ev != nullptr) cudaEventDestroy(*ev);
        *ev = nullptr;
    }
    if (host_pages != nullptr) cudaFreeHost(host_pages);
    host_pages = nullptr;
    if (host_table != nullptr) cudaFreeHost(host_table);
    host_table = nullptr;
    if (stream != nullptr) cudaStreamDestroy(stream);
    stream = nullptr;
}

Workspace::~Workspace() {
    cudaSetDevice(device);
    if (stream != nullptr) cudaStreamSynchronize(stream);
    release();
}

void Workspace::destroy_graphs() noexcept {
    for (auto& kv : graphs) {
        if (kv.second.predictor != nullptr) cudaGraphExecDestroy(kv.second.predictor);
        if (kv.second.talker != nullptr) cudaGraphExecDestroy(kv.second.talker);
    }
    graphs.clear();
}

void Workspace::ensure_scratch(int splits) {
    if (splits <= scratch_splits) return;
    check_cuda(cudaStreamSynchronize(stream), "cudaStreamSynchronize(scratch)");
    destroy_graphs();   // captured launches hold the old scratch pointer
    scratch = DeviceBuffer();
    scratch = DeviceBuffer(attention_scratch_floats(capacity, 16, 128, splits) * sizeof(float));
    scratch_splits = splits;
}

uint64_t Workspace::bytes() const {
    return hidden.bytes() + qkv.bytes() + attention.bytes() + gate.bytes() + logits.bytes()
        + x_in.bytes() + projection.bytes() + normalized.bytes() + table.bytes()
        + talker_pages.bytes() + predictor_pages.bytes() + predictor_positions.bytes()
        + counters.bytes() + scratch.bytes();
}

// ------------------------------------------------------------------ Model

Model::Model(int device) : device_(device) {
    check_cuda(cudaSetDevice(device_), "cudaSetDevice(model)");
    check_cuda(cudaStreamCreateWithFlags(&upload_stream_, cudaStreamNonBlocking),
               "cudaStreamCreate(upload)");
    talker = {2048, 6144, 16, 8, 128, 2048, 1024, kTalkerLayers};
    // The checkpoint's code predictor has head_dim 128 (q 2048 wide, k/v 1024 wide);
    // QWEN3_TTS_PREDICTOR_HEAD_DIM=64 selects the 64-wide variant for experiments.
    const int phd = env_int("QWEN3_TTS_PREDICTOR_HEAD_DIM", 128) == 64 ? 64 : 128;
    predictor = {1024, 3072, 16, 8, phd, 16 * phd, 8 * phd, kPredictorLayers};
    mask_eos = env_int("QWEN3_TTS_MASK_EOS", 0) != 0;
    use_graphs = env_int("QWEN3_TTS_DISABLE_GRAPHS", 0) == 0;

    const uint64_t H = talker.hidden, PH = predictor.hidden;
    add_keep("talker.model.codec_embedding.weight", {kTalkerVocab, H}, &codec_embedding);
    add_keep("talker.model.text_embedding.weight", {kTextVocab, H}, &text_embedding);
    text_fc1 = add_quant_matrix("talker.text_projection.linear_fc1.weight", H, H);
    add_keep("talker.text_projection.linear_fc1.bias", {H}, &text_fc1_bias);
    text_fc2 = add_quant_matrix("talker.text_projection.linear_fc2.weight", H, H);
    add_keep("talker.text_projection.linear_fc2.bias", {H}, &text_fc2_bias);
    add_keep("talker.model.norm.weight", {H}, &talker_norm);
    codec_head = add_quant_matrix("talker.codec_head.weight", kTalkerVocab, H);
    plan_layers("talker.model.layers.", talker, talker_layers);
    small_to_mtp = add_quant_matrix("talker.code_predictor.small_to_mtp_projection.weight", PH, H);
    add_keep("talker.code_predictor.small_to_mtp_projection.bias", {PH}, &small_to_mtp_bias);
    add_keep("talker.code_predictor.model.norm.weight", {PH}, &predictor_norm);
    plan_layers("talker.code_predictor.model.layers.", predictor, predictor_layers);
    for (int g = 0; g < kResidualCodebooks; ++g) {
        add_keep("talker.code_predictor.model.codec_embedding." + std::to_string(g) + ".weight",
                 {(uint64_t)kPredictorVocab, H}, &predictor_embeddings[g]);
        predictor_heads[g] = add_quant_matrix(
            "talker.code_predictor.lm_head." + std::to_string(g) + ".weight", kPredictorVocab, PH);
    }
}

Model::~Model() {
    cudaSetDevice(device_);
    batch_.reset();
    if (upload_stream_ != nullptr) {
        cudaStreamSynchronize(upload_stream_);
        cudaStreamDestroy(upload_stream_);
    }
}

void Model::add_keep(const std::string& name, std::vector<uint64_t> shape, const bf16** slot) {
    size_t elements = 1;
    for (uint64_t d : shape) elements *= d;
    storage_.emplace_back(elements * sizeof(bf16));
    Spec s;
    s.shape = std::move(shape);
    s.destination = storage_.back().as<void>();
    *slot = storage_.back().as<bf16>();
    specs_.emplace(name, std::move(s));
}

void Model::add_quant_rows(const std::string& name, uint64_t rows, uint64_t cols, int8_t* data,
                           float* scales) {
    Spec s;
    s.shape = {rows, cols};
    s.quantize = true;
    s.destination = data;
    s.scales = scales;
    specs_.emplace(name, std::move(s));
    staging_bytes_ = std::max(staging_bytes_, (size_t)(rows * cols * sizeof(bf16)));
}

Quantized Model::allocate_quantized(uint64_t rows, uint64_t cols) {
    storage_.emplace_back(rows * cols);
    int8_t* data = storage_.back().as<int8_t>();
    storage_.emplace_back(rows * sizeof(float));
    float* scales = storage_.back().as<float>();
    return Quantized{data, scales};
}

Quantized Model::add_quant_matrix(const std::string& name, uint64_t rows, uint64_t cols) {
    const Quantized q = allocate_quantized(rows, cols);
    add_quant_rows(name, rows, cols, const_cast<int8_t*>(q.data), const_cast<float*>(q.scales));
    return q;
}

void Model::plan_layers(const std::string& prefix, const ModelDims& d, std::vector<LayerWeights>& out) {
    const uint64_t H = d.hidden, I = d.intermediate, QW = d.q_width, KW = d.kv_width, HD = d.head_dim;
    out.resize(d.layers);
    for (int l = 0; l < d.layers; ++l) {
        LayerWeights& w = out[l];
        const std::string p = prefix + std::to_string(l);
        add_keep(p + ".input_layernorm.weight", {H}, &w.input_norm);
        w.qkv = allocate_quantized(QW + 2 * KW, H);
        int8_t* qd = const_cast<int8_t*>(w.qkv.data);
        float* qs = const_cast<float*>(w.qkv.scales);
        add_quant_rows(p + ".self_attn.q_proj.weight", QW, H, qd, qs);
        add_quant_rows(p + ".self_attn.k_proj.weight", KW, H, qd + QW * H, qs + QW);
        add_quant_rows(p + ".self_attn.v_proj.weight", KW, H, qd + (QW + KW) * H, qs + QW + KW);
        w.o = add_quant_matrix(p + ".self_attn.o_proj.weight", H, QW);
        add_keep(p + ".self_attn.q_norm.weight", {HD}, &w.q_norm);
        add_keep(p + ".self_attn.k_norm.weight", {HD}, &w.k_norm);
        add_keep(p + ".post_attention_layernorm.weight", {H}, &w.post_norm);
        w.gate_up = allocate_quantized(2 * I, H);
        int8_t* gd = const_cast<int8_t*>(w.gate_up.data);
        float* gs = const_cast<float*>(w.gate_up.scales);
        add_quant_rows(p + ".mlp.gate_proj.weight", I, H, gd, gs);
        add_quant_rows(p + ".mlp.up_proj.weight", I, H, gd + I * H, gs + I);
        w.down = add_quant_matrix(p + ".mlp.down_proj.weight", H, I);
    }
}

void Model::upload_tensor(const char* name, const void* data, uint64_t bytes, int rank,
                          const uint64_t* shape) {
    check_cuda(cudaSetDevice(device_), "cudaSetDevice(upload)");
    if (finalized_) throw std::runtime_error("model weights are already finalized");
    if (name == nullptr || *name == '\0' || data == nullptr || shape == nullptr) {
        throw std::runtime_error("tensor upload received a null argument");
    }
    if (rank <= 0 || rank > 4 || bytes == 0) {
        throw std::runtime_error("tensor upload has an invalid rank or byte size");
    }
    uint64_t elements = 1;
    std::vector<uint64_t> dims;
    for (int i = 0; i < rank; ++i) {
        if (shape[i] == 0 || elements > std::numeric_limits<uint64_t>::max() / shape[i]) {
            throw std::runtime_error("tensor shape is empty or overflows");
        }
        elements *= shape[i];
        dims.push_back(shape[i]);
    }
    if (elements > std::numeric_limits<uint64_t>::max() / sizeof(bf16)
        || elements * sizeof(bf16) != bytes) {
        throw std::runtime_error("tensor byte size does not match BF16 shape");
    }
    const auto found = specs_.find(name);
    if (found == specs_.end()) {
        throw std::runtime_error(std::string("tensor is not part of the talker checkpoint: ") + name);
    }
    Spec& spec = found->second;
    if (spec.seen) throw std::runtime_error(std::string("duplicate tensor upload: ") + name);
    if (spec.shape != dims) throw std::runtime_error(std::string("unexpected shape for tensor ") + name);
    if (spec.quantize) {
        if (staging_.bytes() < staging_bytes_) staging_ = DeviceBuffer(staging_bytes_);
        check_cuda(cudaMemcpyAsync(staging_.as<void>(), data, bytes, cudaMemcpyHostToDevice,
                                   upload_stream_), "cudaMemcpyAsync(weight H2D)");
        check_cuda(launch_quantize_weight_rows(staging_.as<bf16>(),
                                               static_cast<int8_t*>(spec.destination), spec.scales,
                                               static_cast<int>(dims[1]), static_cast<int>(dims[0]),
                                               upload_stream_), "quantize decode weight");
        // the staging buffer is reused by the next upload; the host copy above has already
        // left the caller's buffer when cudaMemcpyAsync returns for pageable memory, but a
        // pinned source is read asynchronously, so wait before handing control back
        check_cuda(cudaStreamSynchronize(upload_stream_), "cudaStreamSynchronize(upload)");
    } else {
        check_cuda(cudaMemcpyAsync(spec.destination, data, bytes, cudaMemcpyHostToDevice,
                                   upload_stream_), "cudaMemcpyAsync(weight H2D)");
        check_cuda(cudaStreamSynchronize(upload_stream_), "cudaStreamSynchronize(upload)");
    }
    spec.seen = true;
    weight_bytes_ += bytes;
    ++tensor_count_;
}

Model::TensorImage Model::tensor_image(const char* name) const {
    if (name == nullptr) throw std::runtime_error("tensor name is null");
    const auto found = specs_.find(name);
    if (found == specs_.end()) {
        throw std::runtime_error(std::string("tensor is not part of the talker checkpoint: ") + name);
    }
    const Spec& spec = found->second;
    uint64_t elements = 1;
    for (uint64_t d : spec.shape) elements *= d;
    TensorImage image;
    image.data = spec.destination;
    image.quantized = spec.quantize;
    image.loaded = spec.seen;
    if (spec.quantize) {
        image.data_bytes = elements;                          // one int8 per weight
        image.scales = spec.scales;
        image.scales_bytes = spec.shape[0] * sizeof(float);   // one scale per output row
    } else {
        image.data_bytes = elements * sizeof(bf16);
    }
    return image;
}

void Model::adopt_tensor(const char* name) {
    check_cuda(cudaSetDevice(device_), "cudaSetDevice(adopt)");
    if (finalized_) throw std::runtime_error("model weights are already finalized");
    if (name == nullptr) throw std::runtime_error("tensor name is null");
    const auto found = specs_.find(name);
    if (found == specs_.end()) {
        throw std::runtime_error(std::string("tensor is not part of the talker checkpoint: ") + name);
    }
    Spec& spec = found->second;
    if (spec.seen) throw std::runtime_error(std::string("duplicate tensor upload: ") + name);
    uint64_t elements = 1;
    for (uint64_t d : spec.shape) elements *= d;
    spec.seen = true;
    weight_bytes_ += elements * sizeof(bf16);     // counted as the checkpoint tensor it stands for
    ++tensor_count_;
}

void Model::finalize(uint64_t* weight_bytes, uint32_t* tensor_count) {
    check_cuda(cudaSetDevice(device_), "cudaSetDevice(finalize)");
    if (finalized_) throw std::runtime_error("model weights are already finalized");
    if (tensor_count_ != 404 || specs_.size() != 404) {
        for (const auto& kv : specs_) {
            if (!kv.second.seen) {
                throw std::runtime_error("checkpoint is missing required tensor " + kv.first);
            }
        }
        throw std::runtime_error("expected exactly 404 VoiceDesign tensors, found "
                                 + std::to_string(tensor_count_));
    }
    check_cuda(cudaStreamSynchronize(upload_stream_), "cudaStreamSynchronize(upload)");
    staging_ = DeviceBuffer();
    embedding_ptrs_ = DeviceBuffer(kResidualCodebooks * sizeof(const bf16*));
    check_cuda(cudaMemcpy(embedding_ptrs_.as<void>(), predictor_embeddings.data(),
                          kResidualCodebooks * sizeof(const bf16*), cudaMemcpyHostToDevice),
               "cudaMemcpy(embedding table)");
    predictor_embedding_table = embedding_ptrs_.as<const bf16*>();
    talker_rope_ = DeviceBuffer((size_t)kRopePositions * (talker.head_dim / 2) * sizeof(uint32_t));
    check_cuda(launch_build_rope_table(talker_rope_.as<uint32_t>(), kRopePositions, talker.head_dim,
                                       kRopeTheta, upload_stream_), "rope table");
    talker_rope = talker_rope_.as<uint32_t>();
    if (predictor.head_dim == talker.head_dim) {
        predictor_rope = talker_rope;
    } else {
        predictor_rope_ = DeviceBuffer((size_t)kRopePositions * (predictor.head_dim / 2) * sizeof(uint32_t));
        check_cuda(launch_build_rope_table(predictor_rope_.as<uint32_t>(), kRopePositions, predictor.head_dim,
                                           kRopeTheta, upload_stream_), "rope table");
        predictor_rope = predictor_rope_.as<uint32_t>();
    }
    check_cuda(cudaStreamSynchronize(upload_stream_), "cudaStreamSynchronize(rope tables)");
    talker_pool.reset(new KvPool(talker.layers, talker.kv_width, 8));
    predictor_pool.reset(new KvPool(predictor.layers, predictor.kv_width, 6));
    finalized_ = true;
    *weight_bytes = weight_bytes_;
    *tensor_count = tensor_count_;
}

unsigned int Model::device_errors() const {
    volatile unsigned int* word = device_error_word(device_);
    return word != nullptr ? *word : 0u;
}

void Model::check_device_errors(unsigned int count_at_enqueue) const {
    if (device_errors() != count_at_enqueue) {
        throw CudaFailure("a bounded device-side wait ran out: the results of this call cannot be trusted");
    }
}

Workspace& Model::batch_workspace() {
    std::lock_guard<std::mutex> lock(mutex);
    if (!batch_) batch_.reset(new Workspace(kMaxRows, device_));
    return *batch_;
}

Workspace& Model::prefill_workspace() {
    std::lock_guard<std::mutex> lock(mutex);
    if (!prefill_) prefill_.reset(new Workspace(kMaxRows, device_));
    return *prefill_;
}

// ------------------------------------------------------------------ frame enqueue

namespace {

// Observation points of a prompt pass for the parity hooks (QWEN3_TTS_PARITY_TRACE,
// QWEN3_TTS_STAGE_DUMP): called with the stage name, the layer and one activation row in device
// memory.  Each call synchronises the stream, so a probed pass is never captured in a graph.
struct Probe {
    int row = 0;       // which row of the pass is observed (the last prompt position)
    std::function<void(const char* stage, int layer, const bf16* values, int width)> emit;
};

void enqueue_layers(Workspace& w, const ModelDims& d, const std::vector<LayerWeights>& layers,
                    const uint32_t* rope_table, const KvPool& pool, const int* page_table, int table_stride,
                    const int* positions, int n, int splits, cudaStream_t s, bool shared_cache = false,
                    const Probe* probe = nullptr) {
    const int qkv_width = d.q_width + 2 * d.kv_width;
    for (size_t l = 0; l < layers.size(); ++l) {
        const LayerWeights& lw = layers[l];
        const int layer = static_cast<int>(l);
        auto observe = [&](const char* stage, const bf16* base, int stride, int width) {
            if (probe != nullptr) probe->emit(stage, layer, base + (size_t)probe->row * stride, width);
        };
        GemvArgs g;
        g.w = lw.qkv.data; g.scales = lw.qkv.scales;
        g.x = w.hidden.as<bf16>(); g.y = w.qkv.as<bf16>();
        g.norm_w = lw.input_norm;
        if (probe != nullptr) g.norm_out = w.normalized.as<bf16>();
        g.in_features = d.hidden; g.out_features = qkv_width; g.rows = n; g.epilogue = EPI_PLAIN;
        check_launch(launch_int8_gemm(g, s), "qkv projection");
        observe("input_norm", w.normalized.as<bf16>(), d.hidden, d.hidden);
        observe("q_projection", w.qkv.as<bf16>(), qkv_width, d.q_width);
        observe("k_projection", w.qkv.as<bf16>() + d.q_width, qkv_width, d.kv_width);
        observe("v_projection", w.qkv.as<bf16>() + d.q_width + d.kv_width, qkv_width, d.kv_width);

        AttentionArgs a;
        a.q = w.qkv.as<bf16>();
        a.k_new = w.qkv.as<bf16>() + d.q_width;
        a.v_new = w.qkv.as<bf16>() + d.q_width + d.kv_width;
        a.q_stride = qkv_width; a.kv_new_stride = qkv_width;
        a.q_norm_w = lw.q_norm; a.k_norm_w = lw.k_norm;
        a.positions = positions;
        a.out = w.attention.as<bf16>();
        a.kv = pool.layout(static_cast<int>(l), page_table, table_stride);
        a.scratch = w.scratch.as<float>();
        a.counters = w.counters.as<unsigned int>();
        a.rows = n; a.q_heads = d.q_heads; a.kv_heads = d.kv_heads; a.head_dim = d.head_dim;
        a.max_splits = splits; a.fused = 1;
        a.rope_table = rope_table; a.rope_positions = Model::kRopePositions;
        // The kernel directly before attention is the qkv projection; positions, page table and
        // the older cache rows all date from earlier launches (the kernel ignores this outside
        // plain decode steps).
        a.inputs_settled = 1;
        if (shared_cache) {
            // the rows are consecutive positions of one session: every row's K/V goes into the
            // cache first, then every row attends up to its own position
            a.append_mode = 1;
            check_launch(launch_attention(a, s), "prompt KV append");
            a.append_mode = 2;
        }
        check_launch(launch_attention(a, s), "decode attention");
        observe("attention", w.attention.as<bf16>(), d.q_width, d.q_width);

        GemvArgs o;
        o.w = lw.o.data; o.scales = lw.o.scales;
        o.x = w.attention.as<bf16>(); o.y = w.hidden.as<bf16>();
        o.in_features = d.q_width; o.out_features = d.hidden; o.rows = n; o.epilogue = EPI_ADD;
        o.residual_settled = true;     // hidden was last written before the qkv projection
        check_launch(launch_int8_gemm(o, s), "attention output projection");
        observe("attention_residual", w.hidden.as<bf16>(), d.hidden, d.hidden);

        GemvArgs u;
        u.w = lw.gate_up.data; u.scales = lw.gate_up.scales;
        u.x = w.hidden.as<bf16>(); u.y = w.gate.as<bf16>();
        u.norm_w = lw.post_norm;
        if (probe != nullptr) u.norm_out = w.normalized.as<bf16>();
        u.in_features = d.hidden; u.out_features = d.intermediate; u.rows = n;
        u.epilogue = EPI_GATE_UP_SILU;
        check_launch(launch_int8_gemm(u, s), "gate/up projection");
        observe("post_attention_norm", w.normalized.as<bf16>(), d.hidden, d.hidden);
        observe("gated_activation", w.gate.as<bf16>(), d.intermediate, d.intermediate);

        GemvArgs dn;
        dn.w = lw.down.data; dn.scales = lw.down.scales;
        dn.x = w.gate.as<bf16>(); dn.y = w.hidden.as<bf16>();
        dn.in_features = d.intermediate; dn.out_features = d.hidden; dn.rows = n;
        dn.epilogue = EPI_ADD;
        dn.residual_settled = true;    // hidden was last written by the output projection, two launches up
        check_launch(launch_int8_gemm(dn, s), "down projection");
        observe("layer_output", w.hidden.as<bf16>(), d.hidden, d.hidden);
    }
}

// 16 predictor positions, 15 sampled codebooks, packed codes (talker.cu:1549-1701)
void enqueue_predictor(Workspace& w, Model& m, int n, cudaStream_t s) {
    const FrameTable* table = w.table.as<FrameTable>();
    const int H = m.talker.hidden, PH = m.predictor.hidden;
    check_launch(launch_frame_begin(table, n, s), "frame begin");
    for (int p = 0; p < kPredictorSequence; ++p) {
        check_launch(launch_predictor_input(table, p, m.codec_embedding, m.predictor_embedding_table,
                                          w.x_in.as<bf16>(), H, n, s), "predictor input");
        GemvArgs g;
        g.w = m.small_to_mtp.data; g.scales = m.small_to_mtp.scales;
        g.x = w.x_in.as<bf16>(); g.y = w.hidden.as<bf16>(); g.bias = m.small_to_mtp_bias;
        g.in_features = H; g.out_features = PH; g.rows = n; g.epilogue = EPI_BIAS;
        check_launch(launch_int8_gemm(g, s), "predictor input projection");
        enqueue_layers(w, m.predictor, m.predictor_layers, m.predictor_rope, *m.predictor_pool,
                       w.predictor_pages.as<int>(), 1,
                       w.predictor_positions.as<int>() + (size_t)p * kMaxRows, n, 1, s);
        if (p >= 1) {
            GemvArgs h;
            h.w = m.predictor_heads[p - 1].data; h.scales = m.predictor_heads[p - 1].scales;
            h.x = w.hidden.as<bf16>(); h.y = w.logits.as<bf16>(); h.norm_w = m.predictor_norm;
            h.in_features = PH; h.out_features = kPredictorVocab; h.rows = n; h.epilogue = EPI_PLAIN;
            check_launch(launch_int8_gemm(h, s), "predictor head");
            check_launch(launch_sample_table(table, w.logits.as<bf16>(), kPredictorVocab,
                                           kPredictorVocab, 0, p, 0, kEos, n, s),
                       "sample predictor logits");
        }
    }
    check_launch(launch_pack_codes(table, n, s), "pack codec frame");
}

void enqueue_text_projection(Workspace& w, Model& m, int n, bool residual, cudaStream_t s) {
    const int H = m.talker.hidden;
    GemvArgs f1;
    f1.w = m.text_fc1.data; f1.scales = m.text_fc1.scales;
    f1.x = w.x_in.as<bf16>(); f1.y = w.projection.as<bf16>(); f1.bias = m.text_fc1_bias;
    f1.in_features = H; f1.out_features = H; f1.rows = n; f1.epilogue = EPI_BIAS_SILU;
    check_launch(launch_int8_gemm(f1, s), "text projection fc1");
    GemvArgs f2;
    f2.w = m.text_fc2.data; f2.scales = m.text_fc2.scales;
    f2.x = w.projection.as<bf16>(); f2.bias = m.text_fc2_bias;
    f2.in_features = H; f2.out_features = H; f2.rows = n;
    if (residual) {
        f2.resid = w.hidden.as<bf16>(); f2.epilogue = EPI_BIAS_ADD;
    } else {
        f2.y = w.hidden.as<bf16>(); f2.epilogue = EPI_BIAS;
    }
    check_launch(launch_int8_gemm(f2, s), "text projection fc2");
}

void enqueue_talker_head(Workspace& w, Model& m, int n, int advance, cudaStream_t s) {
    FrameTable* table = w.table.as<FrameTable>();
    const int H = m.talker.hidden;
    GemvArgs h;
    h.w = m.codec_head.data; h.scales = m.codec_head.scales;
    h.x = w.hidden.as<bf16>(); h.y = w.logits.as<bf16>();
    h.norm_w = m.talker_norm; h.norm_out = w.normalized.as<bf16>();
    h.in_features = H; h.out_features = kTalkerVocab; h.rows = n; h.epilogue = EPI_PLAIN;
    check_launch(launch_int8_gemm(h, s), "codec head");
    check_launch(launch_sample_table(table, w.logits.as<bf16>(), kTalkerVocab, kTalkerVocab, 1, 0,
                                   m.mask_eos, kEos, n, s), "sample talker logits");
    check_launch(launch_frame_end(table, w.normalized.as<bf16>(), H, n, advance, s), "frame end");
}

// next talker input, 28 layers, head, sample (talker.cu:1703-1880)
void enqueue_talker(Workspace& w, Model& m, int n, int splits, cudaStream_t s) {
    FrameTable* table = w.table.as<FrameTable>();
    const int H = m.talker.hidden;
    check_launch(launch_talker_input(table, m.codec_embedding, m.predictor_embedding_table,
                                   m.text_embedding, kTextVocab, w.hidden.as<bf16>(),
                                   w.x_in.as<bf16>(), H, n, s), "talker input");
    enqueue_text_projection(w, m, n, true, s);
    enqueue_layers(w, m.talker, m.talker_layers, m.talker_rope, *m.talker_pool, w.talker_pages.as<int>(),
                   Workspace::kMaxPagesPerRow, table->position, n, splits, s);
    enqueue_talker_head(w, m, n, 1, s);
}

// one prompt position of row 0 (talker.cu:1058-1064 + one decoder pass)
void enqueue_prompt_step(Workspace& w, Model& m, const int* text_ids, const int* codec_ids,
                         int splits, cudaStream_t s) {
    FrameTable* table = w.table.as<FrameTable>();
    const int H = m.talker.hidden;
    check_launch(launch_prompt_gather(table, text_ids, m.text_embedding, kTextVocab,
                                    w.x_in.as<bf16>(), H, s), "prompt gather");
    enqueue_text_projection(w, m, 1, false, s);
    check_launch(launch_prompt_combine(table, text_ids, codec_ids, m.codec_embedding, kTalkerVocab,
                                     w.hidden.as<bf16>(), H, s), "prompt combine");
    enqueue_layers(w, m.talker, m.talker_layers, m.talker_rope, *m.talker_pool, w.talker_pages.as<int>(),
                   Workspace::kMaxPagesPerRow, table->position, 1, splits, s);
    check_launch(launch_advance_position(table, s), "advance position");
}

// prompt positions base .. base + rows - 1 of row 0's session as the rows of one decoder pass
void enqueue_prompt_chunk(Workspace& w, Model& m, const int* text_ids, const int* codec_ids, int base,
                          int rows, int splits, cudaStream_t s, const Probe* probe = nullptr) {
    const int H = m.talker.hidden;
    check_launch(launch_prompt_rows(text_ids, codec_ids, base, rows, m.text_embedding, kTextVocab,
                                  w.x_in.as<bf16>(), w.prompt_positions.as<int>(), H, s), "prompt rows");
    enqueue_text_projection(w, m, rows, false, s);
    check_launch(launch_prompt_combine_rows(text_ids, codec_ids, base, rows, m.codec_embedding, kTalkerVocab,
                                          w.hidden.as<bf16>(), H, s), "prompt combine");
    if (probe != nullptr) probe->emit("input", -1, w.hidden.as<bf16>() + (size_t)probe->row * H, H);
    // page-table stride 0: every row reads and writes the cache of the session bound to row 0
    enqueue_layers(w, m.talker, m.talker_layers, m.talker_rope, *m.talker_pool, w.talker_pages.as<int>(), 0,
                   w.prompt_positions.as<int>(), rows, splits, s, true, probe);
}

// ---- parity hooks of the prompt path --------------------------------------------------------
// QWEN3_TTS_PARITY_TRACE: one line per observed vector on stderr, in the reference's format
// (talker.cu:2342-2432: "QWEN3_TTS_TRACE {json}" with stage, layer, mean, rms, maximum and the first
// 16 values; the 20 largest logits at the end), for the input row, every layer's output, the final
// norm and the logits of the last prompt position.  QWEN3_TTS_STAGE_DUMP: the layer-0 stages and the
// final logits as raw bf16 files named <stage>.bf16, in the directory the variable names (a value
// without a slash selects the reference's /tmp/native_stages, talker.cu:2503-2538).
struct ParityHooks {
    bool trace = false;
    std::string dump_dir;
    cudaStream_t stream = nullptr;

    static ParityHooks from_environment(cudaStream_t s) {
        ParityHooks h;
        h.stream = s;
        h.trace = std::getenv("QWEN3_TTS_PARITY_TRACE") != nullptr;
        if (const char* d = std::getenv("QWEN3_TTS_STAGE_DUMP")) {
            h.dump_dir = std::strchr(d, '/') != nullptr ? d : "/tmp/native_stages";
        }
        return h;
    }
    bool active() const { return trace || !dump_dir.empty(); }

    std::vector<float> fetch(const bf16* values, int width) const {
        std::vector<bf16> raw(width);
        check_cuda(cudaMemcpyAsync(raw.data(), values, (size_t)width * sizeof(bf16), cudaMemcpyDeviceToHost,
                                   stream), "copy parity vector to host");
        check_cuda(cudaStreamSynchronize(stream), "synchronize parity vector");
        std::vector<float> out(width);
        for (int i = 0; i < width; ++i) out[i] = __bfloat162float(raw[i]);
        return out;
    }
    void dump(const char* stage, const bf16* values, int width) const {
        if (dump_dir.empty()) return;
        std::vector<bf16> raw(width);
        check_cuda(cudaMemcpyAsync(raw.data(), values, (size_t)width * sizeof(bf16), cudaMemcpyDeviceToHost,
                                   stream), "copy stage dump to host");
        check_cuda(cudaStreamSynchronize(stream), "synchronize stage dump");
        const std::string path = dump_dir + "/" + stage + ".bf16";
        std::FILE* f = std::fopen(path.c_str(), "wb");
        if (f == nullptr) throw std::runtime_error("failed to create stage dump " + path);
        const size_t written = std::fwrite(raw.data(), sizeof(bf16), raw.size(), f);
        if (std::fclose(f) != 0 || written != raw.size()) throw std::runtime_error("failed to write stage dump " + path);
    }
    void vector_line(const char* stage, int layer, const bf16* values, int width) const {
        if (!trace) return;
        const std::vector<float> v = fetch(values, width);
        double sum = 0.0, squares = 0.0;
        float largest = 0.0f;
        for (float x : v) {
            sum += x;
            squares += (double)x * x;
            largest = std::max(largest, std::fabs(x));
        }
        std::string line = "QWEN3_TTS_TRACE {\"stage\":\"" + std::string(stage) + "\",\"layer\":" + std::to_string(layer);
        char number[64];
        std::snprintf(number, sizeof(number), ",\"mean\":%.9g", sum / width); line += number;
        std::snprintf(number, sizeof(number), ",\"rms\":%.9g", std::sqrt(squares / width)); line += number;
        std::snprintf(number, sizeof(number), ",\"maximum\":%.9g,\"first\":[", largest); line += number;
        for (int i = 0; i < std::min(width, 16); ++i) {
            std::snprintf(number, sizeof(number), "%s%.9g", i == 0 ? "" : ",", v[i]);
            line += number;
        }
        std::fprintf(stderr, "%s]}\n", line.c_str());
    }
    void logits_line(const bf16* logits, int vocabulary) const {
        if (!trace) return;
        const std::vector<float> v = fetch(logits, vocabulary);
        std::vector<int> order(vocabulary);
        std::iota(order.begin(), order.end(), 0);
        const int top = std::min(20, vocabulary);
        std::partial_sort(order.begin(), order.begin() + top, order.end(),
                          [&v](int a, int b) { return v[a] == v[b] ? a < b : v[a] > v[b]; });
        std::string line = "QWEN3_TTS_TRACE {\"stage\":\"logits\",\"top\":[";
        char item[96];
        for (int r = 0; r < top; ++r) {
            std::snprintf(item, sizeof(item), "%s{\"token\":%d,\"logit\":%.9g}", r == 0 ? "" : ",", order[r], v[order[r]]);
            line += item;
        }
        std::fprintf(stderr, "%s]}\n", line.c_str());
    }
    // the probe a prompt pass is run with
    Probe probe(int row) const {
        Probe p;
        p.row = row;
        const ParityHooks* self = this;
        p.emit = [self](const char* stage, int layer, const bf16* values, int width) {
            const bool input = std::strcmp(stage, "input") == 0;
            const bool output = std::strcmp(stage, "layer_output") == 0;
            if (input) self->vector_line("input", -1, values, width);
            if (output) self->vector_line("layer", layer, values, width);
            if (input || layer == 0) self->dump(stage, values, width);
        };
        return p;
    }
};

int count_kernel_nodes(cudaGraph_t graph) {
    size_t total = 0;
    if (cudaGraphGetNodes(graph, nullptr, &total) != cudaSuccess || total == 0) return 0;
    std::vector<cudaGraphNode_t> nodes(total);
    if (cudaGraphGetNodes(graph, nodes.data(), &total) != cudaSuccess) return 0;
    int kernels = 0;
    for (size_t i = 0; i < total; ++i) {
        cudaGraphNodeType type;
        if (cudaGraphNodeGetType(nodes[i], &type) == cudaSuccess && type == cudaGraphNodeTypeKernel) {
            ++kernels;
        }
    }
    return kernels;
}

template <class Enqueue>
cudaGraphExec_t capture(cudaStream_t s, Enqueue&& enqueue, int* kernel_nodes = nullptr) {
    check_cuda(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
    cudaGraph_t graph = nullptr;
    try {
        enqueue();
    } catch (...) {
        cudaStreamEndCapture(s, &graph);
        if (graph != nullptr) cudaGraphDestroy(graph);
        throw;
    }
    check_cuda(cudaStreamEndCapture(s, &graph), "cudaStreamEndCapture");
    if (kernel_nodes != nullptr) *kernel_nodes = count_kernel_nodes(graph);
    cudaGraphExec_t exec = nullptr;
    const cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    check_cuda(e, "cudaGraphInstantiate");
    return exec;
}

int split_bucket(int max_length) {
    const int splits = (max_length + kAttnChunk - 1) / kAttnChunk;
    return (splits + 7) / 8 * 8;
}

void validate_sampling_params(const SamplingParams& p) {
    if (p.top_k < 0 || !(p.top_p > 0.0f) || p.top_p > 1.0f || !(p.temperature > 0.0f)
        || !(p.penalty > 0.0f)) {
        throw std::runtime_error("invalid sampling configuration");
    }
}

}  // namespace

// ------------------------------------------------------------------ Session

Session::Session(std::shared_ptr<Model> model, int max_sequence_length, uint64_t seed)
    : model_(std::move(model)), id_(g_next_session_id.fetch_add(1)), device_(model_->device()),
      max_seq_(max_sequence_length) {
    if (max_sequence_length < 16 || max_sequence_length > 8192) {
        throw std::runtime_error("max sequence length must be in [16, 8192]");
    }
    if (!model_->finalized()) {
        throw std::runtime_error("model weights must be finalized before creating a session");
    }
    check_cuda(cudaSetDevice(device_), "cudaSetDevice(session)");
    solo_.reset(new Workspace(1, device_));
    stream_ = solo_->stream;
    try {
        check_cuda(cudaEventCreateWithFlags(&codes_ready_, cudaEventDisableTiming), "cudaEventCreate");
        check_cuda(cudaEventCreateWithFlags(&semantic_ready_, cudaEventDisableTiming), "cudaEventCreate");
        const size_t off_tokens = 0;
        const size_t off_codes = align_up(off_tokens + kCodebooks * sizeof(int), 256);
        const size_t off_sampled = align_up(off_codes + kCodebooks * sizeof(unsigned short), 256);
        const size_t off_rng = align_up(off_sampled + sizeof(int), 256);
        const size_t off_hidden = align_up(off_rng + sizeof(unsigned long long), 256);
        const size_t off_history = align_up(off_hidden + 2048 * sizeof(bf16), 256);
        const size_t total = off_history + (size_t)max_seq_ * sizeof(int);
        state_ = DeviceBuffer(total);
        check_cuda(cudaMemset(state_.as<void>(), 0, total), "cudaMemset(session state)");
        char* base = state_.as<char>();
        d_frame_tokens_ = reinterpret_cast<int*>(base + off_tokens);
        d_frame_codes_ = reinterpret_cast<unsigned short*>(base + off_codes);
        d_sampled_ = reinterpret_cast<int*>(base + off_sampled);
        d_rng_ = reinterpret_cast<unsigned long long*>(base + off_rng);
        d_last_hidden_ = reinterpret_cast<bf16*>(base + off_hidden);
        d_history_ = reinterpret_cast<int*>(base + off_history);
        check_cuda(cudaHostAlloc(reinterpret_cast<void**>(&h_token_), sizeof(int), cudaHostAllocMapped),
                   "cudaHostAlloc(sampled token)");
        check_cuda(cudaHostAlloc(reinterpret_cast<void**>(&h_codes_), kCodebooks * sizeof(unsigned short),
                                 cudaHostAllocMapped), "cudaHostAlloc(frame codes)");
        *h_token_ = -1;
        {
            std::lock_guard<std::mutex> lock(model_->mutex);
            const int pages = (max_seq_ + kPageTokens - 1) / kPageTokens;
            for (int i = 0; i < pages; ++i) talker_pages_.push_back(model_->talker_pool->allocate());
            predictor_page_ = model_->predictor_pool->allocate();
            talker_kv_bytes = (uint64_t)pages * model_->talker_pool->page_bytes();
            predictor_kv_bytes = model_->predictor_pool->page_bytes();
        }
        solo_->ensure_scratch(split_bucket(max_seq_ < 512 ? max_seq_ : 512));
        workspace_bytes = solo_->bytes() + state_.bytes();
        reset(seed);
    } catch (...) {
        release();
        throw;
    }
}

void Session::release() noexcept {
    if (model_) {
        std::lock_guard<std::mutex> lock(model_->mutex);
        for (int page : talker_pages_) model_->talker_pool->release(page);
        talker_pages_.clear();
        if (predictor_page_ >= 0) model_->predictor_pool->release(predictor_page_);
        predictor_page_ = -1;
    }
    if (h_codes_ != nullptr) cudaFreeHost(h_codes_);
    h_codes_ = nullptr;
    if (h_token_ != nullptr) cudaFreeHost(h_token_);
    h_token_ = nullptr;
    if (semantic_ready_ != nullptr) cudaEventDestroy(semantic_ready_);
    semantic_ready_ = nullptr;
    if (codes_ready_ != nullptr) cudaEventDestroy(codes_ready_);
    codes_ready_ = nullptr;
}

Session::~Session() {
    cudaSetDevice(device_);
    // A lockstep frame of this session that was begun and never finished may still be running on
    // the shared workspace: its last event is this session's own, so no other thread's stream (which
    // may be capturing a graph at this moment) has to be touched.  Workspaces remember bound sessions
    // by id, and ids are never reused, so nothing has to be erased from them either.
    if (frame_in_flight_ && semantic_ready_ != nullptr) cudaEventSynchronize(semantic_ready_);
    if (stream_ != nullptr) cudaStreamSynchronize(stream_);
    release();
    solo_.reset();
}

void Session::reset(uint64_t seed) {
    own_stream_busy_ = true;
    check_cuda(cudaSetDevice(device_), "cudaSetDevice(reset)");
    if (frame_in_flight_) throw std::runtime_error("cannot reset while a device frame lease is in flight");
    position_ = 0;
    generated_ = 0;
    frames_generated = 0;
    device_sample_count = 0;
    host_sync_count = 0;
    current_token_ = 0;
    phase_ = model_->finalized() ? kPhaseReady : kPhaseCreated;
    const unsigned long long state = seed == 0 ? 0x9e3779b97f4a7c15ULL : seed;
    check_cuda(cudaMemcpyAsync(d_rng_, &state, sizeof(state), cudaMemcpyHostToDevice, stream_),
               "reset device random state");
    check_cuda(cudaStreamSynchronize(stream_), "synchronize reset random state");
}

void Session::fill_row(FrameTable& t, int row, int trailing_text, const SamplingParams& talker,
                       const SamplingParams& predictor, bool host_codes) const {
    t.position[row] = position_;
    t.history_count[row] = generated_;
    t.trailing_text[row] = trailing_text;
    t.frame_tokens[row] = d_frame_tokens_;
    t.frame_codes[row] = d_frame_codes_;
    t.history[row] = d_history_;
    t.rng[row] = d_rng_;
    t.sampled[row] = d_sampled_;
    t.last_hidden[row] = d_last_hidden_;
    t.host_token[row] = h_token_;
    t.host_codes[row] = host_codes ? h_codes_ : nullptr;
    t.talker[row] = talker;
    t.predictor[row] = predictor;
}

// the checks of the reference's begin_frame, in its order (talker.cu:1103-1127)
void Session::validate_begin(int semantic_token, int trailing_text, const SamplingParams& talker,
                             const SamplingParams& predictor) const {
    if (poisoned_) throw std::runtime_error("talker session is poisoned and must be destroyed");
    if (frame_in_flight_) throw std::runtime_error("a device frame lease is already in flight");
    if (phase_ != kPhasePrefilled) {
        throw std::runtime_error("talker must be prefilled before frame generation");
    }
    if (semantic_token == kEos) throw std::runtime_error("EOS must not be expanded into a codec frame");
    if (semantic_token >= kTalkerVocab) {
        throw std::runtime_error("semantic token is outside the talker vocabulary");
    }
    if (semantic_token != current_token_) {
        throw std::runtime_error("semantic token does not match talker session state");
    }
    if (trailing_text < 0 || trailing_text >= kTextVocab) {
        throw std::runtime_error("next-frame text token is outside the text vocabulary");
    }
    if (position_ >= max_seq_) throw std::runtime_error("talker KV cache is full");
    if (generated_ >= max_seq_) {
        throw std::runtime_error("semantic history exceeds configured sequence capacity");
    }
    validate_sampling_params(talker);
    validate_sampling_params(predictor);
}

// Makes the page lists of s[0..n) resident in the workspace's page tables.
void Session::bind_rows(Workspace& w, Session** s, int n) {
    bool same = static_cast<int>(w.bound.size()) == n;
    for (int i = 0; same && i < n; ++i) same = w.bound[i] == s[i]->id_;
    if (same) return;
    check_cuda(cudaStreamSynchronize(w.stream), "cudaStreamSynchronize(rebind)");
    const int stride = Workspace::kMaxPagesPerRow;
    int* talker_rows = w.host_pages;
    int* predictor_rows = w.host_pages + (size_t)w.capacity * stride;
    for (int i = 0; i < n; ++i) {
        const std::vector<int>& pages = s[i]->talker_pages_;
        std::copy(pages.begin(), pages.end(), talker_rows + (size_t)i * stride);
        predictor_rows[i] = s[i]->predictor_page_;
    }
    check_cuda(cudaMemcpyAsync(w.talker_pages.as<void>(), talker_rows,
                               (size_t)n * stride * sizeof(int), cudaMemcpyHostToDevice, w.stream),
               "upload talker page table");
    check_cuda(cudaMemcpyAsync(w.predictor_pages.as<void>(), predictor_rows, (size_t)n * sizeof(int),
                               cudaMemcpyHostToDevice, w.stream), "upload predictor page table");
    w.bound.resize(n);
    for (int i = 0; i < n; ++i) w.bound[i] = s[i]->id_;
}

Workspace::Graphs& Session::frame_graphs(Workspace& w, Model& m, int n, int splits) {
    const auto key = std::make_pair(n, splits);
    auto found = w.graphs.find(key);
    if (found != w.graphs.end()) return found->second;
    Workspace::Graphs g;
    g.predictor = capture(w.stream, [&] { enqueue_predictor(w, m, n, w.stream); },
                          &g.predictor_kernels);
    try {
        g.talker = capture(w.stream, [&] { enqueue_talker(w, m, n, splits, w.stream); },
                           &g.talker_kernels);
    } catch (...) {
        cudaGraphExecDestroy(g.predictor);
        throw;
    }
    return w.graphs.emplace(key, g).first->second;
}

// Enqueues one frame for rows s[0..n) on w.stream.  The host table must be filled.
void Session::launch_frame(Workspace& w, Model& m, Session** s, int n, bool upload_table,
                           bool record_session_events) {
    int max_length = 1;
    for (int i = 0; i < n; ++i) max_length = std::max(max_length, w.host_table->position[i] + 1);
    const int splits = split_bucket(max_length);
    ++w.frame_serial;
    if (w.option_epoch != m.option_epoch) {
        check_cuda(cudaStreamSynchronize(w.stream), "cudaStreamSynchronize(options)");
        w.destroy_graphs();
        w.option_epoch = m.option_epoch;
    }
    w.ensure_scratch(splits);
    bind_rows(w, s, n);
    if (upload_table) {
        check_cuda(cudaMemcpyAsync(w.table.as<void>(), w.host_table, sizeof(FrameTable),
                                   cudaMemcpyHostToDevice, w.stream), "upload frame table");
        check_cuda(cudaEventRecord(w.table_uploaded, w.stream), "cudaEventRecord(table)");
    }
    if (m.use_graphs) {
        Workspace::Graphs& g = frame_graphs(w, m, n, splits);
        check_cuda(cudaEventRecord(w.predictor_start, w.stream), "cudaEventRecord");
        check_cuda(cudaGraphLaunch(g.predictor, w.stream), "cudaGraphLaunch(predictor)");
        check_cuda(cudaEventRecord(w.predictor_stop, w.stream), "cudaEventRecord");
        if (record_session_events) {
            for (int i = 0; i < n; ++i) {
                check_cuda(cudaEventRecord(s[i]->codes_ready_, w.stream), "cudaEventRecord(codes)");
            }
        }
        check_cuda(cudaEventRecord(w.talker_start, w.stream), "cudaEventRecord");
        check_cuda(cudaGraphLaunch(g.talker, w.stream), "cudaGraphLaunch(talker)");
        check_cuda(cudaEventRecord(w.talker_stop, w.stream), "cudaEventRecord");
        m.kernel_launches += static_cast<uint64_t>(g.predictor_kernels + g.talker_kernels);
    } else {
        check_cuda(cudaEventRecord(w.predictor_start, w.stream), "cudaEventRecord");
        enqueue_predictor(w, m, n, w.stream);
        check_cuda(cudaEventRecord(w.predictor_stop, w.stream), "cudaEventRecord");
        if (record_session_events) {
            for (int i = 0; i < n; ++i) {
                check_cuda(cudaEventRecord(s[i]->codes_ready_, w.stream), "cudaEventRecord(codes)");
            }
        }
        check_cuda(cudaEventRecord(w.talker_start, w.stream), "cudaEventRecord");
        enqueue_talker(w, m, n, splits, w.stream);
        check_cuda(cudaEventRecord(w.talker_stop, w.stream), "cudaEventRecord");
    }
    if (record_session_events) {
        for (int i = 0; i < n; ++i) {
            check_cuda(cudaEventRecord(s[i]->semantic_ready_, w.stream), "cudaEventRecord(semantic)");
        }
    }
}

uint64_t Session::take_lease(Workspace* w, bool host_codes) {
    const uint64_t lease = next_lease_++;
    if (next_lease_ == 0) next_lease_ = 1;
    frame_in_flight_ = true;
    pending_host_codes_ = host_codes;
    pending_lease_ = lease;
    pending_position_ = static_cast<uint32_t>(position_);
    pending_workspace_ = w;
    pending_frame_serial_ = w != nullptr ? w->frame_serial + 1 : 0;    // the frame about to be launched
    pending_errors_ = model_->device_errors();
    return lease;
}

void Session::drop_lease_poisoned() noexcept {
    poisoned_ = true;
    frame_in_flight_ = false;
    pending_host_codes_ = false;
    pending_lease_ = 0;
    pending_workspace_ = nullptr;
}

FrameView Session::begin_frame(uint16_t semantic_token, int trailing_text, const SamplingParams& talker,
                               const SamplingParams& predictor, bool host_codes) {
    check_cuda(cudaSetDevice(device_), "cudaSetDevice(begin frame)");
    validate_begin(semantic_token, trailing_text, talker, predictor);
    Workspace& w = *solo_;
    own_stream_busy_ = true;
    const uint64_t lease = take_lease(&w, host_codes);
    try {
        check_cuda(cudaEventSynchronize(w.table_uploaded), "cudaEventSynchronize(table)");
        fill_row(*w.host_table, 0, trailing_text, talker, predictor, host_codes);
        Session* self = this;
        launch_frame(w, *model_, &self, 1, true, true);
    } catch (...) {
        cudaStreamSynchronize(stream_);
        drop_lease_poisoned();
        throw;
    }
    device_sample_count += kPredictorSequence;
    ++generated_;
    ++position_;
    FrameView view;
    view.device_codes = d_frame_codes_;
    view.ready_event = codes_ready_;
    view.lease_id = lease;
    view.device = device_;
    return view;
}

void Session::batch_begin(Model* model, Session** s, int n, const int* trailing_text,
                          const SamplingParams* talker, const SamplingParams* predictor,
                          FrameView* views) {
    if (model == nullptr || s == nullptr || n <= 0 || n > kMaxRows) {
        throw std::runtime_error("invalid batch frame arguments");
    }
    check_cuda(cudaSetDevice(model->device()), "cudaSetDevice(batch frame)");
    for (int i = 0; i < n; ++i) {
        if (s[i]->model_.get() != model) {
            throw std::runtime_error("batched session belongs to a different model");
        }
        for (int j = 0; j < i; ++j) {
            if (s[j] == s[i]) throw std::runtime_error("a session appears twice in one batch");
        }
        s[i]->validate_begin(s[i]->current_token_, trailing_text[i], talker[i], predictor[i]);
    }
    std::lock_guard<std::mutex> one_batch(model->batch_mutex);
    Workspace& w = model->batch_workspace();
    const bool host_codes = model->batch_host_codes != 0;
    for (int i = 0; i < n; ++i) s[i]->take_lease(&w, host_codes);
    try {
        check_cuda(cudaEventSynchronize(w.table_uploaded), "cudaEventSynchronize(table)");
        for (int i = 0; i < n; ++i) {
            s[i]->fill_row(*w.host_table, i, trailing_text[i], talker[i], predictor[i], host_codes);
        }
        // order the batch stream after each session's earlier work
        for (int i = 0; i < n; ++i) {
            if (!s[i]->own_stream_busy_) continue;      // nothing of its own since the last lockstep frame
            check_cuda(cudaEventRecord(w.join_events[i], s[i]->stream_), "cudaEventRecord(join)");
            check_cuda(cudaStreamWaitEvent(w.stream, w.join_events[i], 0), "cudaStreamWaitEvent(join)");
            s[i]->own_stream_busy_ = false;
        }
        launch_frame(w, *model, s, n, true, true);
        for (int i = 0; i < n; ++i) {
            s[i]->device_sample_count += kPredictorSequence;
            ++s[i]->generated_;
            ++s[i]->position_;
            check_cuda(cudaStreamWaitEvent(s[i]->stream_, s[i]->semantic_ready_, 0),
                       "cudaStreamWaitEvent(rejoin)");
        }
    } catch (...) {
        cudaStreamSynchronize(w.stream);
        for (int i = 0; i < n; ++i) s[i]->drop_lease_poisoned();
        w.destroy_graphs();
        throw;
    }
    for (int i = 0; i < n; ++i) {
        views[i].device_codes = s[i]->d_frame_codes_;
        views[i].ready_event = s[i]->codes_ready_;
        views[i].lease_id = s[i]->pending_lease_;
        views[i].device = s[i]->device_;
    }
}

FrameResult Session::finish_frame(uint64_t lease_id, cudaEvent_t consumer_done) {
    check_cuda(cudaSetDevice(device_), "cudaSetDevice(finish frame)");
    if (poisoned_) throw std::runtime_error("talker session is poisoned and must be destroyed");
    if (!frame_in_flight_) throw std::runtime_error("no device frame lease is in flight");
    if (lease_id == 0 || lease_id != pending_lease_) {
        throw std::runtime_error("device frame lease ID is stale or invalid");
    }
    if (consumer_done != nullptr) {
        check_cuda(cudaStreamWaitEvent(stream_, consumer_done, 0), "cudaStreamWaitEvent(consumer done)");
        own_stream_busy_ = true;
    }
    check_cuda(cudaEventSynchronize(semantic_ready_), "cudaEventSynchronize(semantic ready)");
    ++host_sync_count;
    const int next = *h_token_;
    try {
        model_->check_device_errors(pending_errors_);
        if (next < 0 || next >= kTalkerVocab) {
            throw std::runtime_error("device sampler returned an invalid token");
        }
    } catch (...) {
        drop_lease_poisoned();
        throw;
    }
    FrameResult r{};
    r.talker_position = pending_position_;
    Workspace* w = pending_workspace_;
    if (w != nullptr && w->timed_frame == pending_frame_serial_ && pending_frame_serial_ != 0) {
        r.predictor_ms = w->timed_predictor_ms;      // a sibling of this lockstep frame already asked
        r.talker_ms = w->timed_talker_ms;
    } else if (w == nullptr || w->frame_serial != pending_frame_serial_
               || cudaEventElapsedTime(&r.predictor_ms, w->predictor_start, w->predictor_stop) != cudaSuccess
               || cudaEventElapsedTime(&r.talker_ms, w->talker_start, w->talker_stop) != cudaSuccess) {
        // a later frame of a shared workspace has re-recorded the timing events
        cudaGetLastError();
        r.predictor_ms = 0.0f;
        r.talker_ms = 0.0f;
    } else {
        w->timed_frame = pending_frame_serial_;
        w->timed_predictor_ms = r.predictor_ms;
        w->timed_talker_ms = r.talker_ms;
    }
    if (pending_host_codes_) std::copy_n(h_codes_, kCodebooks, r.codes);
    r.next_semantic = static_cast<uint16_t>(next);
    r.ended = next == kEos ? 1u : 0u;
    current_token_ = r.next_semantic;
    ++frames_generated;
    phase_ = r.ended ? kPhaseEnded : kPhasePrefilled;
    frame_in_flight_ = false;
    pending_host_codes_ = false;
    pending_lease_ = 0;
    pending_workspace_ = nullptr;
    return r;
}

void Session::prefill(const int32_t* text_ids, const int32_t* codec_ids, int count,
                      const SamplingParams& sampling, uint16_t* first_token, float* gpu_ms) {
    own_stream_busy_ = true;
    check_cuda(cudaSetDevice(device_), "cudaSetDevice(prefill)");
    if (poisoned_) throw std::runtime_error("talker session is poisoned and must be destroyed");
    if (frame_in_flight_) throw std::runtime_error("cannot prefill while a device frame lease is in flight");
    if (text_ids == nullptr || codec_ids == nullptr || count <= 0) {
        throw std::runtime_error("prefill requires non-empty text and codec ID arrays");
    }
    if (count > max_seq_) throw std::runtime_error("prompt exceeds the configured KV-cache capacity");
    for (int i = 0; i < count; ++i) {
        if (text_ids[i] < 0 && codec_ids[i] < 0) {
            throw std::runtime_error("a prompt position must contain text or codec input");
        }
        if (text_ids[i] >= kTextVocab || codec_ids[i] >= kTalkerVocab) {
            throw std::runtime_error("embedding token is outside its vocabulary");
        }
    }
    validate_sampling_params(sampling);
    Model& m = *model_;
    // A prompt runs as chunks of up to prefill_chunk positions per decoder pass (the rows of a
    // skinny GEMM) on the model's prompt workspace, one prompt at a time; with prefill_chunk = 1,
    // or a prompt of one position, it runs position by position on the session's own workspace.
    const int chunk = std::min(std::max(m.prefill_chunk, 1), kMaxRows);
    const ParityHooks hooks = ParityHooks::from_environment(nullptr);
    // the parity hooks observe the chunked pass (they synchronise, so nothing of it may be captured)
    const bool chunked = (chunk > 1 && count > 1) || hooks.active();
    std::unique_lock<std::mutex> one_prompt(m.prefill_mutex, std::defer_lock);
    if (chunked) one_prompt.lock();
    Workspace& w = chunked ? m.prefill_workspace() : *solo_;
    position_ = 0;
    generated_ = 0;
    const unsigned int errors_before = m.device_errors();
    try {
        DeviceBuffer ids(2 * (size_t)count * sizeof(int));
        int* d_text = ids.as<int>();
        int* d_codec = d_text + count;
        check_cuda(cudaMemcpyAsync(d_text, text_ids, (size_t)count * sizeof(int),
                                   cudaMemcpyHostToDevice, w.stream), "upload prompt text ids");
        check_cuda(cudaMemcpyAsync(d_codec, codec_ids, (size_t)count * sizeof(int),
                                   cudaMemcpyHostToDevice, w.stream), "upload prompt codec ids");
        check_cuda(cudaEventSynchronize(w.table_uploaded), "cudaEventSynchronize(table)");
        fill_row(*w.host_table, 0, 0, sampling, sampling, false);
        const int splits = split_bucket(count);
        w.ensure_scratch(splits);
        Session* self = this;
        bind_rows(w, &self, 1);
        check_cuda(cudaMemcpyAsync(w.table.as<void>(), w.host_table, sizeof(FrameTable),
                                   cudaMemcpyHostToDevice, w.stream), "upload frame table");
        check_cuda(cudaEventRecord(w.table_uploaded, w.stream), "cudaEventRecord(table)");
        check_cuda(cudaEventRecord(w.talker_start, w.stream), "cudaEventRecord");
        if (chunked) {
            int last_rows = 0;
            ParityHooks observed = hooks;
            observed.stream = w.stream;
            for (int base = 0; base < count; base += chunk) {
                last_rows = std::min(chunk, count - base);
                if (hooks.active() && base + last_rows == count) {
                    const Probe probe = observed.probe(last_rows - 1);     // the last prompt position
                    enqueue_prompt_chunk(w, m, d_text, d_codec, base, last_rows, splits, w.stream, &probe);
                } else {
                    enqueue_prompt_chunk(w, m, d_text, d_codec, base, last_rows, splits, w.stream);
                }
            }
            if (last_rows > 1) {
                // the head and the sampler read row 0: bring the last position's hidden state there
                const size_t row_bytes = (size_t)m.talker.hidden * sizeof(bf16);
                check_cuda(cudaMemcpyAsync(w.hidden.as<bf16>(),
                                           w.hidden.as<bf16>() + (size_t)(last_rows - 1) * m.talker.hidden,
                                           row_bytes, cudaMemcpyDeviceToDevice, w.stream), "last prompt row");
            }
        } else if (m.use_graphs) {
            // The prompt ids live in a buffer of this call, so the captured step graph is rebuilt
            // per prefill; capture costs far less than the steps it replays.
            cudaGraphExec_t step = capture(w.stream, [&] {
                enqueue_prompt_step(w, m, d_text, d_codec, splits, w.stream);
            });
            try {
                for (int i = 0; i < count; ++i) {
                    check_cuda(cudaGraphLaunch(step, w.stream), "cudaGraphLaunch(prompt step)");
                }
            } catch (...) {
                cudaStreamSynchronize(w.stream);
                cudaGraphExecDestroy(step);
                throw;
            }
            check_cuda(cudaStreamSynchronize(w.stream), "cudaStreamSynchronize(prompt)");
            cudaGraphExecDestroy(step);
        } else {
            for (int i = 0; i < count; ++i) enqueue_prompt_step(w, m, d_text, d_codec, splits, w.stream);
        }
        enqueue_talker_head(w, m, 1, 0, w.stream);
        if (hooks.active()) {
            ParityHooks observed = hooks;
            observed.stream = w.stream;
            observed.vector_line("final_norm", m.talker.layers, w.normalized.as<bf16>(), m.talker.hidden);
            observed.dump("final_logits", w.logits.as<bf16>(), kTalkerVocab);
            observed.logits_line(w.logits.as<bf16>(), kTalkerVocab);
        }
        check_cuda(cudaEventRecord(w.talker_stop, w.stream), "cudaEventRecord");
        check_cuda(cudaStreamSynchronize(w.stream), "synchronize sampled token");
        ++host_sync_count;
        ++device_sample_count;
        check_cuda(cudaEventElapsedTime(gpu_ms, w.talker_start, w.talker_stop), "cudaEventElapsedTime");
        m.check_device_errors(errors_before);
    } catch (...) {
        cudaStreamSynchronize(w.stream);
        poisoned_ = true;
        throw;
    }
    const int first = *h_token_;
    if (first < 0 || first >= kTalkerVocab) throw std::runtime_error("device sampler returned an invalid token");
    position_ = count;
    generated_ = 1;
    current_token_ = static_cast<uint16_t>(first);
    phase_ = first == kEos ? kPhaseEnded : kPhasePrefilled;
    *first_token = current_token_;
}

void Session::run_frames(Model* model, Session** s, int n, int frames, int trailing_text,
                         const SamplingParams& talker, const SamplingParams& predictor,
                         float* frame_ms, float* total_ms) {
    if (model == nullptr || s == nullptr || n <= 0 || n > kMaxRows || frames <= 0) {
        throw std::runtime_error("invalid frame-loop arguments");
    }
    check_cuda(cudaSetDevice(model->device()), "cudaSetDevice(frame loop)");
    for (int i = 0; i < n; ++i) {
        if (s[i]->model_.get() != model) throw std::runtime_error("session belongs to a different model");
        for (int j = 0; j < i; ++j) {
            if (s[j] == s[i]) throw std::runtime_error("a session appears twice in one batch");
        }
        s[i]->validate_begin(s[i]->current_token_, trailing_text, talker, predictor);
        if (s[i]->position_ + frames > s[i]->max_seq_) {
            throw std::runtime_error("frame loop would overflow the talker KV cache");
        }
    }
    std::unique_lock<std::mutex> one_batch(model->batch_mutex, std::defer_lock);
    if (n > 1) one_batch.lock();
    Workspace& w = n == 1 ? *s[0]->solo_ : model->batch_workspace();
    const unsigned int errors_before = model->device_errors();
    std::vector<cudaEvent_t> marks;
    try {
        check_cuda(cudaEventSynchronize(w.table_uploaded), "cudaEventSynchronize(table)");
        int longest = 0;
        for (int i = 0; i < n; ++i) {
            s[i]->fill_row(*w.host_table, i, trailing_text, talker, predictor, false);
            longest = std::max(longest, s[i]->position_ + frames);
            check_cuda(cudaEventRecord(w.join_events[i], s[i]->stream_), "cudaEventRecord(join)");
            check_cuda(cudaStreamWaitEvent(w.stream, w.join_events[i], 0), "cudaStreamWaitEvent(join)");
        }
        w.ensure_scratch(split_bucket(longest));
        marks.resize(frames + 1, nullptr);
        for (cudaEvent_t& ev : marks) check_cuda(cudaEventCreate(&ev), "cudaEventCreate(frame mark)");
        check_cuda(cudaEventRecord(marks[0], w.stream), "cudaEventRecord(frame mark)");
        for (int f = 0; f < frames; ++f) {
            // the device table advances itself; the host mirror follows for the graph key
            launch_frame(w, *model, s, n, f == 0, false);
            for (int i = 0; i < n; ++i) w.host_table->position[i] += 1;
            check_cuda(cudaEventRecord(marks[f + 1], w.stream), "cudaEventRecord(frame mark)");
        }
        check_cuda(cudaStreamSynchronize(w.stream), "cudaStreamSynchronize(frame loop)");
        model->check_device_errors(errors_before);
        if (frame_ms != nullptr) {
            for (int f = 0; f < frames; ++f) {
                check_cuda(cudaEventElapsedTime(&frame_ms[f], marks[f], marks[f + 1]), "cudaEventElapsedTime");
            }
        }
        if (total_ms != nullptr) {
            check_cuda(cudaEventElapsedTime(total_ms, marks[0], marks[frames]), "cudaEventElapsedTime");
        }
        for (int i = 0; i < n; ++i) {
            Session* c = s[i];
            c->position_ += frames;
            c->generated_ += frames;
            c->frames_generated += frames;
            c->device_sample_count += (uint64_t)frames * kPredictorSequence;
            ++c->host_sync_count;
            const int token = *c->h_token_;
            if (token < 0 || token >= kTalkerVocab) throw std::runtime_error("device sampler returned an invalid token");
            c->current_token_ = static_cast<uint16_t>(token);
            c->phase_ = token == kEos ? kPhaseEnded : kPhasePrefilled;
        }
    } catch (...) {
        cudaStreamSynchronize(w.stream);
        for (cudaEvent_t ev : marks) if (ev != nullptr) cudaEventDestroy(ev);
        for (int i = 0; i < n; ++i) s[i]->poisoned_ = true;
        throw;
    }
    for (cudaEvent_t ev : marks) cudaEventDestroy(ev);
}

void Session::synthetic_prefill(int position, uint64_t seed) {
    own_stream_busy_ = true;
    check_cuda(cudaSetDevice(device_), "cudaSetDevice(synthetic prefill)");
    if (poisoned_) throw std::runtime_error("talker session is poisoned and must be destroyed");
    if (frame_in_flight_) throw std::runtime_error("a device frame lease is in flight");
    if (position < 1 || position >= max_seq_) {
        throw std::runtime_error("synthetic prefill position must be in [1, max_sequence_length)");
    }
    Workspace& w = *solo_;
    Model& m = *model_;
    Session* self = this;
    bind_rows(w, &self, 1);
    const int pages = (position + kPageTokens - 1) / kPageTokens;
    const KvPool& pool = *m.talker_pool;
    check_cuda(launch_fill_kv_pages(pool.slab_table(), pool.slab_shift(), pool.page_elems(),
                                    pool.plane_elems(), w.talker_pages.as<int>(), pages,
                                    pool.layers() * 2, seed * 2 + 1, w.stream), "fill KV pages");
    check_cuda(launch_fill_normal(d_last_hidden_, 2048, seed * 2 + 2, w.stream), "fill last hidden");
    const int token = static_cast<int>(seed % 2048);
    check_cuda(cudaMemcpyAsync(d_sampled_, &token, sizeof(int), cudaMemcpyHostToDevice, w.stream),
               "store semantic token");
    check_cuda(cudaMemcpyAsync(d_history_, &token, sizeof(int), cudaMemcpyHostToDevice, w.stream),
               "store semantic history");
    check_cuda(cudaStreamSynchronize(w.stream), "cudaStreamSynchronize(synthetic prefill)");
    position_ = position;
    generated_ = 1;
    current_token_ = static_cast<uint16_t>(token);
    *h_token_ = token;
    phase_ = kPhasePrefilled;
}

void Session::read_state(uint16_t* last_hidden, int* frame_tokens, unsigned long long* rng) const {
    check_cuda(cudaSetDevice(device_), "cudaSetDevice(read state)");
    check_cuda(cudaStreamSynchronize(stream_), "cudaStreamSynchronize(read state)");
    if (last_hidden != nullptr) {
        check_cuda(cudaMemcpy(last_hidden, d_last_hidden_, 2048 * sizeof(bf16), cudaMemcpyDeviceToHost),
                   "cudaMemcpy(last hidden)");
    }
    if (frame_tokens != nullptr) {
        check_cuda(cudaMemcpy(frame_tokens, d_frame_tokens_, kCodebooks * sizeof(int),
                              cudaMemcpyDeviceToHost), "cudaMemcpy(frame tokens)");
    }
    if (rng != nullptr) {
        check_cuda(cudaMemcpy(rng, d_rng_, sizeof(unsigned long long), cudaMemcpyDeviceToHost),
                   "cudaMemcpy(rng)");
    }
}

void Session::read_kv(int layer, int first, int count, uint16_t* keys, uint16_t* values) const {
    check_cuda(cudaSetDevice(device_), "cudaSetDevice(read kv)");
    if (first < 0 || count < 0 || first + count > position_) {
        throw std::runtime_error("KV positions outside what the session has written");
    }
    check_cuda(cudaStreamSynchronize(stream_), "cudaStreamSynchronize(read kv)");
    const KvPool& pool = *model_->talker_pool;
    const int width = model_->talker.kv_width;
    const int hd = model_->talker.head_dim;
    const int heads = model_->talker.kv_heads;
    // a page holds [kv head][16 tokens][head_dim]: fetch the page whole, hand out token-major rows
    std::vector<uint16_t> page_copy((size_t)kPageTokens * width);
    for (int token = first; token < first + count;) {
        const int in_page = token % kPageTokens;
        const int run = std::min(kPageTokens - in_page, first + count - token);
        const int page = talker_pages_.at(token / kPageTokens);
        for (int plane = 0; plane < 2; ++plane) {
            uint16_t* out = plane == 0 ? keys : values;
            if (out == nullptr) continue;
            check_cuda(cudaMemcpy(page_copy.data(), pool.page_rows(page, layer, plane == 1),
                                  page_copy.size() * sizeof(uint16_t), cudaMemcpyDeviceToHost), "cudaMemcpy(read kv)");
            for (int t = 0; t < run; ++t) {
                for (int h = 0; h < heads; ++h) {
                    std::memcpy(out + (size_t)(token - first + t) * width + (size_t)h * hd,
                                page_copy.data() + ((size_t)h * kPageTokens + in_page + t) * hd, (size_t)hd * sizeof(uint16_t));
                }
            }
        }
        token += run;
    }
}

}  // namespace q3t
