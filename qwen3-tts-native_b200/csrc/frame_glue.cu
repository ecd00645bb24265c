// Row-table kernels that stitch the projections of one codec frame together: token
// stores, embedding gathers and sums, code packing and the end-of-frame bookkeeping.
// They replace the store_token / store_sampled_token / pack_frame_codes / gather_embedding
// launches of the reference (native/qwen3-tts-native/native/src/sampling_kernels.cu:403-452
// and talker_kernels.cu:680-709) -- about 40 single-purpose launches per frame there --
// with one launch per step of the frame, all driven by the device-resident FrameTable.

#include "q3t_kernels.cuh"

namespace q3t {
namespace {

constexpr int kThreads = 256;

__global__ void frame_begin_kernel(const FrameTable* t, int rows) {
    pdl_wait();
    pdl_trigger();
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row < rows) t->frame_tokens[row][0] = *t->sampled[row];
}

__global__ void __launch_bounds__(kThreads)
predictor_input_kernel(const FrameTable* t, int p, const bf16* __restrict__ codec_embedding,
                       const bf16* const* predictor_embeddings, bf16* __restrict__ x, int width) {
    pdl_wait();
    pdl_trigger();
    const int row = blockIdx.x;
    const bf16* src;
    if (p == 0) {
        src = t->last_hidden[row];
    } else if (p == 1) {
        const int token = t->frame_tokens[row][0];
        if (token < 0 || token >= kMaxVocab) return;
        src = codec_embedding + (size_t)token * width;
    } else {
        const int token = t->frame_tokens[row][p - 1];
        if (token < 0 || token >= kPredictorVocab) return;
        src = predictor_embeddings[p - 2] + (size_t)token * width;
    }
    const int4* s4 = reinterpret_cast<const int4*>(src);
    int4* d4 = reinterpret_cast<int4*>(x + (size_t)row * width);
    for (int i = threadIdx.x; i < width / 8; i += kThreads) d4[i] = s4[i];
}

// The reference builds the next talker input with one gather and fifteen add launches,
// each add rounding to bf16 (talker.cu:3546-3570 / 1704-1731); the same chain runs here in
// registers, in the same order.
__global__ void __launch_bounds__(kThreads)
talker_input_kernel(const FrameTable* t, const bf16* __restrict__ codec_embedding,
                    const bf16* const* predictor_embeddings,
                    const bf16* __restrict__ text_embedding, int text_vocabulary,
                    bf16* __restrict__ hidden, bf16* __restrict__ text_in, int width) {
    pdl_wait();
    pdl_trigger();
    const int row = blockIdx.x;
    const int* tokens = t->frame_tokens[row];
    // the sixteen embedding rows of this frame (null: token out of range, nothing is added, as
    // in the reference's gather)
    __shared__ const bf16* rows_of[kCodebooks];
    if (threadIdx.x < kCodebooks) {
        const int r = threadIdx.x;
        const int token = tokens[r];
        const bf16* base = nullptr;
        if (r == 0) {
            if (token >= 0 && token < kMaxVocab) base = codec_embedding + (size_t)token * width;
        } else if (token >= 0 && token < kPredictorVocab) {
            base = predictor_embeddings[r - 1] + (size_t)token * width;
        }
        rows_of[r] = base;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < width; i += kThreads) {
        // all sixteen loads go out together; the sum is then formed in codebook order with the
        // reference's rounding after every addition
        float v[kCodebooks];
#pragma unroll
        for (int r = 0; r < kCodebooks; ++r) {
            const bf16* base = rows_of[r];
            v[r] = base != nullptr ? bf2f(base[i]) : 0.0f;
        }
        float acc = rows_of[0] != nullptr ? v[0] : bf2f(hidden[(size_t)row * width + i]);
#pragma unroll
        for (int r = 1; r < kCodebooks; ++r) {
            if (rows_of[r] != nullptr) acc = rbf(acc + v[r]);
        }
        hidden[(size_t)row * width + i] = f2bf(acc);
    }
    const int text = t->trailing_text[row];
    if (text >= 0 && text < text_vocabulary) {
        const int4* s4 = reinterpret_cast<const int4*>(text_embedding + (size_t)text * width);
        int4* d4 = reinterpret_cast<int4*>(text_in + (size_t)row * width);
        for (int i = threadIdx.x; i < width / 8; i += kThreads) d4[i] = s4[i];
    }
}

__global__ void pack_codes_kernel(const FrameTable* t, int rows) {
    pdl_wait();
    pdl_trigger();
    const int row = blockIdx.x;
    const int i = threadIdx.x;
    if (row < rows && i < kCodebooks) {
        const unsigned short code = static_cast<unsigned short>(t->frame_tokens[row][i]);
        t->frame_codes[row][i] = code;
        if (t->host_codes[row] != nullptr) t->host_codes[row][i] = code;
    }
}

__global__ void __launch_bounds__(kThreads)
frame_end_kernel(FrameTable* t, const bf16* __restrict__ normalized, int width,
                 int advance_position) {
    pdl_wait();
    pdl_trigger();
    const int row = blockIdx.x;
    const int4* s4 = reinterpret_cast<const int4*>(normalized + (size_t)row * width);
    int4* d4 = reinterpret_cast<int4*>(t->last_hidden[row]);
    for (int i = threadIdx.x; i < width / 8; i += kThreads) d4[i] = s4[i];
    if (threadIdx.x == 0) {
        if (t->host_token[row] != nullptr) {
            *t->host_token[row] = *t->sampled[row];
            __threadfence_system();
        }
        if (advance_position) t->position[row] += 1;
        t->history_count[row] += 1;
    }
}

__global__ void __launch_bounds__(kThreads)
prompt_gather_kernel(const FrameTable* t, const int* __restrict__ text_ids,
                     const bf16* __restrict__ text_embedding, int text_vocabulary,
                     bf16* __restrict__ x, int width) {
    const int text = text_ids[t->position[0]];
    if (text < 0 || text >= text_vocabulary) return;
    const int4* s4 = reinterpret_cast<const int4*>(text_embedding + (size_t)text * width);
    int4* d4 = reinterpret_cast<int4*>(x);
    for (int i = blockIdx.x * kThreads + threadIdx.x; i < width / 8; i += gridDim.x * kThreads) {
        d4[i] = s4[i];
    }
}

// talker.cu:2721-2748: text part (or zeros) plus the codec embedding, one rounded add
__global__ void __launch_bounds__(kThreads)
prompt_combine_kernel(const FrameTable* t, const int* __restrict__ text_ids,
                      const int* __restrict__ codec_ids, const bf16* __restrict__ codec_embedding,
                      int codec_vocabulary, bf16* __restrict__ hidden, int width) {
    const int index = t->position[0];
    const int text = text_ids[index];
    const int codec = codec_ids[index];
    for (int i = blockIdx.x * kThreads + threadIdx.x; i < width; i += gridDim.x * kThreads) {
        float v = text >= 0 ? bf2f(hidden[i]) : 0.0f;
        if (codec >= 0 && codec < codec_vocabulary) {
            v = rbf(v + bf2f(codec_embedding[(size_t)codec * width + i]));
        }
        hidden[i] = f2bf(v);
    }
}

// ---- a chunk of prompt positions as the rows of one pass ------------------------------------------
// Row r is prompt position base + r: the text embedding row goes to text_in (left as it is when
// the position has no text, as in the single-position kernel) and the position to positions[r].
__global__ void __launch_bounds__(kThreads)
prompt_rows_kernel(const int* __restrict__ text_ids, const int* __restrict__ codec_ids, int base,
                   const bf16* __restrict__ text_embedding, int text_vocabulary,
                   bf16* __restrict__ text_in, int* __restrict__ positions, int width) {
    const int row = blockIdx.x;
    if (threadIdx.x == 0) positions[row] = base + row;
    const int text = text_ids[base + row];
    if (text < 0 || text >= text_vocabulary) return;
    const int4* s4 = reinterpret_cast<const int4*>(text_embedding + (size_t)text * width);
    int4* d4 = reinterpret_cast<int4*>(text_in + (size_t)row * width);
    for (int i = threadIdx.x; i < width / 8; i += kThreads) d4[i] = s4[i];
    (void)codec_ids;
}

// text part (or zeros) plus the codec embedding, one rounded add, per row (talker.cu:2721-2748)
__global__ void __launch_bounds__(kThreads)
prompt_combine_rows_kernel(const int* __restrict__ text_ids, const int* __restrict__ codec_ids, int base,
                           const bf16* __restrict__ codec_embedding, int codec_vocabulary,
                           bf16* __restrict__ hidden, int width) {
    const int row = blockIdx.x;
    const int text = text_ids[base + row];
    const int codec = codec_ids[base + row];
    bf16* h = hidden + (size_t)row * width;
    for (int i = threadIdx.x; i < width; i += kThreads) {
        float v = text >= 0 ? bf2f(h[i]) : 0.0f;
        if (codec >= 0 && codec < codec_vocabulary) {
            v = rbf(v + bf2f(codec_embedding[(size_t)codec * width + i]));
        }
        h[i] = f2bf(v);
    }
}

// ---- benchmark harness: seeded pseudo-random N(0,1) fills ------------------------------------

__device__ __forceinline__ float hashed_normal(unsigned long long index, unsigned long long seed) {
    unsigned long long z = index * 0x9e3779b97f4a7c15ULL + seed;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ULL;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebULL;
    z ^= z >> 31;
    const float u1 = (static_cast<float>(z >> 40) + 1.0f) * (1.0f / 16777217.0f);
    const float u2 = static_cast<float>((z >> 16) & 0xffffffull) * (1.0f / 16777216.0f);
    return sqrtf(-2.0f * logf(u1)) * cosf(6.2831853f * u2);
}

__global__ void __launch_bounds__(kThreads)
fill_normal_kernel(bf16* __restrict__ dst, size_t count, unsigned long long seed) {
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < count;
         i += (size_t)gridDim.x * kThreads) {
        dst[i] = f2bf(hashed_normal(i, seed));
    }
}

// seeded pseudo-random int8 weights, uniform in [-127, 127], eight per thread and step
__global__ void __launch_bounds__(kThreads)
fill_bytes_kernel(unsigned char* __restrict__ dst, size_t count, unsigned long long seed) {
    const size_t words = count / 8;
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < words; i += (size_t)gridDim.x * kThreads) {
        unsigned long long z = i * 0x9e3779b97f4a7c15ULL + seed;
        z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ULL;
        z = (z ^ (z >> 27)) * 0x94d049bb133111ebULL;
        z ^= z >> 31;
        unsigned long long out = 0;
#pragma unroll
        for (int b = 0; b < 8; ++b) {
            const int v = static_cast<int>(((z >> (8 * b)) & 0xffull) * 255ull >> 8) - 127;   // -127..127
            out |= static_cast<unsigned long long>(static_cast<unsigned char>(v)) << (8 * b);
        }
        reinterpret_cast<unsigned long long*>(dst)[i] = out;
    }
    if (blockIdx.x == 0 && threadIdx.x < count % 8) dst[words * 8 + threadIdx.x] = 1;
}

// grid (pages, layers*2): block (p, plane) fills the 16 x kv_width page `page_ids[p]` of that
// K or V plane
__global__ void __launch_bounds__(kThreads)
fill_kv_pages_kernel(bf16* const* slabs, int slab_shift, long long page_elems,
                     long long plane_elems, const int* __restrict__ page_ids,
                     unsigned long long seed) {
    const int pid = page_ids[blockIdx.x];
    bf16* dst = slabs[pid >> slab_shift] + (long long)blockIdx.y * plane_elems
        + (long long)(pid & ((1 << slab_shift) - 1)) * page_elems;
    const unsigned long long base =
        ((unsigned long long)blockIdx.y * gridDim.x + blockIdx.x) * (unsigned long long)page_elems;
    for (long long i = threadIdx.x; i < page_elems; i += kThreads) {
        dst[i] = f2bf(hashed_normal(base + i, seed));
    }
}

__global__ void advance_position_kernel(FrameTable* t) {
    if (threadIdx.x == 0 && blockIdx.x == 0) t->position[0] += 1;
}

}  // namespace

cudaError_t launch_frame_begin(const FrameTable* table, int rows, cudaStream_t stream) {
    return launch_pdl(frame_begin_kernel, dim3(1), dim3(kMaxRows), 0, stream, table, rows);
}

cudaError_t launch_predictor_input(const FrameTable* table, int p, const bf16* codec_embedding,
                                   const bf16* const* predictor_embeddings, bf16* x, int width,
                                   int rows, cudaStream_t stream) {
    return launch_pdl(predictor_input_kernel, dim3(rows), dim3(kThreads), 0, stream, table, p, codec_embedding,
                      predictor_embeddings, x, width);
}

cudaError_t launch_talker_input(const FrameTable* table, const bf16* codec_embedding,
                                const bf16* const* predictor_embeddings, const bf16* text_embedding,
                                int text_vocabulary, bf16* hidden, bf16* text_in, int width, int rows,
                                cudaStream_t stream) {
    return launch_pdl(talker_input_kernel, dim3(rows), dim3(kThreads), 0, stream, table, codec_embedding,
                      predictor_embeddings, text_embedding, text_vocabulary, hidden, text_in, width);
}

cudaError_t launch_pack_codes(const FrameTable* table, int rows, cudaStream_t stream) {
    return launch_pdl(pack_codes_kernel, dim3(rows), dim3(32), 0, stream, table, rows);
}

cudaError_t launch_frame_end(FrameTable* table, const bf16* normalized, int width, int rows,
                             int advance_position, cudaStream_t stream) {
    return launch_pdl(frame_end_kernel, dim3(rows), dim3(kThreads), 0, stream, table, normalized, width,
                      advance_position);
}

cudaError_t launch_prompt_gather(const FrameTable* table, const int* text_ids,
                                 const bf16* text_embedding, int text_vocabulary, bf16* x, int width,
                                 cudaStream_t stream) {
    prompt_gather_kernel<<<1, kThreads, 0, stream>>>(table, text_ids, text_embedding,
                                                     text_vocabulary, x, width);
    return cudaGetLastError();
}

cudaError_t launch_prompt_combine(const FrameTable* table, const int* text_ids, const int* codec_ids,
                                  const bf16* codec_embedding, int codec_vocabulary, bf16* hidden,
                                  int width, cudaStream_t stream) {
    prompt_combine_kernel<<<4, kThreads, 0, stream>>>(table, text_ids, codec_ids, codec_embedding,
                                                      codec_vocabulary, hidden, width);
    return cudaGetLastError();
}

cudaError_t launch_prompt_rows(const int* text_ids, const int* codec_ids, int base, int rows,
                               const bf16* text_embedding, int text_vocabulary, bf16* text_in,
                               int* positions, int width, cudaStream_t stream) {
    if (rows < 1 || rows > kMaxRows) return cudaErrorInvalidValue;
    prompt_rows_kernel<<<rows, kThreads, 0, stream>>>(text_ids, codec_ids, base, text_embedding,
                                                      text_vocabulary, text_in, positions, width);
    return cudaGetLastError();
}

cudaError_t launch_prompt_combine_rows(const int* text_ids, const int* codec_ids, int base, int rows,
                                       const bf16* codec_embedding, int codec_vocabulary, bf16* hidden,
                                       int width, cudaStream_t stream) {
    if (rows < 1 || rows > kMaxRows) return cudaErrorInvalidValue;
    prompt_combine_rows_kernel<<<rows, kThreads, 0, stream>>>(text_ids, codec_ids, base, codec_embedding,
                                                              codec_vocabulary, hidden, width);
    return cudaGetLastError();
}

cudaError_t launch_fill_normal(bf16* dst, size_t count, unsigned long long seed, cudaStream_t stream) {
    if (dst == nullptr || count == 0) return cudaErrorInvalidValue;
    size_t blocks = (count + kThreads - 1) / kThreads;
    if (blocks > 2048) blocks = 2048;
    fill_normal_kernel<<<static_cast<unsigned int>(blocks), kThreads, 0, stream>>>(dst, count, seed);
    return cudaGetLastError();
}

cudaError_t launch_fill_bytes(unsigned char* dst, size_t count, unsigned long long seed, cudaStream_t stream) {
    if (dst == nullptr || count == 0 || (reinterpret_cast<uintptr_t>(dst) & 7u) != 0) return cudaErrorInvalidValue;
    size_t blocks = (count / 8 + kThreads - 1) / kThreads;
    if (blocks > 4096) blocks = 4096;
    if (blocks < 1) blocks = 1;
    fill_bytes_kernel<<<static_cast<unsigned int>(blocks), kThreads, 0, stream>>>(dst, count, seed);
    return cudaGetLastError();
}

cudaError_t launch_fill_kv_pages(bf16* const* slabs, int slab_shift, long long page_elems,
                                 long long plane_elems, const int* page_ids, int pages, int planes,
                                 unsigned long long seed, cudaStream_t stream) {
    if (pages < 1 || planes < 1) return cudaErrorInvalidValue;
    fill_kv_pages_kernel<<<dim3(pages, planes), kThreads, 0, stream>>>(slabs, slab_shift, page_elems,
                                                                      plane_elems, page_ids, seed);
    return cudaGetLastError();
}

cudaError_t launch_advance_position(FrameTable* table, cudaStream_t stream) {
    advance_position_kernel<<<1, 32, 0, stream>>>(table);
    return cudaGetLastError();
}

}  // namespace q3t
