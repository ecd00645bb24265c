// Seeded temperature / top-k / top-p sampler, one CTA per session row.
//
// Token-for-token and RNG-state-for-RNG-state equal to the reference's
// sample_logits_kernel (native/qwen3-tts-native/native/src/sampling_kernels.cu:143-389):
//   * adjusted logits: reserved-token mask and repetition penalty (:30-51);
//   * do_sample == 0: argmax, ties to the lower index, no RNG draw (:208-240);
//   * top_k == 0 and top_p >= 1: categorical over the whole vocabulary in index order
//     with a sequential fp64 sum (:242-265);
//   * otherwise the top-min(k, V) logits in the total order "value descending, ties by
//     lower index" (:71-84), w_r = exp((double)(v_r/T - v_0/T)), sequential fp64
//     denominator, top-p cut on cumulative w_r/denominator, sequential re-sum of the
//     retained weights, one xorshift64* draw, first prefix >= target (:352-388).
// What differs is how the ordered top-k is found.  Every logit gets a unique 44-bit key
// (order-preserving float bits << 12 | 4095 - index), so "value descending, lower index
// first" is plain descending key order with no ties.  A byte-wise radix select finds the
// k-th key (stopping as soon as a bucket boundary coincides with k), the k survivors are
// compacted and ranked by counting.  The fp64 tail keeps the reference's sequential
// summation order: the prefix sums of the weights are computed once on one thread, and the
// denominator, the retained total and the final cumulative scan all read that one prefix.

#include "q3t_kernels.cuh"

namespace q3t {
namespace {

constexpr int kSampleThreads = 512;
constexpr int kSampleWarps = kSampleThreads / kWarp;

__device__ __forceinline__ unsigned int order_key(float v) {
    unsigned int u = __float_as_uint(v);
    if (u == 0x80000000u) u = 0u;   // -0 ties with +0
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ float key_value(unsigned long long ckey) {
    const unsigned int k = static_cast<unsigned int>(ckey >> 12);
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

__device__ __forceinline__ int key_index(unsigned long long ckey) {
    return 4095 - static_cast<int>(ckey & 0xfffull);
}

// xorshift64* (sampling_kernels.cu:53-69)
__device__ float uniform_random(unsigned long long* state) {
    unsigned long long v = *state;
    if (v == 0) v = 0x9e3779b97f4a7c15ULL;
    v ^= v >> 12;
    v ^= v << 25;
    v ^= v >> 27;
    *state = v;
    const unsigned long long r = v * 0x2545f4914f6cdd1dULL;
    constexpr double scale = 1.0 / 9007199254740992.0;
    return static_cast<float>(static_cast<double>(r >> 11) * scale);
}

__device__ __forceinline__ unsigned long long block_max_u64(unsigned long long v,
                                                           unsigned long long* warp_slots) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, v, o);
        v = other > v ? other : v;
    }
    if (threadIdx.x % kWarp == 0) warp_slots[threadIdx.x / kWarp] = v;
    __syncthreads();
    unsigned long long m = warp_slots[0];
    for (int w = 1; w < kSampleWarps; ++w) m = warp_slots[w] > m ? warp_slots[w] : m;
    return m;
}

__device__ __forceinline__ void sample_one(const SamplerRow& r, unsigned char* smem_raw) {
    const int V = r.vocabulary;
    // [0, 8V): keys, later the fp64 prefix sums | [8V, 16V): candidates, later the fp64
    // weights | [16V, 20V): sorted values | [20V, 24V): sorted indices
    unsigned long long* keys = reinterpret_cast<unsigned long long*>(smem_raw);
    double* prefix = reinterpret_cast<double*>(smem_raw);
    unsigned long long* cand = keys + V;
    double* weights = reinterpret_cast<double*>(cand);
    float* sval = reinterpret_cast<float*>(cand + V);
    int* sidx = reinterpret_cast<int*>(sval + V);

    __shared__ unsigned int seen[kMaxVocab / 32];
    __shared__ unsigned int hist[256];
    __shared__ unsigned long long warp_slots[kSampleWarps];
    __shared__ unsigned long long s_prefix;
    __shared__ int s_above;
    __shared__ int s_done;
    __shared__ int s_counter;
    __shared__ int s_retained;

    const int tid = threadIdx.x;
    const int lane = tid % kWarp;
    const float neg_inf = -INFINITY;

    // ---- adjusted logits -> keys ---------------------------------------------------
    const int count = r.history_count != nullptr ? *r.history_count : r.history_count_value;
    const bool penalise = r.suppress && r.penalty != 1.0f && count > 0;
    if (penalise) {
        for (int i = tid; i < kMaxVocab / 32; i += kSampleThreads) seen[i] = 0u;
        __syncthreads();
        for (int i = tid; i < count; i += kSampleThreads) {
            const int t = r.history[i];
            if (t >= 0 && t < V) atomicOr(&seen[t >> 5], 1u << (t & 31));
        }
        __syncthreads();
    }
    for (int t = tid; t < V; t += kSampleThreads) {
        float v;
        if (r.suppress && t >= kPredictorVocab && (t != r.eos || r.mask_eos)) {
            v = neg_inf;
        } else if (r.mask_eos && t == r.eos) {
            v = neg_inf;
        } else {
            v = bf2f(r.logits[t]);
            if (penalise && ((seen[t >> 5] >> (t & 31)) & 1u)) {
                v = v < 0.0f ? v * r.penalty : v / r.penalty;
            }
        }
        keys[t] = (static_cast<unsigned long long>(order_key(v)) << 12)
                  | static_cast<unsigned long long>(4095 - t);
    }
    __syncthreads();

    const bool direct = r.do_sample != 0 && r.top_k == 0 && r.top_p >= 1.0f;
    const int selections = r.do_sample == 0 ? 1 : (r.top_k == 0 ? V : min(r.top_k, V));
    int retained = 0;     // number of ordered candidates the final draw runs over
    int fallback = 0;     // token when no prefix reaches the target

    if (r.do_sample == 0 || direct) {
        unsigned long long best = 0ull;
        for (int t = tid; t < V; t += kSampleThreads) best = keys[t] > best ? keys[t] : best;
        best = block_max_u64(best, warp_slots);
        const int best_index = key_index(best);
        if (r.do_sample == 0) {
            if (tid == 0) {
                *r.selected = best_index;
                if (r.store_a != nullptr) r.store_a[r.store_a_index] = best_index;
                if (r.store_b != nullptr) r.store_b[count] = best_index;
            }
            return;
        }
        // categorical over the whole vocabulary, index order
        const float maximum = key_value(best) / r.temperature;
        for (int t = tid; t < V; t += kSampleThreads) {
            const float v = key_value(keys[t]);
            sidx[t] = t;
            weights[t] = exp(static_cast<double>(v / r.temperature - maximum));
        }
        retained = V;
        fallback = best_index;
        __syncthreads();
        if (tid == 0) {
            double running = 0.0;
            for (int t = 0; t < V; ++t) {
                running += weights[t];
                prefix[t] = running;
            }
        }
        __syncthreads();
    } else {
        // ---- radix select of the `selections`-th largest key --------------------------
        if (tid == 0) {
            s_prefix = 0ull;
            s_above = 0;
            s_done = 0;
        }
        __syncthreads();
        for (int pass = 0; pass < 6; ++pass) {
            const int shift = pass < 5 ? 36 - 8 * pass : 0;
            const int width = pass < 5 ? 8 : 4;
            if (s_done) break;
            if (!penalise && (pass == 2 || pass == 3)) {
                // bf16 logits: the low 16 bits of every value are zero, so those of the order key are
                // all zeros (non-negative values) or all ones (negative ones), and every key still in
                // the running has the sign of the prefix: the digit is known without counting
                if (tid == 0 && ((s_prefix >> 43) & 1ull) == 0ull) s_prefix |= 0xffull << shift;
                __syncthreads();
                continue;
            }
            for (int i = tid; i < 256; i += kSampleThreads) hist[i] = 0u;
            __syncthreads();
            const unsigned long long pref = s_prefix;
            const int hs = shift + width;
            for (int t = tid; t < V; t += kSampleThreads) {
                const unsigned long long k = keys[t];
                if ((k >> hs) == (pref >> hs)) {
                    atomicAdd(&hist[static_cast<unsigned int>(k >> shift) & ((1u << width) - 1u)], 1u);
                }
            }
            __syncthreads();
            if (tid < kWarp) {
                // lane l owns bins 255-8l .. 248-8l (descending)
                unsigned int mine[8];
                unsigned int local = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    mine[j] = hist[255 - 8 * lane - j];
                    local += mine[j];
                }
                unsigned int incl = local;
#pragma unroll
                for (int o = 1; o < kWarp; o <<= 1) {
                    const unsigned int n = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += n;
                }
                const int above = s_above;
                const bool crosses = above + static_cast<int>(incl) >= selections;
                const unsigned int ballot = __ballot_sync(0xffffffffu, crosses);
                const int owner = __ffs(ballot) - 1;
                if (lane == owner) {
                    int c = above + static_cast<int>(incl - local);
                    int chosen = 0;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (c + static_cast<int>(mine[j]) >= selections) {
                            chosen = 255 - 8 * lane - j;
                            if (c + static_cast<int>(mine[j]) == selections) s_done = 1;
                            break;
                        }
                        c += static_cast<int>(mine[j]);
                    }
                    s_above = c;
                    s_prefix = pref | (static_cast<unsigned long long>(chosen) << shift);
                }
            }
            __syncthreads();
        }
        const unsigned long long threshold = s_prefix;
        if (tid == 0) s_counter = 0;
        __syncthreads();
        for (int t = tid; t < V; t += kSampleThreads) {
            const unsigned long long k = keys[t];
            if (k >= threshold) {
                const int p = atomicAdd(&s_counter, 1);
                if (p < V) cand[p] = k;
            }
        }
        __syncthreads();
        // ---- rank the survivors by counting (keys are unique) --------------------------
        for (int i = tid; i < selections; i += kSampleThreads) {
            const unsigned long long k = cand[i];
            int rank = 0;
#pragma unroll 8
            for (int j = 0; j < selections; ++j) rank += cand[j] > k ? 1 : 0;
            sval[rank] = key_value(k);
            sidx[rank] = key_index(k);
        }
        __syncthreads();   // candidates are dead from here: their storage becomes `weights`
        const float maximum = sval[0] / r.temperature;
        for (int i = tid; i < selections; i += kSampleThreads) {
            weights[i] = exp(static_cast<double>(sval[i] / r.temperature - maximum));
        }
        __syncthreads();
        if (tid == 0) {
            // one thread, the reference's order of additions; eight loads at a time ahead of the chain
            double running = 0.0;
            int i = 0;
            for (; i + 8 <= selections; i += 8) {
                double w8[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) w8[u] = weights[i + u];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    running += w8[u];
                    prefix[i + u] = running;
                }
            }
            for (; i < selections; ++i) {
                running += weights[i];
                prefix[i] = running;
            }
        }
        __syncthreads();
        const double denominator = prefix[selections - 1];
        for (int i = tid; i < selections; i += kSampleThreads) weights[i] = weights[i] / denominator;
        __syncthreads();
        if (tid == 0) {
            double cumulative = 0.0;
            int keep = selections;
            const double limit = static_cast<double>(r.top_p);
            int i = 0;
            bool found = false;
            for (; !found && i + 8 <= selections; i += 8) {
                double w8[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) w8[u] = weights[i + u];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    cumulative += w8[u];
                    if (!found && cumulative >= limit) {
                        keep = i + u + 1;
                        found = true;
                    }
                }
            }
            for (; !found && i < selections; ++i) {
                cumulative += weights[i];
                if (cumulative >= limit) {
                    keep = i + 1;
                    found = true;
                }
            }
            s_retained = keep;
        }
        __syncthreads();
        retained = s_retained;
        fallback = sidx[retained - 1];
    }

    // ---- one draw; first prefix that reaches the target ------------------------------------
    if (tid == 0) {
        const double total = prefix[retained - 1];
        const double target = static_cast<double>(uniform_random(r.rng)) * total;
        int selected = fallback;
        int first = retained;            // first prefix that reaches the target
        for (int i = 0; i < retained && first == retained; i += 8) {
            double p8[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) p8[u] = i + u < retained ? prefix[i + u] : 0.0;
#pragma unroll
            for (int u = 7; u >= 0; --u) {
                if (i + u < retained && p8[u] >= target) first = i + u;
            }
        }
        if (first < retained) selected = sidx[first];
        *r.selected = selected;
        if (r.store_a != nullptr) r.store_a[r.store_a_index] = selected;
        if (r.store_b != nullptr) r.store_b[count] = selected;
    }
}

__global__ void __launch_bounds__(kSampleThreads) sample_rows_kernel(const SamplerRow* rows) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const SamplerRow r = rows[blockIdx.x];
    sample_one(r, smem_raw);
}

__global__ void __launch_bounds__(kSampleThreads)
sample_table_kernel(const FrameTable* table, const bf16* logits, int logits_stride, int vocabulary,
                    int talker, int store_index, int mask_eos, int eos) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int row = blockIdx.x;
    const SamplingParams p = talker ? table->talker[row] : table->predictor[row];
    SamplerRow r;
    r.logits = logits + (size_t)row * logits_stride;
    r.history = table->history[row];
    r.history_count = nullptr;
    r.history_count_value = table->history_count[row];
    r.rng = table->rng[row];
    r.vocabulary = vocabulary;
    r.suppress = talker;
    r.mask_eos = talker ? mask_eos : 0;
    r.eos = eos;
    r.do_sample = p.do_sample;
    r.top_k = p.top_k;
    r.top_p = p.top_p;
    r.temperature = p.temperature;
    r.penalty = p.penalty;
    if (talker) {
        r.selected = table->sampled[row];
        r.store_a = nullptr;
        r.store_a_index = 0;
        r.store_b = table->history[row];
    } else {
        r.selected = table->frame_tokens[row] + store_index;
        r.store_a = nullptr;
        r.store_a_index = 0;
        r.store_b = nullptr;
    }
    sample_one(r, smem_raw);
}

// one row whose descriptor travels as the kernel argument (no device-side descriptor needed)
__global__ void __launch_bounds__(kSampleThreads) sample_value_kernel(const SamplerRow r) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    sample_one(r, smem_raw);
}

constexpr size_t kSampleSmem = (size_t)kMaxVocab * 24;

}  // namespace

cudaError_t launch_sample_value(const SamplerRow& row, cudaStream_t stream) {
    if (row.logits == nullptr || row.selected == nullptr || row.rng == nullptr
        || row.vocabulary < 1 || row.vocabulary > kMaxVocab) {
        return cudaErrorInvalidValue;
    }
    sample_value_kernel<<<1, kSampleThreads, kSampleSmem, stream>>>(row);
    return cudaGetLastError();
}

cudaError_t configure_sampler_kernels() {
    cudaError_t e = cudaFuncSetAttribute(sample_value_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(kSampleSmem));
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(sample_rows_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(kSampleSmem));
    if (e == cudaSuccess) {
        e = cudaFuncSetAttribute(sample_table_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(kSampleSmem));
    }
    return e;
}

cudaError_t launch_sample_rows(const SamplerRow* rows, int count, cudaStream_t stream) {
    if (rows == nullptr || count < 1) return cudaErrorInvalidValue;
    sample_rows_kernel<<<count, kSampleThreads, kSampleSmem, stream>>>(rows);
    return cudaGetLastError();
}

cudaError_t launch_sample_table(const FrameTable* table, const bf16* logits, int logits_stride,
                                int vocabulary, int talker, int store_index, int mask_eos,
                                int eos, int rows, cudaStream_t stream) {
    if (table == nullptr || logits == nullptr || rows < 1 || rows > kMaxRows || vocabulary < 1
        || vocabulary > kMaxVocab) {
        return cudaErrorInvalidValue;
    }
    return launch_pdl(sample_table_kernel, dim3(rows), dim3(kSampleThreads), kSampleSmem, stream, 
        table, logits, logits_stride, vocabulary, talker, store_index, mask_eos, eos);
    return cudaGetLastError();
}

}  // namespace q3t
