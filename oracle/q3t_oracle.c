/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of the reference's decode hot path.
 *
 * Plain C (gcc, -ffp-contract=off) restatement of the arithmetic of the kernels in
 * luka-loehr/qwen3-tts-native, native/qwen3-tts-native/native/src/{int8_gemv,
 * talker_kernels,sampling_kernels}.cu.  Each function cites the reference lines it
 * follows.  Where the reference's fp32 summation order is observable in the result
 * (per-lane partial sums, shuffle/shared-memory trees) the order is reproduced, so
 * the outputs equal the reference kernels' bit for bit except where a transcendental
 * (expf, powf, cosf, sinf, rsqrtf, exp) of the host libm differs from CUDA's by an ulp.
 *
 * Pinning: the four closed-form fixtures of the reference's primitive_parity.cu
 * (regenerated from their formulas in tests/golden/) and, on a GPU box, the
 * reference's own kernels compiled for sm_100a (oracle/_ref, see build_ref.sh).
 *
 * Only tests/, the smoke check and the benchmark's cpu_baseline / reference legs may
 * load this file.  The product library never does.
 *
 * bf16 values travel as uint16_t bit patterns.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ bf16 -- */

static inline float bf2f(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* round-to-nearest-even, NaN -> 0x7fff: the behaviour of __float2bfloat16 */
static inline uint16_t f2bf(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fff;
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

static inline float rbf(float f) { return bf2f(f2bf(f)); }

/* correctly rounded 1/sqrt(x); CUDA's rsqrtf may differ from it by up to 2 ulp */
static inline float rsqrt_f(float x) { return (float)(1.0 / sqrt((double)x)); }

ORC_API int orc_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

ORC_API void orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

ORC_API void orc_f2bf(const float* in, uint16_t* out, long n) {
    for (long i = 0; i < n; ++i) out[i] = f2bf(in[i]);
}

ORC_API void orc_bf2f(const uint16_t* in, float* out, long n) {
    for (long i = 0; i < n; ++i) out[i] = bf2f(in[i]);
}

/* ------------------------------------------------- int8 weight-only GEMV -- */

/* One output channel, one activation row, in the reference's order
 * (int8_gemv.cu:73-121): lane l owns the 16-element vectors l, l+32, ...; inside a
 * vector 16 sequential fmaf; the vector sum is added to the lane accumulator; the 32
 * lane accumulators are folded by the __shfl_down_sync tree (offsets 16..1). */
static float gemv_channel_f32(const int8_t* w, const uint16_t* x, int k) {
    float lane[32];
    const int vectors = k / 16;
    for (int l = 0; l < 32; ++l) {
        float acc = 0.0f;
        for (int v = l; v < vectors; v += 32) {
            const int8_t* wv = w + (size_t)v * 16;
            const uint16_t* xv = x + (size_t)v * 16;
            float sum = 0.0f;
            for (int j = 0; j < 16; ++j) sum = fmaf((float)wv[j], bf2f(xv[j]), sum);
            acc += sum;
        }
        lane[l] = acc;
    }
    for (int off = 16; off > 0; off >>= 1)
        for (int l = 0; l < off; ++l) lane[l] += lane[l + off];
    return lane[0];
}

/* mode 0: y = bf16(acc*scale)                       int8_gemv.cu:122-125
 * mode 1: y = bf16(y + acc*scale), contracted to one fma by nvcc (-fmad default)
 *                                                   int8_gemv.cu:190-196
 * acc_out (optional, [rows][n]) receives the fp32 value before the bf16 round. */
ORC_API void orc_int8_gemm_rows(const int8_t* w, const float* scales, const uint16_t* x,
                                uint16_t* y, float* acc_out, int k, int n, int rows, int mode) {
#pragma omp parallel for schedule(static)
    for (int c = 0; c < n; ++c) {
        const int8_t* wc = w + (size_t)c * k;
        for (int r = 0; r < rows; ++r) {
            const float acc = gemv_channel_f32(wc, x + (size_t)r * k, k);
            const size_t o = (size_t)r * n + c;
            float val;
            if (mode == 1) val = fmaf(acc, scales[c], bf2f(y[o]));
            else val = acc * scales[c];
            if (acc_out) acc_out[o] = val;
            y[o] = f2bf(val);
        }
    }
}

/* Fused gate/up/SiLU: W is [2n][k] (gate rows first), scales [2n]
 * (int8_gemv.cu:221-291): out = bf16( g/(1+expf(-g)) * u ). */
ORC_API void orc_int8_gate_up_silu_rows(const int8_t* w, const float* scales, const uint16_t* x,
                                        uint16_t* y, float* acc_out, int k, int n, int rows) {
#pragma omp parallel for schedule(static)
    for (int c = 0; c < n; ++c) {
        const int8_t* wg = w + (size_t)c * k;
        const int8_t* wu = w + ((size_t)n + c) * k;
        for (int r = 0; r < rows; ++r) {
            const uint16_t* xr = x + (size_t)r * k;
            const float g = gemv_channel_f32(wg, xr, k) * scales[c];
            const float u = gemv_channel_f32(wu, xr, k) * scales[n + c];
            const float act = g / (1.0f + expf(-g));
            const float val = act * u;
            const size_t o = (size_t)r * n + c;
            if (acc_out) acc_out[o] = val;
            y[o] = f2bf(val);
        }
    }
}

/* fp64 truth for the same contraction: out[r][c] = scale[c] * sum_k w[c][k]*x[r][k] */
ORC_API void orc_int8_gemm_rows_f64(const int8_t* w, const float* scales, const uint16_t* x,
                                    double* out, int k, int n, int rows) {
#pragma omp parallel for schedule(static)
    for (int c = 0; c < n; ++c) {
        const int8_t* wc = w + (size_t)c * k;
        for (int r = 0; r < rows; ++r) {
            const uint16_t* xr = x + (size_t)r * k;
            double acc = 0.0;
            for (int i = 0; i < k; ++i) acc += (double)wc[i] * (double)bf2f(xr[i]);
            out[(size_t)r * n + c] = acc * (double)scales[c];
        }
    }
}

/* Per-row symmetric quantizer (int8_gemv.cu:20-52): absmax -> scale = max/127
 * (1.0 when the row is all zero) -> lrintf(clamp(w * (1/scale), +-127)). */
ORC_API void orc_quantize_rows(const uint16_t* weight, int8_t* q, float* scales, int k, int n) {
#pragma omp parallel for schedule(static)
    for (int c = 0; c < n; ++c) {
        const uint16_t* row = weight + (size_t)c * k;
        float maximum = 0.0f;
        for (int i = 0; i < k; ++i) maximum = fmaxf(maximum, fabsf(bf2f(row[i])));
        const float scale = maximum > 0.0f ? maximum / 127.0f : 1.0f;
        const float inverse = 1.0f / scale;
        scales[c] = scale;
        for (int i = 0; i < k; ++i) {
            const float v = bf2f(row[i]) * inverse;
            const float cl = fminf(fmaxf(v, -127.0f), 127.0f);
            q[(size_t)c * k + i] = (int8_t)lrintf(cl);
        }
    }
}

/* --------------------------------------------------------- norms / RoPE -- */

/* The reference's block_sum (talker_kernels.cu:14-25): 256 slots, halving tree. */
static float block_sum_256(float* partial) {
    for (int stride = 128; stride > 0; stride >>= 1)
        for (int t = 0; t < stride; ++t) partial[t] += partial[t + stride];
    return partial[0];
}

/* RMSNorm (talker_kernels.cu:27-48): thread t sums x^2 over t, t+256, ... with fmaf,
 * tree sum, inv = rsqrtf(sum/W + eps), out = bf16( bf16(x*inv) * w ). */
ORC_API void orc_rms_norm_rows(const uint16_t* x, const uint16_t* w, uint16_t* y, int rows,
                               int width, float eps) {
    for (int r = 0; r < rows; ++r) {
        const uint16_t* xr = x + (size_t)r * width;
        float partial[256];
        for (int t = 0; t < 256; ++t) {
            float ss = 0.0f;
            for (int i = t; i < width; i += 256) {
                const float v = bf2f(xr[i]);
                ss = fmaf(v, v, ss);
            }
            partial[t] = ss;
        }
        const float inv = rsqrt_f(block_sum_256(partial) / (float)width + eps);
        for (int i = 0; i < width; ++i) {
            const float normalized = rbf(bf2f(xr[i]) * inv);
            y[(size_t)r * width + i] = f2bf(normalized * bf2f(w[i]));
        }
    }
}

/* Per-head RMSNorm in place (talker_kernels.cu:50-70); `heads` counts rows*heads. */
ORC_API void orc_head_rms_norm(uint16_t* v, const uint16_t* w, int heads, int head_dim,
                               float eps) {
    orc_rms_norm_rows(v, w, v, heads, head_dim, eps);
}

/* Rotate-half RoPE with the reference's bf16 rounding chain
 * (talker_kernels.cu:597-639): cos/sin rounded to bf16, each product rounded,
 * the sum/difference rounded. */
ORC_API void orc_rope_rows_at(uint16_t* v, int rows, int heads, int head_dim,
                              const int* positions, float theta) {
    const int half = head_dim / 2;
    for (int r = 0; r < rows; ++r) {
        for (int h = 0; h < heads; ++h) {
            uint16_t* base = v + ((size_t)r * heads + h) * head_dim;
            for (int d = 0; d < half; ++d) {
                const float exponent = (float)(2 * d) / (float)head_dim;
                const float angle = (float)positions[r] * powf(theta, -exponent);
                const float c = rbf(cosf(angle));
                const float s = rbf(sinf(angle));
                const float first = bf2f(base[d]);
                const float second = bf2f(base[d + half]);
                const float fc = rbf(first * c);
                const float ss = rbf(second * s);
                const float sc = rbf(second * c);
                const float fs = rbf(first * s);
                base[d] = f2bf(fc - ss);
                base[d + half] = f2bf(sc + fs);
            }
        }
    }
}

/* ------------------------------------------------------------ attention -- */

/* "Fast" decode attention (talker_kernels.cu:506-595), the semantic reference for the
 * int8 decode path: fp32 scores, expf, per-thread strided partial sums folded by a
 * 256-slot tree, out = bf16(acc * (1/sum)).  K and V of row r start at k + r*row_stride
 * (elements) and are laid out [position][kv_heads][head_dim].  out_f32 (optional)
 * receives the value before the final bf16 round. */
ORC_API void orc_attention_fast(const uint16_t* q, const uint16_t* k, const uint16_t* v,
                                const int* positions, uint16_t* out, float* out_f32, int rows,
                                int q_heads, int kv_heads, int head_dim, long row_stride) {
    const int groups = q_heads / kv_heads;
    const float scale = rsqrt_f((float)head_dim);
#pragma omp parallel for schedule(dynamic) collapse(2)
    for (int r = 0; r < rows; ++r) {
        for (int h = 0; h < q_heads; ++h) {
            const int len = positions[r] + 1;
            const int kvh = h / groups;
            const uint16_t* qv = q + ((size_t)r * q_heads + h) * head_dim;
            const uint16_t* kc = k + (size_t)r * row_stride;
            const uint16_t* vc = v + (size_t)r * row_stride;
            float* scores = (float*)malloc(sizeof(float) * (size_t)len);
            float maximum = -INFINITY;
            for (int p = 0; p < len; ++p) {
                const uint16_t* key = kc + ((size_t)p * kv_heads + kvh) * head_dim;
                float dot = 0.0f;
                for (int d = 0; d < head_dim; ++d) dot = fmaf(bf2f(qv[d]), bf2f(key[d]), dot);
                scores[p] = dot * scale;
                maximum = fmaxf(maximum, scores[p]);
            }
            float partial[256];
            for (int t = 0; t < 256; ++t) {
                float local = 0.0f;
                for (int p = t; p < len; p += 256) {
                    const float wgt = expf(scores[p] - maximum);
                    scores[p] = wgt;
                    local += wgt;
                }
                partial[t] = local;
            }
            const float inverse = 1.0f / block_sum_256(partial);
            for (int d = 0; d < head_dim; ++d) {
                float acc = 0.0f;
                for (int p = 0; p < len; ++p) {
                    const uint16_t* val = vc + ((size_t)p * kv_heads + kvh) * head_dim;
                    acc = fmaf(scores[p], bf2f(val[d]), acc);
                }
                const size_t o = ((size_t)r * q_heads + h) * head_dim + d;
                if (out_f32) out_f32[o] = acc * inverse;
                out[o] = f2bf(acc * inverse);
            }
            free(scores);
        }
    }
}

/* "Exact" decode attention (talker_kernels.cu:423-497): per-position dot through the
 * 256-slot tree (thread d holds q[d]*k[d]), dot and scaled score rounded to bf16, serial
 * max/exp/sum, probabilities rounded to bf16, PV in fp32.  Used only to report the
 * distance between the two reference kernels. */
ORC_API void orc_attention_exact(const uint16_t* q, const uint16_t* k, const uint16_t* v,
                                 const int* positions, uint16_t* out, int rows, int q_heads,
                                 int kv_heads, int head_dim, long row_stride) {
    const int groups = q_heads / kv_heads;
    const float scale = rsqrt_f((float)head_dim);
#pragma omp parallel for schedule(dynamic) collapse(2)
    for (int r = 0; r < rows; ++r) {
        for (int h = 0; h < q_heads; ++h) {
            const int len = positions[r] + 1;
            const int kvh = h / groups;
            const uint16_t* qv = q + ((size_t)r * q_heads + h) * head_dim;
            const uint16_t* kc = k + (size_t)r * row_stride;
            const uint16_t* vc = v + (size_t)r * row_stride;
            float* scores = (float*)malloc(sizeof(float) * (size_t)len);
            for (int p = 0; p < len; ++p) {
                const uint16_t* key = kc + ((size_t)p * kv_heads + kvh) * head_dim;
                float partial[256];
                for (int t = 0; t < 256; ++t) {
                    float dot = 0.0f;
                    for (int d = t; d < head_dim; d += 256)
                        dot = fmaf(bf2f(qv[d]), bf2f(key[d]), dot);
                    partial[t] = dot;
                }
                const float dp = rbf(block_sum_256(partial));
                scores[p] = rbf(dp * scale);
            }
            float maximum = -INFINITY;
            for (int p = 0; p < len; ++p) maximum = fmaxf(maximum, scores[p]);
            float denominator = 0.0f;
            for (int p = 0; p < len; ++p) {
                scores[p] = expf(scores[p] - maximum);
                denominator += scores[p];
            }
            const float inverse = 1.0f / denominator;
            for (int p = 0; p < len; ++p) scores[p] = rbf(scores[p] * inverse);
            for (int d = 0; d < head_dim; ++d) {
                float acc = 0.0f;
                for (int p = 0; p < len; ++p) {
                    const uint16_t* val = vc + ((size_t)p * kv_heads + kvh) * head_dim;
                    acc = fmaf(scores[p], bf2f(val[d]), acc);
                }
                out[((size_t)r * q_heads + h) * head_dim + d] = f2bf(acc);
            }
            free(scores);
        }
    }
}

/* ------------------------------------------------------ elementwise glue -- */

/* talker_kernels.cu:660-678: v = bf16( (v + b) [ * 1/(1+expf(-(v+b))) ] ) */
ORC_API void orc_bias_activation_rows(uint16_t* v, const uint16_t* bias, int rows, int width,
                                      int silu) {
    for (long i = 0; i < (long)rows * width; ++i) {
        float val = bf2f(v[i]) + bf2f(bias[i % width]);
        if (silu) val *= 1.0f / (1.0f + expf(-val));
        v[i] = f2bf(val);
    }
}

/* talker_kernels.cu:405-421 (the unfused path; intermediate bf16 round of silu(g)) */
ORC_API void orc_silu_gate(uint16_t* gate, const uint16_t* up, int width) {
    for (int i = 0; i < width; ++i) {
        const float g = bf2f(gate[i]);
        const float act = rbf(g / (1.0f + expf(-g)));
        gate[i] = f2bf(act * bf2f(up[i]));
    }
}

/* talker_kernels.cu:359-371 */
ORC_API void orc_add_in_place(uint16_t* dst, const uint16_t* src, long n) {
    for (long i = 0; i < n; ++i) dst[i] = f2bf(bf2f(dst[i]) + bf2f(src[i]));
}

/* ---------------------------------------------------------------- sampler -- */

/* xorshift64* (sampling_kernels.cu:53-69) */
static uint64_t next_random(uint64_t* state) {
    uint64_t v = *state;
    if (v == 0) v = 0x9e3779b97f4a7c15ULL;
    v ^= v >> 12;
    v ^= v << 25;
    v ^= v >> 27;
    *state = v;
    return v * 0x2545f4914f6cdd1dULL;
}

static float uniform_random(uint64_t* state) {
    const double scale = 1.0 / 9007199254740992.0;
    return (float)((double)(next_random(state) >> 11) * scale);
}

ORC_API float orc_uniform(uint64_t* state) { return uniform_random(state); }

/* sampling_kernels.cu:30-51 */
static float adjusted_logit(const uint16_t* logits, int token, int suppress, int eos,
                            const int* history, int count, float penalty) {
    if (suppress && token >= 2048 && token != eos) return -INFINITY;
    float value = bf2f(logits[token]);
    if (suppress && penalty != 1.0f) {
        int hit = 0;
        for (int i = 0; i < count; ++i)
            if (history[i] == token) { hit = 1; break; }
        if (hit) value = value < 0.0f ? value * penalty : value / penalty;
    }
    return value;
}

typedef struct { float v; int i; } cand_t;

/* total order of sampling_kernels.cu:73-75: value descending, ties by lower index
 * (IEEE ==, so -0 ties with +0) */
static int cand_cmp(const void* a, const void* b) {
    const cand_t* x = (const cand_t*)a;
    const cand_t* y = (const cand_t*)b;
    if (x->v > y->v) return -1;
    if (x->v < y->v) return 1;
    return (x->i > y->i) - (x->i < y->i);
}

/* One sampler call (sampling_kernels.cu:143-389).  Returns the selected token and
 * advances *rng exactly when the reference does (not for do_sample == 0). */
ORC_API int orc_sample(const uint16_t* logits, int vocabulary, int suppress, int eos,
                       const int* history, int count, int do_sample, int top_k, float top_p,
                       float temperature, float penalty, uint64_t* rng) {
    cand_t* c = (cand_t*)malloc(sizeof(cand_t) * (size_t)vocabulary);
    double* weights = (double*)malloc(sizeof(double) * (size_t)vocabulary);
    for (int t = 0; t < vocabulary; ++t) {
        c[t].v = adjusted_logit(logits, t, suppress, eos, history, count, penalty);
        c[t].i = t;
    }
    const int direct = do_sample != 0 && top_k == 0 && top_p >= 1.0f;
    const int selections =
        do_sample == 0 ? 1 : (top_k == 0 ? vocabulary : (top_k < vocabulary ? top_k : vocabulary));
    int selected;
    if (do_sample == 0 || direct) {
        /* argmax, ties to the lower index (:208-233) */
        float best = -INFINITY;
        int best_i = -1;
        for (int t = 0; t < vocabulary; ++t) {
            if (c[t].v > best || (c[t].v == best && best_i < 0)) { best = c[t].v; best_i = t; }
        }
        if (do_sample == 0) {
            selected = best_i;
        } else {
            /* direct categorical over the whole vocabulary in index order (:242-264) */
            const float maximum = best / temperature;
            for (int t = 0; t < vocabulary; ++t)
                weights[t] = exp((double)(c[t].v / temperature - maximum));
            double total = 0.0;
            for (int t = 0; t < vocabulary; ++t) total += weights[t];
            const double target = (double)uniform_random(rng) * total;
            double cumulative = 0.0;
            selected = best_i;
            for (int t = 0; t < vocabulary; ++t) {
                cumulative += weights[t];
                if (cumulative >= target) { selected = t; break; }
            }
        }
    } else {
        /* top-`selections` in the total order (:268-350), then the fp64 tail (:352-388) */
        qsort(c, (size_t)vocabulary, sizeof(cand_t), cand_cmp);
        const float maximum = c[0].v / temperature;
        for (int r = 0; r < selections; ++r)
            weights[r] = exp((double)(c[r].v / temperature - maximum));
        double denominator = 0.0;
        for (int r = 0; r < selections; ++r) denominator += weights[r];
        double cumulative = 0.0;
        int retained = selections;
        for (int r = 0; r < selections; ++r) {
            cumulative += weights[r] / denominator;
            if (cumulative >= (double)top_p) { retained = r + 1; break; }
        }
        double retained_total = 0.0;
        for (int r = 0; r < retained; ++r) retained_total += weights[r];
        const double target = (double)uniform_random(rng) * retained_total;
        cumulative = 0.0;
        selected = c[retained - 1].i;
        for (int r = 0; r < retained; ++r) {
            cumulative += weights[r];
            if (cumulative >= target) { selected = c[r].i; break; }
        }
    }
    free(c);
    free(weights);
    return selected;
}

/* Embedding row copy / add (sampling_kernels.cu:428-452): out-of-range token = no-op */
ORC_API void orc_embedding(const uint16_t* table, int vocabulary, int width, int token,
                           uint16_t* out, int add) {
    if (token < 0 || token >= vocabulary) return;
    const uint16_t* src = table + (size_t)token * width;
    for (int i = 0; i < width; ++i)
        out[i] = add ? f2bf(bf2f(out[i]) + bf2f(src[i])) : src[i];
}
