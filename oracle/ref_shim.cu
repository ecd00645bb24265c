// TEST INFRASTRUCTURE ONLY -- not part of the shipped library.
//
// Thin extern "C" wrappers around the reference project's own kernel launchers
// (namespace qwen3_tts, declared in its native/src/talker_internal.cuh).  The
// reference sources are compiled where they lie (see build_ref.sh) for sm_100a
// and linked with this file into oracle/_ref/libq3t_ref.so, so that the GPU
// parity tests can run the *unmodified reference kernels* on the same seeded
// inputs as our kernels.  Every wrapper takes HOST pointers, stages them through
// cudaMalloc'd buffers, runs one reference launch and copies the result back.
//
// Nothing in the product library links against or loads this file.

#include "talker_internal.cuh"   // resolved with -I<reference>/native/qwen3-tts-native/native/src

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <vector>

namespace {

struct Dev {
    void* p = nullptr;
    size_t n = 0;
    Dev() = default;
    explicit Dev(size_t bytes) : n(bytes) { if (bytes) cudaMalloc(&p, bytes); }
    Dev(const Dev&) = delete;
    Dev& operator=(const Dev&) = delete;
    ~Dev() { if (p) cudaFree(p); }
    template <class T> T* as() { return static_cast<T*>(p); }
    void up(const void* h) { if (n) cudaMemcpy(p, h, n, cudaMemcpyHostToDevice); }
    void down(void* h) { if (n) cudaMemcpy(h, p, n, cudaMemcpyDeviceToHost); }
};

int finish(cudaError_t launch) {
    if (launch != cudaSuccess) return static_cast<int>(launch);
    return static_cast<int>(cudaDeviceSynchronize());
}

}  // namespace

extern "C" {

// mode 0: y = bf16(scale*(W x)); 1: y = bf16(y + scale*(W x)); 2: fused gate/up/SiLU
// (W is [2N][K], scales [2N], y [rows][N]).
int ref_int8_gemm(const int8_t* w, const float* scales, const uint16_t* x, uint16_t* y,
                  int in_features, int out_features, int rows, int mode) {
    const size_t wrows = mode == 2 ? 2 * (size_t)out_features : (size_t)out_features;
    Dev dw(wrows * in_features), ds(wrows * sizeof(float));
    Dev dx((size_t)rows * in_features * 2), dy((size_t)rows * out_features * 2);
    dw.up(w); ds.up(scales); dx.up(x); dy.up(y);
    cudaError_t e;
    if (mode == 0) {
        e = qwen3_tts::launch_int8_gemm_rows(dw.as<int8_t>(), ds.as<float>(),
            dx.as<__nv_bfloat16>(), dy.as<__nv_bfloat16>(), in_features, out_features, rows, 0);
    } else if (mode == 1) {
        e = qwen3_tts::launch_int8_gemm_rows_add(dw.as<int8_t>(), ds.as<float>(),
            dx.as<__nv_bfloat16>(), dy.as<__nv_bfloat16>(), in_features, out_features, rows, 0);
    } else {
        e = qwen3_tts::launch_int8_gate_up_silu_rows(dw.as<int8_t>(), ds.as<float>(),
            dx.as<__nv_bfloat16>(), dy.as<__nv_bfloat16>(), in_features, out_features, rows, 0);
    }
    const int r = finish(e);
    dy.down(y);
    return r;
}

int ref_quantize_rows(const uint16_t* weight, int8_t* q, float* scales,
                      int in_features, int out_features) {
    Dev dw((size_t)out_features * in_features * 2), dq((size_t)out_features * in_features);
    Dev ds((size_t)out_features * sizeof(float));
    dw.up(weight);
    const int r = finish(qwen3_tts::launch_quantize_weight_rows(
        dw.as<__nv_bfloat16>(), dq.as<int8_t>(), ds.as<float>(), in_features, out_features, 0));
    dq.down(q); ds.down(scales);
    return r;
}

int ref_rms_norm_rows(const uint16_t* x, const uint16_t* w, uint16_t* y, int rows, int width,
                      float eps) {
    Dev dx((size_t)rows * width * 2), dw((size_t)width * 2), dy((size_t)rows * width * 2);
    dx.up(x); dw.up(w);
    const int r = finish(qwen3_tts::launch_rms_norm_rows(dx.as<__nv_bfloat16>(),
        dw.as<__nv_bfloat16>(), dy.as<__nv_bfloat16>(), rows, width, eps, 0));
    dy.down(y);
    return r;
}

int ref_head_rms_norm_rows(uint16_t* v, const uint16_t* w, int rows, int heads, int head_dim,
                           float eps) {
    Dev dv((size_t)rows * heads * head_dim * 2), dw((size_t)head_dim * 2);
    dv.up(v); dw.up(w);
    const int r = finish(qwen3_tts::launch_head_rms_norm_rows(dv.as<__nv_bfloat16>(),
        dw.as<__nv_bfloat16>(), rows, heads, head_dim, eps, 0));
    dv.down(v);
    return r;
}

int ref_rope_rows_at(uint16_t* v, int rows, int heads, int head_dim, const int* positions,
                     float theta) {
    Dev dv((size_t)rows * heads * head_dim * 2), dp((size_t)rows * sizeof(int));
    dv.up(v); dp.up(positions);
    const int r = finish(qwen3_tts::launch_rope_rows_at(dv.as<__nv_bfloat16>(), rows, heads,
        head_dim, dp.as<int>(), theta, 0));
    dv.down(v);
    return r;
}

// K and V are [rows][capacity][kv_heads*head_dim]; positions[r] is the last valid index.
int ref_attention(const uint16_t* q, const uint16_t* k, const uint16_t* v, const int* positions,
                  uint16_t* out, int rows, int q_heads, int kv_heads, int head_dim, int capacity,
                  int fast) {
    const size_t per_row = (size_t)capacity * kv_heads * head_dim;
    Dev dq((size_t)rows * q_heads * head_dim * 2), dk(rows * per_row * 2), dv(rows * per_row * 2);
    Dev dp((size_t)rows * sizeof(int)), dout((size_t)rows * q_heads * head_dim * 2);
    Dev dkb((size_t)rows * sizeof(void*)), dvb((size_t)rows * sizeof(void*));
    dq.up(q); dk.up(k); dv.up(v); dp.up(positions);
    std::vector<__nv_bfloat16*> kb(rows), vb(rows);
    for (int r = 0; r < rows; ++r) {
        kb[r] = dk.as<__nv_bfloat16>() + r * per_row;
        vb[r] = dv.as<__nv_bfloat16>() + r * per_row;
    }
    dkb.up(kb.data()); dvb.up(vb.data());
    cudaError_t e;
    if (fast) {
        e = qwen3_tts::launch_batch_causal_gqa_attention_fast(dq.as<__nv_bfloat16>(),
            dkb.as<__nv_bfloat16*>(), dvb.as<__nv_bfloat16*>(), dp.as<int>(),
            dout.as<__nv_bfloat16>(), rows, q_heads, kv_heads, head_dim, capacity, 0);
    } else {
        e = qwen3_tts::launch_batch_causal_gqa_attention(dq.as<__nv_bfloat16>(),
            dkb.as<__nv_bfloat16*>(), dvb.as<__nv_bfloat16*>(), dp.as<int>(),
            dout.as<__nv_bfloat16>(), rows, q_heads, kv_heads, head_dim, capacity, 0);
    }
    const int r = finish(e);
    dout.down(out);
    return r;
}

// One sampler launch; rng_state is read and written back.
int ref_sample(const uint16_t* logits, int vocabulary, int suppress, int eos, const int* history,
               int history_count, int do_sample, int top_k, float top_p, float temperature,
               float penalty, uint64_t* rng_state, int* token) {
    Dev dl((size_t)vocabulary * 2), dh((size_t)(history_count > 0 ? history_count : 1) * sizeof(int));
    Dev dr(sizeof(uint64_t)), dt(sizeof(int));
    dl.up(logits);
    if (history_count > 0) cudaMemcpy(dh.p, history, (size_t)history_count * sizeof(int),
                                      cudaMemcpyHostToDevice);
    dr.up(rng_state);
    cudaMemset(dt.p, 0xff, sizeof(int));
    const int r = finish(qwen3_tts::launch_sample_logits(dl.as<__nv_bfloat16>(), vocabulary,
        suppress != 0, eos, dh.as<int>(), history_count, do_sample, top_k, top_p, temperature,
        penalty, dr.as<uint64_t>(), dt.as<int>(), 0));
    dr.down(rng_state); dt.down(token);
    return r;
}

int ref_bias_activation_rows(uint16_t* v, const uint16_t* bias, int rows, int width, int silu) {
    Dev dv((size_t)rows * width * 2), db((size_t)width * 2);
    dv.up(v); db.up(bias);
    const int r = finish(qwen3_tts::launch_bias_activation_rows(dv.as<__nv_bfloat16>(),
        db.as<__nv_bfloat16>(), rows, width, silu != 0, 0));
    dv.down(v);
    return r;
}

int ref_silu_gate(uint16_t* gate, const uint16_t* up, int width) {
    Dev dg((size_t)width * 2), du((size_t)width * 2);
    dg.up(gate); du.up(up);
    const int r = finish(qwen3_tts::launch_silu_gate(dg.as<__nv_bfloat16>(),
        du.as<__nv_bfloat16>(), width, 0));
    dg.down(gate);
    return r;
}

int ref_add_in_place(uint16_t* dst, const uint16_t* src, int width) {
    Dev dd((size_t)width * 2), ds((size_t)width * 2);
    dd.up(dst); ds.up(src);
    const int r = finish(qwen3_tts::launch_add_in_place(dd.as<__nv_bfloat16>(),
        ds.as<__nv_bfloat16>(), width, 0));
    dd.down(dst);
    return r;
}

// Same-box comparator: mean microseconds per launch of the reference GEMV kernel,
// rotating over `buffers` distinct weight images (so the stream comes from HBM,
// not L2) for `iterations` launches.  Returns < 0 on a CUDA error.
float ref_time_int8_gemm(int in_features, int out_features, int rows, int mode, int buffers,
                         int iterations) {
    const size_t wrows = mode == 2 ? 2 * (size_t)out_features : (size_t)out_features;
    const size_t wbytes = wrows * in_features;
    Dev dw(wbytes * buffers), ds(wrows * sizeof(float));
    Dev dx((size_t)rows * in_features * 2), dy((size_t)rows * out_features * 2);
    if (!dw.p || !ds.p || !dx.p || !dy.p) return -1.0f;
    cudaMemset(dw.p, 1, wbytes * buffers);
    cudaMemset(ds.p, 0, wrows * sizeof(float));
    cudaMemset(dx.p, 0, dx.n);
    cudaMemset(dy.p, 0, dy.n);
    cudaEvent_t a, b;
    cudaEventCreate(&a); cudaEventCreate(&b);
    auto run = [&](int i) {
        const int8_t* w = dw.as<int8_t>() + (size_t)(i % buffers) * wbytes;
        if (mode == 0) return qwen3_tts::launch_int8_gemm_rows(w, ds.as<float>(),
            dx.as<__nv_bfloat16>(), dy.as<__nv_bfloat16>(), in_features, out_features, rows, 0);
        if (mode == 1) return qwen3_tts::launch_int8_gemm_rows_add(w, ds.as<float>(),
            dx.as<__nv_bfloat16>(), dy.as<__nv_bfloat16>(), in_features, out_features, rows, 0);
        return qwen3_tts::launch_int8_gate_up_silu_rows(w, ds.as<float>(),
            dx.as<__nv_bfloat16>(), dy.as<__nv_bfloat16>(), in_features, out_features, rows, 0);
    };
    for (int i = 0; i < buffers; ++i) run(i);
    cudaDeviceSynchronize();
    cudaEventRecord(a, 0);
    for (int i = 0; i < iterations; ++i) run(i);
    cudaEventRecord(b, 0);
    float ms = -1.0f;
    if (cudaEventSynchronize(b) != cudaSuccess || cudaEventElapsedTime(&ms, a, b) != cudaSuccess) {
        ms = -1.0f;
    }
    cudaEventDestroy(a); cudaEventDestroy(b);
    return ms < 0 ? -1.0f : ms * 1000.0f / iterations;
}

}  // extern "C"
