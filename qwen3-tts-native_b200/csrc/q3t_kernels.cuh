// Internal launcher interface of the sm_100a decode kernels.  Every launcher takes raw
// device pointers and a stream and returns a cudaError_t, like the launchers of the
// reference's native/qwen3-tts-native/native/src/talker_internal.cuh that they replace.
#pragma once

#include "q3t_common.cuh"

namespace q3t {

// Per-device one-time set-up (dynamic shared-memory ceilings).  Call with the device current
// before the first launch on it and never inside a stream capture; later calls are no-ops.
cudaError_t configure_device();
cudaError_t configure_gemv_kernels();
cudaError_t configure_sampler_kernels();

// ---------------------------------------------------------------- int8 GEMV / GEMM
enum Epilogue : int {
    EPI_PLAIN = 0,       // y = bf16(acc*scale)
    EPI_ADD = 1,         // y = bf16(fma(acc, scale, y))                      (residual)
    EPI_BIAS = 2,        // y = bf16(bf16(acc*scale) + bias)
    EPI_BIAS_SILU = 3,   // v = bf16(acc*scale) + bias; y = bf16(v * 1/(1+exp(-v)))
    EPI_BIAS_ADD = 4,    // t = bf16(bf16(acc*scale) + bias); resid = bf16(resid + t)
    EPI_GATE_UP_SILU = 5 // W is [2N][K]: y = bf16(silu(g*sg) * (u*su))
};

struct GemvArgs {
    const int8_t* w = nullptr;       // [N][K] row-major (EPI_GATE_UP_SILU: [2N][K])
    const float* scales = nullptr;   // [N] (or [2N])
    const bf16* x = nullptr;         // [rows][K]
    bf16* y = nullptr;               // [rows][N]
    float* y32 = nullptr;            // optional fp32 value before the final bf16 round
    const bf16* norm_w = nullptr;    // non-null: RMSNorm(x) * norm_w is applied to x first
    bf16* norm_out = nullptr;        // optional [rows][K]: the normalized activations
    const bf16* bias = nullptr;      // [N] for the bias epilogues
    bf16* resid = nullptr;           // [rows][N] for EPI_BIAS_ADD
    int in_features = 0;             // K, multiple of 16
    int out_features = 0;            // N
    int rows = 0;                    // 1..kMaxRows
    int epilogue = EPI_PLAIN;
    float eps = kRmsEps;
    // EPI_ADD / EPI_BIAS_ADD: the accumulated-into values (y, resid) were last written two or more
    // launches upstream of this one in its stream (never by the launch directly before it), so
    // they may be fetched ahead of the dependency wait.  Set only by callers that build the whole
    // launch sequence; false is always correct.
    bool residual_settled = false;
};

// Launch with programmatic stream serialisation (QWEN3_TTS_PDL=0 turns it into an ordinary
// launch).  Only for kernels that call pdl_wait() before they read anything a predecessor wrote.
bool pdl_enabled();
template <typename... Params, typename... Args>
cudaError_t launch_pdl(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                       Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
}

// Dispatcher over the kernels below (see its definition for the rule)
cudaError_t launch_int8_gemm(const GemvArgs& args, cudaStream_t stream);
cudaError_t launch_int8_gemm_simt(const GemvArgs& args, cudaStream_t stream);
// 1..8 rows on mma.sync with the weights bulk-copied ahead of the dependency wait (gemv_int8_mma.cu):
// K = 512 * {2, 3, 4, 6, 8, 9, 12, ...}; same value as the SIMT kernel up to the order of summation
bool gemv_mma_supports(const GemvArgs& args);
cudaError_t launch_int8_gemv_mma(const GemvArgs& args, cudaStream_t stream);
// the shared-memory plan of one launch (host arithmetic only; see gemv_int8_mma.cu)
struct GemvMmaPlan {
    int grid, stages, group, tiles, rows_per_launch;
    long long stage_bytes, ring_bytes, shared_bytes;
};
bool gemv_mma_plan(int in_features, int out_features, int rows, bool gate_up, bool norm, GemvMmaPlan* out);
cudaError_t configure_gemv_mma_kernels();
unsigned int gemv_mma_error_count();
// which kernel launch_int8_gemm picks for 1..8 rows: 0 SIMT (the reference's summation order, bit for
// bit), 1 the int8 mma.sync kernel where it applies (default).
// Process-wide; returns the previous mode.
int set_gemv_mode(int mode);
int gemv_mode();
// tensor-core path (tcgen05, TMEM accumulators): rows >= tc_min_rows() and K % 64 == 0
bool gemm_tc_supports(const GemvArgs& args);
cudaError_t launch_int8_gemm_tc(const GemvArgs& args, cudaStream_t stream);
cudaError_t configure_tc_kernels();      // also allocates the per-device scratch of that path
void set_tc_min_rows(int rows);          // 65 or more: never use the tensor-core path
int tc_min_rows();
unsigned int gemm_tc_error_count();

cudaError_t launch_quantize_weight_rows(const bf16* weight, int8_t* quantized, float* scales,
                                        int in_features, int out_features, cudaStream_t stream);

// ---------------------------------------------------------------- norms / RoPE / glue
cudaError_t launch_rms_norm_rows(const bf16* input, const bf16* weight, bf16* output, int rows,
                                 int width, float eps, cudaStream_t stream);
cudaError_t launch_head_rms_norm_rows(bf16* values, const bf16* weight, int rows, int heads,
                                      int head_dim, float eps, cudaStream_t stream);
cudaError_t launch_rope_rows_at(bf16* values, int rows, int heads, int head_dim,
                                const int* positions, float theta, cudaStream_t stream);
cudaError_t launch_kv_scatter_rows(const bf16* rows_data, bf16* const* cache_bases,
                                   const int* positions, int rows, int width, cudaStream_t stream);
cudaError_t launch_bias_activation_rows(bf16* values, const bf16* bias, int rows, int width,
                                        bool silu, cudaStream_t stream);
cudaError_t launch_add_in_place(bf16* destination, const bf16* source, int count,
                                cudaStream_t stream);
cudaError_t launch_silu_gate(bf16* gate, const bf16* up, int count, cudaStream_t stream);
// tokens[row] points at that row's token array; out-of-range tokens leave the row untouched
cudaError_t launch_gather_embedding_rows(const bf16* table, int vocabulary, int width,
                                         const int* const* tokens, int token_offset, bf16* output,
                                         int rows, bool add, cudaStream_t stream);

// ---------------------------------------------------------------- decode attention
// Where the K/V rows of one batch row live.  Contiguous: base[row] + token*kv_width.
// Paged: pages of kPageTokens tokens; page id p of a row lives at
// slabs[p >> slab_shift] + (p & slab_mask) * page_elems + layer_offset, and holds
// [kv head][kPageTokens][head_dim]: the tokens of one KV head are one contiguous block (what a CTA
// of the attention kernel reads), not interleaved with the other heads.
struct KvLayout {
    bf16* const* k_bases = nullptr;     // contiguous mode: [rows]
    bf16* const* v_bases = nullptr;
    const int* page_table = nullptr;    // paged mode: [rows][table_stride] page ids
    int table_stride = 0;
    bf16* const* slabs = nullptr;       // paged mode: slab base pointers
    int slab_shift = 0;
    long long page_elems = 0;           // elements between consecutive pages of a slab
    long long k_offset = 0;             // element offset of this layer's K plane in a slab
    long long v_offset = 0;             // ... and of its V plane
};

struct AttentionArgs {
    const bf16* q = nullptr;            // [rows][q_heads*head_dim]
    const bf16* k_new = nullptr;        // fused mode: [rows][kv_heads*head_dim], raw projections
    const bf16* v_new = nullptr;
    const bf16* q_norm_w = nullptr;     // fused mode: per-head RMSNorm weights [head_dim]
    const bf16* k_norm_w = nullptr;
    const int* positions = nullptr;     // [rows] index of the newest token (length-1)
    bf16* out = nullptr;                // [rows][q_heads*head_dim]
    float* out32 = nullptr;             // optional fp32 value before the final round
    KvLayout kv;
    const uint32_t* rope_table = nullptr;   // optional [rope_positions][head_dim/2] bf16 cos | sin << 16
    int rope_positions = 0;                 //   (launch_build_rope_table); positions beyond it are computed
    float* scratch = nullptr;           // split-KV partials, see attention_scratch_floats()
    unsigned int* counters = nullptr;   // [rows*kv_heads], zero before the first launch
    int q_stride = 0;                   // elements between rows of q (0: q_heads*head_dim)
    int kv_new_stride = 0;              // elements between rows of k_new / v_new (0: packed)
    int rows = 0;
    int q_heads = 0;
    int kv_heads = 0;
    int head_dim = 0;                   // 64 or 128 (32 allowed when not fused)
    int max_splits = 0;                 // grid.x; >= ceil(max length / kAttnChunk)
    int fused = 0;                      // 1: head-norm + RoPE on q/k_new, append k/v at position
    int append_mode = 0;                // fused only.  0: append, then attend (decode).  1: append only.
                                        // 2: attend only.  Rows that share one cache (a prompt chunk)
                                        // need every row's K/V in place before any row attends: 1, then 2.
    // Decode steps only (fused, append_mode 0): positions, the page table and every cache row older
    // than this step's token were written two or more launches upstream in the stream, so the kernel
    // may fetch them ahead of its dependency wait (only q / k_new / v_new come from the launch directly
    // before).  Set by callers that build the whole launch sequence; 0 is always correct.
    int inputs_settled = 0;
    int units_per_cta = 0;              // splits one CTA walks (0: chosen from the grid size); no effect on results
    float eps = kRmsEps;
    float theta = kRopeTheta;
};

constexpr int kAttnChunk = 64;          // tokens per split
size_t attention_scratch_floats(int rows, int q_heads, int head_dim, int max_splits);
cudaError_t launch_decode_attention(const AttentionArgs& args, cudaStream_t stream);
// Layout of a caller's scratch buffer for the split-KV kernel, shared by every entry point that
// carves one up: ticket counters first (rounded to 256 bytes), the chunk partials behind them.
inline size_t attention_counters_bytes(int rows, int kv_heads) {
    return ((size_t)rows * kv_heads * sizeof(unsigned int) + 255) / 256 * 256;
}
inline int attention_splits_for(int max_sequence_length) {
    const int s = (max_sequence_length + kAttnChunk - 1) / kAttnChunk;
    return s < 1 ? 1 : s;
}
// Parity mode: the same attention with every fp32 sum formed in the order of the reference's
// kernel (bit-identical bf16 output; slow).  Fused mode normalises and rotates the query heads;
// the new token's K/V must already be in the cache (launch_decode_attention with append_mode 1).
// Positions must be below 8192.
cudaError_t launch_attention_reference_order(const AttentionArgs& args, cudaStream_t stream);
// Process-wide choice between the two (1, default: split-KV kernel; 0: reference order) and the
// launcher that honours it: in mode 0 a fused call appends with the split-KV kernel's prologue,
// then attends in the reference's order.
// rows seen so far whose position lay outside what the launch was sized for (clamped and counted)
unsigned int attention_range_error_count();
cudaError_t set_attention_error_sink(unsigned int* device_visible_word);
int set_attention_mode(int mode);
int attention_mode();
cudaError_t launch_attention(const AttentionArgs& args, cudaStream_t stream);
// cos/sin of every (position, rotary pair), rounded to bf16 as the fused prologue rounds them;
// computed by the same device expressions, so using the table changes no bit
cudaError_t launch_build_rope_table(uint32_t* table, int positions, int head_dim, float theta,
                                    cudaStream_t stream);

// ---------------------------------------------------------------- sampler
struct SamplerRow {
    const bf16* logits;          // [vocabulary]
    const int* history;          // semantic history (talker rows)
    const int* history_count;    // device count (may be null -> history_count_value)
    unsigned long long* rng;     // xorshift64* state
    int* selected;               // sampled token
    int* store_a;                // optional: store_a[store_a_index] = token
    int* store_b;                // optional: store_b[*history_count] = token (history append)
    int store_a_index;
    int history_count_value;
    int vocabulary;
    int suppress;                // talker rows: tokens >= 2048 other than EOS are masked
    int mask_eos;                // harness option: also mask EOS (synthetic weights)
    int eos;
    int do_sample;
    int top_k;
    float top_p;
    float temperature;
    float penalty;
};

// rows[] lives in device memory; one CTA per row
cudaError_t launch_sample_rows(const SamplerRow* rows, int count, cudaStream_t stream);
// a single row passed by value
cudaError_t launch_sample_value(const SamplerRow& row, cudaStream_t stream);

// ---------------------------------------------------------------- frame table
struct SamplingParams {      // same field order as the ABI's Qwen3TtsSamplingConfig
    int do_sample;
    int top_k;
    float top_p;
    float temperature;
    float penalty;
};

// Per-row state of one lockstep frame, resident in device memory and refreshed by the
// host before a frame.  Everything that differs between sessions or frames reaches the
// kernels through this table, so a captured frame graph stays valid for any session set.
struct FrameTable {
    int position[kMaxRows];            // talker KV slot written by this frame
    int history_count[kMaxRows];       // semantic tokens generated so far
    int trailing_text[kMaxRows];       // text token mixed into the next talker input
    int* frame_tokens[kMaxRows];       // [16] codebook tokens of the frame
    unsigned short* frame_codes[kMaxRows];   // [16] packed codes handed to the codec
    int* history[kMaxRows];            // semantic history (repetition penalty)
    unsigned long long* rng[kMaxRows]; // xorshift64* state
    int* sampled[kMaxRows];            // current semantic token in, next semantic token out
    bf16* last_hidden[kMaxRows];       // [talker hidden] final-normed hidden of the last step
    int* host_token[kMaxRows];         // pinned, device-mapped: next semantic token
    unsigned short* host_codes[kMaxRows];    // pinned, device-mapped: the 16 codes
    SamplingParams talker[kMaxRows];
    SamplingParams predictor[kMaxRows];
};

// Sampler over table rows: row r reads logits + r*logits_stride.  talker != 0: reserved
// tokens masked, repetition penalty, token -> sampled[r] and appended to history[r];
// talker == 0: token -> frame_tokens[r][store_index].
cudaError_t launch_sample_table(const FrameTable* table, const bf16* logits, int logits_stride,
                                int vocabulary, int talker, int store_index, int mask_eos,
                                int eos, int rows, cudaStream_t stream);

// frame_tokens[r][0] = *sampled[r]
cudaError_t launch_frame_begin(const FrameTable* table, int rows, cudaStream_t stream);
// input of predictor position p: p == 0 last_hidden, p == 1 codec_embedding[tok 0],
// else predictor_embedding[p-2][tok p-1]; written to x[r][width]
cudaError_t launch_predictor_input(const FrameTable* table, int p, const bf16* codec_embedding,
                                   const bf16* const* predictor_embeddings, bf16* x, int width,
                                   int rows, cudaStream_t stream);
// hidden[r] = codec_embedding[tok0] (+) predictor_embedding[i][tok i+1] for i = 0..14, each add
// rounded to bf16 in that order; text_in[r] = text_embedding[trailing_text[r]]
cudaError_t launch_talker_input(const FrameTable* table, const bf16* codec_embedding,
                                const bf16* const* predictor_embeddings, const bf16* text_embedding,
                                int text_vocabulary, bf16* hidden, bf16* text_in, int width, int rows,
                                cudaStream_t stream);
// frame_codes[r][i] = (u16) frame_tokens[r][i]; also mirrored to host_codes[r]
cudaError_t launch_pack_codes(const FrameTable* table, int rows, cudaStream_t stream);
// last_hidden[r] = normalized[r]; host_token[r] = *sampled[r]; history_count += 1 and, when
// advance_position != 0, position += 1
cudaError_t launch_frame_end(FrameTable* table, const bf16* normalized, int width, int rows,
                             int advance_position, cudaStream_t stream);
// prompt row: x = text_embedding[text_ids[index]] (skipped when negative)
cudaError_t launch_prompt_gather(const FrameTable* table, const int* text_ids,
                                 const bf16* text_embedding, int text_vocabulary, bf16* x, int width,
                                 cudaStream_t stream);
// prompt row: hidden = (text id < 0 ? 0 : hidden) (+) codec_embedding[codec id] when >= 0
cudaError_t launch_prompt_combine(const FrameTable* table, const int* text_ids, const int* codec_ids,
                                  const bf16* codec_embedding, int codec_vocabulary, bf16* hidden,
                                  int width, cudaStream_t stream);
// benchmark harness: seeded pseudo-random N(0,1) fills of a flat buffer / of whole KV pages
// (grid over `pages` page ids and `planes` = layers*2 K/V planes of every slab)
cudaError_t launch_fill_normal(bf16* dst, size_t count, unsigned long long seed, cudaStream_t stream);
// seeded pseudo-random int8 values uniform in [-127, 127]; dst 8-byte aligned
cudaError_t launch_fill_bytes(unsigned char* dst, size_t count, unsigned long long seed, cudaStream_t stream);
cudaError_t launch_fill_kv_pages(bf16* const* slabs, int slab_shift, long long page_elems,
                                 long long plane_elems, const int* page_ids, int pages, int planes,
                                 unsigned long long seed, cudaStream_t stream);
// position[0] += 1 (prompt rows advance one KV slot per step)
cudaError_t launch_advance_position(FrameTable* table, cudaStream_t stream);
// prompt positions base .. base + rows - 1 as rows of one pass (chunked prefill)
cudaError_t launch_prompt_rows(const int* text_ids, const int* codec_ids, int base, int rows,
                               const bf16* text_embedding, int text_vocabulary, bf16* text_in,
                               int* positions, int width, cudaStream_t stream);
cudaError_t launch_prompt_combine_rows(const int* text_ids, const int* codec_ids, int base, int rows,
                                       const bf16* codec_embedding, int codec_vocabulary, bf16* hidden,
                                       int width, cudaStream_t stream);

cudaError_t launch_pack_frame_codes_rows(const int* const* tokens, unsigned short* const* codes,
                                         int rows, cudaStream_t stream);

}  // namespace q3t
