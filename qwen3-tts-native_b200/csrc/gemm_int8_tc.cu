// Skinny int8 weight-only GEMM for 9..64 activation rows on the 5th-generation tensor cores.
//
// y[r][n] = epilogue( scale[n] * sum_k W[n][k] * x[r][k] ) like the SIMT kernels, but the weights
// are the UMMA "A" operand: a CTA owns 128 output channels (one TMEM lane each) and a slice of K,
// the sessions are the UMMA "N" dimension (16, 32 or 64 columns of fp32 accumulators in TMEM).
//
//   TMA (cp.async.bulk.tensor.2d)   int8 W tile 128 x 64  -> shared ring (8 stages)
//   TMA, 128-byte swizzle           bf16 x tile  MT x 64  -> shared, already in UMMA K-major layout
//   4 warps                         int8 -> bf16 in registers (exact; XOR + PRMT into the mantissa
//                                   of 2^23, packed subtract, PRMT of the high halves) -> shared,
//                                   128-byte-swizzled K-major A tile
//   1 thread                        tcgen05.mma.cta_group::1.kind::f16, 128 x MT x 16 per
//                                   instruction, accumulators in TMEM; tcgen05.commit frees stages
//   4 warps                         tcgen05.ld the accumulators, per-channel scale and the same
//                                   epilogues as the SIMT path
// K is split across CTAs so that every SM streams weights; the K-slices of a channel tile are
// summed in slice order by the CTA that takes the tile's last ticket (deterministic).
//
// The reference has no counterpart: its int8 path stops at 8 rows of SIMT FMAs
// (int8_gemv.cu:329) and its larger row counts go through cuBLAS bf16 GEMMs.
//
// Every wait is bounded by a wall-clock budget; a kernel that runs out records an error, lets
// its copies land, frees its TMEM columns and returns.

#include "q3t_kernels.cuh"

#include <cuda.h>

#include <mutex>

namespace q3t {
namespace {

constexpr int kTcThreads = 256;
constexpr int kTileN = 128;            // output channels per CTA = TMEM lanes
constexpr int kBK = 64;                // K elements per pipeline chunk
constexpr int kWStages = 8;            // int8 ring
constexpr int kAStages = 3;            // bf16 A / x ring
constexpr int kWStageBytes = kTileN * kBK;          // 8 KB
constexpr int kAStageBytes = kTileN * kBK * 2;      // 16 KB
constexpr unsigned long long kBudgetNs = 2000000000ull;   // 2 s for the whole kernel

__device__ unsigned int g_tc_errors = 0;

struct TcParams {
    const float* scales;
    bf16* y;
    float* y32;
    const bf16* bias;
    bf16* resid;
    float* partials;          // [tile][split][MT][128] fp32, only when splits > 1
    unsigned int* tickets;    // [tiles]
    int out_features;         // N (GATEUP: channels, the matrix has 2N rows)
    int rows;                 // valid sessions
    int epilogue;
    int splits;
    int chunks_per_split;     // K chunks of 64 per split
    int tiles;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Shared by all roles of a CTA: deadline and an abort flag that turns every later wait into a no-op.
struct Guard {
    unsigned long long deadline;
    volatile int* abort_flag;
    __device__ __forceinline__ bool wait(uint64_t* bar, uint32_t parity) const {
        while (!mbar_try_wait(bar, parity)) {
            if (*abort_flag) return false;
            if (now_ns() > deadline) {
                *abort_flag = 1;
                return false;
            }
        }
        return true;
    }
};

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

// K-major, 128-byte-swizzled operand tile: rows at a 128-byte pitch, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// four int8 (one word) -> four bf16 (two words), exact
__device__ __forceinline__ void dequant4(uint32_t word, uint32_t& lo, uint32_t& hi) {
    const uint32_t u = word ^ 0x80808080u;
    const unsigned long long bias = pack2(-8388736.0f, -8388736.0f);
    const unsigned long long a = add2(pack2(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)),
                                            __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651))), bias);
    const unsigned long long b = add2(pack2(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)),
                                            __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653))), bias);
    // a small integer as fp32 has a zero low half: its high half is the bf16 of the same value
    lo = __byte_perm(static_cast<uint32_t>(a), static_cast<uint32_t>(a >> 32), 0x7632);
    hi = __byte_perm(static_cast<uint32_t>(b), static_cast<uint32_t>(b >> 32), 0x7632);
}

__device__ __forceinline__ float finish(const TcParams& p, float acc, int channel, size_t o) {
    const float scale = p.scales[channel];
    switch (p.epilogue) {
        case EPI_ADD: return fmaf(acc, scale, bf2f(p.y[o]));
        case EPI_BIAS: return rbf(acc * scale) + bf2f(p.bias[channel]);
        case EPI_BIAS_SILU: {
            float v = rbf(acc * scale) + bf2f(p.bias[channel]);
            v *= 1.0f / (1.0f + expf(-v));
            return v;
        }
        case EPI_BIAS_ADD: return bf2f(p.resid[o]) + rbf(rbf(acc * scale) + bf2f(p.bias[channel]));
        default: return acc * scale;
    }
}

template <int MT>
__device__ __forceinline__ void tmem_load_row(uint32_t taddr, float (&v)[MT]) {
#pragma unroll
    for (int c = 0; c < MT; c += 16) {
        uint32_t r[16];
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(taddr + c));
#pragma unroll
        for (int i = 0; i < 16; ++i) v[c + i] = __uint_as_float(r[i]);
    }
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <int MT, bool GATEUP>
__global__ void __launch_bounds__(kTcThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap x_map,
               const TcParams p) {
    constexpr int kXStageBytes = MT * 128;
    constexpr uint32_t kTmemCols = MT < 32 ? 32 : MT;
    constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(MT >> 3) << 17)
                                | ((uint32_t)(kTileN >> 4) << 24);
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char* a16 = smem;
    unsigned char* xs = a16 + kAStages * kAStageBytes;
    unsigned char* w8 = xs + kAStages * kXStageBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(w8 + kWStages * kWStageBytes);
    uint64_t* full_w = bars;
    uint64_t* empty_w = full_w + kWStages;
    uint64_t* full_a = empty_w + kWStages;
    uint64_t* full_x = full_a + kAStages;
    uint64_t* empty_ax = full_x + kAStages;
    uint64_t* acc_done = empty_ax + kAStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_done + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* last_flag = const_cast<int*>(abort_flag) + 1;

    const int tid = threadIdx.x;
    const int warp = tid / kWarp;
    const int lane = tid % kWarp;
    const int tile = blockIdx.x % p.tiles;
    const int split = blockIdx.x / p.tiles;
    const int nk = p.chunks_per_split;
    const int k_first = split * nk * kBK;
    const int N = p.out_features;
    const int row_a = GATEUP ? tile * 64 : tile * kTileN;          // first W row of box 0
    const int row_b = GATEUP ? N + tile * 64 : tile * kTileN + 64;  // first W row of box 1

    Guard guard;
    guard.deadline = now_ns() + kBudgetNs;
    guard.abort_flag = abort_flag;

    if (tid == 0) {
        for (int s = 0; s < kWStages; ++s) {
            mbar_init(&full_w[s], 1);
            mbar_init(&empty_w[s], 4);
        }
        for (int s = 0; s < kAStages; ++s) {
            mbar_init(&full_a[s], 4);
            mbar_init(&full_x[s], 1);
            mbar_init(&empty_ax[s], 1);
        }
        mbar_init(acc_done, 1);
        *abort_flag = 0;
        *last_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 3) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---- weight producer --------------------------------------------------------------
        for (int i = 0; i < nk; ++i) {
            const int s = i % kWStages;
            if (i >= kWStages && !guard.wait(&empty_w[s], ((i / kWStages) - 1) & 1)) break;
            mbar_expect_tx(&full_w[s], kWStageBytes);
            unsigned char* dst = w8 + s * kWStageBytes;
            tma_load_2d(dst, &w_map, k_first + i * kBK, row_a, &full_w[s]);
            tma_load_2d(dst + kWStageBytes / 2, &w_map, k_first + i * kBK, row_b, &full_w[s]);
        }
    } else if (warp == 2 && lane == 0) {
        // ---- activation producer ----------------------------------------------------------
        for (int i = 0; i < nk; ++i) {
            const int sa = i % kAStages;
            if (i >= kAStages && !guard.wait(&empty_ax[sa], ((i / kAStages) - 1) & 1)) break;
            mbar_expect_tx(&full_x[sa], kXStageBytes);
            tma_load_2d(xs + sa * kXStageBytes, &x_map, k_first + i * kBK, 0, &full_x[sa]);
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer -------------------------------------------------------------------
        bool ok = true;
        for (int i = 0; i < nk && ok; ++i) {
            const int sa = i % kAStages;
            const uint32_t parity = (i / kAStages) & 1;
            ok = guard.wait(&full_a[sa], parity) && guard.wait(&full_x[sa], parity);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_addr = smem_u32(a16 + sa * kAStageBytes);
            const uint32_t b_addr = smem_u32(xs + sa * kXStageBytes);
#pragma unroll
            for (int j = 0; j < kBK / 16; ++j) {
                umma_f16(tmem_base, umma_desc(a_addr + 32 * j), umma_desc(b_addr + 32 * j), kIdesc,
                         (i | j) != 0 ? 1u : 0u);
            }
            umma_commit(&empty_ax[sa]);
        }
        umma_commit(acc_done);   // fires when every MMA issued above has completed
    } else if (warp >= 4) {
        // ---- dequantisers, then epilogue ----------------------------------------------------
        const int t = tid - 128;          // 0..127 = tile row = TMEM lane
        bool ok = true;
        for (int i = 0; i < nk && ok; ++i) {
            const int s = i % kWStages;
            const int sa = i % kAStages;
            // a wait that gives up does so for the whole warp: the warp-level sync below must be
            // reached by all 32 lanes or by none
            if (!__all_sync(0xffffffffu, guard.wait(&full_w[s], (i / kWStages) & 1))) { ok = false; break; }
            const unsigned char* src = w8 + s * kWStageBytes;
            uint32_t out[4][8];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                // 32 consecutive 16-byte chunks per warp: conflict-free reads
                const int chunk = q * 128 + t;
                const int4 raw = *reinterpret_cast<const int4*>(src + (size_t)chunk * 16);
                dequant4(static_cast<uint32_t>(raw.x), out[q][0], out[q][1]);
                dequant4(static_cast<uint32_t>(raw.y), out[q][2], out[q][3]);
                dequant4(static_cast<uint32_t>(raw.z), out[q][4], out[q][5]);
                dequant4(static_cast<uint32_t>(raw.w), out[q][6], out[q][7]);
            }
            if (i >= kAStages
                && !__all_sync(0xffffffffu, guard.wait(&empty_ax[sa], ((i / kAStages) - 1) & 1))) {
                ok = false;
                break;
            }
            unsigned char* dst = a16 + sa * kAStageBytes;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int chunk = q * 128 + t;
                const int row = chunk >> 2;
                const int c = chunk & 3;       // 16 int8 = bf16 chunks 2c and 2c+1 of the row
                unsigned char* rowp = dst + row * 128;
                *reinterpret_cast<int4*>(rowp + (((2 * c) ^ (row & 7)) << 4)) =
                    make_int4(out[q][0], out[q][1], out[q][2], out[q][3]);
                *reinterpret_cast<int4*>(rowp + (((2 * c + 1) ^ (row & 7)) << 4)) =
                    make_int4(out[q][4], out[q][5], out[q][6], out[q][7]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&full_a[sa]);
                mbar_arrive(&empty_w[s]);
            }
        }
        if (ok) ok = guard.wait(acc_done, 0);
        if (!ok) *abort_flag = 1;
        // all 128 epilogue threads meet here, so that they agree on whether the tile is complete
        // (the named barriers below must be reached by all of them or by none)
        epilogue_barrier();
        if (*abort_flag == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float v[MT];
            tmem_load_row<MT>(tmem_base + ((uint32_t)((warp - 4) * 32) << 16), v);
            const int channel = GATEUP ? tile * 64 + (t & 63) : tile * kTileN + t;
            if (p.splits == 1) {
                if (GATEUP) {
                    float* stage = reinterpret_cast<float*>(w8);   // the weight ring is drained
                    if (t >= 64) {
#pragma unroll
                        for (int s = 0; s < MT; ++s) stage[s * 64 + (t - 64)] = v[s];
                    }
                    epilogue_barrier();
                    if (t < 64 && channel < N) {
                        const float sg = p.scales[channel];
                        const float su = p.scales[N + channel];
#pragma unroll
                        for (int s = 0; s < MT; ++s) {
                            if (s < p.rows) {
                                const float gate = v[s] * sg;
                                const float up = stage[s * 64 + t] * su;
                                const float val = gate / (1.0f + expf(-gate)) * up;
                                const size_t o = (size_t)s * N + channel;
                                if (p.y32 != nullptr) p.y32[o] = val;
                                p.y[o] = f2bf(val);
                            }
                        }
                    }
                } else if (channel < N) {
#pragma unroll
                    for (int s = 0; s < MT; ++s) {
                        if (s < p.rows) {
                            const size_t o = (size_t)s * N + channel;
                            const float val = finish(p, v[s], channel, o);
                            if (p.y32 != nullptr) p.y32[o] = val;
                            if (p.epilogue == EPI_BIAS_ADD) p.resid[o] = f2bf(val);
                            else p.y[o] = f2bf(val);
                        }
                    }
                }
            } else {
                // ---- K was split: park the slice, the last CTA of the tile sums in slice order ----
                float* mine = p.partials + ((size_t)(tile * p.splits + split) * MT) * kTileN;
#pragma unroll
                for (int s = 0; s < MT; ++s) mine[s * kTileN + t] = v[s];
                __threadfence();
                epilogue_barrier();
                if (t == 0) {
                    const unsigned int ticket = atomicAdd(&p.tickets[tile], 1u);
                    *last_flag = ticket == static_cast<unsigned int>(p.splits - 1);
                }
                epilogue_barrier();
                if (*last_flag) {
                    __threadfence();
                    const float* base = p.partials + ((size_t)tile * p.splits * MT) * kTileN;
                    const bool active = GATEUP ? (t < 64 && channel < N) : channel < N;
                    if (active) {
                        for (int s = 0; s < p.rows; ++s) {
                            float acc = 0.0f, acc_up = 0.0f;
                            for (int sp = 0; sp < p.splits; ++sp) {
                                const float* slice = base + ((size_t)sp * MT + s) * kTileN;
                                acc += __ldcg(slice + t);
                                if (GATEUP) acc_up += __ldcg(slice + t + 64);
                            }
                            const size_t o = (size_t)s * N + channel;
                            float val;
                            if (GATEUP) {
                                const float gate = acc * p.scales[channel];
                                const float up = acc_up * p.scales[N + channel];
                                val = gate / (1.0f + expf(-gate)) * up;
                            } else {
                                val = finish(p, acc, channel, o);
                            }
                            if (p.y32 != nullptr) p.y32[o] = val;
                            if (!GATEUP && p.epilogue == EPI_BIAS_ADD) p.resid[o] = f2bf(val);
                            else p.y[o] = f2bf(val);
                        }
                    }
                    if (t == 0) p.tickets[tile] = 0u;
                }
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*abort_flag) {
        // give copies that are still in flight time to land before the CTA's memory is released
        if (tid == 0) atomicAdd(&g_tc_errors, 1u);
        const unsigned long long until = now_ns() + 200000ull;
        while (now_ns() < until) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 3) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------------- host side

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                 CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                 CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
    static EncodeTiled fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &result) != cudaSuccess
            || result != cudaDriverEntryPointSuccess) {
            p = nullptr;
        }
        return reinterpret_cast<EncodeTiled>(p);
    }();
    return fn;
}

bool make_map(CUtensorMap* map, CUtensorMapDataType type, const void* base, uint64_t inner, uint64_t outer,
              uint64_t row_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swizzle) {
    EncodeTiled fn = encode_tiled();
    if (fn == nullptr) return false;
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t elem[2] = {1, 1};
    return fn(map, type, 2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
              swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Per-device scratch of the tensor-core path: K-slice partials, tile tickets and a buffer for
// normalised activations.  Allocated once per device by configure_tc_kernels(); launches on one
// device that use it must be ordered (the engine issues them on one stream).
struct TcScratch {
    float* partials = nullptr;
    unsigned int* tickets = nullptr;
    bf16* normalized = nullptr;
    int sms = 148;
    bool ready = false;
};
constexpr size_t kPartialFloats = (size_t)512 * 64 * kTileN;     // up to 512 (tile, slice) pairs
constexpr int kTicketCount = 4096;
constexpr size_t kNormalizedElems = (size_t)kMaxRows * 8192;
TcScratch g_scratch[64];
std::mutex g_scratch_guard;

TcScratch* scratch_for_current_device() {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return nullptr;
    return g_scratch[device].ready ? &g_scratch[device] : nullptr;
}

template <int MT, bool GATEUP>
size_t tc_smem_bytes() {
    return 1024 + (size_t)kAStages * kAStageBytes + (size_t)kAStages * MT * 128
        + (size_t)kWStages * kWStageBytes + 26 * sizeof(uint64_t) + 64;
}

template <int MT, bool GATEUP>
cudaError_t configure_one() {
    return cudaFuncSetAttribute(gemm_tc_kernel<MT, GATEUP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(tc_smem_bytes<MT, GATEUP>()));
}

template <int MT, bool GATEUP>
cudaError_t launch_mt(const CUtensorMap& wm, const CUtensorMap& xm, const TcParams& p, cudaStream_t stream) {
    gemm_tc_kernel<MT, GATEUP>
        <<<p.tiles * p.splits, kTcThreads, tc_smem_bytes<MT, GATEUP>(), stream>>>(wm, xm, p);
    return cudaGetLastError();
}

int g_tc_min_rows = 9;

}  // namespace

void set_tc_min_rows(int rows) { g_tc_min_rows = rows < 2 ? 2 : rows; }
int tc_min_rows() { return g_tc_min_rows; }

cudaError_t configure_tc_kernels() {
    cudaError_t e = configure_one<16, false>();
    if (e == cudaSuccess) e = configure_one<16, true>();
    if (e == cudaSuccess) e = configure_one<32, false>();
    if (e == cudaSuccess) e = configure_one<32, true>();
    if (e == cudaSuccess) e = configure_one<64, false>();
    if (e == cudaSuccess) e = configure_one<64, true>();
    if (e != cudaSuccess) return e;
    int device = 0;
    e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_scratch_guard);
    TcScratch& s = g_scratch[device];
    if (s.ready) return cudaSuccess;
    e = cudaMalloc(&s.partials, kPartialFloats * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&s.tickets, kTicketCount * sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMemset(s.tickets, 0, kTicketCount * sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMalloc(&s.normalized, kNormalizedElems * sizeof(bf16));
    if (e != cudaSuccess) return e;
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) == cudaSuccess && sms > 0) s.sms = sms;
    s.ready = encode_tiled() != nullptr;
    return s.ready ? cudaSuccess : cudaErrorNotSupported;
}

bool gemm_tc_supports(const GemvArgs& a) {
    if (a.rows < g_tc_min_rows || a.rows > kMaxRows) return false;
    if (a.in_features % kBK != 0 || a.in_features > 8192) return false;
    if ((reinterpret_cast<uintptr_t>(a.w) & 15u) != 0 || (reinterpret_cast<uintptr_t>(a.x) & 15u) != 0) return false;
    return scratch_for_current_device() != nullptr;
}

cudaError_t launch_int8_gemm_tc(const GemvArgs& a, cudaStream_t stream) {
    TcScratch* scratch = scratch_for_current_device();
    if (scratch == nullptr || !gemm_tc_supports(a) || a.out_features < 1 || a.w == nullptr
        || a.scales == nullptr || a.x == nullptr) {
        return cudaErrorInvalidValue;
    }
    const bool gateup = a.epilogue == EPI_GATE_UP_SILU;
    if (a.epilogue == EPI_BIAS_ADD ? (a.resid == nullptr) : (a.y == nullptr)) return cudaErrorInvalidValue;
    if ((a.epilogue == EPI_BIAS || a.epilogue == EPI_BIAS_SILU || a.epilogue == EPI_BIAS_ADD)
        && a.bias == nullptr) {
        return cudaErrorInvalidValue;
    }
    const int K = a.in_features;
    const int N = a.out_features;
    const bf16* x = a.x;
    if (a.norm_w != nullptr) {
        // RMSNorm as its own launch here: at 9+ rows one more launch is noise, and every CTA of the
        // GEMM reads the normalised rows
        bf16* normalized = a.norm_out != nullptr ? a.norm_out : scratch->normalized;
        const cudaError_t e = launch_rms_norm_rows(a.x, a.norm_w, normalized, a.rows, K, a.eps, stream);
        if (e != cudaSuccess) return e;
        x = normalized;
    }
    const int mt = a.rows <= 16 ? 16 : (a.rows <= 32 ? 32 : 64);
    TcParams p;
    p.scales = a.scales; p.y = a.y; p.y32 = a.y32; p.bias = a.bias; p.resid = a.resid;
    p.partials = scratch->partials; p.tickets = scratch->tickets;
    p.out_features = N; p.rows = a.rows; p.epilogue = a.epilogue;
    p.tiles = gateup ? (N + 63) / 64 : (N + kTileN - 1) / kTileN;
    const int nk = K / kBK;
    int splits = 1;
    for (int s = 1; s <= nk; ++s) {
        if (nk % s == 0 && (long long)p.tiles * s <= scratch->sms) splits = s;
    }
    if ((size_t)p.tiles * splits * mt * kTileN > kPartialFloats || p.tiles > kTicketCount) splits = 1;
    p.splits = splits;
    p.chunks_per_split = nk / splits;

    alignas(64) CUtensorMap wm, xm;
    const uint64_t w_rows = gateup ? 2ull * N : (uint64_t)N;
    if (!make_map(&wm, CU_TENSOR_MAP_DATA_TYPE_UINT8, a.w, K, w_rows, K, kBK, 64, CU_TENSOR_MAP_SWIZZLE_NONE)
        || !make_map(&xm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, x, K, a.rows, (uint64_t)K * 2, kBK, mt,
                     CU_TENSOR_MAP_SWIZZLE_128B)) {
        return cudaErrorInvalidValue;
    }
    if (gateup) {
        switch (mt) {
            case 16: return launch_mt<16, true>(wm, xm, p, stream);
            case 32: return launch_mt<32, true>(wm, xm, p, stream);
            default: return launch_mt<64, true>(wm, xm, p, stream);
        }
    }
    switch (mt) {
        case 16: return launch_mt<16, false>(wm, xm, p, stream);
        case 32: return launch_mt<32, false>(wm, xm, p, stream);
        default: return launch_mt<64, false>(wm, xm, p, stream);
    }
}

unsigned int gemm_tc_error_count() {
    unsigned int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_errors, sizeof(v)) != cudaSuccess) return ~0u;
    return v;
}

}  // namespace q3t
