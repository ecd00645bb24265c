// Skinny int8 weight-only GEMM for 9..64 activation rows on the 5th-generation tensor cores.
//
// y[r][n] = epilogue( scale[n] * sum_k W[n][k] * x[r][k] ) like the SIMT kernels, but the weights
// are the UMMA "A" operand: a CTA owns 128 output channels (one TMEM lane each) and a slice of K,
// the sessions are the UMMA "N" dimension (16, 32 or 64 columns of fp32 accumulators in TMEM).
//
//   TMA, 128-byte swizzle           int8 W tile 128 x 128 -> shared ring (6 stages of 16 KB)
//   TMA, 128-byte swizzle           bf16 x tile MT x 128  -> shared ring (4 stages), UMMA K-major
//   2 x 4 warps, steps in turn      a thread owns a channel: 128 int8 of its row -> bf16 in
//                                   registers (exact: XOR, PRMT into the mantissa of 2^23, packed
//                                   subtract, PRMT of the high halves) -> tcgen05.st into the TMEM
//                                   columns of an A stage.  The dequantised weights never touch
//                                   shared memory, whose bandwidth bounds this kernel.
//   1 thread                        tcgen05.mma.cta_group::1.kind::f16 with A from TMEM and B
//                                   (activations) from shared memory, 128 x MT x 16 per
//                                   instruction; tcgen05.commit frees the stages
//   the same 8 warps                tcgen05.ld the accumulators, then the K-slice exchange below
//                                   and the same epilogues as the SIMT path
// K is split across the CTAs of a thread-block cluster (up to 8) so that every SM streams
// weights; each CTA pushes the rows of its slice into the shared memory of the CTA that owns
// them (distributed shared memory) and, after one cluster barrier, sums the rows it owns over
// all slices in slice order (deterministic).
//
// The reference has no counterpart: its int8 path stops at 8 rows of SIMT FMAs
// (int8_gemv.cu:329) and its larger row counts go through cuBLAS bf16 GEMMs.
//
// Every wait is bounded by a wall-clock budget; a kernel that runs out records an error, lets
// its copies land, frees its TMEM columns and returns.

#include "q3t_kernels.cuh"

#include <cuda.h>

#include <cstdlib>
#include <mutex>

namespace q3t {
namespace {

// Warp roles: 0 weight copies, 1 MMA issue, 2 activation copies, 3 TMEM allocation (one elected
// thread each); 4..7 and 8..11 are the two dequantiser groups.  Warp w may touch TMEM lanes
// 32 * (w % 4) .. + 31 only, so a dequantiser owns the channel (w % 4) * 32 + lane.
constexpr int kGroups = 2;
constexpr int kTcThreads = 128 + 128 * kGroups;
constexpr int kTileN = 128;            // output channels per CTA = TMEM lanes
constexpr int kBK = 128;               // K elements per pipeline step
constexpr int kWStages = 6;            // int8 ring in shared memory
constexpr int kXStages = 4;            // activation ring in shared memory (stage i pairs with A stage i)
constexpr int kAStages = 4;            // dequantised A stages in TMEM
constexpr int kWStageBytes = kTileN * kBK;          // 16 KB
static_assert(kXStages == kAStages, "activation stage i and TMEM A stage i share their barriers");
constexpr int kAStageCols = kBK / 2;   // 64 TMEM columns: two bf16 per 32-bit column
constexpr int kAccCols = 64;           // accumulators sit in columns [0, 64), A stages follow
constexpr uint32_t kTmemCols = 512;    // 64 + 4 * 64 rounded up to a power of two
constexpr int kRedBytes = 36 * 1024;   // K-slice exchange: up to 8 slices x ceil(64 / slices) rows x 128 fp32
constexpr unsigned long long kBudgetNs = 2000000000ull;   // 2 s for the whole kernel

__device__ unsigned int g_tc_errors = 0;

__device__ unsigned int* g_tc_error_sink = nullptr;   // host-mapped word of the engine, if any

struct TcParams {
    const float* scales;
    bf16* y;
    float* y32;
    const bf16* bias;
    bf16* resid;
    int out_features;         // N (GATEUP: channels, the matrix has 2N rows)
    int rows;                 // valid sessions
    int epilogue;
    int splits;               // K-slices per channel tile = CTAs per cluster
    int chunks;               // K chunks of 64 in the whole contraction
    int tiles;
    int residual_settled;     // GemvArgs::residual_settled
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

// One lane of a converged warp.  Unlike a test of the lane index, this tells the compiler that
// the code below runs in exactly one thread, which the instructions that take their operands
// from uniform registers (TMA copies, MMA issue) need in order to be emitted without a loop
// over the active lanes.
__device__ __forceinline__ bool elect_one() {
    uint32_t chosen;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(chosen));
    return chosen != 0;
}

// Shared by all roles of a CTA: deadline and an abort flag that turns every later wait into a no-op.
struct Guard {
    unsigned long long deadline;
    volatile int* abort_flag;
    __device__ __forceinline__ bool wait(uint64_t* bar, uint32_t parity) const {
        // the clock is read once per 1024 polls: a read of the global timer costs about as much
        // as a whole pipeline stage
        uint32_t polls = 0;
        while (!mbar_try_wait(bar, parity)) {
            if ((++polls & 63u) != 0) continue;
            if (*abort_flag) return false;
            if ((polls & 1023u) == 0 && now_ns() > deadline) {
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

// Hardware barrier over every thread of the cluster (one CTA per K-slice of a channel tile).
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// address of the same shared-memory location in the CTA of another rank of the cluster
__device__ __forceinline__ uint32_t peer_smem(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

// K-major, 128-byte-swizzled operand tile: rows at a 128-byte pitch, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

// A (128 x 16 bf16) from TMEM columns, B from shared memory
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}

// 32 consecutive columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_store_32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr),
          "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(smem_u32(bar)) : "memory");
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

__device__ __forceinline__ float finish(const TcParams& p, float acc, float scale, int channel, size_t o,
                                        bool have_base, float base) {
    switch (p.epilogue) {
        case EPI_ADD: return fmaf(acc, scale, have_base ? base : bf2f(p.y[o]));
        case EPI_BIAS: return rbf(acc * scale) + bf2f(p.bias[channel]);
        case EPI_BIAS_SILU: {
            float v = rbf(acc * scale) + bf2f(p.bias[channel]);
            return __fdividef(v, 1.0f + __expf(-v));
        }
        case EPI_BIAS_ADD: return (have_base ? base : bf2f(p.resid[o])) + rbf(rbf(acc * scale) + bf2f(p.bias[channel]));
        default: return acc * scale;
    }
}

// NCOL consecutive fp32 accumulator columns of this thread's TMEM lane
template <int NCOL>
__device__ __forceinline__ void tmem_load_row(uint32_t taddr, float (&v)[NCOL]) {
#pragma unroll
    for (int c = 0; c < NCOL; c += 8) {
        uint32_t r[8];
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
            : "r"(taddr + c));
#pragma unroll
        for (int i = 0; i < 8; ++i) v[c + i] = __uint_as_float(r[i]);
    }
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}


__device__ __forceinline__ void dequant_barrier() {
    asm volatile("bar.sync 1, %0;" ::"n"(128 * kGroups) : "memory");
}

template <int MT, bool GATEUP>
__global__ void __launch_bounds__(kTcThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap x_map,
               const TcParams p) {
    constexpr int kXAtomBytes = MT * 128;          // MT rows x 64 bf16, one 128-byte-swizzled atom
    constexpr int kXStageBytes = 2 * kXAtomBytes;  // 128 K elements per step
    // fp32 accumulate, A and B bf16 (format 1), both K-major
    constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(MT >> 3) << 17)
                                | ((uint32_t)(kTileN >> 4) << 24);
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char* w8 = smem;
    unsigned char* xs = w8 + kWStages * kWStageBytes;
    float* red = reinterpret_cast<float*>(xs + kXStages * kXStageBytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(red) + kRedBytes);
    uint64_t* full_w = bars;
    uint64_t* empty_w = full_w + kWStages;
    uint64_t* full_x = empty_w + kWStages;
    uint64_t* empty_x = full_x + kXStages;
    uint64_t* full_a = empty_x + kXStages;
    uint64_t* empty_a = full_a + kAStages;
    uint64_t* acc_done = empty_a + kAStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_done + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x;
    const int warp = __shfl_sync(0xffffffffu, tid / kWarp, 0);      // warp-uniform by construction
    const int lane = tid % kWarp;
    const int split = (int)cluster_rank();           // cluster = the K-slices of one channel tile
    const int tile = blockIdx.x / p.splits;
    const int step_first = p.chunks * split / p.splits;             // slices may differ by one step
    const int nk = p.chunks * (split + 1) / p.splits - step_first;
    const int k_first = step_first * kBK;
    const int N = p.out_features;
    const int rows_share = (MT + p.splits - 1) / p.splits;      // rows a CTA owns in the K-slice sum
    const int row_a = GATEUP ? tile * 64 : tile * kTileN;          // first W row of the tile
    const int row_b = N + tile * 64;                               // GATEUP: first row of the "up" half

    // the channel this thread finishes in the K-slice sum, and its scales: asked for now, so that
    // the (cold) loads are long back when the epilogue needs them
    constexpr int kPerRow = GATEUP ? 64 : kTileN;
    const int c = tid % kPerRow;                       // kTcThreads is a multiple of kPerRow
    const int channel = tile * kPerRow + c;
    float scale = 0.0f, scale_up = 0.0f;
    if (channel < N) {
        scale = p.scales[channel];
        if (GATEUP) scale_up = p.scales[N + channel];
    }
    Guard guard;
    guard.deadline = now_ns() + kBudgetNs;
    guard.abort_flag = abort_flag;

    if (tid == 0) {
        for (int s = 0; s < kWStages; ++s) {
            mbar_init(&full_w[s], 1);
            mbar_init(&empty_w[s], 4);
        }
        for (int s = 0; s < kXStages; ++s) {
            mbar_init(&full_x[s], 1);
            mbar_init(&empty_x[s], 1);
        }
        for (int s = 0; s < kAStages; ++s) {
            mbar_init(&full_a[s], 4 + 1);     // four dequantiser warps + the activation copy (bytes)
            mbar_init(&empty_a[s], 1);
        }
        mbar_init(acc_done, 1);
        *abort_flag = 0;
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
    // The weight copies (warp 0) start at once: weights never depend on the kernel before this
    // one.  Everyone else first waits for that kernel to complete (activations, residual), and
    // only then is the kernel after this one let in: every kernel of the library signals its
    // dependents after its own wait, so that a kernel may read, ahead of its wait, whatever was
    // written two or more launches upstream.
    // The dequantisers (warps 4..) touch only weights and tensor memory until the K-slice sum, so
    // they too run ahead and wait there.
    if (warp >= 1 && warp <= 3) {
        pdl_wait();
        if (warp == 1) pdl_trigger();
    }

    if (warp == 0) {
        if (elect_one()) {
            // ---- weight producer ----------------------------------------------------------
            for (int i = 0; i < nk; ++i) {
                const int s = i % kWStages;
                if (i >= kWStages && !guard.wait(&empty_w[s], ((i / kWStages) - 1) & 1)) break;
                mbar_expect_tx(&full_w[s], kWStageBytes);
                unsigned char* dst = w8 + s * kWStageBytes;
                if (GATEUP) {
                    tma_load_2d(dst, &w_map, k_first + i * kBK, row_a, &full_w[s]);
                    tma_load_2d(dst + kWStageBytes / 2, &w_map, k_first + i * kBK, row_b, &full_w[s]);
                } else {
                    tma_load_2d(dst, &w_map, k_first + i * kBK, row_a, &full_w[s]);
                }
            }
        }
    } else if (warp == 2) {
        if (elect_one()) {
            // ---- activation producer ------------------------------------------------------
            for (int i = 0; i < nk; ++i) {
                const int sx = i % kXStages;
                if (i >= kXStages && !guard.wait(&empty_a[sx], ((i / kXStages) - 1) & 1)) break;
                // the activation tile lands on the same barrier the dequantisers arrive on, so
                // that the MMA issuer has one thing to wait for per step
                mbar_expect_tx(&full_a[sx], kXStageBytes);
                unsigned char* dst = xs + sx * kXStageBytes;
                tma_load_2d(dst, &x_map, k_first + i * kBK, 0, &full_a[sx]);
                tma_load_2d(dst + kXAtomBytes, &x_map, k_first + i * kBK + 64, 0, &full_a[sx]);
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            // ---- MMA issuer ---------------------------------------------------------------
            for (int i = 0; i < nk; ++i) {
                const int sa = i % kAStages;
                const int sx = i % kXStages;
                bool ok = true;
                ok = ok && guard.wait(&full_a[sa], (i / kAStages) & 1);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_col = tmem_base + kAccCols + sa * kAStageCols;
                const uint32_t b_addr = smem_u32(xs + sx * kXStageBytes);
#pragma unroll
                for (int j = 0; j < kBK / 16; ++j) {
                    // 16 K elements = 8 TMEM columns of A, 32 bytes within a row of the B atom
                    umma_f16_ts(tmem_base, a_col + 8 * j,
                                umma_desc(b_addr + (j / 4) * kXAtomBytes + 32 * (j % 4)), kIdesc,
                                (i | j) != 0 ? 1u : 0u);
                }
                umma_commit(&empty_a[sa]);       // frees the TMEM stage and the activation stage
            }
            umma_commit(acc_done);   // fires when every MMA issued above has completed
        }
    } else if (warp >= 4) {
        // ---- dequantisers, then accumulator readers -----------------------------------------
        const int group = (warp - 4) / 4;            // steps group, group + kGroups, ...
        const int t = (warp % 4) * 32 + lane;        // channel within the tile = TMEM lane
        const uint32_t lane_base = tmem_base + ((uint32_t)((warp % 4) * 32) << 16);
        bool ok = true;
        for (int i = group; i < nk && ok; i += kGroups) {
            const int s = i % kWStages;
            const int sa = i % kAStages;
            // a wait that gives up does so for the whole warp: the warp-level syncs below must be
            // reached by all 32 lanes or by none
            if (!__all_sync(0xffffffffu, guard.wait(&full_w[s], (i / kWStages) & 1))) { ok = false; break; }
            // this thread's row: 128 bytes, whose 16-byte pieces sit at piece ^ (row & 7)
            const unsigned char* rowp = w8 + s * kWStageBytes + t * 128;
            int4 raw[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                raw[c] = *reinterpret_cast<const int4*>(rowp + ((c ^ (t & 7)) << 4));
            }
            if (i >= kAStages
                && !__all_sync(0xffffffffu, guard.wait(&empty_a[sa], ((i / kAStages) - 1) & 1))) {
                ok = false;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t out[32];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int4 v = raw[4 * h + c];
                    dequant4(static_cast<uint32_t>(v.x), out[8 * c + 0], out[8 * c + 1]);
                    dequant4(static_cast<uint32_t>(v.y), out[8 * c + 2], out[8 * c + 3]);
                    dequant4(static_cast<uint32_t>(v.z), out[8 * c + 4], out[8 * c + 5]);
                    dequant4(static_cast<uint32_t>(v.w), out[8 * c + 6], out[8 * c + 7]);
                }
                tmem_store_32(lane_base + kAccCols + sa * kAStageCols + 32 * h, out);
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&full_a[sa]);
                mbar_arrive(&empty_w[s]);
            }
        }
        if (ok) ok = guard.wait(acc_done, 0);
        if (!ok) *abort_flag = 1;
        // all accumulator readers meet here, so that they agree on whether the tile is complete
        dequant_barrier();
        if (*abort_flag == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // each group takes half of the accumulator columns (= activation rows); every row of
            // this K-slice goes to the shared memory of the CTA that owns the row
            constexpr int kCols = MT / kGroups;
            float v[kCols];
            tmem_load_row<kCols>(lane_base + group * kCols, v);
            if (p.splits == 1) {
                // nothing to exchange: park the rows in this CTA's own shared memory
#pragma unroll
                for (int j = 0; j < kCols; ++j) red[(group * kCols + j) * kTileN + t] = v[j];
            } else {
                const uint32_t slot0 = smem_u32(red) + (uint32_t)(split * rows_share * kTileN + t) * 4u;
                int owner = (group * kCols) / rows_share;            // one division, then counted up
                int within = group * kCols - owner * rows_share;
#pragma unroll
                for (int j = 0; j < kCols; ++j) {
                    if (group * kCols + j < p.rows) {
                        st_cluster(peer_smem(slot0 + (uint32_t)(within * kTileN) * 4u, (uint32_t)owner), v[j]);
                    }
                    if (++within == rows_share) {
                        within = 0;
                        ++owner;
                    }
                }
            }
        }
    }

    // ---- the K-slices of a channel tile live in the CTAs of one cluster; CTA s owns rows
    // [s * rows_share, (s + 1) * rows_share) and sums them over all slices in slice order ----------
    // The values a residual epilogue adds to, requested before the cluster barrier hides their
    // latency (and, when their writer is known to be long done, before the dependency wait).
    constexpr int kBasePre = 3;
    float base_pre[kBasePre];
    const bool base_wanted = !GATEUP && channel < N && (p.epilogue == EPI_ADD || p.epilogue == EPI_BIAS_ADD);
    const bf16* base_src = p.epilogue == EPI_ADD ? p.y : p.resid;
    auto fetch_bases = [&]() {
        const int row0 = split * rows_share;
        const int my_rows = min(rows_share, p.rows - row0);
#pragma unroll
        for (int u = 0; u < kBasePre; ++u) {
            const int j = tid / kPerRow + u * (kTcThreads / kPerRow);
            base_pre[u] = j < my_rows ? bf2f(base_src[(size_t)(row0 + j) * N + channel]) : 0.0f;
        }
    };
    if (base_wanted && p.residual_settled != 0) fetch_bases();
    if (warp == 0 || warp >= 4) pdl_wait();
    if (base_wanted && p.residual_settled == 0) fetch_bases();
    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    cluster_sync();       // the only cluster barrier: nothing remote is touched after it
    if (*abort_flag == 0 && channel < N) {
        const int row0 = split * rows_share;
        const int my_rows = min(rows_share, p.rows - row0);
        int u = 0;
#pragma unroll 2
        for (int j = tid / kPerRow; j < my_rows; j += kTcThreads / kPerRow, ++u) {
            const float* at = red + j * kTileN + c;
            float acc = at[0], acc_up = GATEUP ? at[64] : 0.0f;
            if (p.splits > 1) {
                float part[8], part_up[8];
#pragma unroll
                for (int sp = 1; sp < 8; ++sp) {
                    part[sp] = 0.0f;
                    part_up[sp] = 0.0f;
                    if (sp < p.splits) {
                        part[sp] = at[sp * rows_share * kTileN];
                        if (GATEUP) part_up[sp] = at[sp * rows_share * kTileN + 64];
                    }
                }
#pragma unroll
                for (int sp = 1; sp < 8; ++sp) {
                    acc += part[sp];
                    acc_up += part_up[sp];
                }
            }
            const size_t out = (size_t)(row0 + j) * N + channel;
            float val;
            if (GATEUP) {
                const float gate = acc * scale;
                const float up = acc_up * scale_up;
                // hardware exp2/reciprocal (good to about 2^-21); this path is compared at bf16 tolerance
                val = __fdividef(gate, 1.0f + __expf(-gate)) * up;
            } else {
                const float base = u == 0 ? base_pre[0] : (u == 1 ? base_pre[1] : base_pre[2]);
                val = finish(p, acc, scale, channel, out, base_wanted && u < kBasePre, base);
            }
            if (p.y32 != nullptr) p.y32[out] = val;
            if (!GATEUP && p.epilogue == EPI_BIAS_ADD) p.resid[out] = f2bf(val);
            else p.y[out] = f2bf(val);
        }
    }
    __syncthreads();
    if (*abort_flag) {
        // give copies that are still in flight time to land before the CTA's memory is released
        if (tid == 0) {
            atomicAdd(&g_tc_errors, 1u);
            if (g_tc_error_sink != nullptr) atomicAdd_system(g_tc_error_sink, 1u);
        }
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

// Per-device scratch of the tensor-core path: a buffer for normalised activations.  Allocated
// once per device by configure_tc_kernels(); launches on one device that use it must be ordered
// (the engine issues them on one stream).
struct TcScratch {
    bf16* normalized = nullptr;
    int sms = 148;
    // clusters of 1..8 CTAs that the device can hold at once, per kernel variant [MT index][GATEUP]
    int resident_clusters[3][2][9] = {};
    bool ready = false;
};
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
    return 1024 + (size_t)kWStages * kWStageBytes + (size_t)kXStages * MT * 256 + kRedBytes
        + (2 * kWStages + 2 * kAStages + 2 * kXStages + 1) * sizeof(uint64_t) + 64;
}

template <int MT, bool GATEUP>
cudaError_t configure_one(int (&resident)[9]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<MT, GATEUP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(tc_smem_bytes<MT, GATEUP>()));
    for (int size = 1; size <= 8 && e == cudaSuccess; ++size) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(size * 64), 1, 1);
        cfg.blockDim = dim3(kTcThreads, 1, 1);
        cfg.dynamicSmemBytes = tc_smem_bytes<MT, GATEUP>();
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)size;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int clusters = 0;
        e = cudaOccupancyMaxActiveClusters(&clusters, gemm_tc_kernel<MT, GATEUP>, &cfg);
        resident[size] = clusters;
    }
    return e;
}

template <int MT, bool GATEUP>
cudaError_t launch_mt(const CUtensorMap& wm, const CUtensorMap& xm, const TcParams& p, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(p.tiles * p.splits), 1, 1);
    cfg.blockDim = dim3(kTcThreads, 1, 1);
    cfg.dynamicSmemBytes = tc_smem_bytes<MT, GATEUP>();
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)p.splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, gemm_tc_kernel<MT, GATEUP>, wm, xm, p);
}

int g_tc_min_rows = 9;

}  // namespace

void set_tc_min_rows(int rows) { g_tc_min_rows = rows < 2 ? 2 : rows; }
int tc_min_rows() { return g_tc_min_rows; }

cudaError_t configure_tc_kernels() {
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_scratch_guard);
    TcScratch& s = g_scratch[device];
    if (s.ready) return cudaSuccess;
    e = configure_one<16, false>(s.resident_clusters[0][0]);
    if (e == cudaSuccess) e = configure_one<16, true>(s.resident_clusters[0][1]);
    if (e == cudaSuccess) e = configure_one<32, false>(s.resident_clusters[1][0]);
    if (e == cudaSuccess) e = configure_one<32, true>(s.resident_clusters[1][1]);
    if (e == cudaSuccess) e = configure_one<64, false>(s.resident_clusters[2][0]);
    if (e == cudaSuccess) e = configure_one<64, true>(s.resident_clusters[2][1]);
    if (e != cudaSuccess) return e;
    e = cudaMalloc(&s.normalized, kNormalizedElems * sizeof(bf16));
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
    p.out_features = N; p.rows = a.rows; p.epilogue = a.epilogue;
    p.tiles = gateup ? (N + 63) / 64 : (N + kTileN - 1) / kTileN;
    p.residual_settled = a.residual_settled ? 1 : 0;
    const int nk = K / kBK;
    // K-slices per tile = cluster size: as many as still let every cluster be resident at once (a
    // second wave would double the time); slices and row shares may be ragged
    const int (&resident)[9] = scratch->resident_clusters[mt == 16 ? 0 : (mt == 32 ? 1 : 2)][gateup ? 1 : 0];
    static const int split_cap = [] {
        const char* v = std::getenv("QWEN3_TTS_TC_MAX_SPLITS");
        const int n = v != nullptr ? std::atoi(v) : 8;
        return n < 1 ? 1 : (n > 8 ? 8 : n);
    }();
    int splits = 1;
    for (int s = 2; s <= split_cap && s <= nk; ++s) {
        if (p.tiles <= resident[s]) splits = s;
    }
    p.splits = splits;
    p.chunks = nk;

    alignas(64) CUtensorMap wm, xm;
    const uint64_t w_rows = gateup ? 2ull * N : (uint64_t)N;
    if (!make_map(&wm, CU_TENSOR_MAP_DATA_TYPE_UINT8, a.w, K, w_rows, K, kBK, gateup ? 64 : kTileN,
                  CU_TENSOR_MAP_SWIZZLE_128B)
        || !make_map(&xm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, x, K, a.rows, (uint64_t)K * 2, 64, mt,
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

cudaError_t set_tc_error_sink(unsigned int* device_visible_word) {
    return cudaMemcpyToSymbol(g_tc_error_sink, &device_visible_word, sizeof(device_visible_word));
}

}  // namespace q3t
