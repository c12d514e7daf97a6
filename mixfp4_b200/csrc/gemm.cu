// Prefill-shape dequant-linear on the Blackwell tensor cores:
//   y[M,N] = x[M,K] * W[N,K]^T,  x bf16, W packed mixed-FP4, fp32 accumulation in TMEM.
// Replaces F.linear on the dequantized weight (project_quant/modeling.py:629) and, with
// rotation_block = 128, the activation pre-hook (modeling.py:662-668).
//
// Tile: one CTA computes (1 or 2) x 128 rows of x by 128 or 256 weight rows, K in steps of 64;
// with two 128-row sub-tiles the transcoded weight tile feeds two accumulators, which
// halves the transcode work per flop.  Warp roles (figures for the 128 x 128 tile):
//   warp 0      TMA producer: one lane issues cp.async.bulk.tensor.2d loads of the x tile
//               (128 rows x 64 bf16, 128-byte swizzle) into a 6-stage shared-memory ring.
//   warp 1      MMA issuer: allocates 128 TMEM columns, then one lane issues four
//               tcgen05.mma.cta_group::1.kind::f16 (128x128x16, bf16 x bf16 -> fp32) per
//               stage and commits the stage's "empty" barrier; after the last K step it
//               commits the accumulator barrier.
//   warps 2-9   weight transcoders, then epilogue.  Each thread owns half a row of the
//               128 x 64 weight tile (a whole row of a 256-row tile): it reads 16 or 32 B of
//               codes from the shared-memory code ring one K step ahead, takes its scale bytes (8 B per row and two K steps)
//               straight from global memory, decodes with the shared (format, scale) ->
//               bf16 table into exactly the reference's dequantized bf16 values and writes
//               them into the K-major 128B-swizzled operand layout tcgen05 reads
//               (conflict-free 16-byte stores), fences the async proxy and arrives on the
//               stage's "full" barrier.  At the end the same warps read the accumulator
//               with tcgen05.ld and store y.
//   warp 10     TMA producer of the packed codes: a box of 32 bytes x tile rows per K step
//               into its own ring (a per-thread global load of a row's 32 bytes touches 32
//               lines per warp and made the load/store pipe the limiter).
// Every mbarrier wait is bounded (wall-clock limit); on expiry the kernel records a code
// in the caller's status word, stops issuing work, waits for its own TMA loads, frees
// TMEM and returns.
//
// Tensor-pipe roofline: 2*M*N*K flops against the measured dense bf16 peak.  The weight
// tile is transcoded once per CTA, i.e. N*K elements are decoded M/128 times over.
//
// Large problems run gemm_pair_kernel (further down): two CTAs of a cluster share each
// decoded weight tile through tcgen05.mma.cta_group::2.

#include <cuda.h>
#include <stdio.h>
#include <stdlib.h>

#include <mutex>

#include "common.cuh"
#include "decode.cuh"

namespace mixfp4 {
namespace {

constexpr int BK = 64;                     // K elements per pipeline stage (one 128-byte swizzle row)
constexpr int kDecodeWarps = 8;             // more transcoder warps were measured: no gain alone, a loss in CTA pairs
constexpr int kThreads = (3 + kDecodeWarps) * 32;   // x producer, MMA issuer, transcoders, code producer
constexpr uint64_t kWaitLimitNs = 2000000000ull;   // 2 s: far beyond any legitimate wait
constexpr uint32_t kMinSpins = 1u << 16;            // ... and at least this many polls

// Tile configuration: kMT sub-tiles of 128 rows of x (each its own TMEM accumulator, all
// sharing the transcoded weight tile) by kBN weight rows.
template <int kMT, int kBN>
struct Cfg {
    static constexpr int BM = 128 * kMT, BN = kBN;
    static constexpr uint32_t kABytes = BM * BK * 2, kBBytes = BN * BK * 2;
    static constexpr uint32_t kStageBytes = kABytes + kBBytes;
    static constexpr int kStages = (196608 / kStageBytes) < 6 ? (196608 / kStageBytes) : 6;
    static constexpr uint32_t kTmemCols = kMT * kBN;            // 128, 256 or 512: powers of two
    // shared-memory map (offsets from a 1024-aligned base)
    static constexpr uint32_t kOffA = 0;
    static constexpr uint32_t kOffB = kStages * kABytes;
    static constexpr uint32_t kOffLut = kOffB + kStages * kBBytes;
    // ring of packed code tiles (kBN rows x 32 bytes per K step), filled by TMA
    static constexpr uint32_t kWBytes = BN * (BK / 2);
    static constexpr int kWStages = 24576 / kWBytes;            // 3 (256 rows) or 6 (128 rows)
    static constexpr uint32_t kOffW = kOffLut + 4096;
    static constexpr uint32_t kOffBar = kOffW + kWStages * kWBytes;   // full_a[S] full_b[S] empty[S] accum full_w[WS] empty_w[WS]
    static constexpr uint32_t kOffMisc = kOffBar + (3 * kStages + 1 + 2 * kWStages) * 8;   // tmem base, abort flag
    static constexpr uint32_t kSmemBytes = kOffMisc + 16 + 1024;   // + alignment slack
    // tcgen05 instruction descriptor, kind::f16: D fp32 (bits 4-5 = 1), A and B bf16 (bits 7-9
    // and 10-12 = 1), both K-major (bits 15, 16 = 0), N >> 3 at bits 17-22, M >> 4 at bits 24-28.
    static constexpr uint32_t kInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kBN >> 3) << 17) |
                                           ((uint32_t)(128 >> 4) << 24);
    // transcoders: 256 threads over kBN rows
    static constexpr int kThreadsPerRow = kDecodeWarps * 32 / kBN;   // 2 or 1
    static constexpr int kWords = 8 / kThreadsPerRow;           // 32-bit code words per thread and K step: 4 or 8
};

struct GemmArgs {
    const uint8_t* codes;
    const uint8_t* scales;
    const uint8_t* fmt;
    const float* global_scale;
    const uint4* lut;           // optional prebuilt decode table
    int64_t m, n, k, kpad;
    void* y;
    int out_dtype;
    int64_t ldy;
    int* status;
    int tma_store;              // pair kernel: epilogue through shared memory and TMA stores
    int kt_per_split;           // K steps per CTA along grid.z (all of them without split K)
    float* partial;             // split K: fp32 partial sums [splits][m][ld_partial]
    int64_t ld_partial;
    int stream_layout;          // `codes` is the chunk buffer of the stream layout (decode.cuh), `scales` unused
    int subs;                   // chunks per row tile (kpad / 128)
};

// Sum of the split-K partials in split order (deterministic), converted to the output type.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ partial, int splits, int64_t m,
                                                            int64_t n, int64_t ld_partial, void* __restrict__ y,
                                                            int out_dtype, int64_t ldy) {
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= m * n) return;
    const int64_t r = i / n, c = i - r * n;
    float sum = partial[r * ld_partial + c];
    for (int z = 1; z < splits; ++z) sum += partial[((int64_t)z * m + r) * ld_partial + c];
    if (out_dtype == MIXFP4_F32) static_cast<float*>(y)[r * ldy + c] = sum;
    else static_cast<__nv_bfloat16*>(y)[r * ldy + c] = __float2bfloat16_rn(sum);
}

// ------------------------------------------------------------------------- PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

struct WaitCtx {
    volatile int* abort_flag;   // shared memory
    int* status;                // global, may be null
};

// Bounded wait: false if the limit expired or another thread of the CTA already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtx& ctx, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 63u) == 0) {
            if (*ctx.abort_flag) return false;
            // both a long time and many polls: a discontinuity of the timer alone never aborts a wait
            if (spins > kMinSpins && global_timer_ns() - t0 > kWaitLimitNs) {
                *ctx.abort_flag = 1;
                if (ctx.status) atomicCAS(ctx.status, 0, code);
                return false;
            }
        }
    }
    return true;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}

// Box of the stream layout's code bytes: coordinates (byte in a row's 64, row in the tile, chunk along K, row tile).
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2,
                                            int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc], bf16 inputs, fp32 accumulate.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// mbarrier arrive once all previously issued tcgen05.mma of this thread have completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 TMEM lanes x 32 columns of 32-bit: thread i of the warp gets lane base+i, columns c..c+31.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major bf16 tile with 128-byte swizzle: rows are
// 128 B apart inside an 8-row group, groups 1024 B apart (stride byte offset), descriptor
// version 1 (sm_100), layout type 2 (SWIZZLE_128B).  The tile base must be 1024-aligned;
// a K step of 16 elements advances the start address by 32 B.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
    const uint64_t lo = ((saddr & 0x3ffffu) >> 4) | (1ull << 16);
    const uint64_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
    return lo | (hi << 32);
}

__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint4 lds128_lut(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// Epilogue of one CTA: the transcoder warps read the accumulators from TMEM (lane quarter =
// warp % 4, a hardware rule; columns split between the warp groups) and store y.
template <int kMT, int kBN>
__device__ __forceinline__ void store_accumulators(const GemmArgs& a, uint32_t tmem_base, uint32_t m0, uint32_t n0,
                                                   int warp, int lane) {
    tcgen05_fence_after();
    constexpr int kColGroups = kDecodeWarps / 4;                 // warp groups that split the tile's columns
    const int q = warp & 3, ch = (warp - 2) >> 2;
    constexpr int kChunks = kBN / (32 * kColGroups);             // 32-column chunks per warp and sub-tile
#pragma unroll 1
    for (int it = 0; it < kMT * kChunks; ++it) {
        const int mt = it / kChunks, c = it % kChunks;
        const int64_t mrow = (int64_t)m0 + mt * 128 + q * 32 + lane;
        const int col0 = ch * (kBN / kColGroups) + c * 32;
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(mt * kBN + col0), r);
        const int64_t ncol = (int64_t)n0 + col0;
        if (mrow < a.m && ncol < a.n) {
            const bool full = ncol + 32 <= a.n;
            if (a.out_dtype == MIXFP4_F32) {
                float* out = static_cast<float*>(a.y) + mrow * a.ldy + ncol;
                if (full && (a.ldy & 3) == 0 && (reinterpret_cast<uintptr_t>(a.y) & 15) == 0) {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        reinterpret_cast<uint4*>(out)[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (ncol + j < a.n) out[j] = __uint_as_float(r[j]);
                }
            } else {
                __nv_bfloat16* out = static_cast<__nv_bfloat16*>(a.y) + mrow * a.ldy + ncol;
                uint32_t pk[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
                    pk[j] = *reinterpret_cast<const uint32_t*>(&v);
                }
                if (full && (a.ldy & 7) == 0 && (reinterpret_cast<uintptr_t>(a.y) & 15) == 0) {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        reinterpret_cast<uint4*>(out)[j] = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (ncol + j < a.n)
                            out[j] = __ushort_as_bfloat16((unsigned short)((pk[j >> 1] >> (16 * (j & 1))) & 0xffffu));
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------ kernel
template <int kMT, int kBN, bool kKL>
__global__ void __launch_bounds__(kThreads, 1) gemm_kernel(const __grid_constant__ CUtensorMap tmap_x,
                                                           const __grid_constant__ CUtensorMap tmap_w,
                                                           const GemmArgs a) {
    using C = Cfg<kMT, kBN>;
    constexpr int kStages = C::kStages, kWStages = C::kWStages;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (base - raw);            // generic pointer to the aligned base

    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;   // provably warp-uniform
    const uint32_t n0 = blockIdx.x * C::BN, m0 = blockIdx.y * C::BM;
    // split K: grid.z CTAs share an output tile, each takes a run of K steps (an even number, so
    // scale pairs and format bytes stay aligned) and stores fp32 partial sums
    const int total_kt = static_cast<int>(a.kpad / BK);
    const int kt0 = blockIdx.z * a.kt_per_split;
    const int num_kt = min(a.kt_per_split, total_kt - kt0);

    auto full_a = [&](int s) { return base + C::kOffBar + 8u * s; };
    auto full_b = [&](int s) { return base + C::kOffBar + 8u * (kStages + s); };
    auto empty = [&](int s) { return base + C::kOffBar + 8u * (2 * kStages + s); };
    const uint32_t accum_bar = base + C::kOffBar + 8u * (3 * kStages);
    auto full_w = [&](int s) { return base + C::kOffBar + 8u * (3 * kStages + 1 + s); };
    auto empty_w = [&](int s) { return base + C::kOffBar + 8u * (3 * kStages + 1 + kWStages + s); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + C::kOffMisc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + C::kOffMisc + 4);
    const WaitCtx ctx{abort_flag, a.status};

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_a(s), 1);
            mbar_init(full_b(s), kDecodeWarps);
            mbar_init(empty(s), 1);
        }
        mbar_init(accum_bar, 1);
        for (int s = 0; s < kWStages; ++s) {
            mbar_init(full_w(s), 1);
            mbar_init(empty_w(s), kDecodeWarps);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_proxy();
    }
    if (warp == 1) tmem_alloc(base + C::kOffMisc, C::kTmemCols);
    if (warp >= 2 && warp < 2 + 8) {   // the (format, scale) -> magnitudes table: 256 entries, one thread each
        const int e = threadIdx.x - 64;
        reinterpret_cast<uint4*>(gen + C::kOffLut)[e] =
            a.lut ? __ldg(a.lut + e) : make_lut_entry(e & 127, e >> 7, *a.global_scale);
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            // x may come from the kernel launched just before (see launch_gemm's after_producer)
            asm volatile("griddepcontrol.wait;" ::: "memory");
            asm volatile("fence.proxy.async.global;" ::: "memory");
            int issued = 0;
            for (int kt = 0; kt < num_kt; ++kt) {
                const int s = kt % kStages;
                const uint32_t ph = (kt / kStages) & 1;
                if (!mbar_wait(empty(s), ph ^ 1, ctx, 1)) break;
                mbar_arrive_expect_tx(full_a(s), C::kABytes);
                tma_load_2d(base + C::kOffA + s * C::kABytes, &tmap_x, full_a(s), (kt0 + kt) * BK, (int)m0);
                issued = kt + 1;
            }
            // never leave with a bulk copy still writing into this CTA's shared memory
            for (int kt = max(0, issued - kStages); kt < issued; ++kt)
                if (!mbar_wait(full_a(kt % kStages), (kt / kStages) & 1, ctx, 2)) break;
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            bool ok = true;
            for (int kt = 0; kt < num_kt && ok; ++kt) {
                const int s = kt % kStages;
                const uint32_t ph = (kt / kStages) & 1;
                ok = mbar_wait(full_a(s), ph, ctx, 3) && mbar_wait(full_b(s), ph, ctx, 4);
                if (!ok) break;
                tcgen05_fence_after();
                const uint64_t db = make_smem_desc(base + C::kOffB + s * C::kBBytes);
#pragma unroll
                for (int mt = 0; mt < kMT; ++mt) {     // 128-row sub-tile mt starts 16 KB further
                    const uint64_t da = make_smem_desc(base + C::kOffA + s * C::kABytes + mt * 16384u);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)  // +32 B per K step of 16: +2 in the address field
                        umma_bf16(tmem_base + mt * kBN, da + 2u * k, db + 2u * k, C::kInstrDesc,
                                  (kt | k) != 0 ? 1u : 0u);
                }
                umma_commit(empty(s));                  // frees the stage when these MMAs are done
            }
            if (ok) umma_commit(accum_bar);
        }
    } else if (warp == 2 + kDecodeWarps) {
        // ------------------------------------------------- TMA producer of the code tiles
        if (lane == 0) {
            int issued = 0;
            for (int kt = 0; kt < num_kt; ++kt) {
                const int s = kt % kWStages;
                const uint32_t ph = (kt / kWStages) & 1;
                if (!mbar_wait(empty_w(s), ph ^ 1, ctx, 7)) break;
                mbar_arrive_expect_tx(full_w(s), C::kWBytes);
                if (a.stream_layout)
                    tma_load_4d(base + C::kOffW + s * C::kWBytes, &tmap_w, full_w(s), ((kt0 + kt) & 1) * (BK / 2), 0,
                                (kt0 + kt) >> 1, (int)(n0 >> 4));
                else
                    tma_load_2d(base + C::kOffW + s * C::kWBytes, &tmap_w, full_w(s), (kt0 + kt) * (BK / 2), (int)n0);
                issued = kt + 1;
            }
            for (int kt = max(0, issued - kWStages); kt < issued; ++kt)
                if (!mbar_wait(full_w(kt % kWStages), (kt / kWStages) & 1, ctx, 8)) break;
        }
    } else {
        // -------------------------------------------------- weight transcoders / epilogue
        constexpr int kWords = C::kWords, kBlocks = kWords / 2;
        // The threads of a row are neighbouring lanes, so a warp reads whole 32-byte code rows
        // (conflict-free) and its 16-byte stores into the swizzled tile never share a bank.
        constexpr int kTPR = C::kThreadsPerRow;
        const int dt = threadIdx.x - 64;                // transcoder thread index
        const int row = dt / kTPR, part = dt % kTPR;    // tile row, which part of the K step
        const uint32_t last_row = (uint32_t)a.n - 1;
        const uint32_t grow = min(n0 + row, last_row);  // rows past N re-read the last row; never stored
        // a row's 8 scale bytes per 128 K elements: 8 bytes apart in a scale row, one chunk apart in the stream layout
        const uint8_t* srow = a.stream_layout
            ? a.codes + (size_t)(grow >> 4) * a.subs * kChunkBytes + kChunkCodeBytes + (grow & 15) * 8
            : a.scales + (size_t)grow * (a.kpad / 16);
        const size_t sstep = a.stream_layout ? kChunkBytes : 8;
        const uint8_t* fptr = kKL ? a.scales : a.fmt + (size_t)grow * (a.kpad / 128);   // unused for the kernel layout
        const uint32_t lut_base = base + C::kOffLut;
        // destination of this thread's 16-byte chunks: row r, logical chunk c -> c ^ (r & 7)
        const uint32_t row_off = (row >> 3) * 1024u + (row & 7) * 128u;
        const uint32_t sw = row & 7;

        // The code tile of a K step is in shared memory (32 bytes per row, rows past N zero-filled
        // by TMA).
        auto load_codes = [&](uint32_t (&w)[kWords], int kt) -> bool {
            const int ws = kt % kWStages;
            if (!__all_sync(0xffffffffu, mbar_wait(full_w(ws), (kt / kWStages) & 1, ctx, 9))) return false;
            const uint32_t src = base + C::kOffW + ws * C::kWBytes + row * 32 + part * (kWords * 4);
            if constexpr (kWords == 8) {   // one thread per row: read the halves in an order that spreads the banks
                const uint32_t c0 = (lane >> 2) & 1;
                const uint4 va = lds128_lut(src + c0 * 16), vb = lds128_lut(src + (c0 ^ 1) * 16);
                const uint4 lo = c0 ? vb : va, hi = c0 ? va : vb;
                w[0] = lo.x; w[1] = lo.y; w[2] = lo.z; w[3] = lo.w;
                w[4] = hi.x; w[5] = hi.y; w[6] = hi.z; w[7] = hi.w;
            } else if constexpr (kWords == 4) {
                const uint4 v = lds128_lut(src);
                w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
            } else {
                asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(w[0]), "=r"(w[1]) : "r"(src));
            }
            __syncwarp();                               // every lane has read: the stage may be refilled
            if (lane == 0) mbar_arrive(empty_w(ws));
            return true;
        };
        // Scales: 8 bytes of a row cover two K steps.
        auto load_scale_pair = [&](int pair) -> uint2 {
            return __ldg(reinterpret_cast<const uint2*>(srow + (size_t)pair * sstep));
        };

        uint32_t codes[kWords], ncodes[kWords];
        bool ok = load_codes(codes, 0);
        // scale pairs are fetched two pairs (four K steps) ahead: a global load takes longer than two steps
        uint2 sc2 = load_scale_pair(kt0 >> 1), nsc2 = num_kt > 2 ? load_scale_pair((kt0 >> 1) + 1) : sc2, nnsc2 = nsc2;
        uint32_t fb = kKL ? 0u : __ldg(fptr + (kt0 >> 1));
        for (int kt = 0; kt < num_kt && ok; ++kt) {
            const int s = kt % kStages;
            const uint32_t ph = (kt / kStages) & 1;
            uint32_t nfb = fb;
            if (kt + 1 < num_kt) {                      // next K step's packed data, one step ahead
                ok = load_codes(ncodes, kt + 1);
                if (!ok) break;
                if ((kt & 1) == 0 && kt + 4 < num_kt) nnsc2 = load_scale_pair(((kt0 + kt) >> 1) + 2);
                if constexpr (!kKL) nfb = __ldg(fptr + ((kt0 + kt + 1) >> 1));
            }
            const uint32_t scs = ((kt & 1) ? sc2.y : sc2.x) >> (8 * part * kBlocks);
            ok = __all_sync(0xffffffffu, mbar_wait(empty(s), ph ^ 1, ctx, 5));   // warp-uniform: lanes stay together
            if (!ok) break;
            const uint32_t dst = base + C::kOffB + s * C::kBBytes + row_off;
            const uint32_t fbits = fb >> ((kt & 1) * 4 + part * kBlocks);     // this thread's blocks
#pragma unroll
            for (int b = 0; b < kBlocks; ++b) {
                const uint32_t idx = kKL ? ((scs >> (8 * b)) & 0xffu)
                                         : ((((fbits >> b) & 1u) << 7) | ((scs >> (8 * b)) & 0x7fu));
                const uint4 tab = lds128_lut(lut_base + idx * 16);
#pragma unroll
                for (int w = 0; w < 2; ++w) {
                    const int i = 2 * b + w;
                    uint32_t p[4];
                    decode_word<kKL>(codes[i], tab, p);
                    const uint32_t chunk = (uint32_t)(part * kWords + i) ^ sw;
                    sts128(dst + chunk * 16, p[0], p[1], p[2], p[3]);
                }
            }
            fence_async_proxy();                        // generic-proxy stores -> visible to tcgen05
            __syncwarp();
            if (lane == 0) mbar_arrive(full_b(s));
#pragma unroll
            for (int i = 0; i < kWords; ++i) codes[i] = ncodes[i];
            if (kt & 1) { sc2 = nsc2; nsc2 = nnsc2; }
            fb = nfb;
        }

        if (ok && mbar_wait(accum_bar, 0, ctx, 6)) {
            if (gridDim.z == 1) {
                store_accumulators<kMT, kBN>(a, tmem_base, m0, n0, warp, lane);
            } else {                     // this split's partial sums, fp32 [m, ld_partial]
                GemmArgs p = a;
                p.y = a.partial + (size_t)blockIdx.z * a.m * a.ld_partial;
                p.out_dtype = MIXFP4_F32;
                p.ldy = a.ld_partial;
                store_accumulators<kMT, kBN>(p, tmem_base, m0, n0, warp, lane);
            }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

// Epilogue through shared memory and TMA stores (bf16 output with 16-byte aligned rows): every
// lane owns one accumulator row, so direct stores touch 32 different lines per instruction and
// cost about a tenth of a tile's time.  Here the warps write their bf16 values into boxes of
// 128 rows x 64 columns in the 128-byte swizzle (conflict-free), and one thread hands the boxes
// to the TMA unit, which also clips them at the edges of y.  `stage` is operand memory that is
// free once the accumulator barrier has completed (1024-byte aligned, kMT * kBN / 64 * 16 KB).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(c0), "r"(c1) : "memory");
}
// AND over the epilogue warps (named barrier 1): they take the shared-memory epilogue together or not at all.
__device__ __forceinline__ bool epilogue_warps_all(bool pred) {
    uint32_t out;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 q, %1, 0;\n\t"
        "bar.red.and.pred p, 1, %2, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(out)
        : "r"((uint32_t)pred), "n"(kDecodeWarps * 32)
        : "memory");
    return out != 0;
}
template <int kMT, int kBN>
__device__ __forceinline__ void store_accumulators_tma(const GemmArgs& a, const CUtensorMap* tmap_y, uint32_t stage,
                                                       uint32_t tmem_base, uint32_t m0, uint32_t n0, int warp, int lane) {
    tcgen05_fence_after();
    constexpr int kColGroups = kDecodeWarps / 4;
    const int q = warp & 3, ch = (warp - 2) >> 2;
    constexpr int kChunks = kBN / (32 * kColGroups);
    constexpr int kBoxesPerSub = kBN / 64;
    const uint32_t row = q * 32 + lane;                       // row inside a 128-row box
#pragma unroll 1
    for (int it = 0; it < kMT * kChunks; ++it) {
        const int mt = it / kChunks, c = it % kChunks;
        const int col0 = ch * (kBN / kColGroups) + c * 32;
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(mt * kBN + col0), r);
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
            pk[j] = *reinterpret_cast<const uint32_t*>(&v);
        }
        const uint32_t box = stage + (uint32_t)(mt * kBoxesPerSub + col0 / 64) * 16384u + row * 128u;
        const uint32_t chunk0 = (uint32_t)(col0 % 64) / 8;
#pragma unroll
        for (int j = 0; j < 4; ++j)
            sts128(box + (((chunk0 + j) ^ (row & 7u)) * 16u), pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
    }
    fence_async_proxy();
    asm volatile("bar.sync 1, %0;" ::"n"(kDecodeWarps * 32) : "memory");      // the epilogue warps only
    if (warp == 2 && lane == 0) {
#pragma unroll
        for (int mt = 0; mt < kMT; ++mt) {
#pragma unroll
            for (int bx = 0; bx < kBoxesPerSub; ++bx) {
                const int64_t r0 = (int64_t)m0 + mt * 128, c0 = (int64_t)n0 + bx * 64;
                if (r0 < a.m && c0 < a.n)
                    tma_store_2d(tmap_y, stage + (uint32_t)(mt * kBoxesPerSub + bx) * 16384u, (int)c0, (int)r0);
            }
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");    // the boxes are read before the CTA leaves
    }
}

// ------------------------------------------------------------------- CTA-pair kernel
// The single-CTA kernel above is bound by the shared-memory data path: per K step the
// transcoders store and the tensor core re-reads the whole decoded 256-row weight tile, once
// per 128-row accumulator.  Here two CTAs of a cluster share one weight tile of 256 rows:
// each decodes only its own 128 rows, and one tcgen05.mma.cta_group::2 (M = 256: 128 token
// rows from each CTA, N = 256: 128 weight rows from each CTA's shared memory) feeds both
// SMs' tensor cores, so each CTA stores half as much and the hardware reads every half once.
// The even CTA of the pair (the leader) issues all MMAs; its "full" barriers collect the TMA
// bytes and the transcoder arrivals of both CTAs, and its commits release the stages of both
// CTAs (tcgen05.commit with a cluster multicast mask).  No TMA load is multicast.
constexpr uint32_t kPeerMask = 0xFEFFFFFFu;          // clears the CTA-rank bit of a shared::cluster address

template <int kMT>
struct PairCfg {
    static constexpr int BM = 128 * kMT;             // token rows per CTA
    static constexpr int BN = 256, BNH = 128;        // weight rows per pair / per CTA
    static constexpr uint32_t kABytes = BM * BK * 2, kBBytes = BNH * BK * 2;
    static constexpr uint32_t kStageBytes = kABytes + kBBytes;
    static constexpr int kStages = (196608 / kStageBytes) < 6 ? (196608 / kStageBytes) : 6;
    static constexpr uint32_t kTmemCols = kMT * BN;
    static constexpr uint32_t kWBytes = BNH * (BK / 2);
    static constexpr int kWStages = 4;
    static constexpr uint32_t kOffA = 0;
    static constexpr uint32_t kOffB = kStages * kABytes;
    static constexpr uint32_t kOffLut = kOffB + kStages * kBBytes;
    static constexpr uint32_t kOffW = kOffLut + 4096;
    static constexpr uint32_t kOffBar = kOffW + kWStages * kWBytes;   // full_a[S] full_b[S] empty[S] accum full_w[WS] empty_w[WS]
    static constexpr uint32_t kOffMisc = kOffBar + (3 * kStages + 1 + 2 * kWStages) * 8;
    static constexpr uint32_t kSmemBytes = kOffMisc + 16 + 1024;
    // kind::f16 instruction descriptor as above with M = 256 (the pair), N = 256
    static constexpr uint32_t kInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                                           ((uint32_t)(256 >> 4) << 24);
    static constexpr int kThreadsPerRow = kDecodeWarps * 32 / BNH;   // 2
    static constexpr int kWords = 8 / kThreadsPerRow;                // 4
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on the leader CTA's copy of a barrier (from either CTA of the pair).
__device__ __forceinline__ void mbar_arrive_leader(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar & kPeerMask) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait with cluster-scope acquire (the barrier is also signalled by the peer CTA).
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, const WaitCtx& ctx, int code) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait_cluster(bar, parity)) {
        if ((++spins & 63u) == 0) {
            if (*ctx.abort_flag) return false;
            // both a long time and many polls: a discontinuity of the timer alone never aborts a wait
            if (spins > kMinSpins && global_timer_ns() - t0 > kWaitLimitNs) {
                *ctx.abort_flag = 1;
                if (ctx.status) atomicCAS(ctx.status, 0, code);
                return false;
            }
        }
    }
    return true;
}
// TMA load into this CTA's shared memory whose bytes are counted on the leader's barrier.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar & kPeerMask), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_pair_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive on the barrier at this shared-memory offset in both CTAs once all MMAs issued so far are done.
__device__ __forceinline__ void umma_pair_commit(uint32_t bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(mask) : "memory");
}

template <int kMT, bool kKL>
__global__ void __launch_bounds__(kThreads, 1) gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_x,
                                                                const __grid_constant__ CUtensorMap tmap_w,
                                                                const __grid_constant__ CUtensorMap tmap_y,
                                                                const GemmArgs a) {
    using C = PairCfg<kMT>;
    constexpr int kStages = C::kStages, kWStages = C::kWStages;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;      // same offset in both CTAs of the pair
    uint8_t* gen = smem_raw + (base - raw);

    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;   // provably warp-uniform
    const uint32_t rank = cluster_ctarank();           // 0 = leader
    const uint32_t m0 = blockIdx.x * C::BM;            // this CTA's token rows
    const uint32_t n0 = blockIdx.y * C::BN;            // the pair's weight rows; this CTA decodes n0 + rank*128 ...
    const uint32_t nh0 = n0 + rank * C::BNH;
    const int num_kt = static_cast<int>(a.kpad / BK);

    auto full_a = [&](int s) { return base + C::kOffBar + 8u * s; };
    auto full_b = [&](int s) { return base + C::kOffBar + 8u * (kStages + s); };
    auto empty = [&](int s) { return base + C::kOffBar + 8u * (2 * kStages + s); };
    const uint32_t accum_bar = base + C::kOffBar + 8u * (3 * kStages);
    auto full_w = [&](int s) { return base + C::kOffBar + 8u * (3 * kStages + 1 + s); };
    auto empty_w = [&](int s) { return base + C::kOffBar + 8u * (3 * kStages + 1 + kWStages + s); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + C::kOffMisc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + C::kOffMisc + 4);
    const WaitCtx ctx{abort_flag, a.status};

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_a(s), 1);                    // leader: its own expect_tx arrival; bytes of both CTAs
            mbar_init(full_b(s), 2 * kDecodeWarps);     // leader: the transcoder warps of both CTAs
            mbar_init(empty(s), 1);                     // each CTA: the leader's commit
        }
        mbar_init(accum_bar, 1);
        for (int s = 0; s < kWStages; ++s) {
            mbar_init(full_w(s), 1);
            mbar_init(empty_w(s), kDecodeWarps);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_proxy();
    }
    if (warp == 1) tmem_alloc_pair(base + C::kOffMisc, C::kTmemCols);   // the same warp in both CTAs
    if (warp >= 2 && warp < 2 + 8) {
        const int e = threadIdx.x - 64;
        reinterpret_cast<uint4*>(gen + C::kOffLut)[e] =
            a.lut ? __ldg(a.lut + e) : make_lut_entry(e & 127, e >> 7, *a.global_scale);
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();          // the peer's barriers are initialised before anything signals them
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------- TMA producer of this CTA's x tile
        if (lane == 0) {
            // x may be written by the kernel launched just before (the rotation pass): with programmatic
            // dependent launch everything above and the weight side below run under that kernel's tail,
            // and only the x loads wait for it (a no-op without the launch attribute)
            asm volatile("griddepcontrol.wait;" ::: "memory");
            asm volatile("fence.proxy.async.global;" ::: "memory");      // ordinary stores of that kernel, read by TMA
            int issued = 0;
            for (int kt = 0; kt < num_kt; ++kt) {
                const int s = kt % kStages;
                const uint32_t ph = (kt / kStages) & 1;
                if (!mbar_wait_cluster(empty(s), ph ^ 1, ctx, 1)) break;
                if (rank == 0) mbar_arrive_expect_tx(full_a(s), 2 * C::kABytes);   // both CTAs' tiles
                tma_load_2d_pair(base + C::kOffA + s * C::kABytes, &tmap_x, full_a(s), kt * BK, (int)m0);
                issued = kt + 1;
            }
            // never leave with a bulk copy still writing into this CTA's shared memory: the stage's
            // "empty" barrier completes only after the MMAs that read the landed tile
            for (int kt = max(0, issued - kStages); kt < issued; ++kt)
                if (!mbar_wait_cluster(empty(kt % kStages), (kt / kStages) & 1, ctx, 2)) break;
        }
    } else if (warp == 1) {
        // ------------------------------------------------------ MMA issuer (leader only)
        if (rank == 0 && lane == 0) {
            bool ok = true;
            for (int kt = 0; kt < num_kt && ok; ++kt) {
                const int s = kt % kStages;
                const uint32_t ph = (kt / kStages) & 1;
                ok = mbar_wait_cluster(full_a(s), ph, ctx, 3) && mbar_wait_cluster(full_b(s), ph, ctx, 4);
                if (!ok) break;
                tcgen05_fence_after();
                const uint64_t db = make_smem_desc(base + C::kOffB + s * C::kBBytes);
#pragma unroll
                for (int mt = 0; mt < kMT; ++mt) {
                    const uint64_t da = make_smem_desc(base + C::kOffA + s * C::kABytes + mt * 16384u);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        umma_pair_bf16(tmem_base + mt * C::BN, da + 2u * k, db + 2u * k, C::kInstrDesc,
                                       (kt | k) != 0 ? 1u : 0u);
                }
                umma_pair_commit(empty(s));             // frees the stage in both CTAs
            }
            if (ok) umma_pair_commit(accum_bar);
        }
    } else if (warp == 2 + kDecodeWarps) {
        // ------------------------------------------ TMA producer of this CTA's code tiles
        if (lane == 0) {
            int issued = 0;
            for (int kt = 0; kt < num_kt; ++kt) {
                const int s = kt % kWStages;
                const uint32_t ph = (kt / kWStages) & 1;
                if (!mbar_wait(empty_w(s), ph ^ 1, ctx, 7)) break;
                mbar_arrive_expect_tx(full_w(s), C::kWBytes);
                if (a.stream_layout)
                    tma_load_4d(base + C::kOffW + s * C::kWBytes, &tmap_w, full_w(s), (kt & 1) * (BK / 2), 0, kt >> 1,
                                (int)(nh0 >> 4));
                else
                    tma_load_2d(base + C::kOffW + s * C::kWBytes, &tmap_w, full_w(s), kt * (BK / 2), (int)nh0);
                issued = kt + 1;
            }
            for (int kt = max(0, issued - kWStages); kt < issued; ++kt)
                if (!mbar_wait(full_w(kt % kWStages), (kt / kWStages) & 1, ctx, 8)) break;
        }
    } else {
        // -------------------------------------------------- weight transcoders / epilogue
        constexpr int kWords = C::kWords, kBlocks = kWords / 2, kTPR = C::kThreadsPerRow;
        const int dt = threadIdx.x - 64;                // transcoder thread index
        const int row = dt / kTPR, part = dt % kTPR;    // row of this CTA's half tile, part of the K step
        const uint32_t last_row = (uint32_t)a.n - 1;
        const uint32_t grow = min(nh0 + row, last_row);
        const uint8_t* srow = a.stream_layout
            ? a.codes + (size_t)(grow >> 4) * a.subs * kChunkBytes + kChunkCodeBytes + (grow & 15) * 8
            : a.scales + (size_t)grow * (a.kpad / 16);
        const size_t sstep = a.stream_layout ? kChunkBytes : 8;
        const uint8_t* fptr = kKL ? a.scales : a.fmt + (size_t)grow * (a.kpad / 128);
        const uint32_t lut_base = base + C::kOffLut;
        const uint32_t row_off = (row >> 3) * 1024u + (row & 7) * 128u;
        const uint32_t sw = row & 7;

        auto load_codes = [&](uint32_t (&w)[kWords], int kt) -> bool {
            const int ws = kt % kWStages;
            if (!__all_sync(0xffffffffu, mbar_wait(full_w(ws), (kt / kWStages) & 1, ctx, 9))) return false;
            const uint32_t src = base + C::kOffW + ws * C::kWBytes + row * 32 + part * (kWords * 4);
            if constexpr (kWords == 4) {
                const uint4 v = lds128_lut(src);
                w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
            } else {
                asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(w[0]), "=r"(w[1]) : "r"(src));
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_w(ws));
            return true;
        };
        auto load_scale_pair = [&](int pair) -> uint2 { return __ldg(reinterpret_cast<const uint2*>(srow + (size_t)pair * sstep)); };

        uint32_t codes[kWords], ncodes[kWords];
        bool ok = load_codes(codes, 0);
        uint2 sc2 = load_scale_pair(0), nsc2 = num_kt > 2 ? load_scale_pair(1) : sc2, nnsc2 = nsc2;   // two pairs ahead
        uint32_t fb = kKL ? 0u : __ldg(fptr);
        for (int kt = 0; kt < num_kt && ok; ++kt) {
            const int s = kt % kStages;
            const uint32_t ph = (kt / kStages) & 1;
            uint32_t nfb = fb;
            if (kt + 1 < num_kt) {
                ok = load_codes(ncodes, kt + 1);
                if (!ok) break;
                if ((kt & 1) == 0 && kt + 4 < num_kt) nnsc2 = load_scale_pair((kt >> 1) + 2);
                if constexpr (!kKL) nfb = __ldg(fptr + ((kt + 1) >> 1));
            }
            const uint32_t scs = ((kt & 1) ? sc2.y : sc2.x) >> (8 * part * kBlocks);
            ok = __all_sync(0xffffffffu, mbar_wait_cluster(empty(s), ph ^ 1, ctx, 5));
            if (!ok) break;
            const uint32_t dst = base + C::kOffB + s * C::kBBytes + row_off;
            const uint32_t fbits = fb >> ((kt & 1) * 4 + part * kBlocks);
#pragma unroll
            for (int b = 0; b < kBlocks; ++b) {
                const uint32_t idx = kKL ? ((scs >> (8 * b)) & 0xffu)
                                         : ((((fbits >> b) & 1u) << 7) | ((scs >> (8 * b)) & 0x7fu));
                const uint4 tab = lds128_lut(lut_base + idx * 16);
#pragma unroll
                for (int w = 0; w < 2; ++w) {
                    const int i = 2 * b + w;
                    uint32_t p[4];
                    decode_word<kKL>(codes[i], tab, p);
                    const uint32_t chunk = (uint32_t)(part * kWords + i) ^ sw;
                    sts128(dst + chunk * 16, p[0], p[1], p[2], p[3]);
                }
            }
            fence_async_proxy();
            __syncwarp();
            if (lane == 0) mbar_arrive_leader(full_b(s));   // this CTA's half is in place
#pragma unroll
            for (int i = 0; i < kWords; ++i) codes[i] = ncodes[i];
            if (kt & 1) { sc2 = nsc2; nsc2 = nnsc2; }
            fb = nfb;
        }

        // a.tma_store is the same for every thread, so the named barrier inside is reached by all or none
        const bool done = ok && mbar_wait_cluster(accum_bar, 0, ctx, 6);
        if (a.tma_store) {
            if (epilogue_warps_all(done))
                store_accumulators_tma<kMT, C::BN>(a, &tmap_y, base + C::kOffA, tmem_base, m0, n0, warp, lane);
        } else if (done) {
            store_accumulators<kMT, C::BN>(a, tmem_base, m0, n0, warp, lane);
        }
    }

    // Both CTAs stay until the pair is done: the leader's MMAs read the peer's shared memory and
    // its commits signal the peer's barriers.
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tcgen05_fence_after();
        tmem_dealloc_pair(tmem_base, C::kTmemCols);
    }
}

// ------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// Tensor map of the packed codes; a box is one K step (32 bytes per row) of `box_rows` weight rows.
// Row-major layouts: the byte matrix [n, kpad/2].  Stream layout: (64 code bytes of a row in a chunk,
// 16 rows, chunks along K, row tiles), whose box of box_rows/16 tiles lands in shared memory in the
// same row-major order.
bool encode_code_map(EncodeTiledFn encode, CUtensorMap* map, const GemmArgs& a, int box_rows) {
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    if (a.stream_layout) {
        const cuuint64_t dims[4] = {64, kChunkRows, (cuuint64_t)a.subs, (cuuint64_t)stream_tiles(a.n)};
        const cuuint64_t strides[3] = {64, kChunkBytes, (cuuint64_t)a.subs * kChunkBytes};
        const cuuint32_t box[4] = {BK / 2, kChunkRows, 1, (cuuint32_t)(box_rows / (int)kChunkRows)};
        return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<uint8_t*>(a.codes), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    }
    const cuuint64_t dims[2] = {(cuuint64_t)(a.kpad / 2), (cuuint64_t)a.n};
    const cuuint64_t strides[1] = {(cuuint64_t)(a.kpad / 2)};
    const cuuint32_t box[2] = {BK / 2, (cuuint32_t)box_rows};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(a.codes), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int64_t x_staging_bytes(int64_t m, int64_t k) { return m * ((k + 7) / 8 * 8) * 2; }
constexpr int64_t kAmaxSlotBytes = 256;

// after_producer: the kernel launched just before on this stream wrote xa (and nothing else this kernel
// reads) and signals its dependents early; this launch may then start under its tail.
template <int kMT, int kBN, bool kKL>
int launch_gemm(const void* xa, int64_t lda, const GemmArgs& a, cudaStream_t st, bool after_producer = false) {
    using C = Cfg<kMT, kBN>;
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) return record_error_text("cuTensorMapEncodeTiled is not available from the driver");
    CUtensorMap tmap;
    const cuuint64_t dims[2] = {(cuuint64_t)a.k, (cuuint64_t)a.m};
    const cuuint64_t strides[1] = {(cuuint64_t)lda * 2};
    const cuuint32_t box[2] = {BK, (cuuint32_t)C::BM};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult cr = encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(xa), dims, strides, box,
                               estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return record_error_text("cuTensorMapEncodeTiled failed");
    // the packed codes as a byte matrix [n, kpad/2]; a box is one K step (32 bytes) of BN rows
    CUtensorMap tmap_w;
    if (!encode_code_map(encode, &tmap_w, a, C::BN)) return record_error_text("cuTensorMapEncodeTiled failed for the code matrix");
    static unsigned long long configured = 0;          // one per instantiation, one bit per device
    if (const int rc = ensure_dynamic_smem(gemm_kernel<kMT, kBN, kKL>, (int)C::kSmemBytes, configured)) return rc;
    const int total_kt = static_cast<int>(a.kpad / BK);
    const int splits = (total_kt + a.kt_per_split - 1) / a.kt_per_split;
    const dim3 grid((unsigned)((a.n + C::BN - 1) / C::BN), (unsigned)((a.m + C::BM - 1) / C::BM), (unsigned)splits);
    if (grid.y > 65535) return MIXFP4_E_SHAPE;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = after_producer ? 1 : 0;
    MIXFP4_CUDA_CHECK(cudaLaunchKernelEx(&cfg, gemm_kernel<kMT, kBN, kKL>, tmap, tmap_w, a));
    int rc = check_launch("gemm_kernel");
    if (rc == MIXFP4_OK && splits > 1) {
        const int64_t total = a.m * a.n;
        splitk_reduce_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(a.partial, splits, a.m, a.n, a.ld_partial,
                                                                             a.y, a.out_dtype, a.ldy);
        rc = check_launch("splitk_reduce_kernel");
    }
    return rc;
}

// Tile choice of the single-CTA kernel: estimated time = waves over the 148 SMs x relative time of
// one tile (measured: a tile with two 128-row sub-tiles or 256 weight rows amortises the transcode
// better), and how many CTAs share a tile along K when the tiles alone would leave SMs idle.
struct GemmPlan {
    int mt, bn, splits, kt_per_split;
};
GemmPlan plan_gemm(int64_t m, int64_t n, int64_t k) {
    const int total_kt = static_cast<int>(padded_k(k) / BK);
    GemmPlan p = {1, 128, 1, total_kt};
    const int mts[4] = {1, 2, 1, 2}, bns[4] = {128, 128, 256, 256};
    const double cost[4] = {1.0, 1.35, 1.78, 2.2};      // time of one K step of a tile, in units of ~0.45 us
    // Each K step costs a CTA about the same whatever M is (the weight tile has to be decoded), so
    // a problem with few tiles and a long K can run several CTAs per tile: fp32 partial sums go to
    // the workspace and are added in split order.  At least 8 K steps per CTA, even counts; the
    // partial sums cost their bytes once written and once read (about 3 TB/s through L2).
    double best = 1e300;
    for (int i = 0; i < 4; ++i) {
        const int64_t tiles = ((m + 128 * mts[i] - 1) / (128 * mts[i])) * ((n + bns[i] - 1) / bns[i]);
        for (int splits = 1; splits <= 8; ++splits) {
            if (splits > 1 && (splits > total_kt / 8 || tiles * splits > 148)) break;
            int per = (total_kt + splits - 1) / splits;
            per += (splits > 1) ? (per & 1) : 0;
            const int real_splits = (total_kt + per - 1) / per;
            const double waves = (double)((tiles * real_splits + 147) / 148);
            double t = waves * per * cost[i];
            if (real_splits > 1) t += (double)real_splits * m * n * 8.0 / 3.0e6 / 0.45;
            if (t < best) { best = t; p.mt = mts[i]; p.bn = bns[i]; p.splits = real_splits; p.kt_per_split = per; }
        }
    }
    return p;
}
int64_t partial_ld(int64_t n) { return (n + 3) / 4 * 4; }

// after_producer: the kernel launched just before on this stream wrote xa (and nothing else this kernel
// reads) and signals its dependents early; this launch may then start under its tail.
template <int kMT, bool kKL>
int launch_gemm_pair(const void* xa, int64_t lda, const GemmArgs& args, cudaStream_t st, bool after_producer = false) {
    using C = PairCfg<kMT>;
    GemmArgs a = args;
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) return record_error_text("cuTensorMapEncodeTiled is not available from the driver");
    CUtensorMap tmap, tmap_w, tmap_y;
    const cuuint32_t estr[2] = {1, 1};
    // bf16 output with 16-byte aligned rows: boxes of 128 rows x 64 columns leave through TMA stores
    a.tma_store = a.out_dtype == MIXFP4_BF16 && aligned(a.y, 16) && (a.ldy * 2) % 16 == 0;
    {
        const cuuint64_t ydims[2] = {(cuuint64_t)a.n, (cuuint64_t)a.m};
        const cuuint64_t ystrides[1] = {(cuuint64_t)a.ldy * 2};
        const cuuint32_t ybox[2] = {64, 128};
        if (a.tma_store &&
            encode(&tmap_y, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.y, ydims, ystrides, ybox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            a.tma_store = 0;
        if (!a.tma_store) memset(&tmap_y, 0, sizeof(tmap_y));
    }
    const cuuint64_t dims[2] = {(cuuint64_t)a.k, (cuuint64_t)a.m};
    const cuuint64_t strides[1] = {(cuuint64_t)lda * 2};
    const cuuint32_t box[2] = {BK, (cuuint32_t)C::BM};
    if (encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(xa), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return record_error_text("cuTensorMapEncodeTiled failed");
    if (!encode_code_map(encode, &tmap_w, a, C::BNH)) return record_error_text("cuTensorMapEncodeTiled failed for the code matrix");
    static unsigned long long configured = 0;          // one per instantiation, one bit per device
    if (const int rc = ensure_dynamic_smem(gemm_pair_kernel<kMT, kKL>, (int)C::kSmemBytes, configured)) return rc;
    const int64_t pairs = (a.m + 2 * C::BM - 1) / (2 * C::BM);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * pairs), (unsigned)((a.n + C::BN - 1) / C::BN));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cfg.stream = st;
    if (cfg.gridDim.y > 65535) return MIXFP4_E_SHAPE;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = after_producer ? 2 : 1;
    MIXFP4_CUDA_CHECK(cudaLaunchKernelEx(&cfg, gemm_pair_kernel<kMT, kKL>, tmap, tmap_w, tmap_y, a));
    return check_launch("gemm_pair_kernel");
}

}  // namespace
}  // namespace mixfp4

using namespace mixfp4;

// Argument checks shared by every GEMM entry point; they run before anything is enqueued.
static int check_gemm_args(const void* x, int64_t m, int64_t ldx, const uint8_t* codes, const uint8_t* scales,
                           const uint8_t* fmt, const float* global_scale, int64_t n, int64_t k, int layout,
                           const void* lut, int rotation_block, const void* y, int out_dtype, int64_t ldy) {
    if (layout != MIXFP4_LAYOUT_CANONICAL && layout != MIXFP4_LAYOUT_KERNEL && layout != MIXFP4_LAYOUT_STREAM)
        return MIXFP4_E_MODE;
    const bool streamed = layout == MIXFP4_LAYOUT_STREAM;
    if (!x || !codes || (!scales && !streamed) || (!fmt && layout == MIXFP4_LAYOUT_CANONICAL) || !global_scale || !y)
        return MIXFP4_E_NULL;
    if (m <= 0 || n <= 0 || k <= 0 || ldx < k || ldy < n) return MIXFP4_E_SHAPE;
    if (m > 0x7fffffffLL || n > 0x7fffffffLL || k > 0x7fffffffLL) return MIXFP4_E_SHAPE;
    if (out_dtype != MIXFP4_F32 && out_dtype != MIXFP4_BF16) return MIXFP4_E_DTYPE;
    if (rotation_block != 0 && rotation_block != 128) return MIXFP4_E_MODE;
    if (!aligned(codes, 16) || (!streamed && !aligned(scales, 8)) || (lut && !aligned(lut, 16))) return MIXFP4_E_ALIGN;
    return MIXFP4_OK;
}

extern "C" int64_t mixfp4_gemm_workspace_bytes(int64_t m, int64_t n, int64_t k) {
    if (m <= 0 || k <= 0) return 0;
    int64_t bytes = (x_staging_bytes(m, k) + 255) / 256 * 256;
    if (n > 0) {
        const GemmPlan p = plan_gemm(m, n, k);
        if (p.splits > 1) bytes += (int64_t)p.splits * m * partial_ld(n) * 4;
    }
    return bytes + kAmaxSlotBytes;      // last: the activation amax word of mixfp4_gemm_a4
}

// x_from_previous_kernel: x (16-byte aligned rows) was written by the kernel launched just before on this
// stream, which signals its dependents early and writes nothing else this call reads.
static int gemm_run(const void* x, int64_t m, int64_t ldx, const uint8_t* codes, const uint8_t* scales,
                    const uint8_t* fmt, const float* global_scale, int64_t n, int64_t k, int layout, const void* lut,
                    int rotation_block, void* y, int out_dtype, int64_t ldy, void* workspace, int64_t workspace_bytes,
                    int* status, void* stream, bool x_from_previous_kernel) {
    if (const int rc = check_gemm_args(x, m, ldx, codes, scales, fmt, global_scale, n, k, layout, lut, rotation_block, y,
                                       out_dtype, ldy))
        return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    // The TMA descriptor needs a 16-byte aligned base and row pitch; the rotation needs a
    // place to put bf16(H128 x).  Both go through the caller's workspace.
    const void* xa = x;
    int64_t lda = ldx;
    const bool tma_ok = aligned(x, 16) && (ldx % 8 == 0);
    if (rotation_block == 128 || !tma_ok) {
        const int64_t need = x_staging_bytes(m, k);
        if (!workspace || workspace_bytes < need) return MIXFP4_E_WORKSPACE;
        if (!aligned(workspace, 16)) return MIXFP4_E_ALIGN;
        lda = (k + 7) / 8 * 8;
        if (rotation_block == 128) {
            const int rc = mixfp4_fwht(x, workspace, MIXFP4_BF16, m, k, ldx, lda, 128, nullptr, 0, stream);
            if (rc != MIXFP4_OK) return rc;
        } else {
            MIXFP4_CUDA_CHECK(cudaMemcpy2DAsync(workspace, lda * 2, x, ldx * 2, k * 2, m, cudaMemcpyDeviceToDevice, st));
        }
        xa = workspace;
    }

    GemmArgs a;
    a.codes = codes; a.scales = scales; a.fmt = fmt; a.global_scale = global_scale;
    a.lut = static_cast<const uint4*>(lut);
    a.m = m; a.n = n; a.k = k; a.kpad = padded_k(k);
    a.y = y; a.out_dtype = out_dtype; a.ldy = ldy; a.status = status;
    a.kt_per_split = static_cast<int>(a.kpad / BK); a.partial = nullptr; a.ld_partial = 0; a.tma_store = 0;
    a.stream_layout = layout == MIXFP4_LAYOUT_STREAM; a.subs = static_cast<int>(a.kpad / kChunkK);
    const GemmPlan plan = plan_gemm(m, n, k);
    const int mt = plan.mt, bn = plan.bn;
    if (plan.splits > 1) {     // split K needs room for the partial sums after the staging area; without it: one CTA per tile
        const int64_t staging = (x_staging_bytes(m, k) + 255) / 256 * 256;
        const int64_t need = staging + (int64_t)plan.splits * m * partial_ld(n) * 4;
        if (workspace && workspace_bytes >= need && aligned(workspace, 16)) {
            a.kt_per_split = plan.kt_per_split;
            a.partial = reinterpret_cast<float*>(static_cast<char*>(workspace) + staging);
            a.ld_partial = partial_ld(n);
        }
    }
    const bool kl = layout != MIXFP4_LAYOUT_CANONICAL;       // the stream layout keeps the kernel layout's code words
    // More than 256 tokens and enough tiles to occupy most SMs: CTA pairs (two SMs share each decoded
    // weight tile; measured 1.25-1.3 x the single-CTA kernel at M >= 2048, slower below about 100 CTAs).
    // Pairs of 256-row CTAs unless pairs of 128-row CTAs pad the token rows noticeably less.  With at
    // most 256 tokens a pair's second CTA would hold no rows and still decode: measured 88 us against 51
    // for the single-CTA kernel at M = 17 .. 128 on a 28672 x 4096 weight.
    // the rotation pass above (or the caller's last kernel) is this launch's only producer
    const bool dep = rotation_block == 128 || (x_from_previous_kernel && xa == x);
    if (m > 256) {
        const int64_t tiles_n = (n + 255) / 256;
        const int64_t rows2 = (m + 511) / 512 * 512, rows1 = (m + 255) / 256 * 256;
        if (rows2 * 100 <= rows1 * 108 && 2 * (rows2 / 512) * tiles_n >= 112)
            return kl ? launch_gemm_pair<2, true>(xa, lda, a, st, dep) : launch_gemm_pair<2, false>(xa, lda, a, st, dep);
        if (2 * (rows1 / 256) * tiles_n >= 112)
            return kl ? launch_gemm_pair<1, true>(xa, lda, a, st, dep) : launch_gemm_pair<1, false>(xa, lda, a, st, dep);
    }
    if (mt == 1 && bn == 128) return kl ? launch_gemm<1, 128, true>(xa, lda, a, st, dep) : launch_gemm<1, 128, false>(xa, lda, a, st, dep);
    if (mt == 1 && bn == 256) return kl ? launch_gemm<1, 256, true>(xa, lda, a, st, dep) : launch_gemm<1, 256, false>(xa, lda, a, st, dep);
    if (mt == 2 && bn == 128) return kl ? launch_gemm<2, 128, true>(xa, lda, a, st, dep) : launch_gemm<2, 128, false>(xa, lda, a, st, dep);
    return kl ? launch_gemm<2, 256, true>(xa, lda, a, st, dep) : launch_gemm<2, 256, false>(xa, lda, a, st, dep);
}

extern "C" int mixfp4_gemm(const void* x, int64_t m, int64_t ldx, const uint8_t* codes, const uint8_t* scales,
                           const uint8_t* fmt, const float* global_scale, int64_t n, int64_t k, int layout,
                           const void* lut, int rotation_block, void* y, int out_dtype, int64_t ldy, void* workspace,
                           int64_t workspace_bytes, int* status, int flags, void* stream) {
    (void)flags;
    return gemm_run(x, m, ldx, codes, scales, fmt, global_scale, n, k, layout, lut, rotation_block, y, out_dtype, ldy,
                    workspace, workspace_bytes, status, stream, false);
}

extern "C" int mixfp4_gemm_a4(const void* x, int64_t m, int64_t ldx, const uint8_t* codes, const uint8_t* scales,
                              const uint8_t* fmt, const float* global_scale, int64_t n, int64_t k, int layout,
                              const void* lut, int rotation_block, int act_mode, void* y, int out_dtype, int64_t ldy,
                              void* workspace, int64_t workspace_bytes, int* status, int flags, void* stream) {
    if (const int rc = check_gemm_args(x, m, ldx, codes, scales, fmt, global_scale, n, k, layout, lut, rotation_block, y,
                                       out_dtype, ldy))
        return rc;
    if (act_mode < MIXFP4_MODE_ORACLE16 || act_mode > MIXFP4_MODE_ALL_E0M3) return MIXFP4_E_MODE;
    const int64_t total = mixfp4_gemm_workspace_bytes(m, n, k);
    if (!workspace || workspace_bytes < total) return MIXFP4_E_WORKSPACE;
    if (!aligned(workspace, 16)) return MIXFP4_E_ALIGN;
    // staging area: the rotated (every stage rounded to bf16, as the reference's hook computes it on
    // a bf16 tensor), then fake-quantized activations; the amax word sits in the workspace's last slot
    const int64_t lda = (k + 7) / 8 * 8;
    float* amax = reinterpret_cast<float*>(static_cast<char*>(workspace) + total - kAmaxSlotBytes);
    const void* src = x;
    int64_t lds = ldx;
    bool have_amax = false;
    if (rotation_block == 128) {
        // one pass for the rotation and the rotated tensor's maximum where the rows allow it
        int rc = fwht128_stagewise_amax(x, workspace, MIXFP4_BF16, m, k, ldx, lda, amax, static_cast<cudaStream_t>(stream));
        have_amax = rc == MIXFP4_OK;
        if (rc == MIXFP4_E_UNSUPPORTED) rc = mixfp4_fwht(x, workspace, MIXFP4_BF16, m, k, ldx, lda, 128, nullptr, 1, stream);
        if (rc != MIXFP4_OK) return rc;
        src = workspace;
        lds = lda;
    }
    const int rc = have_amax ? fake_quantize_with_amax(src, MIXFP4_BF16, m, k, lds, act_mode, amax, workspace, lda,
                                                       static_cast<cudaStream_t>(stream))
                             : mixfp4_fake_quantize(src, MIXFP4_BF16, m, k, lds, act_mode, amax, workspace, lda, stream);
    if (rc != MIXFP4_OK) return rc;
    (void)flags;
    // the quantizer's kernel is the only producer of the staged activations and lets its dependents start early
    return gemm_run(workspace, m, lda, codes, scales, fmt, global_scale, n, k, layout, lut, 0, y, out_dtype, ldy, workspace,
                    total - kAmaxSlotBytes, status, stream, true);
}


// ------------------------------------------------------------- allocation-free variant
// Staging buffer of mixfp4_gemm_h128_static: lives in the library image, so every GPU that
// loads the library carries these 8 MiB until the process exits.
namespace mixfp4 {
namespace {
constexpr int64_t kStaticScratchBytes = 8ll << 20;
static __device__ __align__(256) uint8_t g_static_scratch[kStaticScratchBytes];
constexpr int kMaxDevices = 64;

// Device address of g_static_scratch on the current device.  In host code the symbol name
// is only a handle, so the address is looked up once per device (with that device current)
// and remembered.
int static_scratch_address(void** out) {
    static std::mutex lock;
    static void* addr[kMaxDevices] = {};
    int dev = 0;
    MIXFP4_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return MIXFP4_E_UNSUPPORTED;
    std::lock_guard<std::mutex> guard(lock);
    if (!addr[dev]) {
        void* p = nullptr;
        MIXFP4_CUDA_CHECK(cudaGetSymbolAddress(&p, g_static_scratch));
        addr[dev] = p;
    }
    *out = addr[dev];
    return MIXFP4_OK;
}
}  // namespace
}  // namespace mixfp4

extern "C" int64_t mixfp4_gemm_h128_static_max_bytes(void) { return mixfp4::kStaticScratchBytes; }

extern "C" int mixfp4_gemm_h128_static(const void* x, int64_t m, int64_t ldx, const uint8_t* codes,
                                       const uint8_t* scales, const uint8_t* fmt, const float* global_scale,
                                       int64_t n, int64_t k, int layout, const void* lut, void* y, int out_dtype,
                                       int64_t ldy, int* status, void* stream) {
    // every argument is checked before the first kernel is enqueued: a rejected call leaves the
    // shared array untouched (the sizes are below 2^31 here, so the product cannot wrap)
    if (const int rc = check_gemm_args(x, m, ldx, codes, scales, fmt, global_scale, n, k, layout, lut, 128, y, out_dtype,
                                       ldy))
        return rc;
    const int64_t lda = (k + 7) / 8 * 8;
    if (m * lda * 2 > kStaticScratchBytes) return MIXFP4_E_TOO_LARGE;
    void* scratch = nullptr;
    int rc = static_scratch_address(&scratch);
    if (rc != MIXFP4_OK) return rc;
    // rotated activations bf16(H128 x) -> static buffer (every element the GEMM reads is
    // rewritten here, so nothing left over from an earlier call is ever consumed)
    rc = mixfp4_fwht(x, scratch, MIXFP4_BF16, m, k, ldx, lda, 128, nullptr, 0, stream);
    if (rc != MIXFP4_OK) return rc;
    // The rest of the array is offered as workspace: mixfp4_gemm puts split-K partial sums behind the
    // staging area (which is where the rotated activations already are) when they fit, exactly as it
    // does with a caller's workspace, so both entry points take the same decisions.
    return mixfp4_gemm(scratch, m, lda, codes, scales, fmt, global_scale, n, k, layout, lut, 0, y, out_dtype, ldy,
                       scratch, kStaticScratchBytes, status, 0, stream);
}
