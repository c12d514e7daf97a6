// Decode-shape dequant-linear (1 <= M <= 16): y[M,N] = x[M,K] * W[N,K]^T, W in the packed
// mixed-FP4 layout.  Replaces F.linear on the dequantized weight
// (project_quant/modeling.py:629 + nn.Linear.forward).  HBM-bound: the packed weight
// (0.5703 B/element) is read exactly once, x stays in L1/L2.
//
// Work split.  A CTA owns 16 consecutive weight rows; its warps split K in interleaved
// 128-element steps and their partial sums are added in a fixed order through shared
// memory (deterministic).  Inside a warp a 16 x 128 step is laid over the
// mma.sync.m16n8k16 A-fragment: lane (g, t) = (lane/4, lane%4) owns rows g and g+8 and
// the 32 consecutive K elements starting at 32*t.  The k index of an MMA is only a
// summation label, so the 16 k-slots of every MMA are filled with whatever 4 consecutive
// elements each lane decodes next; the B fragment takes the same 4 elements of x (batch
// row g).
//
// Data movement.  Every warp runs its own ring of cp.async stages: per step a lane
// copies its 2 x 16 B of codes, (two lanes of each quad) the 8 scale bytes of a row, and
// its 64 B of x, a few steps ahead of the arithmetic, so neither the HBM latency of the
// weights nor the L2 latency of x is exposed.  The format bytes of the CTA's 16 rows are
// read once into shared memory.
//
// Decode.  A 256-entry table in shared memory, built per launch from the tensor scale,
// maps (format bit, E4M3 scale byte) to the block's eight magnitudes
// bf16((level * scale) * global) -- exactly the reference's dequantized weight -- stored
// as 8 low bytes + 8 high bytes.  Eight 4-bit codes (one 32-bit word) become four bf16x2
// registers with byte permutes: two PRMT look up low/high bytes of four elements, the
// sign bits are spread with PRMT's sign-replicate mode, two more PRMT interleave.
// The accumulation is the tensor core's fp32.

#include <stdlib.h>

#include "common.cuh"
#include "decode.cuh"

namespace mixfp4 {
namespace {

constexpr int kRowsPerCta = 16;
constexpr int kStepK = 128;               // K elements one warp consumes per step

struct GemvArgs {
    const __nv_bfloat16* x;
    int64_t m, ldx;
    const uint8_t* codes;
    const uint8_t* scales;
    const uint8_t* fmt;
    const float* global_scale;
    int64_t n, k, kpad;
    void* y;
    int out_dtype;
    int64_t ldy;
    bool x_vec;                            // x rows are 16-byte aligned and K % 8 == 0
};

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct Piece {                // what one lane holds for one 128-wide K step: rows g (0) and g+8 (1)
    uint4 c[2];               // 2 x 32 codes
    uint32_t s[2];            // 2 x 2 scale bytes
    uint32_t f[2];            // 2 x format byte of the step (8 blocks)
};

template <int kWarps, int kNTiles, bool kXVec>
__global__ void __launch_bounds__(kWarps * 32, kWarps == 16 ? 2 : 3) gemv_kernel(const GemvArgs a) {
    __shared__ uint4 lut[256];
    __shared__ float red[kWarps][kRowsPerCta][8 * kNTiles];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t row0 = blockIdx.x * kRowsPerCta;
    const uint32_t ld_codes = (uint32_t)(a.kpad >> 1), ld_scales = (uint32_t)(a.kpad >> 4);
    const uint32_t ld_fmt = (uint32_t)(a.kpad >> 7);
    const int steps = static_cast<int>(a.kpad / kStepK);
    const bool row_ok[2] = {row0 + g < a.n, row0 + g + 8 < a.n};
    // byte offsets of this lane's rows (the host checks that they fit 32 bits)
    uint32_t coff[2], soff[2], foff[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t r = row_ok[h] ? row0 + g + 8 * h : 0;
        coff[h] = r * ld_codes + t * 16;
        soff[h] = r * ld_scales + t * 2;
        foff[h] = r * ld_fmt;
    }

    auto load_piece = [&](Piece& p, int step) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            if (row_ok[h]) {
                p.c[h] = ldg_stream(reinterpret_cast<const uint4*>(a.codes + (coff[h] + (uint32_t)step * 64u)));
                p.s[h] = __ldg(reinterpret_cast<const unsigned short*>(a.scales + (soff[h] + (uint32_t)step * 8u)));
                p.f[h] = __ldg(a.fmt + (foff[h] + (uint32_t)step));
            } else {
                p.c[h] = make_uint4(0, 0, 0, 0);
                p.s[h] = 0;                    // scale byte 0 -> table entry of zeros
                p.f[h] = 0;
            }
        }
    };

    Piece cur, nxt;
    if (warp < steps) load_piece(cur, warp);

    {   // build the decode table while the first loads are in flight
        const float gs = *a.global_scale;
        for (int e = threadIdx.x; e < 256; e += kWarps * 32) lut[e] = make_lut_entry(e & 127, e >> 7, gs);
    }
    __syncthreads();

    float acc[kNTiles][4];
#pragma unroll
    for (int nt = 0; nt < kNTiles; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i] = 0.0f;

    // element offsets into x of this lane's batch rows (host checks they fit 32 bits)
    uint32_t xoff[kNTiles];
    bool x_ok[kNTiles];
#pragma unroll
    for (int nt = 0; nt < kNTiles; ++nt) {
        x_ok[nt] = g + 8 * nt < a.m;
        xoff[nt] = (uint32_t)(x_ok[nt] ? g + 8 * nt : 0) * (uint32_t)a.ldx + t * 32;
    }
    const uint32_t k_lim = (uint32_t)a.k;

    for (int step = warp; step < steps; step += kWarps) {
        const bool more = step + kWarps < steps;
        if (more) load_piece(nxt, step + kWarps);
        const uint32_t kp = (uint32_t)step * kStepK;          // K offset of the step; the lane adds 32 t
#pragma unroll
        for (int b = 0; b < 2; ++b) {                        // the 2 blocks of this lane's piece
            uint4 tab[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t scale_byte = (cur.s[h] >> (8 * b)) & 0x7fu;
                const uint32_t fbit = (cur.f[h] >> (2 * t + b)) & 1u;
                tab[h] = lut[(fbit << 7) | scale_byte];
            }
#pragma unroll
            for (int half = 0; half < 2; ++half) {           // 8 elements = 2 MMAs
                const int i = 2 * b + half;                  // word index inside the piece
                uint32_t pl[4], ph[4];
                const uint32_t wl = i == 0 ? cur.c[0].x : i == 1 ? cur.c[0].y : i == 2 ? cur.c[0].z : cur.c[0].w;
                const uint32_t wh = i == 0 ? cur.c[1].x : i == 1 ? cur.c[1].y : i == 2 ? cur.c[1].z : cur.c[1].w;
                decode8(wl, tab[0], pl);
                decode8(wh, tab[1], ph);
                const uint32_t k0 = kp + 8 * i;              // relative to xoff (which holds + 32 t)
#pragma unroll
                for (int nt = 0; nt < kNTiles; ++nt) {
                    uint4 xv = make_uint4(0, 0, 0, 0);
                    if (x_ok[nt]) {
                        const __nv_bfloat16* xp = a.x + (xoff[nt] + k0);
                        if (kXVec) {
                            if (k0 + t * 32 < k_lim) xv = __ldg(reinterpret_cast<const uint4*>(xp));
                        } else {
                            uint32_t e[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                e[j] = k0 + t * 32 + j < k_lim ? __bfloat16_as_ushort(xp[j]) : 0u;
                            xv = make_uint4(e[0] | (e[1] << 16), e[2] | (e[3] << 16), e[4] | (e[5] << 16),
                                            e[6] | (e[7] << 16));
                        }
                    }
                    mma_bf16(acc[nt], pl[0], ph[0], pl[1], ph[1], xv.x, xv.y);
                    mma_bf16(acc[nt], pl[2], ph[2], pl[3], ph[3], xv.z, xv.w);
                }
            }
        }
        if (more) cur = nxt;
    }

    // accumulator fragment: c0,c1 = (row g, batch 2t, 2t+1); c2,c3 = (row g+8, same batches)
#pragma unroll
    for (int nt = 0; nt < kNTiles; ++nt) {
        red[warp][g][8 * nt + 2 * t] = acc[nt][0];
        red[warp][g][8 * nt + 2 * t + 1] = acc[nt][1];
        red[warp][g + 8][8 * nt + 2 * t] = acc[nt][2];
        red[warp][g + 8][8 * nt + 2 * t + 1] = acc[nt][3];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < kRowsPerCta * 8 * kNTiles; idx += kWarps * 32) {
        const int r = idx % kRowsPerCta, b = idx / kRowsPerCta;
        if (b >= a.m || row0 + r >= a.n) continue;
        float sum = red[0][r][b];
#pragma unroll
        for (int w = 1; w < kWarps; ++w) sum += red[w][r][b];
        if (a.out_dtype == MIXFP4_F32) static_cast<float*>(a.y)[(int64_t)b * a.ldy + row0 + r] = sum;
        else static_cast<__nv_bfloat16*>(a.y)[(int64_t)b * a.ldy + row0 + r] = __float2bfloat16_rn(sum);
    }
}

// ------------------------------------------------------------------ cp.async pipeline
constexpr int kDepth = 3;                 // ring stages per warp

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async16_stream(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory"); }

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}

// One ring stage of a warp: x [chunk 0..3][batch row][t] 16 B (m * 256 bytes), then the codes
// [row half][lane] 16 B, then the scales [row 0..15] 8 B.
__host__ __device__ inline uint32_t stage_bytes(int64_t m) { return (uint32_t)m * 256u + 1024u + 128u; }

template <int kWarps, int kNTiles>
__global__ void __launch_bounds__(kWarps * 32, kWarps == 16 ? 2 : 3) gemv_async_kernel(const GemvArgs a) {
    extern __shared__ __align__(16) uint8_t smem[];
    // lut 4096 | red kWarps*16*8*kNTiles*4 | rings kWarps*kDepth*stage | fmt bytes 16*ld_fmt
    uint4* lut = reinterpret_cast<uint4*>(smem);
    float* red = reinterpret_cast<float*>(smem + 4096);
    constexpr int kRedBytes = kWarps * kRowsPerCta * 8 * kNTiles * 4;
    const uint32_t x_bytes = (uint32_t)a.m * 256u, stage = stage_bytes(a.m);
    const uint32_t off_codes = x_bytes, off_scales = x_bytes + 1024u, x_chunk = (uint32_t)a.m * 64u;
    uint8_t* fmt_tab = smem + 4096 + kRedBytes + kWarps * kDepth * stage;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t row0 = blockIdx.x * kRowsPerCta;
    const uint32_t ld_codes = (uint32_t)(a.kpad >> 1), ld_scales = (uint32_t)(a.kpad >> 4);
    const uint32_t ld_fmt = (uint32_t)(a.kpad >> 7);
    const int steps = static_cast<int>(a.kpad / kStepK);
    const uint32_t last_row = (uint32_t)a.n - 1;
    // rows past N re-read the last row; their sums are never stored
    const uint32_t r0 = min(row0 + g, last_row), r1 = min(row0 + g + 8, last_row);
    const uint8_t* cptr[2] = {a.codes + (size_t)r0 * ld_codes + t * 16, a.codes + (size_t)r1 * ld_codes + t * 16};
    const uint8_t* sptr = a.scales + (size_t)(t == 0 ? r0 : r1) * ld_scales;   // used by lanes t < 2
    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(smem + 4096 + kRedBytes) + warp * kDepth * stage;
    const uint32_t k_lim = (uint32_t)a.k;
    bool x_ok[kNTiles];
    const __nv_bfloat16* xptr[kNTiles];
#pragma unroll
    for (int nt = 0; nt < kNTiles; ++nt) {
        x_ok[nt] = g + 8 * nt < a.m;
        xptr[nt] = a.x + (size_t)(x_ok[nt] ? g + 8 * nt : 0) * a.ldx + t * 32;
    }

    auto issue = [&](int step) {
        const uint32_t base = ring + (uint32_t)(step / kWarps % kDepth) * stage;
#pragma unroll
        for (int h = 0; h < 2; ++h)
            cp_async16_stream(base + off_codes + h * 512 + lane * 16, cptr[h] + (size_t)step * 64);
        if (t < 2) cp_async8(base + off_scales + (g + 8 * t) * 8, sptr + (size_t)step * 8);
#pragma unroll
        for (int nt = 0; nt < kNTiles; ++nt) {
            if (x_ok[nt]) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint32_t kk = (uint32_t)step * kStepK + t * 32 + c * 8;
                    const bool in = kk < k_lim;      // K % 8 == 0: a chunk is all inside or all outside
                    cp_async16(base + c * x_chunk + (g + 8 * nt) * 64 + t * 16,
                               in ? static_cast<const void*>(xptr[nt] + (size_t)step * kStepK + c * 8)
                                  : static_cast<const void*>(a.x),
                               in ? 16u : 0u);
                }
            }
        }
    };

    // prologue: first kDepth-1 steps of this warp in flight, then the CTA-wide tables
#pragma unroll
    for (int d = 0; d < kDepth - 1; ++d) {
        if (warp + d * kWarps < steps) issue(warp + d * kWarps);
        cp_async_commit();
    }
    {
        const float gs = *a.global_scale;
        for (int e = threadIdx.x; e < 256; e += kWarps * 32) lut[e] = make_lut_entry(e & 127, e >> 7, gs);
        for (uint32_t i = threadIdx.x; i < kRowsPerCta * ld_fmt; i += kWarps * 32) {
            const uint32_t r = min(row0 + i / ld_fmt, last_row);
            fmt_tab[i] = __ldg(a.fmt + (size_t)r * ld_fmt + i % ld_fmt);
        }
    }
    __syncthreads();

    float acc[kNTiles][4];
#pragma unroll
    for (int nt = 0; nt < kNTiles; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i] = 0.0f;
    const uint32_t lut_base = (uint32_t)__cvta_generic_to_shared(lut);

    for (int step = warp; step < steps; step += kWarps) {
        // the stage written now was read in the previous iteration: all lanes must be done with it
        __syncwarp();
        const int ahead = step + (kDepth - 1) * kWarps;
        if (ahead < steps) issue(ahead);
        cp_async_commit();
        cp_async_wait<kDepth - 1>();
        __syncwarp();                                        // scale bytes come from another lane's copy
        const uint32_t base = ring + (uint32_t)(step / kWarps % kDepth) * stage;
        const uint4 cl = lds128(base + off_codes + lane * 16);
        const uint4 ch = lds128(base + off_codes + 512 + lane * 16);
        const uint32_t sl = lds16(base + off_scales + g * 8 + t * 2);
        const uint32_t sh = lds16(base + off_scales + (g + 8) * 8 + t * 2);
        const uint32_t fl = fmt_tab[g * ld_fmt + step] >> (2 * t);
        const uint32_t fh = fmt_tab[(g + 8) * ld_fmt + step] >> (2 * t);
#pragma unroll
        for (int b = 0; b < 2; ++b) {                        // the 2 blocks of this lane's piece
            const uint4 tl = lds128(lut_base + ((((fl >> b) & 1u) << 7) | ((sl >> (8 * b)) & 0x7fu)) * 16);
            const uint4 th = lds128(lut_base + ((((fh >> b) & 1u) << 7) | ((sh >> (8 * b)) & 0x7fu)) * 16);
#pragma unroll
            for (int half = 0; half < 2; ++half) {           // 8 elements = 2 MMAs
                const int i = 2 * b + half;                  // word index inside the piece
                uint32_t pl[4], ph[4];
                decode8(i == 0 ? cl.x : i == 1 ? cl.y : i == 2 ? cl.z : cl.w, tl, pl);
                decode8(i == 0 ? ch.x : i == 1 ? ch.y : i == 2 ? ch.z : ch.w, th, ph);
#pragma unroll
                for (int nt = 0; nt < kNTiles; ++nt) {
                    uint4 xv = make_uint4(0, 0, 0, 0);
                    if (x_ok[nt]) xv = lds128(base + i * x_chunk + (g + 8 * nt) * 64 + t * 16);
                    mma_bf16(acc[nt], pl[0], ph[0], pl[1], ph[1], xv.x, xv.y);
                    mma_bf16(acc[nt], pl[2], ph[2], pl[3], ph[3], xv.z, xv.w);
                }
            }
        }
    }
    cp_async_wait<0>();

    // accumulator fragment: c0,c1 = (row g, batch 2t, 2t+1); c2,c3 = (row g+8, same batches)
    constexpr int kCols = 8 * kNTiles;
#pragma unroll
    for (int nt = 0; nt < kNTiles; ++nt) {
        float* rw = red + warp * kRowsPerCta * kCols;
        rw[g * kCols + 8 * nt + 2 * t] = acc[nt][0];
        rw[g * kCols + 8 * nt + 2 * t + 1] = acc[nt][1];
        rw[(g + 8) * kCols + 8 * nt + 2 * t] = acc[nt][2];
        rw[(g + 8) * kCols + 8 * nt + 2 * t + 1] = acc[nt][3];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < kRowsPerCta * kCols; idx += kWarps * 32) {
        const int r = idx % kRowsPerCta, b = idx / kRowsPerCta;
        if (b >= a.m || row0 + r >= a.n) continue;
        float sum = red[r * kCols + b];
#pragma unroll
        for (int w = 1; w < kWarps; ++w) sum += red[(w * kRowsPerCta + r) * kCols + b];
        if (a.out_dtype == MIXFP4_F32) static_cast<float*>(a.y)[(int64_t)b * a.ldy + row0 + r] = sum;
        else static_cast<__nv_bfloat16*>(a.y)[(int64_t)b * a.ldy + row0 + r] = __float2bfloat16_rn(sum);
    }
}

template <int kWarps, int kNTiles>
int launch_async(const GemvArgs& a, cudaStream_t st) {
    const int64_t ctas = (a.n + kRowsPerCta - 1) / kRowsPerCta;
    const size_t smem = 4096 + (size_t)kWarps * kRowsPerCta * 8 * kNTiles * 4 +
                        (size_t)kWarps * kDepth * stage_bytes(a.m) + (size_t)kRowsPerCta * (a.kpad / 128);
    if (smem > 200 * 1024) return MIXFP4_E_SHAPE;
    static bool configured = false;          // per instantiation
    if (!configured) {
        MIXFP4_CUDA_CHECK(cudaFuncSetAttribute(gemv_async_kernel<kWarps, kNTiles>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        configured = true;
    }
    gemv_async_kernel<kWarps, kNTiles><<<(unsigned)ctas, kWarps * 32, smem, st>>>(a);
    return check_launch("gemv_async_kernel");
}

template <int kWarps>
int launch(const GemvArgs& a, cudaStream_t st) {
    const int64_t ctas = (a.n + kRowsPerCta - 1) / kRowsPerCta;
    const unsigned grid = (unsigned)ctas, block = kWarps * 32;
    if (a.m <= 8) gemv_kernel<kWarps, 1, false><<<grid, block, 0, st>>>(a);
    else gemv_kernel<kWarps, 2, false><<<grid, block, 0, st>>>(a);
    return check_launch("gemv_kernel");
}

}  // namespace
}  // namespace mixfp4

using namespace mixfp4;

extern "C" int mixfp4_gemv(const void* x, int64_t m, int64_t ldx, const uint8_t* codes, const uint8_t* scales,
                           const uint8_t* fmt, const float* global_scale, int64_t n, int64_t k, void* y,
                           int out_dtype, int64_t ldy, void* stream) {
    if (!x || !codes || !scales || !fmt || !global_scale || !y) return MIXFP4_E_NULL;
    if (m < 1 || m > 16 || n <= 0 || k <= 0 || ldx < k || ldy < n) return MIXFP4_E_SHAPE;
    if (out_dtype != MIXFP4_F32 && out_dtype != MIXFP4_BF16) return MIXFP4_E_DTYPE;
    if (!aligned(codes, 16) || !aligned(scales, 8) || !aligned(x, 2)) return MIXFP4_E_ALIGN;
    // the kernel addresses the packed arrays and x with 32-bit offsets
    if (n * (padded_k(k) / 2) > 0xffffffffLL || m * ldx > 0xffffffffLL || n > 0x7fffffffLL - 16) return MIXFP4_E_SHAPE;
    GemvArgs a;
    a.x = static_cast<const __nv_bfloat16*>(x);
    a.m = m; a.ldx = ldx;
    a.codes = codes; a.scales = scales; a.fmt = fmt; a.global_scale = global_scale;
    a.n = n; a.k = k; a.kpad = padded_k(k);
    a.y = y; a.out_dtype = out_dtype; a.ldy = ldy;
    a.x_vec = aligned(x, 16) && (ldx % 8 == 0) && (k % 8 == 0);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!a.x_vec) return launch<8>(a, st);     // unaligned x: synchronous-load variant
    int warps = (a.kpad / kStepK >= 32 && m <= 4) ? 16 : 8;
    if (const char* e = getenv("MIXFP4_GEMV_WARPS")) warps = atoi(e);   // TEMP tuning knob
    if (m <= 8) return warps == 16 ? launch_async<16, 1>(a, st) : launch_async<8, 1>(a, st);
    return warps == 16 ? launch_async<16, 2>(a, st) : launch_async<8, 2>(a, st);
}
