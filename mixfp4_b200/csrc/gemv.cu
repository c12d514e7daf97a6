// Decode-shape dequant-linear (1 <= M <= 16): y[M,N] = x[M,K] * W[N,K]^T, W in the packed
// mixed-FP4 layout.  Replaces F.linear on the dequantized weight
// (project_quant/modeling.py:629 + nn.Linear.forward).  HBM-bound by design: the packed
// weight (0.5703 B/element) is read exactly once, x stays in L1/L2.
//
// Two kernels share the work split below.  gemv_sm_kernel (further down) is the main one: one
// persistent CTA per SM, kernel layout, x resident in shared memory, an eightfold decode table;
// it also carries the grouped launch (several weights that share x) and the row-parallel form
// with the all-reduce in its epilogue.  gemv_kernel (first) serves the canonical layout and
// activations too large for shared memory, with two or three CTAs per SM.
//
// Work split.  A row tile is 16 consecutive weight rows; the warps of a CTA (or of a warp group)
// split its K range in interleaved 128-element steps and their partial sums are added in a fixed
// order through shared memory (deterministic).  CTAs are persistent and walk over row tiles.
// Inside a warp a 16 x 128 step is laid over the mma.sync.m16n8k16 A-fragment: lane (g, t) =
// (lane/4, lane%4) owns rows g and g+8 and the 32 consecutive K elements starting at 32*t.  The
// k index of an MMA is only a summation label, so the 16 k-slots of every MMA are filled with
// whatever 4 consecutive elements each lane decodes next; the B fragment takes the same 4
// elements of x (batch row g).  Two accumulator sets alternate to shorten the MMA dependency
// chain.  The limiter is the ALU pipe (the byte-permute decode), then the shared-memory data path.
//
// Data movement.  Every warp runs its own ring of cp.async stages: per step a lane copies its
// 2 x 16 B of codes and (two lanes of each quad) the 8 scale bytes of a row, a few steps ahead
// of the arithmetic and across tile boundaries, so the weight stream never drains.  x is
// copied into shared memory once per CTA when M*K is small (decode), else staged per step like
// the weights.  With MIXFP4_FLAG_OVERLAP_PREVIOUS the kernel is launched as a programmatic
// dependent: weight copies start while the previous kernel drains, x is touched only after
// griddepcontrol.wait.
//
// Decode.  A 256-entry table (from mixfp4_decode_table, or built here) maps
// (format bit, E4M3 scale byte) to the block's eight magnitudes
// bf16((level * scale) * global) -- exactly the reference's dequantized weight.  Eight
// 4-bit codes (one 32-bit word) become four bf16x2 registers with byte permutes
// (decode.cuh).  The accumulation is the tensor core's fp32.

#include "gemv_common.cuh"

namespace mixfp4 {
namespace {

template <int kWarps, int kNTiles, bool kKL, int kU, int kDepth, bool kXRes, int kMinCtas>
__global__ void __launch_bounds__(kWarps * 32, kMinCtas) gemv_kernel(const GemvArgs a) {
    extern __shared__ __align__(16) uint8_t smem[];
    // lut kLutBytes | red 2*kWarps*16*8*kNTiles*4 | rings kWarps*kDepth*kU*stage | (canonical) fmt bytes 16*ld_fmt
    constexpr int kCols = 8 * kNTiles;
    constexpr int kRedBytes = 2 * kWarps * kRowsPerCta * kCols * 4;
    float* red = reinterpret_cast<float*>(smem + kLutBytes);
    const uint32_t x_bytes = kXRes ? 0u : (uint32_t)a.m * 256u, stage = stage_bytes(a.m, kXRes);
    const uint32_t off_codes = x_bytes, off_scales = x_bytes + 1024u, x_chunk = (uint32_t)a.m * 64u;
    uint8_t* fmt_tab = smem + kLutBytes + kRedBytes + kWarps * kDepth * kU * stage;
    // resident x (if any) sits after the format bytes, 16-byte aligned
    const uint32_t xres_off = ((uint32_t)kLutBytes + kRedBytes + kWarps * kDepth * kU * stage +
                               (kKL ? 0u : (uint32_t)kRowsPerCta * (uint32_t)(a.kpad >> 7)) + 15u) & ~15u;
    const uint32_t xres_rs = xres_row_bytes(a.kpad);

    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;   // provably warp-uniform
    const int g = lane >> 2, t = lane & 3;
    const uint32_t ld_codes = (uint32_t)(a.kpad >> 1), ld_scales = (uint32_t)(a.kpad >> 4);
    const uint32_t ld_fmt = (uint32_t)(a.kpad >> 7);
    const int subs = static_cast<int>(a.kpad / kStepK);     // 128-element sub-steps along K
    const int steps = (subs + kU - 1) / kU;                 // steps of a tile
    const int spw = (steps + kWarps - 1) / kWarps;          // steps per warp and tile (some may be empty)
    const uint32_t last_row = (uint32_t)a.n - 1;
    const int ntiles = static_cast<int>((a.n + kRowsPerCta - 1) / kRowsPerCta);
    const uint32_t lut_base = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t ring = lut_base + kLutBytes + kRedBytes + warp * kDepth * kU * stage;
    const uint32_t k_lim = (uint32_t)a.k;
    const bool full_k = a.k == a.kpad;                      // no K tail: every x chunk is in range
    bool x_ok[kNTiles];
    const __nv_bfloat16* xptr[kNTiles];
    uint32_t xrow_off[kNTiles];
#pragma unroll
    for (int nt = 0; nt < kNTiles; ++nt) {
        x_ok[nt] = g + 8 * nt < a.m;
        xptr[nt] = a.x + (size_t)(x_ok[nt] ? g + 8 * nt : 0) * a.ldx + t * 32;
        if (kXRes) xrow_off[nt] = (x_ok[nt] ? (uint32_t)(g + 8 * nt) * xres_rs : 0u) + t * 64;
        else xrow_off[nt] = (x_ok[nt] ? (uint32_t)(g + 8 * nt) * 64u : 0u) + t * 16;
    }

    // The CTA walks over row tiles blockIdx.x, blockIdx.x + gridDim.x, ...; every warp sees the
    // flat sequence (tile, its j-th step of that tile) and prefetches kDepth-1 entries ahead of
    // the arithmetic, across tile boundaries, so the weight stream never drains.
    // Prefetch cursor:
    int p_tile = blockIdx.x, p_j = 0;
    const uint8_t* pc[2] = {a.codes, a.codes};
    const uint8_t* ps = a.scales;
    auto set_rows = [&]() {     // rows past N re-read the last row; their sums are never stored
        if (a.stream) {         // chunk (tile, sub): codes [16 rows][64 B], then scales [16 rows][8 B]
            const uint8_t* tb = a.codes + (size_t)p_tile * subs * kChunkBytes;
            pc[0] = tb + lane * 16;
            pc[1] = tb + 512 + lane * 16;
            ps = tb + kChunkCodeBytes + (g + 8 * t) * 8;
            return;
        }
        const uint32_t row0 = (uint32_t)p_tile * kRowsPerCta;
        const uint32_t r0 = min(row0 + g, last_row), r1 = min(row0 + g + 8, last_row);
        pc[0] = a.codes + (size_t)r0 * ld_codes + t * 16;
        pc[1] = a.codes + (size_t)r1 * ld_codes + t * 16;
        ps = a.scales + (size_t)(t == 0 ? r0 : r1) * ld_scales;   // used by lanes t < 2
    };
    const uint32_t slot_bytes = kU * stage;
    auto issue_weights = [&](int step, uint32_t slot) {
#pragma unroll
        for (int j = 0; j < kU; ++j) {
            const int sub = step * kU + j;
            if (sub >= subs) break;
            const uint32_t base = ring + slot * slot_bytes + j * stage;
#pragma unroll
            for (int h = 0; h < 2; ++h)
                cp_async16_stream(base + off_codes + h * 512 + lane * 16, pc[h] + (size_t)sub * a.code_step);
            if (t < 2) cp_async8(base + off_scales + (g + 8 * t) * 8, ps + (size_t)sub * a.scale_step);
        }
    };
    auto issue_x = [&](int step, uint32_t slot) {
#pragma unroll
        for (int j = 0; j < kU; ++j) {
            const int sub = step * kU + j;
            if (sub >= subs) break;
            const uint32_t base = ring + slot * slot_bytes + j * stage;
#pragma unroll
            for (int nt = 0; nt < kNTiles; ++nt) {
                if (!x_ok[nt]) continue;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint32_t kk = (uint32_t)sub * kStepK + t * 32 + c * 8;
                    const uint32_t dst = base + c * x_chunk + (g + 8 * nt) * 64 + t * 16;
                    const __nv_bfloat16* src = xptr[nt] + (size_t)sub * kStepK + c * 8;
                    if (a.x_vec && full_k) {
                        cp_async16(dst, src, 16u);
                    } else if (a.x_vec) {   // K % 8 == 0: a chunk is all inside or all outside (zero-filled)
                        const bool in = kk < k_lim;
                        cp_async16(dst, in ? static_cast<const void*>(src) : static_cast<const void*>(a.x), in ? 16u : 0u);
                    } else {         // unaligned x: plain guarded loads, stored by the lane that reads them back
                        uint32_t e[8];
#pragma unroll
                        for (int q = 0; q < 8; ++q) e[q] = kk + q < k_lim ? __bfloat16_as_ushort(src[q]) : 0u;
                        sts128(dst, make_uint4(e[0] | (e[1] << 16), e[2] | (e[3] << 16), e[4] | (e[5] << 16), e[6] | (e[7] << 16)));
                    }
                }
            }
        }
    };
    // Issue the entry under the prefetch cursor (if any) into `slot`, then advance the cursor.
    auto prefetch = [&](uint32_t slot, bool weights, bool xs) {
        if (p_tile < ntiles) {
            const int step = warp + p_j * kWarps;
            if (step < steps) {
                if (weights) issue_weights(step, slot);
                if (xs && !kXRes) issue_x(step, slot);
            }
        }
    };
    auto advance = [&]() {
        if (++p_j == spw) { p_j = 0; p_tile += gridDim.x; if (p_tile < ntiles) set_rows(); }
    };

    // Prologue.  Weights first: they never depend on the previous kernel in the stream.
    set_rows();
#pragma unroll
    for (int d = 0; d < kDepth - 1; ++d) { prefetch(d, true, false); advance(); }
    {
        const float gs = a.lut ? 0.0f : *a.global_scale;
        for (int e = threadIdx.x; e < 256; e += kWarps * 32) {
            const uint4 v = a.lut ? __ldg(a.lut + e) : make_lut_entry(e & 127, e >> 7, gs);
#pragma unroll
            for (int r = 0; r < kLutRep; ++r) sts128(lut_base + e * (16 * kLutRep) + r * 16, v);
        }
    }
    if constexpr (!kKL) {   // canonical layout: the host launches one tile per CTA
        const uint32_t row0 = blockIdx.x * kRowsPerCta;
        for (uint32_t i = threadIdx.x; i < kRowsPerCta * ld_fmt; i += kWarps * 32) {
            const uint32_t r = min(row0 + i / ld_fmt, last_row);
            fmt_tab[i] = __ldg(a.fmt + (size_t)r * ld_fmt + i % ld_fmt);
        }
    }
    // x may be the previous kernel's output: wait for it (no-op without the launch attribute),
    // and let the next kernel in the stream start its own weight prefetch.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if constexpr (kXRes) {   // the whole x (m rows, zero-filled to kpad) once per CTA
        const uint32_t chunks_per_row = (uint32_t)(a.kpad >> 3);
        const uint32_t xres_base = lut_base + xres_off;
        for (uint32_t i = threadIdx.x; i < (uint32_t)a.m * chunks_per_row; i += kWarps * 32) {
            const uint32_t r = i / chunks_per_row, c = i - r * chunks_per_row;
            const uint32_t dst = xres_base + r * xres_rs + c * 16;
            const __nv_bfloat16* src = a.x + (size_t)r * a.ldx + c * 8;
            if (a.x_vec) {
                const bool in = c * 8 < k_lim;
                cp_async16(dst, in ? static_cast<const void*>(src) : static_cast<const void*>(a.x), in ? 16u : 0u);
            } else {
                uint32_t e[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) e[q] = c * 8 + q < k_lim ? __bfloat16_as_ushort(src[q]) : 0u;
                sts128(dst, make_uint4(e[0] | (e[1] << 16), e[2] | (e[3] << 16), e[4] | (e[5] << 16), e[6] | (e[7] << 16)));
            }
        }
    }
    p_tile = blockIdx.x; p_j = 0;
    set_rows();
#pragma unroll
    for (int d = 0; d < kDepth - 1; ++d) {
        prefetch(d, false, true);
        advance();
        cp_async_commit();                 // group d: x of entry d (+ every earlier copy)
    }
    cp_async_wait<kDepth - 2>();           // table copies (part of the first group) have landed
    __syncthreads();

    float acc[kNTiles][2][4];           // two independent accumulation chains per output tile
#pragma unroll
    for (int nt = 0; nt < kNTiles; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][0][i] = acc[nt][1][i] = 0.0f;
    const uint32_t xres_base = lut_base + xres_off;

    uint32_t use_slot = 0, fill_slot = kDepth - 1, parity = 0;
    for (int c_tile = blockIdx.x; c_tile < ntiles; c_tile += gridDim.x) {
        for (int c_j = 0; c_j < spw; ++c_j) {
            // the slot written now was read in the previous iteration: all lanes must be done with it
            __syncwarp();
            prefetch(fill_slot, true, true);
            advance();
            cp_async_commit();
            cp_async_wait<kDepth - 1>();
            __syncwarp();                                    // scale bytes come from another lane's copy
            const int step = warp + c_j * kWarps;
            if (step < steps) {
#pragma unroll
                for (int j = 0; j < kU; ++j) {
                    const int sub = step * kU + j;
                    if (sub >= subs) break;
                    const uint32_t base = ring + use_slot * slot_bytes + j * stage;
                    const uint4 cl = lds128(base + off_codes + lane * 16);
                    const uint4 ch = lds128(base + off_codes + 512 + lane * 16);
                    uint32_t sl = lds16(base + off_scales + g * 8 + t * 2);
                    uint32_t sh = lds16(base + off_scales + (g + 8) * 8 + t * 2);
                    if constexpr (!kKL) {   // canonical: merge the format bits into bit 7 of each scale byte
                        const uint32_t fl = fmt_tab[g * ld_fmt + sub] >> (2 * t);
                        const uint32_t fh = fmt_tab[(g + 8) * ld_fmt + sub] >> (2 * t);
                        sl = (sl & 0x7f7fu) | ((fl & 1u) << 7) | ((fl & 2u) << 14);
                        sh = (sh & 0x7f7fu) | ((fh & 1u) << 7) | ((fh & 2u) << 14);
                    }
#pragma unroll
                    for (int b = 0; b < 2; ++b) {                    // the 2 blocks of this lane's piece
                        const uint4 tl = lds128(lut_base + ((sl >> (8 * b)) & 0xffu) * (16 * kLutRep) + (t % kLutRep) * 16);
                        const uint4 th = lds128(lut_base + ((sh >> (8 * b)) & 0xffu) * (16 * kLutRep) + (t % kLutRep) * 16);
#pragma unroll
                        for (int half = 0; half < 2; ++half) {       // 8 elements = 2 MMAs
                            const int i = 2 * b + half;              // word index inside the piece
                            uint32_t pl[4], ph[4];
                            decode_word<kKL>(i == 0 ? cl.x : i == 1 ? cl.y : i == 2 ? cl.z : cl.w, tl, pl);
                            decode_word<kKL>(i == 0 ? ch.x : i == 1 ? ch.y : i == 2 ? ch.z : ch.w, th, ph);
#pragma unroll
                            for (int nt = 0; nt < kNTiles; ++nt) {
                                // lanes of absent batch rows re-read row 0 (same address: a broadcast);
                                // their accumulator columns are never stored
                                const uint4 xv = kXRes ? lds128(xres_base + xrow_off[nt] + (uint32_t)sub * 256u + i * 16)
                                                       : lds128(base + i * x_chunk + xrow_off[nt]);
                                mma_bf16(acc[nt][0], pl[0], ph[0], pl[1], ph[1], xv.x, xv.y);
                                mma_bf16(acc[nt][1], pl[2], ph[2], pl[3], ph[3], xv.z, xv.w);
                            }
                        }
                    }
                }
            }
            use_slot = use_slot + 1 == kDepth ? 0 : use_slot + 1;
            fill_slot = fill_slot + 1 == kDepth ? 0 : fill_slot + 1;
        }

        // Tile done: add the warps' partial sums in a fixed order.  The buffer alternates between
        // tiles, so one barrier per tile is enough.
        // accumulator fragment: c0,c1 = (row g, batch 2t, 2t+1); c2,c3 = (row g+8, same batches)
        float* rbuf = red + parity * (kWarps * kRowsPerCta * kCols);
#pragma unroll
        for (int nt = 0; nt < kNTiles; ++nt) {
            float* rw = rbuf + warp * kRowsPerCta * kCols;
            rw[g * kCols + 8 * nt + 2 * t] = acc[nt][0][0] + acc[nt][1][0];
            rw[g * kCols + 8 * nt + 2 * t + 1] = acc[nt][0][1] + acc[nt][1][1];
            rw[(g + 8) * kCols + 8 * nt + 2 * t] = acc[nt][0][2] + acc[nt][1][2];
            rw[(g + 8) * kCols + 8 * nt + 2 * t + 1] = acc[nt][0][3] + acc[nt][1][3];
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[nt][0][i] = acc[nt][1][i] = 0.0f;
        }
        __syncthreads();
        const uint32_t row0 = (uint32_t)c_tile * kRowsPerCta;
        for (int idx = threadIdx.x; idx < kRowsPerCta * kCols; idx += kWarps * 32) {
            const int r = idx % kRowsPerCta, b = idx / kRowsPerCta;
            if (b >= a.m || row0 + r >= a.n) continue;
            float sum = rbuf[r * kCols + b];
#pragma unroll
            for (int w = 1; w < kWarps; ++w) sum += rbuf[(w * kRowsPerCta + r) * kCols + b];
            if (a.out_dtype == MIXFP4_F32) static_cast<float*>(a.y)[(int64_t)b * a.ldy + row0 + r] = sum;
            else static_cast<__nv_bfloat16*>(a.y)[(int64_t)b * a.ldy + row0 + r] = __float2bfloat16_rn(sum);
        }
        parity ^= 1u;
    }
    cp_async_wait<0>();
}

template <int kWarps, int kNTiles, bool kKL, int kU, int kDepth, bool kXRes, int kMinCtas>
int launch(const GemvArgs& a, int flags, cudaStream_t st) {
    constexpr int ctas_per_sm = kMinCtas;
    const int64_t tiles = (a.n + kRowsPerCta - 1) / kRowsPerCta;
    // kernel layout: persistent CTAs stream over several row tiles each; the canonical layout
    // keeps per-CTA format bytes in shared memory, so one tile per CTA
    int64_t ctas = tiles;
    if (kKL && ctas > (int64_t)ctas_per_sm * 148) ctas = (int64_t)ctas_per_sm * 148;
    const size_t smem = kLutBytes + 2 * (size_t)kWarps * kRowsPerCta * 8 * kNTiles * 4 +
                        (size_t)kWarps * kDepth * kU * stage_bytes(a.m, kXRes) +
                        (kKL ? 0 : (size_t)kRowsPerCta * (a.kpad / 128)) + 16 +
                        (kXRes ? (size_t)a.m * xres_row_bytes(a.kpad) : 0);
    if (smem > 200 * 1024 || ctas > 0x7fffffffLL) return MIXFP4_E_SHAPE;
    static unsigned long long configured = 0;          // one per instantiation, one bit per device
    if (const int rc = ensure_dynamic_smem(gemv_kernel<kWarps, kNTiles, kKL, kU, kDepth, kXRes, kMinCtas>, 200 * 1024, configured))
        return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctas);
    cfg.blockDim = dim3(kWarps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (flags & MIXFP4_FLAG_OVERLAP_PREVIOUS) ? 1 : 0;
    MIXFP4_CUDA_CHECK(cudaLaunchKernelEx(&cfg, gemv_kernel<kWarps, kNTiles, kKL, kU, kDepth, kXRes, kMinCtas>, a));
    return MIXFP4_OK;
}

// ------------------------------------------------------------------------------------------
// One CTA per SM, several warp groups (kernel layout, x resident, M <= 8).
//
// The shared-memory data path, not the arithmetic, limits the kernel above: of about 100
// shared-memory wavefronts per warp and 128-element step, 43 are the four random table
// look-ups (lanes of a quarter-warp collide on banks) and 16 are x loads that lanes of
// unused batch columns do not need.  Here the CTA owns the SM: one decode table holds every
// entry eight times, copy j in bank group j (entry e, copy j at e*128 + j*16), and a lane
// reads copy (lane & 7), so a quarter-warp never collides; x is loaded only by the lanes
// whose MMA column is a real batch row.  kGroups groups of kGW warps each work on their own
// row tile (tile = blockIdx.x + gridDim.x * (group + kGroups * i)), split K between the
// group's warps as above and synchronise with a named barrier per group.
// Up to kMaxSegments weights that share x (q/k/v, gate/up) run as one launch: their row tiles
// are numbered through, every segment has its own table in shared memory.
constexpr int kMaxSegments = 3;

struct GemvSegment {
    const uint8_t* codes;
    const uint8_t* scales;
    const float* global_scale;
    const uint4* lut;                      // optional prebuilt decode table
    void* y;
    int64_t ldy;
    int n;
    int tile_end;                          // first tile index after this segment's tiles
};
struct GemvSmArgs {
    const __nv_bfloat16* x;
    int64_t ldx, k, kpad;
    int m, nseg, ntiles, out_dtype;
    bool x_vec;
    GemvSegment seg[kMaxSegments];
    AllReduceArgs ar;            // used by the all-reduce instantiation only
};
constexpr uint32_t kStageSm = 1024u + 128u;          // codes [row half][lane] 16 B, scales [row] 8 B

__host__ __device__ inline uint32_t red_bytes_sm(int groups, int gw, int64_t m) {
    return (uint32_t)(groups * 2 * gw * kRowsPerCta * (int)m * 4);
}

// kNT: MMA column tiles (8 batch rows each).  kLutRep: copies of the decode table (8: no bank
// conflicts; 1: 9..16 batch rows, where x takes the shared memory the copies would need).
template <int kGroups, int kGW, int kDepth, bool kAR = false, int kNT = 1, int kLutRep = 8>
__global__ void __launch_bounds__(kGroups * kGW * 32, 1) gemv_sm_kernel(const GemvSmArgs a) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int kThreadsSm = kGroups * kGW * 32;
    // the warp index through a shuffle: the compiler then knows it is warp-uniform and keeps the loop
    // and ring bookkeeping that derives from it on the uniform datapath, off the (saturated) ALU pipe
    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    const int grp = warp / kGW, gw = warp % kGW;
    const int g = lane >> 2, t = lane & 3;
    const int m = a.m;
    const uint32_t xres_rs = xres_row_bytes(a.kpad);
    const uint32_t x_bytes = ((uint32_t)m * xres_rs + 15u) & ~15u;
    const uint32_t lut_base = (uint32_t)__cvta_generic_to_shared(smem);
    constexpr uint32_t kLutBytesSm = 256u * 16u * kLutRep;
    const uint32_t x_base = lut_base + a.nseg * kLutBytesSm;
    float* red = reinterpret_cast<float*>(smem + a.nseg * kLutBytesSm + x_bytes) + grp * (2 * kGW * kRowsPerCta * m);
    const uint32_t ring = x_base + x_bytes + red_bytes_sm(kGroups, kGW, m) + warp * kDepth * kStageSm;

    const uint32_t ld_codes = (uint32_t)(a.kpad >> 1), ld_scales = (uint32_t)(a.kpad >> 4);
    const int subs = static_cast<int>(a.kpad / kStepK);
    const int spw = (subs + kGW - 1) / kGW;                  // steps per warp and tile
    const int ntiles = a.ntiles;
    const int tile0 = blockIdx.x + gridDim.x * grp, tile_stride = gridDim.x * kGroups;
    const uint32_t k_lim = (uint32_t)a.k;
    bool x_ok[kNT];                                          // this lane's MMA column is a batch row
    uint32_t xrow_off[kNT];
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) {
        x_ok[nt] = g + 8 * nt < m;
        xrow_off[nt] = (x_ok[nt] ? (uint32_t)(g + 8 * nt) * xres_rs : 0u) + t * 64;
    }
    const uint32_t lut_lane = lut_base + (lane & (kLutRep - 1)) * 16;

    int p_tile = tile0, p_j = 0;
    const uint8_t* pc[2] = {a.seg[0].codes, a.seg[0].codes};
    const uint8_t* ps = a.seg[0].scales;
    auto set_rows = [&]() {     // rows past N re-read the last row; their sums are never stored
        const int s = (p_tile >= a.seg[0].tile_end) + (p_tile >= a.seg[1].tile_end);
        const int first = s == 0 ? 0 : s == 1 ? a.seg[0].tile_end : a.seg[1].tile_end;
        const uint8_t* codes = s == 0 ? a.seg[0].codes : s == 1 ? a.seg[1].codes : a.seg[2].codes;
        const uint8_t* scales = s == 0 ? a.seg[0].scales : s == 1 ? a.seg[1].scales : a.seg[2].scales;
        const uint32_t last_row = (uint32_t)(s == 0 ? a.seg[0].n : s == 1 ? a.seg[1].n : a.seg[2].n) - 1;
        const uint32_t row0 = (uint32_t)(p_tile - first) * kRowsPerCta;
        const uint32_t r0 = min(row0 + g, last_row), r1 = min(row0 + g + 8, last_row);
        pc[0] = codes + (size_t)r0 * ld_codes + t * 16;
        pc[1] = codes + (size_t)r1 * ld_codes + t * 16;
        ps = scales + (size_t)(t == 0 ? r0 : r1) * ld_scales;   // used by lanes t < 2
    };
    auto prefetch = [&](uint32_t slot_off) {
        if (p_tile < ntiles) {
            const int sub = gw + p_j * kGW;
            if (sub < subs) {
                const uint32_t base = ring + slot_off;
#pragma unroll
                for (int h = 0; h < 2; ++h) cp_async16_stream(base + h * 512 + lane * 16, pc[h] + (size_t)sub * 64);
                if (t < 2) cp_async8(base + 1024 + (g + 8 * t) * 8, ps + (size_t)sub * 8);
            }
        }
        if (++p_j == spw) { p_j = 0; p_tile += tile_stride; if (p_tile < ntiles) set_rows(); }
    };

    // Prologue.  Weights first: they never depend on the previous kernel in the stream.
    if (p_tile < ntiles) set_rows();
#pragma unroll
    for (int d = 0; d < kDepth - 1; ++d) { prefetch(d * kStageSm); cp_async_commit(); }
    // Table entries go through registers: loaded here, stored after the x copies have been issued,
    // so the two latencies overlap.  (entry, copy) pairs: a warp writes 512 contiguous bytes; the
    // eight lanes that want the same entry share one L1 access (cp.async copies measured slower).
    constexpr int kLutIters = (256 * kLutRep + kThreadsSm - 1) / kThreadsSm;
    uint4 tv[kMaxSegments][kLutIters];
#pragma unroll
    for (int s = 0; s < kMaxSegments; ++s) {
        if (s >= a.nseg) break;
        const uint4* lut = a.seg[s].lut;
        const float gs = lut ? 0.0f : *a.seg[s].global_scale;
#pragma unroll
        for (int it = 0; it < kLutIters; ++it) {
            const int e = min((int)threadIdx.x + it * kThreadsSm, 256 * kLutRep - 1) / kLutRep;
            tv[s][it] = lut ? __ldg(lut + e) : make_lut_entry(e & 127, e >> 7, gs);
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // sequence number of this launch (advanced by the previous launch's last CTA); flags are seq + 1
    uint32_t seq = 0;
    if constexpr (kAR) seq = *reinterpret_cast<volatile uint32_t*>(a.ar.words);
    {   // the whole x (m rows, zero-filled to kpad) once per CTA
        const uint32_t chunks_per_row = (uint32_t)(a.kpad >> 3);
        for (uint32_t i = threadIdx.x; i < (uint32_t)m * chunks_per_row; i += kThreadsSm) {
            const uint32_t r = i / chunks_per_row, c = i - r * chunks_per_row;
            const uint32_t dst = x_base + r * xres_rs + c * 16;
            const __nv_bfloat16* src = a.x + (size_t)r * a.ldx + c * 8;
            if (a.x_vec) {
                const bool in = c * 8 < k_lim;
                cp_async16(dst, in ? static_cast<const void*>(src) : static_cast<const void*>(a.x), in ? 16u : 0u);
            } else {
                uint32_t e[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) e[q] = c * 8 + q < k_lim ? __bfloat16_as_ushort(src[q]) : 0u;
                sts128(dst, make_uint4(e[0] | (e[1] << 16), e[2] | (e[3] << 16), e[4] | (e[5] << 16), e[6] | (e[7] << 16)));
            }
        }
    }
    cp_async_commit();
#pragma unroll
    for (int s = 0; s < kMaxSegments; ++s) {
        if (s >= a.nseg) break;
#pragma unroll
        for (int it = 0; it < kLutIters; ++it) {
            const int i = threadIdx.x + it * kThreadsSm;
            if (i < 256 * kLutRep) sts128(lut_base + s * kLutBytesSm + i * 16, tv[s][it]);
        }
    }
    cp_async_wait<0>();
    __syncthreads();

    float acc[kNT][2][4];                // two independent accumulation chains per column tile
    uint4 xv[kNT];                       // lanes of unused batch columns keep zeros (never stored)
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) {
        xv[nt] = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][0][i] = acc[nt][1][i] = 0.0f;
    }

    uint32_t use_off = 0, fill_off = (kDepth - 1) * kStageSm, parity = 0;
    for (int c_tile = tile0; c_tile < ntiles; c_tile += tile_stride) {
        const int cs = (c_tile >= a.seg[0].tile_end) + (c_tile >= a.seg[1].tile_end);
        const uint32_t lut_seg = lut_lane + cs * kLutBytesSm;
        for (int c_j = 0; c_j < spw; ++c_j) {
            __syncwarp();                // the slot written now was read in the previous iteration
            prefetch(fill_off);
            cp_async_commit();
            cp_async_wait<kDepth - 1>();
            __syncwarp();                // scale bytes come from another lane's copy
            const int sub = gw + c_j * kGW;
            if (sub < subs) {
                const uint32_t base = ring + use_off;
                const uint4 cl = lds128(base + lane * 16);
                const uint4 ch = lds128(base + 512 + lane * 16);
                const uint32_t sl = lds16(base + 1024 + g * 8 + t * 2);
                const uint32_t sh = lds16(base + 1024 + (g + 8) * 8 + t * 2);
#pragma unroll
                for (int b = 0; b < 2; ++b) {                    // the 2 blocks of this lane's piece
                    const uint4 tl = lds128(lut_seg + ((sl >> (8 * b)) & 0xffu) * (16u * kLutRep));
                    const uint4 th = lds128(lut_seg + ((sh >> (8 * b)) & 0xffu) * (16u * kLutRep));
#pragma unroll
                    for (int half = 0; half < 2; ++half) {       // 8 elements = 2 MMAs
                        const int i = 2 * b + half;              // word index inside the piece
                        uint32_t pl[4], ph[4];
                        decode8_kl(i == 0 ? cl.x : i == 1 ? cl.y : i == 2 ? cl.z : cl.w, tl, pl);
                        decode8_kl(i == 0 ? ch.x : i == 1 ? ch.y : i == 2 ? ch.z : ch.w, th, ph);
#pragma unroll
                        for (int nt = 0; nt < kNT; ++nt) {
                            lds128_if(xv[nt], x_base + xrow_off[nt] + (uint32_t)sub * 256u + i * 16, x_ok[nt]);
                            mma_bf16(acc[nt][0], pl[0], ph[0], pl[1], ph[1], xv[nt].x, xv[nt].y);
                            mma_bf16(acc[nt][1], pl[2], ph[2], pl[3], ph[3], xv[nt].z, xv[nt].w);
                        }
                    }
                }
            }
            use_off = use_off + kStageSm == kDepth * kStageSm ? 0 : use_off + kStageSm;
            fill_off = fill_off + kStageSm == kDepth * kStageSm ? 0 : fill_off + kStageSm;
        }

        // Tile done: the group's warps add their partial sums in a fixed order.  The buffer
        // alternates between tiles, so one barrier per tile is enough.
        // accumulator fragment: c0,c1 = (row g, batch 2t, 2t+1); c2,c3 = (row g+8, same batches)
        float* rbuf = red + parity * (kGW * kRowsPerCta * m);
        float* rw = rbuf + gw * kRowsPerCta * m;
#pragma unroll
        for (int nt = 0; nt < kNT; ++nt) {
            const int b0 = 8 * nt + 2 * t;
            if (b0 < m) {
                rw[g * m + b0] = acc[nt][0][0] + acc[nt][1][0];
                rw[(g + 8) * m + b0] = acc[nt][0][2] + acc[nt][1][2];
            }
            if (b0 + 1 < m) {
                rw[g * m + b0 + 1] = acc[nt][0][1] + acc[nt][1][1];
                rw[(g + 8) * m + b0 + 1] = acc[nt][0][3] + acc[nt][1][3];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[nt][0][i] = acc[nt][1][i] = 0.0f;
        }
        asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "n"(kGW * 32) : "memory");
        const int first = cs == 0 ? 0 : cs == 1 ? a.seg[0].tile_end : a.seg[1].tile_end;
        const uint32_t row0 = (uint32_t)(c_tile - first) * kRowsPerCta;
        const uint32_t n_seg = (uint32_t)(cs == 0 ? a.seg[0].n : cs == 1 ? a.seg[1].n : a.seg[2].n);
        void* y_seg = cs == 0 ? a.seg[0].y : cs == 1 ? a.seg[1].y : a.seg[2].y;
        const int64_t ldy = cs == 0 ? a.seg[0].ldy : cs == 1 ? a.seg[1].ldy : a.seg[2].ldy;
        for (int idx = gw * 32 + lane; idx < kRowsPerCta * m; idx += kGW * 32) {
            const int r = idx % kRowsPerCta, b = idx / kRowsPerCta;
            if (row0 + r >= n_seg) continue;
            float sum = rbuf[r * m + b];
#pragma unroll
            for (int w = 1; w < kGW; ++w) sum += rbuf[(w * kRowsPerCta + r) * m + b];
            if constexpr (kAR) {
                const int64_t slot = (int64_t)b * n_seg + row0 + r;
                const int64_t par = (int64_t)(seq & 1u) * a.ar.world * a.ar.slot_packets;
                const uint32_t flag = seq + 1u;
                for (int p = 0; p < a.ar.world; ++p)
                    if (p != a.ar.rank)
                        st_packet(a.ar.peer[p] + par + a.ar.rank * a.ar.slot_packets + slot, __float_as_uint(sum), flag);
                float total = 0.0f;
                for (int src = 0; src < a.ar.world; ++src) {
                    float v = sum;
                    if (src != a.ar.rank) {
                        const uint2* q = a.ar.recv + par + src * a.ar.slot_packets + slot;
                        uint2 pk = ld_packet(q);
                        if (pk.y != flag) {     // bounded wait for the peer's packet
                            const uint64_t t0 = gemv_timer_ns();
                            uint32_t spins = 0;
                            while ((pk = ld_packet(q)).y != flag) {
                                if ((++spins & 63u) == 0 && spins > 4096u && gemv_timer_ns() - t0 > a.ar.wait_ns) {
                                    if (a.ar.status) atomicCAS(a.ar.status, 0, 100 + src);
                                    break;
                                }
                            }
                        }
                        v = __uint_as_float(pk.x);
                    }
                    total = src == 0 ? v : total + v;
                }
                sum = total;
            }
            if (a.out_dtype == MIXFP4_F32) static_cast<float*>(y_seg)[(int64_t)b * ldy + row0 + r] = sum;
            else static_cast<__nv_bfloat16*>(y_seg)[(int64_t)b * ldy + row0 + r] = __float2bfloat16_rn(sum);
        }
        parity ^= 1u;
    }
    cp_async_wait<0>();
    if constexpr (kAR) {   // the last CTA to finish advances the sequence number for the next launch
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            if (atomicAdd(a.ar.words + 1, 1u) == gridDim.x - 1) {
                a.ar.words[1] = 0;
                __threadfence();
                *reinterpret_cast<volatile uint32_t*>(a.ar.words) = seq + 1u;
            }
        }
    }
}

template <int kGroups, int kGW, int kDepth, bool kAR = false, int kNT = 1, int kLutRep = 8>
int launch_sm(const GemvSmArgs& a, int flags, cudaStream_t st) {
    const int64_t ctas = a.ntiles < 148 ? a.ntiles : 148;
    const size_t smem = (size_t)a.nseg * 256 * 16 * kLutRep + (((size_t)a.m * xres_row_bytes(a.kpad) + 15) & ~(size_t)15) +
                        red_bytes_sm(kGroups, kGW, a.m) + (size_t)kGroups * kGW * kDepth * kStageSm;
    if (smem > 227 * 1024) return MIXFP4_E_SHAPE;
    static unsigned long long configured = 0;          // one per instantiation, one bit per device
    if (const int rc = ensure_dynamic_smem(gemv_sm_kernel<kGroups, kGW, kDepth, kAR, kNT, kLutRep>, 227 * 1024, configured))
        return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctas);
    cfg.blockDim = dim3(kGroups * kGW * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (flags & MIXFP4_FLAG_OVERLAP_PREVIOUS) ? 1 : 0;
    MIXFP4_CUDA_CHECK(cudaLaunchKernelEx(&cfg, gemv_sm_kernel<kGroups, kGW, kDepth, kAR, kNT, kLutRep>, a));
    return MIXFP4_OK;
}

// One CTA per SM: three groups of 8 warps when there are row tiles for all of them, else two
// groups of 16 warps (more warps per tile keep the SM busy).
int dispatch_sm(const GemvSmArgs& g, int flags, cudaStream_t st) {
    return g.ntiles >= 2 * 148 ? launch_sm<3, 8, 4>(g, flags, st) : launch_sm<2, 16, 3>(g, flags, st);
}

// Largest configuration whose shared memory (tables + resident x + rings) fits; each launch_sm
// answers MIXFP4_E_SHAPE when it does not, and so does this when nothing fits.
int dispatch_sm_chain(const GemvSmArgs& g, int flags, cudaStream_t st) {
    if (g.m > 8) return launch_sm<2, 8, 3, false, 2, 1>(g, flags, st);               // 9..16 rows: single table copy
    int rc = dispatch_sm(g, flags, st);
    if (rc == MIXFP4_E_SHAPE) rc = launch_sm<3, 8, 3>(g, flags, st);                  // shallower rings
    if (rc == MIXFP4_E_SHAPE) rc = launch_sm<2, 8, 3, false, 1, 1>(g, flags, st);     // single table copy
    return rc;
}

template <bool kKL>
int dispatch(const GemvArgs& a, int flags, cudaStream_t st) {
    // x stays resident in shared memory when it is small (decode at M = 1..4 for Llama shapes)
    const bool xres = (int64_t)a.m * xres_row_bytes(a.kpad) <= 40 * 1024;
    const int64_t tiles = (a.n + kRowsPerCta - 1) / kRowsPerCta;
    if constexpr (kKL) {
        GemvSmArgs g = {};
        g.x = a.x; g.ldx = a.ldx; g.k = a.k; g.kpad = a.kpad;
        g.m = (int)a.m; g.nseg = 1; g.ntiles = (int)tiles; g.out_dtype = a.out_dtype; g.x_vec = a.x_vec;
        g.seg[0] = GemvSegment{a.codes, a.scales, a.global_scale, a.lut, a.y, a.ldy, (int)a.n, (int)tiles};
        g.seg[1] = g.seg[2] = GemvSegment{a.codes, a.scales, a.global_scale, a.lut, a.y, a.ldy, (int)a.n, 0x7fffffff};
        const int rc = dispatch_sm_chain(g, flags, st);
        if (rc != MIXFP4_E_SHAPE) return rc;     // x too large for shared memory: kernels above
    }
    if (a.m > 8) return launch<8, 2, kKL, 1, 3, false, 2>(a, flags, st);
    if (!xres) return launch<8, 1, kKL, 1, 3, false, 2>(a, flags, st);
    // few row tiles: more warps per tile keep the SMs busy; many: three 8-warp CTAs per SM
    if (tiles < 2 * 148) return launch<16, 1, kKL, 1, 3, true, 2>(a, flags, st);
    return launch<8, 1, kKL, 1, 4, true, 3>(a, flags, st);
}

}  // namespace
}  // namespace mixfp4

using namespace mixfp4;

extern "C" int mixfp4_gemv(const void* x, int64_t m, int64_t ldx, const uint8_t* codes, const uint8_t* scales,
                           const uint8_t* fmt, const float* global_scale, int64_t n, int64_t k, int layout,
                           const void* lut, void* y, int out_dtype, int64_t ldy, int flags, void* stream) {
    if (layout != MIXFP4_LAYOUT_CANONICAL && layout != MIXFP4_LAYOUT_KERNEL && layout != MIXFP4_LAYOUT_STREAM)
        return MIXFP4_E_MODE;
    const bool streamed = layout == MIXFP4_LAYOUT_STREAM;
    if (!x || !codes || (!scales && !streamed) || (!fmt && layout == MIXFP4_LAYOUT_CANONICAL) || !global_scale || !y)
        return MIXFP4_E_NULL;
    if (m < 1 || m > 16 || n <= 0 || k <= 0 || ldx < k || ldy < n) return MIXFP4_E_SHAPE;
    if (out_dtype != MIXFP4_F32 && out_dtype != MIXFP4_BF16) return MIXFP4_E_DTYPE;
    if (!aligned(codes, 16) || (!streamed && !aligned(scales, 8)) || !aligned(x, 2) || (lut && !aligned(lut, 16)))
        return MIXFP4_E_ALIGN;
    if (n > 0x7fffffffLL - 16) return MIXFP4_E_SHAPE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (streamed) {
        const mixfp4_gemv_segment seg = {codes, nullptr, global_scale, lut, y, ldy, n};
        const int rc = gemv_stream(x, m, ldx, k, &seg, 1, out_dtype, flags, nullptr, nullptr, st);
        if (rc != MIXFP4_E_SHAPE) return rc;     // x too large for shared memory: the kernel below stages it
    }
    GemvArgs a;
    a.x = static_cast<const __nv_bfloat16*>(x);
    a.m = m; a.ldx = ldx;
    a.codes = codes; a.scales = scales; a.fmt = fmt; a.global_scale = global_scale;
    a.lut = static_cast<const uint4*>(lut);
    a.n = n; a.k = k; a.kpad = padded_k(k);
    a.y = y; a.out_dtype = out_dtype; a.ldy = ldy;
    a.x_vec = aligned(x, 16) && (ldx % 8 == 0) && (k % 8 == 0);
    a.stream = streamed;
    a.code_step = streamed ? kChunkBytes : 64u;
    a.scale_step = streamed ? kChunkBytes : 8u;
    if (streamed) {
        if (a.m > 8) return launch<8, 2, true, 1, 3, false, 2>(a, flags, st);
        return launch<8, 1, true, 1, 3, false, 2>(a, flags, st);
    }
    return layout == MIXFP4_LAYOUT_KERNEL ? dispatch<true>(a, flags, st) : dispatch<false>(a, flags, st);
}

extern "C" int mixfp4_gemv_grouped(const void* x, int64_t m, int64_t ldx, int64_t k,
                                   const mixfp4_gemv_segment* segments, int count, int layout, int out_dtype,
                                   int flags, void* stream) {
    if (layout != MIXFP4_LAYOUT_KERNEL && layout != MIXFP4_LAYOUT_STREAM) return MIXFP4_E_MODE;
    if (!x || !segments) return MIXFP4_E_NULL;
    if (count < 1 || count > kMaxSegments) return MIXFP4_E_SHAPE;
    if (m < 1 || m > 16 || k <= 0 || ldx < k) return MIXFP4_E_SHAPE;
    if (out_dtype != MIXFP4_F32 && out_dtype != MIXFP4_BF16) return MIXFP4_E_DTYPE;
    if (!aligned(x, 2)) return MIXFP4_E_ALIGN;
    if (layout == MIXFP4_LAYOUT_STREAM)
        return gemv_stream(x, m, ldx, k, segments, count, out_dtype, flags, nullptr, nullptr,
                           static_cast<cudaStream_t>(stream));   // MIXFP4_E_SHAPE: x does not fit
    GemvSmArgs g = {};
    g.x = static_cast<const __nv_bfloat16*>(x);
    g.ldx = ldx; g.k = k; g.kpad = padded_k(k);
    g.m = (int)m; g.nseg = count; g.out_dtype = out_dtype;
    g.x_vec = aligned(x, 16) && (ldx % 8 == 0) && (k % 8 == 0);
    int64_t tiles = 0;
    for (int s = 0; s < kMaxSegments; ++s) {
        const mixfp4_gemv_segment& in = segments[s < count ? s : count - 1];
        if (s < count) {
            if (!in.codes || !in.scales || !in.global_scale || !in.y) return MIXFP4_E_NULL;
            if (in.n <= 0 || in.ldy < in.n || in.n > 0x7fffffffLL - 16) return MIXFP4_E_SHAPE;
            if (!aligned(in.codes, 16) || !aligned(in.scales, 8) || (in.lut && !aligned(in.lut, 16))) return MIXFP4_E_ALIGN;
            tiles += (in.n + kRowsPerCta - 1) / kRowsPerCta;
            if (tiles > 0x7ffffff0LL) return MIXFP4_E_SHAPE;
        }
        g.seg[s] = GemvSegment{in.codes, in.scales, in.global_scale, static_cast<const uint4*>(in.lut), in.y, in.ldy,
                               (int)in.n, s < count ? (int)tiles : 0x7fffffff};
    }
    g.ntiles = (int)tiles;
    return dispatch_sm_chain(g, flags, static_cast<cudaStream_t>(stream));   // MIXFP4_E_SHAPE: x does not fit
}

extern "C" int mixfp4_gemv_allreduce(const mixfp4_comm* comm, const void* x, int64_t m, int64_t ldx,
                                     const uint8_t* codes, const uint8_t* scales, const float* global_scale,
                                     const void* lut, int64_t n, int64_t k, int layout, void* y, int out_dtype,
                                     int64_t ldy, int* status, int flags, void* stream) {
    if (layout != MIXFP4_LAYOUT_KERNEL && layout != MIXFP4_LAYOUT_STREAM) return MIXFP4_E_MODE;
    const bool streamed = layout == MIXFP4_LAYOUT_STREAM;
    if (!comm || !x || !codes || (!scales && !streamed) || !global_scale || !y) return MIXFP4_E_NULL;
    if (m < 1 || m > 8 || n <= 0 || k <= 0 || ldx < k || ldy < n || n > 0x7fffffffLL - 16) return MIXFP4_E_SHAPE;
    if (out_dtype != MIXFP4_F32 && out_dtype != MIXFP4_BF16) return MIXFP4_E_DTYPE;
    if (!aligned(codes, 16) || (!streamed && !aligned(scales, 8)) || !aligned(x, 2) || (lut && !aligned(lut, 16)))
        return MIXFP4_E_ALIGN;
    if (streamed) {
        const mixfp4_gemv_segment seg = {codes, nullptr, global_scale, lut, y, ldy, n};
        return gemv_stream(x, m, ldx, k, &seg, 1, out_dtype, flags, comm, status, static_cast<cudaStream_t>(stream));
    }
    GemvSmArgs g = {};
    g.x = static_cast<const __nv_bfloat16*>(x);
    g.ldx = ldx; g.k = k; g.kpad = padded_k(k);
    g.m = (int)m; g.nseg = 1; g.out_dtype = out_dtype;
    g.x_vec = aligned(x, 16) && (ldx % 8 == 0) && (k % 8 == 0);
    if ((int64_t)m * xres_row_bytes(g.kpad) > 40 * 1024) return MIXFP4_E_SHAPE;   // x must fit in shared memory
    const int64_t tiles = (n + kRowsPerCta - 1) / kRowsPerCta;
    g.ntiles = (int)tiles;
    g.seg[0] = GemvSegment{codes, scales, global_scale, static_cast<const uint4*>(lut), y, ldy, (int)n, (int)tiles};
    g.seg[1] = g.seg[2] = GemvSegment{codes, scales, global_scale, static_cast<const uint4*>(lut), y, ldy, (int)n, 0x7fffffff};
    const int rc = comm_view(comm, &g.ar.rank, &g.ar.world, &g.ar.slot_packets, &g.ar.recv, g.ar.peer, &g.ar.words);
    if (rc != MIXFP4_OK) return rc;
    if (m * n > g.ar.slot_packets) return MIXFP4_E_TOO_LARGE;
    g.ar.status = status;
    g.ar.wait_ns = wait_limit_ns();
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return g.ntiles >= 2 * 148 ? launch_sm<3, 8, 4, true>(g, flags, st) : launch_sm<2, 16, 3, true>(g, flags, st);
}
