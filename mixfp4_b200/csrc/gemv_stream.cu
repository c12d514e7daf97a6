// Decode-shape dequant-linear (1 <= M <= 16) on the stream layout of the packed weight:
//   y[M,N] = x[M,K] * W[N,K]^T, replacing F.linear on the dequantized weight
//   (project_quant/modeling.py:629 + nn.Linear.forward).
//
// The stream layout (decode.cuh) stores every 16-row x 128-K step of the weight as one contiguous
// chunk of 1152 bytes (1024 B of codes, 128 B of scale bytes), chunks ordered along K and then by
// row tile.  One persistent CTA per SM takes a contiguous range of row tiles (the ranges differ by
// at most one tile), and the CTA's warps cut that range's chunks into equal contiguous runs, so
// every warp streams one contiguous piece of memory:
//   * lane 0 of a warp keeps kDepth chunks in flight with cp.async.bulk (one instruction per
//     chunk, completion counted on an mbarrier per ring slot); no thread computes addresses of
//     individual rows and nothing is committed or waited per lane;
//   * the 16 x 128 step is laid over the mma.sync.m16n8k16 A fragment exactly as in gemv.cu
//     (lane (g, t) owns rows g, g+8 and 32 consecutive K elements), decoded with the byte-permute
//     table look-up of decode.cuh into the reference's bf16 weights, multiplied with x from shared
//     memory; the accumulators stay in registers across the chunks of a row tile;
//   * a warp whose run covers a whole row tile stores that tile's outputs directly; the partial
//     head and tail of a run go to shared memory (into the warp's own ring once its last chunk has
//     been consumed; the head sums wait in registers until then), and after one barrier the warp
//     that holds the end of a tile adds the partials in warp order (a fixed order: results are
//     deterministic).
// Up to three weights that share x run as one launch (their tiles are numbered through); the
// row-parallel form sends its outputs as packets into the peers' buffers and adds the ranks'
// partial sums in rank order (comm.cu).  Every wait is bounded and reports through a status word.

#include <atomic>
#include <mutex>

#include "gemv_common.cuh"

namespace mixfp4 {
namespace {

constexpr int kMaxSeg = 3;

struct StreamSeg {
    const uint8_t* chunks;
    const float* global_scale;
    const uint4* lut;                      // optional prebuilt decode table
    void* y;
    int64_t ldy;
    int n;
    int tile_end;                          // first tile index after this segment's tiles
};
struct GemvStreamArgs {
    const __nv_bfloat16* x;
    int64_t ldx, k, kpad;
    int m, nseg, ntiles, out_dtype;
    bool x_vec;
    bool wide_lut;                         // every segment's table is followed by its eightfold copy (mixfp4_decode_table_wide)
    StreamSeg seg[kMaxSeg];
    AllReduceArgs ar;                      // used by the all-reduce instantiation only
    int* status;                           // device word: nonzero after an expired wait
    uint64_t wait_ns;                      // limit of every wait on a chunk
};

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
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
// Contiguous global -> shared copy by the bulk-copy engine; both addresses and the size are
// multiples of 16 bytes.  The bytes are counted on the mbarrier.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t lds_u8(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
// Bounded wait for a chunk: false once the limit has passed (and a few thousand polls were made).
__device__ __forceinline__ bool wait_chunk(uint32_t bar, uint32_t parity, uint64_t limit_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = gemv_timer_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity))
        if ((++spins & 255u) == 0 && spins > 4096u && gemv_timer_ns() - t0 > limit_ns) return false;
    return true;
}

// kWarps warps, each with a ring of kDepth chunks.  kNT: MMA column tiles (8 batch rows each).
// kLutRep: copies of the decode table per segment (8: a quarter-warp's look-ups never share a
// bank; fewer when x or several segments need the shared memory).
template <int kWarps, int kDepth, bool kAR, int kNT, int kLutRep>
__global__ void __launch_bounds__(kWarps * 32, 1) gemv_stream_kernel(const GemvStreamArgs a) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int kThreadsS = kWarps * 32;
    constexpr uint32_t kLutBytesS = 256u * 16u * kLutRep;
    constexpr uint32_t kBarBytes = (kWarps * kDepth * 8 + 8 + 127) & ~127;      // the rings' barriers and the tables' one
    // the warp index through a shuffle: provably warp-uniform, so everything derived from it stays
    // on the uniform datapath
    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int m = a.m;
    const int S = static_cast<int>(a.kpad / kChunkK);          // chunks per row tile
    // shared memory: barriers | rings (after the main loop: the warps' partial sums) | tables | x
    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t bars = sbase + warp * (kDepth * 8);
    const uint32_t ring = sbase + kBarBytes + warp * (kDepth * kChunkBytes);
    const uint32_t lut_base = sbase + kBarBytes + kWarps * kDepth * kChunkBytes;
    const uint32_t x_base = lut_base + a.nseg * kLutBytesS;
    const uint32_t xres_rs = xres_row_bytes(a.kpad);
    // partial sums of warp w: [head, tail][16 rows][m] floats at the start of its ring (at most 2 KB of the
    // ring's kDepth * 1152 bytes); written only after the warp's last chunk has been consumed
    constexpr int kPieceStride = kDepth * (int)kChunkBytes / 4;                    // floats from warp to warp
    float* pieces = reinterpret_cast<float*>(smem + kBarBytes);

    // this CTA's row tiles and this warp's run of their chunks
    // (the CTAs with the lowest indices take the odd tiles: under programmatic dependent launch they
    // are the first to get an SM, so the extra work goes where the head start is)
    const int per_cta = a.ntiles / (int)gridDim.x, extra = a.ntiles % (int)gridDim.x;
    const int t0 = (int)blockIdx.x * per_cta + min((int)blockIdx.x, extra);
    const int t1 = t0 + per_cta + ((int)blockIdx.x < extra ? 1 : 0);
    const int nchunks = (t1 - t0) * S;                      // at most 2^31 / kWarps: the host checks
    auto run_start = [&](int w) { return (int)((uint32_t)nchunks * (uint32_t)w / (uint32_t)kWarps); };
    const int wa = run_start(warp), wb = run_start(warp + 1), cnt = wb - wa;

    auto seg_first = [&](int s) { return s == 0 ? 0 : s == 1 ? a.seg[0].tile_end : a.seg[1].tile_end; };
    auto seg_end = [&](int s) { return s == 0 ? a.seg[0].tile_end : s == 1 ? a.seg[1].tile_end : a.seg[2].tile_end; };
    auto seg_chunks = [&](int s) { return s == 0 ? a.seg[0].chunks : s == 1 ? a.seg[1].chunks : a.seg[2].chunks; };
    struct Cursor {
        int tile, sub, seg;
        const uint8_t* ptr;
    };
    auto make_cursor = [&](int local) {
        Cursor c;
        c.tile = t0 + local / S;
        c.sub = local % S;
        c.seg = (c.tile >= a.seg[0].tile_end) + (c.tile >= a.seg[1].tile_end);
        c.ptr = seg_chunks(c.seg) + ((size_t)(c.tile - seg_first(c.seg)) * S + c.sub) * kChunkBytes;
        return c;
    };
    auto advance = [&](Cursor& c) {
        c.ptr += kChunkBytes;
        if (++c.sub == S) {
            c.sub = 0;
            ++c.tile;
            if (c.tile == seg_end(c.seg) && c.seg + 1 < a.nseg) {
                ++c.seg;
                c.ptr = seg_chunks(c.seg);
            }
        }
    };
    auto issue = [&](const Cursor& c, uint32_t slot) {
        if (lane == 0) {
            mbar_expect_tx(bars + slot * 8, kChunkBytes);
            bulk_load(ring + slot * kChunkBytes, c.ptr, kChunkBytes, bars + slot * 8);
        }
    };

    // Prologue.  The next kernel in the stream may be scheduled as soon as every CTA has passed this
    // point (it still waits for this grid's completion before it touches x).  Weights first: they
    // never depend on the previous kernel.  Only the first chunk goes out here: a bulk copy can
    // stall its issuer while the copy engine's queue is full, and nothing below should wait for that;
    // the main loop fills the ring.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // Tables: with the eightfold table in global memory (mixfp4_decode_table_wide) one thread hands each
    // segment's 32 KB to the copy engine before anything else; otherwise every thread loads a few
    // entries and stores their copies.  x goes through cp.async by all threads either way: a bulk copy
    // of x would queue behind the weight chunks already handed to the copy engine.
    const bool bulk = kLutRep == 8 && a.wide_lut;
    const uint32_t bar_lut = sbase + kWarps * kDepth * 8;
    if (lane == 0) {
#pragma unroll
        for (int d = 0; d < kDepth; ++d) mbar_init(bars + d * 8, 1);
        if (warp == kWarps - 1) mbar_init(bar_lut, 1);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the copy engine sees initialised barriers
    }
    __syncwarp();
    Cursor p = make_cursor(wa);
    if (cnt > 0) { issue(p, 0); advance(p); }
    if (bulk && warp == kWarps - 1 && lane == 0) {
        mbar_expect_tx(bar_lut, (uint32_t)a.nseg * kLutBytesS);
        for (int sgm = 0; sgm < a.nseg; ++sgm) {
            const uint4* lut = sgm == 0 ? a.seg[0].lut : sgm == 1 ? a.seg[1].lut : a.seg[2].lut;
            bulk_load(lut_base + sgm * kLutBytesS, reinterpret_cast<const uint8_t*>(lut) + 4096, kLutBytesS, bar_lut);
        }
    }
    if (cnt == 0)                        // a warp without chunks adds zeros where the tile sums are collected
        for (int v = lane; v < kRowsPerCta * m; v += 32) pieces[(size_t)warp * kPieceStride + v] = 0.0f;

    // Without the wide table: entries go through registers, loaded here and stored after the x copies
    // have been issued, so the two latencies overlap.  (entry, copy) pairs: a warp writes 512 contiguous bytes.
    constexpr int kLutIters = (256 * kLutRep + kThreadsS - 1) / kThreadsS;
    uint4 tv[kMaxSeg][kLutIters];
    if (!bulk) {
#pragma unroll
        for (int sgm = 0; sgm < kMaxSeg; ++sgm) {
            if (sgm >= a.nseg) break;
            const uint4* lut = a.seg[sgm].lut;
            const float gs = lut ? 0.0f : *a.seg[sgm].global_scale;
#pragma unroll
            for (int it = 0; it < kLutIters; ++it) {
                const int e = min((int)threadIdx.x + it * kThreadsS, 256 * kLutRep - 1) / kLutRep;
                tv[sgm][it] = lut ? __ldg(lut + e) : make_lut_entry(e & 127, e >> 7, gs);
            }
        }
    }
    // x may be the previous kernel's output: wait for it (no-op without the launch attribute).
    asm volatile("griddepcontrol.wait;" ::: "memory");
    uint32_t seq = 0;       // sequence number of this launch (advanced by the previous launch's last CTA)
    if constexpr (kAR) seq = *reinterpret_cast<volatile uint32_t*>(a.ar.words);
    {   // the whole x (m rows, zero-filled to kpad) once per CTA
        const uint32_t chunks_per_row = (uint32_t)(a.kpad >> 3), k_lim = (uint32_t)a.k;
        for (int r = 0; r < m; ++r) {
            for (uint32_t c = threadIdx.x; c < chunks_per_row; c += kThreadsS) {
                const uint32_t dst = x_base + (uint32_t)r * xres_rs + (c ^ ((c >> 2) & 2u)) * 16;     // see xrow_lo below
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
    }
    cp_async_commit();
    // The rest of the ring, after x has been asked for: a bulk copy stalls its issuer while the copy
    // engine's queue is full (a few microseconds when every warp fills its ring at once), and the
    // first multiply needs only the tables, x and the first chunk.
#pragma unroll
    for (int d = 1; d < kDepth; ++d)
        if (d < cnt) { issue(p, d); advance(p); }
    if (!bulk) {
#pragma unroll
        for (int sgm = 0; sgm < kMaxSeg; ++sgm) {
            if (sgm >= a.nseg) break;
#pragma unroll
            for (int it = 0; it < kLutIters; ++it) {
                const int i2 = threadIdx.x + it * kThreadsS;
                if (i2 < 256 * kLutRep) sts128(lut_base + sgm * kLutBytesS + i2 * 16, tv[sgm][it]);
            }
        }
    }
    cp_async_wait<0>();
    __syncthreads();                     // x and the stored tables; also: the table barrier is initialised
    if (bulk && !wait_chunk(bar_lut, 0, a.wait_ns) && a.status) atomicCAS(a.status, 0, 299);

    // Outputs.  kAR: every value goes as a packet into every rank's buffer (this rank's included)
    // and is added up at the end; else it is stored.
    auto emit = [&](int cs, uint32_t row, int b, float v) {
        const uint32_t n_seg = (uint32_t)(cs == 0 ? a.seg[0].n : cs == 1 ? a.seg[1].n : a.seg[2].n);
        if (row >= n_seg) return;
        if constexpr (kAR) {
            const int64_t slot = (int64_t)b * n_seg + row;
            const int64_t par = (int64_t)(seq & 1u) * a.ar.world * a.ar.slot_packets;
            for (int pr = 0; pr < a.ar.world; ++pr)
                st_packet(a.ar.peer[pr] + par + a.ar.rank * a.ar.slot_packets + slot, __float_as_uint(v), seq + 1u);
        } else {
            void* y = cs == 0 ? a.seg[0].y : cs == 1 ? a.seg[1].y : a.seg[2].y;
            const int64_t ldy = cs == 0 ? a.seg[0].ldy : cs == 1 ? a.seg[1].ldy : a.seg[2].ldy;
            if (a.out_dtype == MIXFP4_F32) static_cast<float*>(y)[(int64_t)b * ldy + row] = v;
            else static_cast<__nv_bfloat16*>(y)[(int64_t)b * ldy + row] = __float2bfloat16_rn(v);
        }
    };

    bool x_ok[kNT];                                          // this lane's MMA column is a batch row
    // x in shared memory: rows of kpad bf16 plus 16 bytes, so that consecutive rows start one 16-byte unit
    // further in the banks, and inside a row unit c sits at c ^ (2 if c & 8): a quarter-warp's 128-bit loads
    // (two rows, units 4 t + w for t = 0..3) then touch eight different units of the 128-byte bank line.
    // A lane reads units w = 0, 1 from xrow_lo and w = 2, 3 from xrow_hi (swapped halves for t >= 2).
    uint32_t xrow_lo[kNT], xrow_hi[kNT];
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) {
        x_ok[nt] = g + 8 * nt < m;
        const uint32_t row_off = x_base + (x_ok[nt] ? (uint32_t)(g + 8 * nt) * xres_rs : 0u) + t * 64;
        xrow_lo[nt] = row_off + (t & 2) * 16;          // units 0, 1 of the lane's four, or 2, 3 swapped in
        xrow_hi[nt] = row_off - (t & 2) * 16;
    }
    const uint32_t lut_lane = lut_base + (lane & (kLutRep - 1)) * 16;
    float acc[kNT][2][4];                // two independent accumulation chains per column tile
    uint4 xv[kNT];                       // lanes of unused batch columns keep zeros (never stored)
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) {
        xv[nt] = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][0][i] = acc[nt][1][i] = 0.0f;
    }

    // Main loop: one row tile (or the part of it inside this run) at a time, its chunks in a counted
    // inner loop.  `issued` chunks have been handed to the copy engine; the cursor p stands at the next.
    Cursor c = make_cursor(wa);
    int issued = cnt < kDepth ? cnt : kDepth, done = 0;
    bool head = true;                    // the sums in the accumulators include this run's first chunk
    bool head_kept = false;              // the run began with a partial tile: its sums wait in head_v
    float head_v[kNT][4];
    int comb_n = 0, comb_seg = 0;        // after the barrier: pieces to add to the first (0: nothing to add up)
    uint32_t comb_row0 = 0;
    const float* comb_first = pieces;
    const float* comb_next = pieces;
    bool ok = true;                      // false after a chunk did not arrive within the wait limit
    uint32_t use = ring, use_bar = bars, phase = 0;          // ring slot of the chunk consumed next
    while (done < cnt) {
        const int sub0 = c.sub;
        const int piece = min(S - sub0, cnt - done);         // chunks of this tile inside the run
        const uint32_t lut_seg = lut_lane + c.seg * kLutBytesS;
        uint32_t xsub = (uint32_t)sub0 * 256u;
        for (int j = 0; j < piece; ++j) {
            if (ok) ok = wait_chunk(use_bar, phase, a.wait_ns);
            const uint4 cl = lds128(use + lane * 16);
            const uint4 ch = lds128(use + 512 + lane * 16);
            const uint32_t sa = use + kChunkCodeBytes + g * 8 + t * 2;
            const uint32_t sl0 = lds_u8(sa), sl1 = lds_u8(sa + 1), sh0 = lds_u8(sa + 64), sh1 = lds_u8(sa + 65);
#pragma unroll
            for (int b = 0; b < 2; ++b) {                    // the 2 blocks of this lane's piece
                const uint4 tl = lds128(lut_seg + (b == 0 ? sl0 : sl1) * (16u * kLutRep));
                const uint4 th = lds128(lut_seg + (b == 0 ? sh0 : sh1) * (16u * kLutRep));
#pragma unroll
                for (int half = 0; half < 2; ++half) {       // 8 elements = 2 MMAs
                    const int w = 2 * b + half;              // word index inside the piece
                    uint32_t pl[4], ph[4];
                    decode8_kl(w == 0 ? cl.x : w == 1 ? cl.y : w == 2 ? cl.z : cl.w, tl, pl);
                    decode8_kl(w == 0 ? ch.x : w == 1 ? ch.y : w == 2 ? ch.z : ch.w, th, ph);
#pragma unroll
                    for (int nt = 0; nt < kNT; ++nt) {
                        if (x_ok[nt]) xv[nt] = lds128((w < 2 ? xrow_lo[nt] : xrow_hi[nt]) + xsub + w * 16);   // other lanes keep zeros
                        mma_bf16(acc[nt][0], pl[0], ph[0], pl[1], ph[1], xv[nt].x, xv[nt].y);
                        mma_bf16(acc[nt][1], pl[2], ph[2], pl[3], ph[3], xv[nt].z, xv[nt].w);
                    }
                }
            }
            __syncwarp();                // every lane has read the slot: refill it
            if (issued < cnt) {
                if (lane == 0) {
                    mbar_expect_tx(use_bar, kChunkBytes);
                    bulk_load(use, p.ptr, kChunkBytes, use_bar);
                }
                advance(p);
                ++issued;
            }
            xsub += 256u;
            use += kChunkBytes;
            use_bar += 8;
            if (use_bar == bars + kDepth * 8) { use = ring; use_bar = bars; phase ^= 1u; }
        }
        // End of a row tile or of the run.  accumulator fragment: c0,c1 = (row g, batch 2t, 2t+1);
        // c2,c3 = (row g+8, same batches)
        const bool whole = sub0 == 0 && piece == S;
        const uint32_t row0 = (uint32_t)(c.tile - seg_first(c.seg)) * kRowsPerCta;
        // a partial tile at the end of the run is the run's last piece: the ring is free by then
        float* rw = pieces + (size_t)warp * kPieceStride + kRowsPerCta * m;
#pragma unroll
        for (int nt = 0; nt < kNT; ++nt) {
            const int b0 = 8 * nt + 2 * t;
            const float v0 = acc[nt][0][0] + acc[nt][1][0], v1 = acc[nt][0][1] + acc[nt][1][1];
            const float v2 = acc[nt][0][2] + acc[nt][1][2], v3 = acc[nt][0][3] + acc[nt][1][3];
            if (whole) {
                if (b0 < m) { emit(c.seg, row0 + g, b0, v0); emit(c.seg, row0 + g + 8, b0, v2); }
                if (b0 + 1 < m) { emit(c.seg, row0 + g, b0 + 1, v1); emit(c.seg, row0 + g + 8, b0 + 1, v3); }
            } else if (head) {
                head_v[nt][0] = v0; head_v[nt][1] = v1; head_v[nt][2] = v2; head_v[nt][3] = v3;
                head_kept = true;
            } else {
                if (b0 < m) { rw[g * m + b0] = v0; rw[(g + 8) * m + b0] = v2; }
                if (b0 + 1 < m) { rw[g * m + b0 + 1] = v1; rw[(g + 8) * m + b0 + 1] = v3; }
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) acc[nt][0][q] = acc[nt][1][q] = 0.0f;
        }
        if (head) {
            // Once, after this run's first piece and off the kernel's last steps: does this warp add up a
            // row tile after the barrier (its run holds the end of a tile that started in an earlier
            // run), and from where.
            const int tl = wa / S, a_sub = wa - tl * S;
            if (a_sub != 0 && (tl + 1) * S <= wb) {
                const int lo = tl * S;
                // the run that holds the tile's first chunk: the largest w with floor(nchunks * w / kWarps) <= lo
                const int wf = (int)(((uint32_t)kWarps * (uint32_t)(lo + 1) - 1u) / (uint32_t)nchunks);
                comb_n = warp - wf;
                comb_seg = c.seg;
                comb_row0 = row0;
                // that run holds the tile as its tail piece unless it starts exactly at the tile; every run
                // after it lies inside the tile (its head piece; zeros for a run without chunks)
                comb_first = pieces + (size_t)wf * kPieceStride + (run_start(wf) < lo ? kRowsPerCta * m : 0);
                comb_next = pieces + (size_t)(wf + 1) * kPieceStride;
            }
        }
        head = false;
        done += piece;
        // the next tile of the run (its first chunk is the tile's first)
        c.sub = 0;
        ++c.tile;
        if (c.tile == seg_end(c.seg) && c.seg + 1 < a.nseg) ++c.seg;
    }
    if (head_kept) {                     // every chunk of the run has been consumed: the ring takes the head sums
        float* rw = pieces + (size_t)warp * kPieceStride;
#pragma unroll
        for (int nt = 0; nt < kNT; ++nt) {
            const int b0 = 8 * nt + 2 * t;
            if (b0 < m) { rw[g * m + b0] = head_v[nt][0]; rw[(g + 8) * m + b0] = head_v[nt][2]; }
            if (b0 + 1 < m) { rw[g * m + b0 + 1] = head_v[nt][1]; rw[(g + 8) * m + b0 + 1] = head_v[nt][3]; }
        }
    }
    if (!__all_sync(0xffffffffu, ok)) {
        // A chunk did not arrive within the limit (the sums are then wrong; later chunks were not
        // waited for): report it.
        if (lane == 0 && a.status) atomicCAS(a.status, 0, 300 + (int)(blockIdx.x & 0xff));
        const uint64_t t0 = gemv_timer_ns(), grace = a.wait_ns < 1000000ull ? a.wait_ns : 1000000ull;
        while (gemv_timer_ns() - t0 < grace) {}      // a last (bounded) chance for copies in flight to land
    }
    __syncthreads();

    // Row tiles cut by run boundaries: the warp whose run holds the end of such a tile adds the
    // partial sums of the runs before it (ascending K) and its own head piece.
    if (comb_n > 0) {
        constexpr int stride = kPieceStride;
        for (int v = lane; v < kRowsPerCta * m; v += 32) {
            const int r = v % kRowsPerCta, b = v / kRowsPerCta;
            float sum = comb_first[r * m + b];
            const float* q = comb_next + r * m + b;
            for (int w2 = 0; w2 < comb_n; ++w2, q += stride) sum += *q;
            emit(comb_seg, comb_row0 + r, b, sum);
        }
    }

    if constexpr (kAR) {
        // Every output of this CTA's tiles: wait (bounded) for the packet of each rank and add them
        // in rank order, so that every rank ends with the same bits.
        const uint32_t n = (uint32_t)a.seg[0].n;
        const int64_t par = (int64_t)(seq & 1u) * a.ar.world * a.ar.slot_packets;
        const uint32_t flag = seq + 1u;
        const int total = (t1 - t0) * kRowsPerCta * m;
        for (int idx = threadIdx.x; idx < total; idx += kThreadsS) {
            const int tile = t0 + idx / (kRowsPerCta * m), rem = idx % (kRowsPerCta * m);
            const uint32_t row = (uint32_t)tile * kRowsPerCta + rem % kRowsPerCta;
            const int b = rem / kRowsPerCta;
            if (row >= n) continue;
            const int64_t slot_i = (int64_t)b * n + row;
            float sum = 0.0f;
            for (int src = 0; src < a.ar.world; ++src) {
                const uint2* q = a.ar.recv + par + src * a.ar.slot_packets + slot_i;
                uint2 pk = ld_packet(q);
                if (pk.y != flag) {
                    const uint64_t tw = gemv_timer_ns();
                    uint32_t spins = 0;
                    while ((pk = ld_packet(q)).y != flag) {
                        if ((++spins & 63u) == 0 && spins > 4096u && gemv_timer_ns() - tw > a.ar.wait_ns) {
                            if (a.ar.status) atomicCAS(a.ar.status, 0, 100 + src);
                            break;
                        }
                    }
                }
                const float v = __uint_as_float(pk.x);
                sum = src == 0 ? v : sum + v;
            }
            if (a.out_dtype == MIXFP4_F32) static_cast<float*>(a.seg[0].y)[(int64_t)b * a.seg[0].ldy + row] = sum;
            else static_cast<__nv_bfloat16*>(a.seg[0].y)[(int64_t)b * a.seg[0].ldy + row] = __float2bfloat16_rn(sum);
        }
        // the last CTA to finish advances the sequence number for the next launch
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

// Status word of the stream kernels: one int per device inside the library image.
static __device__ int g_stream_status;
constexpr int kMaxDevices = 64;
std::atomic<uint64_t> g_wait_limit_ns{2000000000ull};          // 2 s: far beyond any legitimate wait

struct DeviceInfo {
    int* status = nullptr;
    int sms = 0;
};
int device_info(DeviceInfo* out) {
    static std::mutex lock;
    static DeviceInfo info[kMaxDevices];
    int dev = 0;
    MIXFP4_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return MIXFP4_E_UNSUPPORTED;
    std::lock_guard<std::mutex> guard(lock);
    if (!info[dev].status) {
        void* p = nullptr;
        MIXFP4_CUDA_CHECK(cudaGetSymbolAddress(&p, g_stream_status));
        int sms = 0;
        MIXFP4_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        info[dev].status = static_cast<int*>(p);
        info[dev].sms = sms;
    }
    *out = info[dev];
    return MIXFP4_OK;
}

constexpr size_t kSmemLimit = 227 * 1024;

template <int kWarps, int kDepth, bool kAR, int kNT, int kLutRep>
int launch_stream(const GemvStreamArgs& a, int sms, int flags, cudaStream_t st) {
    const size_t smem = ((size_t)(kWarps * kDepth * 8 + 8 + 127) & ~(size_t)127) + (size_t)kWarps * kDepth * kChunkBytes +
                        (size_t)a.nseg * 256 * 16 * kLutRep + (((size_t)a.m * xres_row_bytes(a.kpad) + 15) & ~(size_t)15);
    static_assert(kDepth * kChunkBytes >= 2 * kRowsPerCta * 8 * kNT * 4, "a ring must hold the warp's two partial sums");
    if (smem > kSmemLimit) return MIXFP4_E_SHAPE;
    static unsigned long long configured = 0;          // one per instantiation, one bit per device
    if (const int rc = ensure_dynamic_smem(gemv_stream_kernel<kWarps, kDepth, kAR, kNT, kLutRep>, (int)kSmemLimit, configured))
        return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(a.ntiles < sms ? a.ntiles : sms));
    cfg.blockDim = dim3(kWarps * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (flags & MIXFP4_FLAG_OVERLAP_PREVIOUS) ? 1 : 0;
    MIXFP4_CUDA_CHECK(cudaLaunchKernelEx(&cfg, gemv_stream_kernel<kWarps, kDepth, kAR, kNT, kLutRep>, a));
    return MIXFP4_OK;
}

// Largest configuration whose shared memory (rings + tables + resident x + partial sums) fits;
// MIXFP4_E_SHAPE when none does (x too large to stay resident).
template <bool kAR>
int dispatch_stream(const GemvStreamArgs& a, int sms, int flags, cudaStream_t st) {
    int rc;
    if (a.m > 8) {
        if constexpr (kAR) {
            return MIXFP4_E_SHAPE;                   // the fused all-reduce takes at most 8 rows
        } else {
            rc = launch_stream<24, 2, false, 2, 8>(a, sms, flags, st);      // rings of two leave room for the eightfold table
            if (rc == MIXFP4_E_SHAPE) rc = launch_stream<24, 3, false, 2, 4>(a, sms, flags, st);
            if (rc == MIXFP4_E_SHAPE) rc = launch_stream<24, 3, false, 2, 2>(a, sms, flags, st);
            if (rc == MIXFP4_E_SHAPE) rc = launch_stream<24, 3, false, 2, 1>(a, sms, flags, st);
            if (rc == MIXFP4_E_SHAPE) rc = launch_stream<16, 3, false, 2, 1>(a, sms, flags, st);
            return rc;
        }
    }
    rc = launch_stream<24, 4, kAR, 1, 8>(a, sms, flags, st);
    if (rc == MIXFP4_E_SHAPE) rc = launch_stream<24, 3, kAR, 1, 8>(a, sms, flags, st);
    if (rc == MIXFP4_E_SHAPE) rc = launch_stream<24, 3, kAR, 1, 4>(a, sms, flags, st);
    if (rc == MIXFP4_E_SHAPE) rc = launch_stream<24, 3, kAR, 1, 1>(a, sms, flags, st);
    if (rc == MIXFP4_E_SHAPE) rc = launch_stream<16, 3, kAR, 1, 1>(a, sms, flags, st);
    return rc;
}

}  // namespace

uint64_t wait_limit_ns() { return g_wait_limit_ns.load(std::memory_order_relaxed); }

int gemv_stream(const void* x, int64_t m, int64_t ldx, int64_t k, const mixfp4_gemv_segment* segments, int count,
                int out_dtype, int flags, const mixfp4_comm* comm, int* ar_status, cudaStream_t st) {
    if (count < 1 || count > kMaxSeg || (comm && count != 1)) return MIXFP4_E_SHAPE;
    if (m < 1 || m > (comm ? 8 : 16)) return MIXFP4_E_SHAPE;
    GemvStreamArgs g = {};
    g.x = static_cast<const __nv_bfloat16*>(x);
    g.ldx = ldx; g.k = k; g.kpad = padded_k(k);
    g.m = (int)m; g.nseg = count; g.out_dtype = out_dtype;
    g.x_vec = aligned(x, 16) && (ldx % 8 == 0) && (k % 8 == 0);
    g.wide_lut = (flags & MIXFP4_FLAG_WIDE_TABLE) != 0;
    g.wait_ns = wait_limit_ns();
    const int64_t subs = g.kpad / kChunkK;
    int64_t tiles = 0;
    for (int s = 0; s < kMaxSeg; ++s) {
        const mixfp4_gemv_segment& in = segments[s < count ? s : count - 1];
        if (s < count) {
            if (!in.codes || !in.global_scale || !in.y) return MIXFP4_E_NULL;
            if (in.n <= 0 || in.ldy < in.n) return MIXFP4_E_SHAPE;
            if (!aligned(in.codes, 16) || (in.lut && !aligned(in.lut, 16))) return MIXFP4_E_ALIGN;
            if (!in.lut) g.wide_lut = false;
            tiles += stream_tiles(in.n);
            if (tiles * subs > 0x7ffffff0LL) return MIXFP4_E_SHAPE;
        }
        g.seg[s] = StreamSeg{in.codes, in.global_scale, static_cast<const uint4*>(in.lut), in.y, in.ldy, (int)in.n,
                             s < count ? (int)tiles : 0x7fffffff};
    }
    g.ntiles = (int)tiles;
    DeviceInfo info;
    if (const int rc = device_info(&info)) return rc;
    g.status = info.status;
    if (comm) {
        const int rc = comm_view(comm, &g.ar.rank, &g.ar.world, &g.ar.slot_packets, &g.ar.recv, g.ar.peer, &g.ar.words);
        if (rc != MIXFP4_OK) return rc;
        if (m * segments[0].n > g.ar.slot_packets) return MIXFP4_E_TOO_LARGE;
        g.ar.status = ar_status;
        g.ar.wait_ns = g.wait_ns;
        return dispatch_stream<true>(g, info.sms, flags, st);
    }
    return dispatch_stream<false>(g, info.sms, flags, st);
}

int stream_status_word(int** out) {
    DeviceInfo info;
    if (const int rc = device_info(&info)) return rc;
    *out = info.status;
    return MIXFP4_OK;
}

}  // namespace mixfp4

using namespace mixfp4;

extern "C" int mixfp4_gemv_x_fits(int64_t m, int64_t k, int count) {
    if (m < 1 || m > 16 || k <= 0 || count < 1 || count > kMaxSeg) return 0;
    // the smallest configuration: 16 warps, rings of 3 chunks, one table copy per weight
    const size_t smem = 512 + (size_t)16 * 3 * kChunkBytes + (size_t)count * 4096 +
                        (((size_t)m * xres_row_bytes(padded_k(k)) + 15) & ~(size_t)15);
    return smem <= kSmemLimit ? 1 : 0;
}

extern "C" int mixfp4_set_wait_limit_ns(uint64_t ns) {
    if (ns == 0) return MIXFP4_E_SHAPE;
    g_wait_limit_ns.store(ns, std::memory_order_relaxed);
    return MIXFP4_OK;
}

extern "C" int mixfp4_check_status(const int* dev_status, int* value, void* stream) {
    const int* word = dev_status;
    if (!word) {
        int* own = nullptr;
        if (const int rc = stream_status_word(&own)) return rc;
        word = own;
    }
    int v = 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    MIXFP4_CUDA_CHECK(cudaMemcpyAsync(&v, word, sizeof(int), cudaMemcpyDeviceToHost, st));
    MIXFP4_CUDA_CHECK(cudaStreamSynchronize(st));
    if (value) *value = v;
    return v == 0 ? MIXFP4_OK : MIXFP4_E_DEVICE_WAIT;
}
