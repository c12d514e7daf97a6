// Decode-shape dequant-linear (1 <= M <= 16): y[M,N] = x[M,K] * W[N,K]^T, W in the packed
// mixed-FP4 layout.  Replaces F.linear on the dequantized weight
// (project_quant/modeling.py:629 + nn.Linear.forward).  HBM-bound: the packed weight
// (0.5703 B/element) is read exactly once, x stays in L1/L2.
//
// Work split.  A CTA owns 16 consecutive weight rows; its warps split K in interleaved
// 512-element steps and their partial sums are added in a fixed order through shared
// memory (deterministic).  Inside a warp the 16 x 512 slab is laid over the
// mma.sync.m16n8k16 A-fragment: lane (g, t) = (lane/4, lane%4) owns rows g and g+8 and
// the 128 consecutive K elements starting at 128*t, so per step it issues four 128-bit
// code loads, one 64-bit scale load and one format-byte load per row, one step ahead of
// the arithmetic.  The k index of an MMA is only a summation label, so the 16 k-slots of
// every MMA are filled with whatever 4 consecutive elements each lane decodes next; the
// B fragment takes the same 4 elements of x (batch row g), zero for g >= M.
//
// Decode.  A 256-entry table in shared memory, built per launch from the tensor scale,
// maps (format bit, E4M3 scale byte) to the block's eight magnitudes
// bf16((level * scale) * global) -- exactly the reference's dequantized weight -- stored
// as 8 low bytes + 8 high bytes.  Eight 4-bit codes (one 32-bit word) become four bf16x2
// registers with byte permutes: two PRMT look up low/high bytes of four elements, the
// sign bits are spread with PRMT's sign-replicate mode, two more PRMT interleave.
// The accumulation is the tensor core's fp32.

#include "common.cuh"

namespace mixfp4 {
namespace {

constexpr int kRowsPerCta = 16;
constexpr int kStepK = 512;               // K elements one warp consumes per step

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

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

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

// One table entry: the eight bf16 magnitudes of a block as low bytes (x, y) / high bytes (z, w).
__device__ __forceinline__ uint4 make_lut_entry(uint32_t scale_byte, bool e0m3, float gs) {
    const float sc = e4m3_to_float(scale_byte);
    uint32_t lo[2] = {0, 0}, hi[2] = {0, 0};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float v = __fmul_rn(__fmul_rn(level_value(j, e0m3), sc), gs);
        const uint32_t bits = __bfloat16_as_ushort(__float2bfloat16_rn(v));
        lo[j >> 2] |= (bits & 0xffu) << (8 * (j & 3));
        hi[j >> 2] |= (bits >> 8) << (8 * (j & 3));
    }
    return make_uint4(lo[0], lo[1], hi[0], hi[1]);
}

// Eight codes (nibble j = element j) -> four bf16x2 registers (elements 01, 23, 45, 67).
__device__ __forceinline__ void decode8(uint32_t w, const uint4& t, uint32_t (&p)[4]) {
    const uint32_t mag = w & 0x77777777u;
    const uint32_t mag_hi = mag >> 16;
    const uint32_t w4 = w << 4;
    uint32_t lo_a = prmt(t.x, t.y, mag), hi_a = prmt(t.z, t.w, mag);
    uint32_t lo_b = prmt(t.x, t.y, mag_hi), hi_b = prmt(t.z, t.w, mag_hi);
    // byte i of sign_a is 0xFF iff element i is negative (selector nibble 8+j = replicate the
    // top bit of byte j of {w, w4}); same for elements 4..7 in sign_b
    const uint32_t sign_a = prmt(w, w4, 0x9D8Cu), sign_b = prmt(w, w4, 0xBFAEu);
    hi_a |= sign_a & 0x80808080u;
    hi_b |= sign_b & 0x80808080u;
    p[0] = prmt(lo_a, hi_a, 0x5140u);
    p[1] = prmt(lo_a, hi_a, 0x7362u);
    p[2] = prmt(lo_b, hi_b, 0x5140u);
    p[3] = prmt(lo_b, hi_b, 0x7362u);
}

struct Slab {                 // what one lane holds for one step: rows g (0) and g+8 (1)
    uint4 c[2][4];            // 2 x 128 codes
    uint2 s[2];               // 2 x 8 scale bytes
    uint32_t f[2];            // 2 x 8 format bits
};

template <int kWarps, int kNTiles>
__global__ void __launch_bounds__(kWarps * 32) gemv_kernel(const GemvArgs a) {
    __shared__ uint4 lut[256];
    __shared__ float red[kWarps][kRowsPerCta][8 * kNTiles];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int64_t row0 = (int64_t)blockIdx.x * kRowsPerCta;
    const int64_t ld_codes = a.kpad / 2, ld_scales = a.kpad / 16, ld_fmt = a.kpad / 128;
    const int steps = static_cast<int>((a.kpad + kStepK - 1) / kStepK);
    const bool row_ok[2] = {row0 + g < a.n, row0 + g + 8 < a.n};

    auto load_slab = [&](Slab& s, int step) {
        const int64_t kp = (int64_t)step * kStepK + t * 128;   // first K element of this lane's piece
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            if (row_ok[h] && kp < a.kpad) {
                const int64_t r = row0 + g + 8 * h;
                const uint4* cp = reinterpret_cast<const uint4*>(a.codes + r * ld_codes + kp / 2);
#pragma unroll
                for (int u = 0; u < 4; ++u) s.c[h][u] = ldg_stream(cp + u);
                s.s[h] = __ldg(reinterpret_cast<const uint2*>(a.scales + r * ld_scales + kp / 16));
                s.f[h] = __ldg(a.fmt + r * ld_fmt + kp / 128);
            } else {
#pragma unroll
                for (int u = 0; u < 4; ++u) s.c[h][u] = make_uint4(0, 0, 0, 0);
                s.s[h] = make_uint2(0, 0);     // scale byte 0 -> table entry of zeros
                s.f[h] = 0;
            }
        }
    };

    Slab cur, nxt;
    if (warp < steps) load_slab(cur, warp);

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

    const __nv_bfloat16* xrow[kNTiles];
    bool x_ok[kNTiles];
#pragma unroll
    for (int nt = 0; nt < kNTiles; ++nt) {
        x_ok[nt] = g + 8 * nt < a.m;
        xrow[nt] = a.x + (int64_t)(g + 8 * nt) * a.ldx;
    }

    for (int step = warp; step < steps; step += kWarps) {
        const bool more = step + kWarps < steps;
        if (more) load_slab(nxt, step + kWarps);
        const int64_t kp = (int64_t)step * kStepK + t * 128;
#pragma unroll
        for (int b = 0; b < 8; ++b) {                    // the 8 blocks of this lane's piece
            uint4 tab[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t sw = b < 4 ? cur.s[h].x : cur.s[h].y;
                const uint32_t scale_byte = (sw >> (8 * (b & 3))) & 0x7fu;
                const uint32_t fbit = (cur.f[h] >> b) & 1u;
                tab[h] = lut[(fbit << 7) | scale_byte];
            }
#pragma unroll
            for (int half = 0; half < 2; ++half) {       // 8 elements = 2 MMAs
                const int i = 2 * b + half;              // word index inside the piece
                uint32_t pl[4], ph[4];
                const uint4& cl = cur.c[0][i >> 2];
                const uint4& ch = cur.c[1][i >> 2];
                const uint32_t wl = (i & 3) == 0 ? cl.x : (i & 3) == 1 ? cl.y : (i & 3) == 2 ? cl.z : cl.w;
                const uint32_t wh = (i & 3) == 0 ? ch.x : (i & 3) == 1 ? ch.y : (i & 3) == 2 ? ch.z : ch.w;
                decode8(wl, tab[0], pl);
                decode8(wh, tab[1], ph);
                const int64_t k0 = kp + 8 * i;
#pragma unroll
                for (int nt = 0; nt < kNTiles; ++nt) {
                    uint4 xv = make_uint4(0, 0, 0, 0);
                    if (x_ok[nt]) {
                        if (a.x_vec) {
                            if (k0 < a.k) xv = __ldg(reinterpret_cast<const uint4*>(xrow[nt] + k0));
                        } else {
                            uint32_t e[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                e[j] = k0 + j < a.k ? __bfloat16_as_ushort(xrow[nt][k0 + j]) : 0u;
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

template <int kWarps>
int launch(const GemvArgs& a, cudaStream_t st) {
    const int64_t ctas = (a.n + kRowsPerCta - 1) / kRowsPerCta;
    if (ctas > 0x7fffffffLL) return MIXFP4_E_SHAPE;
    if (a.m <= 8) gemv_kernel<kWarps, 1><<<(unsigned)ctas, kWarps * 32, 0, st>>>(a);
    else gemv_kernel<kWarps, 2><<<(unsigned)ctas, kWarps * 32, 0, st>>>(a);
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
    GemvArgs a;
    a.x = static_cast<const __nv_bfloat16*>(x);
    a.m = m; a.ldx = ldx;
    a.codes = codes; a.scales = scales; a.fmt = fmt; a.global_scale = global_scale;
    a.n = n; a.k = k; a.kpad = padded_k(k);
    a.y = y; a.out_dtype = out_dtype; a.ldy = ldy;
    a.x_vec = aligned(x, 16) && (ldx % 8 == 0) && (k % 8 == 0);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t steps = (a.kpad + kStepK - 1) / kStepK;
    if (steps >= 16) return launch<8>(a, st);
    if (steps >= 4) return launch<4>(a, st);
    return launch<2>(a, st);
}
