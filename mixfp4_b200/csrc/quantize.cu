// Block quantizer (E2M1-or-E0M3 per 16 elements), tensor amax and packed -> dense decode.
//
// Arithmetic contract (bit-exact with the reference's PyTorch CPU path):
//   project_quant/scale.py:28-36     global = amax / 2688 (1 when the tensor is all zero)
//   project_quant/scale.py:185       s = x / global                    (IEEE division)
//   project_quant/scale.py:53-56     ideal = amax16|s| / qmax, clamp [2^-9, 448], E4M3 RNE
//   project_quant/scale.py:57-58     n = s / scale; codes = E2M1 / E0M3 rounding of n
//   project_quant/codebook.py:12-25  E2M1: floor(mantissa + 0.5) on the private mantissa
//   project_quant/codebook.py:41-43  E0M3: round-half-even, saturate 7
//   project_quant/scale.py:59-60     d = (code * scale) * global; err = sum (d - x)^2
//   project_quant/core.py:116        E0M3 iff err_e0 < err_e2
// Every fp32 operation uses a round-to-nearest intrinsic so that nothing is contracted
// into an FMA, and the 16 squared errors are added in the order the reference's CPU
// reduction uses (lane j + lane j+8 first, then the eight sums left to right).
//
// Work split: one thread owns one 16-element block at a time (two candidates, ~35 instructions per
// element -- the kernel is bound by instruction issue, not by HBM); a warp item is 64 consecutive
// blocks of one row (a lane takes blocks lane and lane + 32), so a warp's loads cover 2 x 1 KB of
// contiguous bf16 and its stores 2 x (256 B of codes, 32 B of scales, one word of format bits).

#include <cuda_fp4.h>

#include "common.cuh"
#include "decode.cuh"

namespace mixfp4 {
namespace {

constexpr int kThreads = 256;
constexpr int kWarpsPerCta = kThreads / 32;

// ---------------------------------------------------------------------------- amax
template <typename T>
__global__ void __launch_bounds__(kThreads) amax_kernel(const T* __restrict__ x, int64_t rows, int64_t k,
                                                        int64_t ldx, bool vec, unsigned int* __restrict__ out) {
    float m = 0.0f;
    if (vec) {
        // rows are contiguous 16-byte multiples: walk the tensor as uint4 words
        constexpr int kPer = 16 / sizeof(T);
        const int64_t words_per_row = k / kPer;
        const int64_t total = rows * words_per_row;
        // eight independent 16-byte loads in flight per thread and trip
        constexpr int kInFlight = 8;
        const int64_t stride = (int64_t)gridDim.x * blockDim.x;
        for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += kInFlight * stride) {
            uint4 v[kInFlight];
#pragma unroll
            for (int u = 0; u < kInFlight; ++u) {
                const int64_t iu = i + u * stride;
                const uint4* src = reinterpret_cast<const uint4*>(x) + iu;         // dense rows: one flat array
                if (ldx != k) {
                    const int64_t r = iu / words_per_row, w = iu - r * words_per_row;
                    src = reinterpret_cast<const uint4*>(x + r * ldx) + w;
                }
                v[u] = iu < total ? __ldg(src) : make_uint4(0u, 0u, 0u, 0u);
            }
            const T* e = reinterpret_cast<const T*>(v);
#pragma unroll
            for (int j = 0; j < kInFlight * kPer; ++j) m = fmaxf(m, fabsf(Elem<T>::load(e + j)));
        }
    } else {
        const int64_t total = rows * k;
        for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
             i += (int64_t)gridDim.x * blockDim.x) {
            const int64_t r = i / k, c = i - r * k;
            m = fmaxf(m, fabsf(Elem<T>::load(x + r * ldx + c)));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    __shared__ float warp_max[kWarpsPerCta];
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
#pragma unroll
        for (int w = 1; w < kWarpsPerCta; ++w) m = fmaxf(m, warp_max[w]);
        // non-negative floats order like their bit patterns
        if (m > 0.0f) atomicMax(out, __float_as_uint(m));
    }
}

// ------------------------------------------------------------------------- quantize
struct QuantArgs {
    const void* x;
    int64_t rows, k, ldx;
    int64_t groups;       // ceil(k / 16): real blocks per row
    int64_t blocks_pad;   // kpad / 16: stored blocks per row
    int64_t chunks;       // ceil(blocks_pad / 64): warp items per row (a lane takes two blocks of an item)
    int mode;
    bool vec_in, vec_out;
    bool in_place;        // dequant aliases x: the input is read with ordinary (coherent) loads
    bool any_stats;       // one of the four per-block statistics arrays is wanted
    const float* amax;
    uint8_t* codes;
    uint8_t* scales;
    uint8_t* fmt;
    float* global_scale;
    float* e2_err;
    float* e0_err;
    float* e2_scale;
    float* e0_scale;
    void* dequant;
    int64_t ld_dequant;
};

// a / b from a correctly rounded reciprocal r = RN(1/b): one multiply and two FMAs (the
// classical residual correction).  It returns the IEEE quotient for every a whenever it does
// so for every significand of a, because the three steps scale exactly with powers of two as
// long as the residual (about 2^-24 |a|) stays a normal number.  The quantizer uses it only
// where that has been checked: for the eight significands an E4M3 scale (and the constants 6
// and 7) can have by mixfp4_selftest_division, for the tensor scale by a per-CTA check over
// all significands of the 16-bit input type.  Quotients below 2^-102, where the residual
// would be subnormal, can be off in the last bit; with a 16-bit input and a tensor scale
// below 2^10 they are still nonzero with the right sign, and anything that small is clamped
// away by the 2^-9 scale floor and rounds to code 0, so no output bit depends on it.
__device__ __forceinline__ float div_rcp(float a, float b, float r) {
    const float q = __fmul_rn(a, r);
    const float rem = __fmaf_rn(-q, b, a);
    return __fmaf_rn(rem, r, q);
}
template <bool kFast>
__device__ __forceinline__ float div_exact(float a, float b, float r) {
    if constexpr (kFast) return div_rcp(a, b, r);
    else return __fdiv_rn(a, b);
}

// E2M1 rounding of |n| exactly as codebook.py:12-25 computes it: exponent floor(log2 |n|)
// clamped at 0, floor(mantissa * 2 + 0.5), saturate at 6.  For |n| >= 1 that is round-half-up
// to one mantissa bit, done on the bit pattern; below 1 the grid is {0, 0.5, 1} with
// thresholds 0.75 and -- because the reference adds 0.5 in fp32 -- the float just below 0.25.
// Returns the level value.
__device__ __forceinline__ float e2m1_round(float mag) {
    const uint32_t b = __float_as_uint(mag);
    const uint32_t rb = (b + 0x00200000u) & 0xffc00000u;               // |n| >= 1
    const float q_big = fminf(__uint_as_float(rb), 6.0f);
    const float q_small = b >= 0x3f400000u ? 1.0f : (b >= 0x3e7fffffu ? 0.5f : 0.0f);
    return b >= 0x3f800000u ? q_big : q_small;
}
// The 3-bit code of an E2M1 level, left in bits 22..24: scaled by 2^-126 the level's fp32 bit
// pattern is the E2M1 encoding itself (0.5 becomes the subnormal with only the top mantissa bit,
// 1 the smallest normal, ...), and nothing else is set.
__device__ __forceinline__ uint32_t e2m1_code_at_22(float q) {
    return __float_as_uint(__fmul_rn(q, 1.1754943508222875e-38f));
}

// E0M3 rounding of |n|: round-half-even then saturate at 7 (codebook.py:41-43).  Clamping at 7.25
// first changes nothing (everything above rounds to 7 or saturates) and keeps the sum's low
// mantissa bits equal to the level: t = 2^23 + level.
__device__ __forceinline__ float e0m3_round(float mag) {
    const float t = __fadd_rn(fminf(mag, 7.25f), 8388608.0f);
    return __fsub_rn(t, 8388608.0f);
}
// The same rounding on the FP4 conversion unit.  The hardware rounds to nearest even, the reference
// half up: setting the last mantissa bit lifts an exact tie (whose low bits are zero) above the
// midpoint and leaves every other value on its side of it (the float below a tie already has the
// bit set); the one input the reference's own fp32 addition lifts, the float just below 0.25, is
// replaced by the float just above 0.25.  Two magnitudes -> one byte (first in the low nibble, the canonical code order),
// and the byte back to the two level values.  mixfp4_selftest_division sweeps every fp32 input
// against e2m1_round.
__device__ __forceinline__ float e2m1_nudge(float mag) {
    const uint32_t b = __float_as_uint(mag);
    return __uint_as_float(b == 0x3e7fffffu ? 0x3e800001u : (b | 1u));
}
__device__ __forceinline__ uint32_t e2m1_pair_codes(float mag0, float mag1) {
    return __nv_cvt_float2_to_fp4x2(make_float2(e2m1_nudge(mag0), e2m1_nudge(mag1)), __NV_E2M1, cudaRoundNearest);
}
__device__ __forceinline__ float2 e2m1_pair_levels(uint32_t byte) {
    const __half2_raw h = __nv_cvt_fp4x2_to_halfraw2(static_cast<__nv_fp4x2_storage_t>(byte), __NV_E2M1);
    return __half22float2(__half2(h));
}

// One candidate format of one block.  ax = |x|, s = x / gs.  Produces the block's scale, its
// squared error in the reference's summation order, the magnitudes of the dequantized values
// (kKeep) and the eight-per-word 3-bit level codes without signs (kPack).
template <bool kE0, bool kFast, bool kPack, bool kKeep>
__device__ __forceinline__ void candidate(const float (&ax)[kGroup], const float (&s)[kGroup], float amax_s,
                                          float gs, uint32_t& lo, uint32_t& hi, uint32_t& scale_byte,
                                          float& scale_val, float& err, float (&dmag)[kGroup]) {
    float ideal = div_exact<kFast>(amax_s, kE0 ? 7.0f : 6.0f, kE0 ? (1.0f / 7.0f) : (1.0f / 6.0f));
    ideal = fminf(fmaxf(ideal, 0.001953125f), 448.0f);
    scale_byte = __nv_cvt_float_to_fp8(ideal, __NV_SATFINITE, __NV_E4M3);
    const float sc = e4m3_to_float(scale_byte);
    const float rsc = __frcp_rn(sc);
    scale_val = sc;
    float sq[kGroup];
    float p4[4] = {0.0f, 0.0f, 0.0f, 0.0f};         // E0M3: four levels per float, 16^j weights (exact)
    uint32_t byte[8];                               // E2M1: code bytes of the eight element pairs
#pragma unroll
    for (int i = 0; i < kGroup; i += 2) {
        const float mag0 = fabsf(div_exact<kFast>(s[i], sc, rsc)), mag1 = fabsf(div_exact<kFast>(s[i + 1], sc, rsc));
        float q[2];
        if constexpr (kE0) {
            q[0] = e0m3_round(mag0);
            q[1] = e0m3_round(mag1);
            if constexpr (kPack) {
                const int w = (i >> 1) & 1;                                // pair 0 or 1 of its group of four
                p4[i >> 2] = w == 0 ? __fmaf_rn(q[1], 16.0f, q[0])
                                    : __fmaf_rn(q[1], 4096.0f, __fmaf_rn(q[0], 256.0f, p4[i >> 2]));
            }
        } else {
            byte[i >> 1] = e2m1_pair_codes(mag0, mag1);
            const float2 lv = e2m1_pair_levels(byte[i >> 1]);
            q[0] = lv.x;
            q[1] = lv.y;
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            // (d - x)^2 == (|d| - |x|)^2 bit for bit: d and x never have opposite signs
            const float d = __fmul_rn(__fmul_rn(q[j], sc), gs);
            if constexpr (kKeep) dmag[i + j] = d;
            const float e = __fsub_rn(d, ax[i + j]);
            sq[i + j] = __fmul_rn(e, e);
        }
    }
    float acc = __fadd_rn(sq[0], sq[8]);
#pragma unroll
    for (int j = 1; j < 8; ++j) acc = __fadd_rn(acc, __fadd_rn(sq[j], sq[j + 8]));
    err = acc;
    lo = 0;
    hi = 0;
    if constexpr (kPack && kE0) {
        // 2^23 + p has p in its low mantissa bits; the low halves of two such words make one code word
        lo = __byte_perm(__float_as_uint(__fadd_rn(p4[0], 8388608.0f)), __float_as_uint(__fadd_rn(p4[1], 8388608.0f)), 0x5410);
        hi = __byte_perm(__float_as_uint(__fadd_rn(p4[2], 8388608.0f)), __float_as_uint(__fadd_rn(p4[3], 8388608.0f)), 0x5410);
    }
    if constexpr (kPack && !kE0) {
        lo = __byte_perm(__byte_perm(byte[0], byte[1], 0x0040), __byte_perm(byte[2], byte[3], 0x0040), 0x5410);
        hi = __byte_perm(__byte_perm(byte[4], byte[5], 0x0040), __byte_perm(byte[6], byte[7], 0x0040), 0x5410);
    }
}

// ---- The same two candidates with packed two-element fp32 operations (mul / add / fma .f32x2: each half is
// the IEEE operation, so every value below has the bits of its one-element counterpart above) and on SIGNED
// quotients, which is what the reference itself rounds:
//   * a / b by the reciprocal (div_rcp) on both halves at once, with -b passed in so that the residual is
//     one fma: q * (-b) + a has the same exact product as (-q) * b + a;
//   * the FP4 conversion unit takes the signed quotients, so the E2M1 code nibbles come out with their sign
//     bit, and the sign nibbles of the E0M3 codes are taken from them.  A nibble's sign is (n < 0); on this
//     path a nonzero 16-bit x never reaches n = 0 (scales are at least 2^-9 and the tensor scale is below
//     2^10), and x = +-0 gives +0 (the residual form returns +0 for a -0 dividend), so it equals (x < 0);
//   * E0M3: clamp to +-7.25, then (c + 1.5 * 2^23) - 1.5 * 2^23 is round-half-even for either sign;
//   * the error term is (d - x)^2 on the signed values (the reference's own expression).
__device__ __forceinline__ float2 div_rcp2(float2 a, float2 neg_b, float2 r) {
    const float2 q = __fmul2_rn(a, r);
    const float2 rem = __ffma2_rn(q, neg_b, a);
    return __ffma2_rn(rem, r, q);
}
// The nudge of e2m1_nudge for a signed pair, without a comparison.  Adding 2^-27 with the value's sign first:
// at 0.25 and above that is at most a quarter of the spacing and rounds back to the value; between 0.125 and
// 0.25 it is half the spacing, so values with an odd last bit move up one step -- all of them stay below 0.25
// except the float just below 0.25, which lands on 0.25 and is then lifted above it by the last-bit nudge
// like every exact tie (the reference rounds exactly that float up to 0.5); below 0.125 everything stays far
// below 0.25.  mixfp4_selftest_division sweeps every fp32 magnitude of both signs against e2m1_round.
__device__ __forceinline__ float2 e2m1_nudge_pair(float2 n) {
    const float2 c = make_float2(__uint_as_float((__float_as_uint(n.x) & 0x80000000u) | 0x32000000u),
                                 __uint_as_float((__float_as_uint(n.y) & 0x80000000u) | 0x32000000u));
    const float2 t = __fadd2_rn(n, c);
    return make_float2(__uint_as_float(__float_as_uint(t.x) | 1u), __uint_as_float(__float_as_uint(t.y) | 1u));
}
template <bool kE0>
__device__ __forceinline__ void block_scale_fast(float amax_s, uint32_t& scale_byte, float& sc, float& rsc) {
    float ideal = div_rcp(amax_s, kE0 ? 7.0f : 6.0f, kE0 ? (1.0f / 7.0f) : (1.0f / 6.0f));
    ideal = fminf(fmaxf(ideal, 0.001953125f), 448.0f);
    scale_byte = __nv_cvt_float_to_fp8(ideal, __NV_SATFINITE, __NV_E4M3);
    sc = e4m3_to_float(scale_byte);
    rsc = __frcp_rn(sc);
}
__device__ __forceinline__ float error_sum(const float2 (&sq)[8]) {
    // pairs (j, j + 8) first, then the eight sums left to right.  One-element adds on purpose: the assembler
    // was seen to merge a packed multiply with a packed add that consumes it into one fused operation
    // (different bits), which it never does with the one-element round-to-nearest forms.
    float acc = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float p0 = __fadd_rn(sq[j].x, sq[j + 4].x), p1 = __fadd_rn(sq[j].y, sq[j + 4].y);
        acc = j == 0 ? __fadd_rn(p0, p1) : __fadd_rn(__fadd_rn(acc, p0), p1);
    }
    return acc;
}
// x2[j] = elements (2j, 2j+1) of the block.  d2 / d0: signed dequantized values (kKeep).
template <bool kPack, bool kKeep>
__device__ __forceinline__ void candidates_fast(const float2 (&x2)[8], float gs, float rgs, uint32_t& lo2, uint32_t& hi2,
                                                uint32_t& b2, float& sc2, float& err2, float2 (&d2)[8], uint32_t& lo0,
                                                uint32_t& hi0, uint32_t& b0, float& sc0, float& err0, float2 (&d0)[8]) {
    const float2 rgs2 = make_float2(rgs, rgs), ngs2 = make_float2(-gs, -gs), gs2 = make_float2(gs, gs);
    const float2 neg1 = make_float2(-1.0f, -1.0f);
    float2 s[8];
    float amax_s = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        s[j] = div_rcp2(x2[j], ngs2, rgs2);
        amax_s = fmaxf(amax_s, fmaxf(fabsf(s[j].x), fabsf(s[j].y)));      // |.| folds into the (three-input) maximum
    }
    {   // E2M1
        float rsc;
        block_scale_fast<false>(amax_s, b2, sc2, rsc);
        const float2 rsc2 = make_float2(rsc, rsc), nsc2 = make_float2(-sc2, -sc2), scv = make_float2(sc2, sc2);
        float2 sq[8];
        uint32_t byte[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float2 n = div_rcp2(s[j], nsc2, rsc2);
            byte[j] = __nv_cvt_float2_to_fp4x2(e2m1_nudge_pair(n), __NV_E2M1, cudaRoundNearest);
            const float2 d = __fmul2_rn(__fmul2_rn(e2m1_pair_levels(byte[j]), scv), gs2);
            if constexpr (kKeep) d2[j] = d;
            const float2 e = __ffma2_rn(x2[j], neg1, d);
            sq[j] = __fmul2_rn(e, e);
        }
        err2 = error_sum(sq);
        lo2 = hi2 = 0;
        if constexpr (kPack) {
            lo2 = __byte_perm(__byte_perm(byte[0], byte[1], 0x0040), __byte_perm(byte[2], byte[3], 0x0040), 0x5410);
            hi2 = __byte_perm(__byte_perm(byte[4], byte[5], 0x0040), __byte_perm(byte[6], byte[7], 0x0040), 0x5410);
        }
    }
    {   // E0M3
        float rsc;
        block_scale_fast<true>(amax_s, b0, sc0, rsc);
        const float2 rsc2 = make_float2(rsc, rsc), nsc2 = make_float2(-sc0, -sc0), scv = make_float2(sc0, sc0);
        const float2 magic = make_float2(12582912.0f, 12582912.0f), nmagic = make_float2(-12582912.0f, -12582912.0f);
        float2 sq[8];
        float p4[4] = {0.0f, 0.0f, 0.0f, 0.0f};         // four levels per float, 16^j weights (exact)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float2 n = div_rcp2(s[j], nsc2, rsc2);
            const float2 c = make_float2(fminf(fmaxf(n.x, -7.25f), 7.25f), fminf(fmaxf(n.y, -7.25f), 7.25f));
            const float2 q = __fadd2_rn(__fadd2_rn(c, magic), nmagic);
            if constexpr (kPack)
                p4[j >> 1] = (j & 1) == 0 ? __fmaf_rn(fabsf(q.y), 16.0f, fabsf(q.x))
                                          : __fmaf_rn(fabsf(q.y), 4096.0f, __fmaf_rn(fabsf(q.x), 256.0f, p4[j >> 1]));
            const float2 d = __fmul2_rn(__fmul2_rn(q, scv), gs2);
            if constexpr (kKeep) d0[j] = d;
            const float2 e = __ffma2_rn(x2[j], neg1, d);
            sq[j] = __fmul2_rn(e, e);
        }
        err0 = error_sum(sq);
        lo0 = hi0 = 0;
        if constexpr (kPack) {
            lo0 = __byte_perm(__float_as_uint(__fadd_rn(p4[0], 8388608.0f)), __float_as_uint(__fadd_rn(p4[1], 8388608.0f)), 0x5410);
            hi0 = __byte_perm(__float_as_uint(__fadd_rn(p4[2], 8388608.0f)), __float_as_uint(__fadd_rn(p4[3], 8388608.0f)), 0x5410);
        }
    }
}

// Element-wise codebook rounding (project_quant/codebook.py:12-25 quantize_e2m1, :41-43 quantize_e0m3):
// y = sign(x) * level(|x|), with the reference's signed zero (a negative x that rounds to zero gives -0,
// x = +-0 gives +0 because sign(0) = 0).
__global__ void __launch_bounds__(kThreads) round_codebook_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                                  int64_t n, bool e0) {
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kThreads) {
        const float v = x[i], mag = fabsf(v);
        const float q = e0 ? e0m3_round(mag) : e2m1_round(mag);
        y[i] = v < 0.0f ? -q : (v > 0.0f ? q : __fmul_rn(v != v ? v : 0.0f, q));
    }
}

// The E0M3 candidate under the reference's scale_rule "four_over_six" (project_quant/scale.py:64-103
// _four_over_six_scale_candidate with qmax 7, :207-225 the choice between the x1.0 and the x1.5
// scale).  One thread per block; every fp32 operation in the reference's order, IEEE, no contraction.
__device__ __forceinline__ float e0_four_over_six_block(const float (&x)[kGroup], float amax, float expansion,
                                                        float (&codes)[kGroup], float (&deq)[kGroup], float& scale_out) {
    const float denominator = 1536.0f;
    float bmax = 0.0f;
#pragma unroll
    for (int i = 0; i < kGroup; ++i) bmax = fmaxf(bmax, fabsf(x[i]));
    float ideal = 0.0f;
    if (amax != 0.0f) ideal = __fmul_rn(__fdiv_rn(bmax, 7.0f), __fdiv_rn(denominator, amax));
    ideal = __fmul_rn(ideal, expansion);
    const float scale = e4m3_to_float(__nv_cvt_float_to_fp8(ideal, __NV_SATFINITE, __NV_E4M3));   // no clamp: may be 0
    const float decode_scale = amax > 0.0f ? __fdiv_rn(1.0f, __fdiv_rn(denominator, amax)) : 0.0f;
    const float recip = scale != 0.0f ? __fdiv_rn(1.0f, __fmul_rn(decode_scale, scale)) : 0.0f;
    float sq[kGroup];
#pragma unroll
    for (int i = 0; i < kGroup; ++i) {
        const float n = scale != 0.0f ? __fmul_rn(x[i], recip) : 0.0f;
        const float level = e0m3_round(fabsf(n));
        const float code = n < 0.0f ? -level : (n > 0.0f ? level : 0.0f);
        codes[i] = code;
        const float d = __fdiv_rn(__fmul_rn(__fmul_rn(code, scale), amax), denominator);
        deq[i] = d;
        const float e = __fsub_rn(d, x[i]);
        sq[i] = __fmul_rn(e, e);
    }
    float acc = __fadd_rn(sq[0], sq[8]);
#pragma unroll
    for (int j = 1; j < 8; ++j) acc = __fadd_rn(acc, __fadd_rn(sq[j], sq[j + 8]));
    scale_out = scale;
    return acc;
}

__global__ void __launch_bounds__(128) e0_four_over_six_kernel(const float* __restrict__ x, int64_t nblocks,
                                                               const float* __restrict__ amax_ptr,
                                                               float* __restrict__ codes, float* __restrict__ dequant,
                                                               float* __restrict__ scales, float* __restrict__ errors,
                                                               uint8_t* __restrict__ expanded) {
    const int64_t b = (int64_t)blockIdx.x * 128 + threadIdx.x;
    if (b >= nblocks) return;
    const float amax = *amax_ptr;
    float v[kGroup], c0[kGroup], d0[kGroup], c1[kGroup], d1[kGroup], s0, s1;
#pragma unroll
    for (int i = 0; i < kGroup; ++i) v[i] = x[b * kGroup + i];
    const float e0 = e0_four_over_six_block(v, amax, 1.0f, c0, d0, s0);
    const float e1 = e0_four_over_six_block(v, amax, 1.5f, c1, d1, s1);
    const bool pick = e1 < e0;
#pragma unroll
    for (int i = 0; i < kGroup; ++i) {
        codes[b * kGroup + i] = pick ? c1[i] : c0[i];
        dequant[b * kGroup + i] = pick ? d1[i] : d0[i];
    }
    scales[b] = pick ? s1 : s0;
    errors[b] = pick ? e1 : e0;
    expanded[b] = pick ? 1 : 0;
}

// Exhaustive check of div_rcp against IEEE division: all 2^23 significands of the dividend
// for each of the 8 significands a divisor can have (E4M3 scales; 6 = 1.5 * 4, 7 = 1.75 * 4).
__global__ void selftest_division_kernel(unsigned long long* mismatches) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;          // 2^23 dividends
    const float a = __uint_as_float(0x3f800000u | i);
    unsigned long long bad = 0;
#pragma unroll
    for (int d = 0; d < 8; ++d) {
        const float b = 1.0f + 0.125f * d;
        const float r = __frcp_rn(b);
        bad += __float_as_uint(div_rcp(a, b, r)) != __float_as_uint(__fdiv_rn(a, b));
        bad += __float_as_uint(div_rcp(a * 0.001f, b * 6.0f, __frcp_rn(b * 6.0f))) != __float_as_uint(__fdiv_rn(a * 0.001f, b * 6.0f));
        // the packed form, one half positive and one negative
        const float2 q2 = div_rcp2(make_float2(a, -a * 0.37f), make_float2(-b, -b), make_float2(r, r));
        bad += __float_as_uint(q2.x) != __float_as_uint(__fdiv_rn(a, b));
        bad += __float_as_uint(q2.y) != __float_as_uint(__fdiv_rn(-a * 0.37f, b));
    }
    if (bad) atomicAdd(mismatches, bad);
}

// Exhaustive check of the FP4-unit E2M1 rounding against e2m1_round: every fp32 magnitude from 0
// to 16 (pairs of neighbouring bit patterns), level value and 3-bit code.
constexpr uint32_t kE2m1SweepPairs = 0x41800000u / 2 + 1;
__global__ void selftest_e2m1_kernel(unsigned long long* mismatches) {
    const uint32_t pair = blockIdx.x * blockDim.x + threadIdx.x;
    if (pair >= kE2m1SweepPairs) return;
    const float m0 = __uint_as_float(2 * pair), m1 = __uint_as_float(2 * pair + 1);
    const uint32_t byte = e2m1_pair_codes(m0, m1);
    const float2 lv = e2m1_pair_levels(byte);
    const float q0 = e2m1_round(m0), q1 = e2m1_round(m1);
    unsigned long long bad = 0;
    bad += __float_as_uint(lv.x) != __float_as_uint(q0);
    bad += __float_as_uint(lv.y) != __float_as_uint(q1);
    bad += (byte & 15u) != (e2m1_code_at_22(q0) >> 22);
    bad += (byte >> 4) != (e2m1_code_at_22(q1) >> 22);
    // the signed, comparison-free nudge of the packed path: first magnitude positive, second negative
    const uint32_t sb = __nv_cvt_float2_to_fp4x2(e2m1_nudge_pair(make_float2(m0, -m1)), __NV_E2M1, cudaRoundNearest);
    const float2 sv = e2m1_pair_levels(sb);
    bad += __float_as_uint(sv.x) != __float_as_uint(q0);
    bad += __float_as_uint(sv.y) != (__float_as_uint(q1) | 0x80000000u);
    bad += (sb & 15u) != (e2m1_code_at_22(q0) >> 22);
    bad += (sb >> 4) != ((e2m1_code_at_22(q1) >> 22) | 8u);
    if (bad) atomicAdd(mismatches, bad);
}

// kPack: write codes / scales / format bits; kDequant: write the dequantized tensor.  Each warp
// walks over (row, 64-block chunk) items with the grid's stride; a lane takes the blocks lane and
// lane + 32 of an item, so the index arithmetic of an item is shared by two blocks.
template <typename T, bool kPack, bool kDequant>
__global__ void __launch_bounds__(kThreads, (kPack && !kDequant) ? 3 : 2) quantize_kernel(const QuantArgs a) {
    // a kernel launched behind this one with programmatic dependent launch (the W4A4 GEMM) may set itself up
    // while this grid runs; it waits for this grid's end before it reads the outputs
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int lane = threadIdx.x & 31;
    const int warp_in_cta = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);   // provably warp-uniform
    const float amax = *a.amax;
    const float gs = amax > 0.0f ? __fdiv_rn(amax, 2688.0f) : 1.0f;
    const float rgs = __frcp_rn(gs);
    // The reciprocal form of x / gs is used only if it gives the IEEE quotient for every
    // significand the 16-bit input type has (checked here by the whole CTA, 128 or 1024
    // divisions); fp32 inputs and extreme tensor scales take the IEEE path.
    bool fast = sizeof(T) == 2 && gs > 8.7e-19f && gs < 1024.0f;
    {
        constexpr int kSig = sizeof(T) == 2 ? (Elem<T>::kDtype == MIXFP4_BF16 ? 128 : 1024) : 0;
        bool ok = true;
        for (int i = threadIdx.x; i < kSig; i += kThreads) {
            const float v = 1.0f + static_cast<float>(i) * (1.0f / kSig);
            ok = ok && __float_as_uint(div_rcp(v, gs, rgs)) == __float_as_uint(__fdiv_rn(v, gs));
        }
        fast = __syncthreads_and(ok) && fast;
    }
    if (blockIdx.x == 0 && threadIdx.x == 0 && a.global_scale) *a.global_scale = gs;

    // (row, chunk) of this warp's items: one division here, carries in the loop
    const int64_t first = (int64_t)blockIdx.x * kWarpsPerCta + warp_in_cta, step = (int64_t)gridDim.x * kWarpsPerCta;
    const int64_t step_rows = step / a.chunks, step_chunks = step - step_rows * a.chunks;
    int64_t row = first / a.chunks, chunk = first - row * a.chunks;
    for (; row < a.rows; row += step_rows, chunk += step_chunks) {
        if (chunk >= a.chunks) {
            chunk -= a.chunks;
            if (++row >= a.rows) break;
        }
#pragma unroll 1
      for (int u = 0; u < 2; ++u) {                    // the lane's two blocks of this item, 32 blocks apart
        const int64_t blk = chunk * 64 + u * 32 + lane;         // block index inside the row
        const bool stored = blk < a.blocks_pad;
        const bool real = blk < a.groups;

        uint32_t lo = 0, hi = 0, scale_byte = 0x01;    // what an all-zero block quantizes to
        bool use_e0 = false;
        if (kPack && a.mode == MIXFP4_MODE_GIVEN && real)   // the caller's format bits (read before the byte is rewritten below)
            use_e0 = (a.fmt[row * (a.blocks_pad / 8) + (blk >> 3)] >> (blk & 7)) & 1;

        if (real) {
            const T* xr = static_cast<const T*>(a.x) + row * a.ldx;
            const int64_t c0 = blk * kGroup;
            float x[kGroup];
            if (a.vec_in && c0 + kGroup <= a.k) {
                constexpr int kWords = kGroup * sizeof(T) / 16;
                uint4 w[kWords];
#pragma unroll
                for (int j = 0; j < kWords; ++j) {
                    const uint4* src = reinterpret_cast<const uint4*>(xr + c0) + j;
                    w[j] = a.in_place ? *src : __ldg(src);
                }
                const T* e = reinterpret_cast<const T*>(w);
#pragma unroll
                for (int i = 0; i < kGroup; ++i) x[i] = Elem<T>::load(e + i);
            } else {
#pragma unroll
                for (int i = 0; i < kGroup; ++i) x[i] = c0 + i < a.k ? Elem<T>::load(xr + c0 + i) : 0.0f;
            }

            uint32_t lo2, hi2, b2, lo0, hi0, b0;
            float sc2, sc0, err2, err0;
            float d2[kGroup], d0[kGroup];
            uint32_t sl = 0, sh = 0;                     // sign nibbles of elements 0..7 and 8..15
            if (fast) {
                float2 x2[8], dd2[8], dd0[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) x2[j] = make_float2(x[2 * j], x[2 * j + 1]);
                candidates_fast<kPack, kDequant>(x2, gs, rgs, lo2, hi2, b2, sc2, err2, dd2, lo0, hi0, b0, sc0, err0, dd0);
                if constexpr (kDequant) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        d2[2 * j] = fabsf(dd2[j].x); d2[2 * j + 1] = fabsf(dd2[j].y);
                        d0[2 * j] = fabsf(dd0[j].x); d0[2 * j + 1] = fabsf(dd0[j].y);
                    }
                }
                sl = lo2 & 0x88888888u;                  // the FP4 unit kept the quotients' signs
                sh = hi2 & 0x88888888u;
            } else {
                float s[kGroup], ax[kGroup];
                float amax_s = 0.0f;
#pragma unroll
                for (int i = 0; i < kGroup; ++i) {
                    s[i] = __fdiv_rn(x[i], gs);
                    ax[i] = fabsf(x[i]);
                    amax_s = fmaxf(amax_s, fabsf(s[i]));
                }
                candidate<false, false, kPack, kDequant>(ax, s, amax_s, gs, lo2, hi2, b2, sc2, err2, d2);
                candidate<true, false, kPack, kDequant>(ax, s, amax_s, gs, lo0, hi0, b0, sc0, err0, d0);
                if constexpr (kPack) {
                    // Sign bit of a nibble = (n < 0) = (x < 0): dividing by the positive scales keeps the sign and
                    // never reaches zero from a nonzero x; x = -0 gives n = -0, which is not below zero.
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        if (x[i] < 0.0f) sl |= 8u << (4 * i);
                        if (x[i + 8] < 0.0f) sh |= 8u << (4 * i);
                    }
                }
            }
            if (a.mode != MIXFP4_MODE_GIVEN)
                use_e0 = a.mode == MIXFP4_MODE_ORACLE16 ? (err0 < err2) : (a.mode == MIXFP4_MODE_ALL_E0M3);

            if (a.any_stats) {
                const int64_t g = row * a.groups + blk;
                if (a.e2_err) a.e2_err[g] = err2;
                if (a.e0_err) a.e0_err[g] = err0;
                if (a.e2_scale) a.e2_scale[g] = sc2;
                if (a.e0_scale) a.e0_scale[g] = sc0;
            }

            if constexpr (kPack) {
                lo = (use_e0 ? lo0 : lo2) | sl;
                hi = (use_e0 ? hi0 : hi2) | sh;
                scale_byte = use_e0 ? b0 : b2;
            }

            if constexpr (kDequant) {
                T* out = static_cast<T*>(a.dequant) + row * a.ld_dequant + c0;
                T vals[kGroup];
#pragma unroll
                for (int i = 0; i < kGroup; ++i) {
                    const float mag = use_e0 ? d0[i] : d2[i];
                    vals[i] = Elem<T>::round(x[i] < 0.0f ? -mag : mag);
                }
                if (a.vec_out && c0 + kGroup <= a.k) {
                    constexpr int kWords = kGroup * sizeof(T) / 16;
#pragma unroll
                    for (int j = 0; j < kWords; ++j)
                        reinterpret_cast<uint4*>(out)[j] = reinterpret_cast<const uint4*>(vals)[j];
                } else {
#pragma unroll
                    for (int i = 0; i < kGroup; ++i)
                        if (c0 + i < a.k) out[i] = vals[i];
                }
            }
        }

        if constexpr (kPack) {
            if (stored) {
                const int64_t ld_codes = a.blocks_pad * 8, ld_scales = a.blocks_pad;
                *reinterpret_cast<uint2*>(a.codes + row * ld_codes + blk * 8) = make_uint2(lo, hi);
                a.scales[row * ld_scales + blk] = static_cast<uint8_t>(scale_byte);
            }
            const uint32_t bits = __ballot_sync(0xffffffffu, use_e0);
            const int64_t fmt_col = chunk * 8 + u * 4 + lane;      // lanes 0..3 write one format byte each
            if (lane < 4 && fmt_col < a.blocks_pad / 8)
                a.fmt[row * (a.blocks_pad / 8) + fmt_col] = static_cast<uint8_t>(bits >> (8 * lane));
        }
      }
    }
}

// kLayout: MIXFP4_LAYOUT_CANONICAL, _KERNEL or _STREAM (codes = the chunk buffer, scales unused).
template <typename T, int kLayout>
__global__ void __launch_bounds__(kThreads) dequant_kernel(const uint8_t* __restrict__ codes,
                                                           const uint8_t* __restrict__ scales,
                                                           const uint8_t* __restrict__ fmt,
                                                           const float* __restrict__ global_scale, int64_t rows,
                                                           int64_t k, int64_t groups, int64_t blocks_pad,
                                                           T* __restrict__ out, int64_t ldo, bool vec_out) {
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t row = t / groups;
    if (row >= rows) return;
    const int64_t blk = t - row * groups;
    const float gs = *global_scale;
    constexpr bool kKL = kLayout != MIXFP4_LAYOUT_CANONICAL;
    const uint8_t* cptr = codes + row * blocks_pad * 8 + blk * 8;
    const uint8_t* sptr = scales + row * blocks_pad + blk;
    if constexpr (kLayout == MIXFP4_LAYOUT_STREAM) {
        const uint8_t* chunk = codes + ((row >> 4) * (blocks_pad >> 3) + (blk >> 3)) * kChunkBytes;
        cptr = chunk + (row & 15) * 64 + (blk & 7) * 8;
        sptr = chunk + kChunkCodeBytes + (row & 15) * 8 + (blk & 7);
    }
    uint2 c = __ldg(reinterpret_cast<const uint2*>(cptr));
    const uint32_t sbyte = __ldg(sptr);
    bool e0;
    if constexpr (kKL) {
        c.x = codes_from_kernel_layout(c.x);
        c.y = codes_from_kernel_layout(c.y);
        e0 = (sbyte >> 7) & 1;
    } else {
        e0 = (__ldg(fmt + row * (blocks_pad / 8) + (blk >> 3)) >> (blk & 7)) & 1;
    }
    const float sc = e4m3_to_float(sbyte & 0x7fu);
    T vals[kGroup];
#pragma unroll
    for (int i = 0; i < kGroup; ++i) {
        const uint32_t nib = ((i < 8 ? c.x : c.y) >> (4 * (i & 7))) & 15u;
        const float mag = __fmul_rn(__fmul_rn(level_value(nib & 7u, e0), sc), gs);
        vals[i] = Elem<T>::round((nib & 8u) ? -mag : mag);
    }
    const int64_t c0 = blk * kGroup;
    T* o = out + row * ldo + c0;
    if (vec_out && c0 + kGroup <= k) {
        constexpr int kWords = kGroup * sizeof(T) / 16;
#pragma unroll
        for (int j = 0; j < kWords; ++j) reinterpret_cast<uint4*>(o)[j] = reinterpret_cast<const uint4*>(vals)[j];
    } else {
#pragma unroll
        for (int i = 0; i < kGroup; ++i)
            if (c0 + i < k) o[i] = vals[i];
    }
}

// ---------------------------------------------------------------------------- repack
// canonical <-> kernel layout (see decode.cuh); one thread per block, a warp covers 32
// consecutive blocks of a row like the quantizer, so the format bits of 32 blocks are one
// ballot word.
template <bool kToKernel>
__global__ void __launch_bounds__(kThreads) repack_kernel(const uint8_t* __restrict__ codes,
                                                          const uint8_t* __restrict__ scales,
                                                          const uint8_t* __restrict__ fmt, int64_t rows,
                                                          int64_t blocks_pad, int64_t chunks,
                                                          uint8_t* __restrict__ codes_out,
                                                          uint8_t* __restrict__ scales_out,
                                                          uint8_t* __restrict__ fmt_out) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * kWarpsPerCta + __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);   // provably warp-uniform
    const int64_t row = warp / chunks;
    if (row >= rows) return;
    const int64_t chunk = warp - row * chunks;
    const int64_t blk = chunk * 32 + lane;
    const bool stored = blk < blocks_pad;
    bool fbit = false;
    if (stored) {
        uint2 c = __ldg(reinterpret_cast<const uint2*>(codes + row * blocks_pad * 8 + blk * 8));
        uint32_t sb = __ldg(scales + row * blocks_pad + blk);
        if constexpr (kToKernel) {
            fbit = (__ldg(fmt + row * (blocks_pad / 8) + (blk >> 3)) >> (blk & 7)) & 1;
            c.x = codes_to_kernel_layout(c.x);
            c.y = codes_to_kernel_layout(c.y);
            sb = (sb & 0x7fu) | (fbit ? 0x80u : 0u);
        } else {
            fbit = (sb >> 7) & 1;
            c.x = codes_from_kernel_layout(c.x);
            c.y = codes_from_kernel_layout(c.y);
            sb &= 0x7fu;
        }
        *reinterpret_cast<uint2*>(codes_out + row * blocks_pad * 8 + blk * 8) = c;
        scales_out[row * blocks_pad + blk] = static_cast<uint8_t>(sb);
    }
    if constexpr (!kToKernel) {
        const uint32_t bits = __ballot_sync(0xffffffffu, fbit);
        const int64_t col = chunk * 4 + lane;
        if (lane < 4 && col < blocks_pad / 8) fmt_out[row * (blocks_pad / 8) + col] = static_cast<uint8_t>(bits >> (8 * lane));
    }
}

// canonical <-> stream layout (decode.cuh).  Same split as above; the grid also covers the rows that
// pad the last 16-row tile, which are written as zero codes with the scale byte 0x01.
template <bool kToStream>
__global__ void __launch_bounds__(kThreads) repack_stream_kernel(const uint8_t* __restrict__ codes,
                                                                 const uint8_t* __restrict__ scales,
                                                                 const uint8_t* __restrict__ fmt,
                                                                 uint8_t* __restrict__ chunks, int64_t rows,
                                                                 int64_t rows_pad, int64_t blocks_pad, int64_t groups32,
                                                                 uint8_t* __restrict__ codes_out,
                                                                 uint8_t* __restrict__ scales_out,
                                                                 uint8_t* __restrict__ fmt_out) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * kWarpsPerCta + __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);   // provably warp-uniform
    const int64_t row = warp / groups32;
    if (row >= (kToStream ? rows_pad : rows)) return;
    const int64_t blk = (warp - row * groups32) * 32 + lane;
    const bool stored = blk < blocks_pad;
    uint8_t* chunk = chunks + ((row >> 4) * (blocks_pad >> 3) + (blk >> 3)) * kChunkBytes;
    uint8_t* cptr = chunk + (row & 15) * 64 + (blk & 7) * 8;
    uint8_t* sptr = chunk + kChunkCodeBytes + (row & 15) * 8 + (blk & 7);
    bool fbit = false;
    if (stored) {
        if constexpr (kToStream) {
            uint2 c = make_uint2(0u, 0u);
            uint32_t sb = 0x01u;
            if (row < rows) {
                c = __ldg(reinterpret_cast<const uint2*>(codes + row * blocks_pad * 8 + blk * 8));
                sb = __ldg(scales + row * blocks_pad + blk);
                fbit = (__ldg(fmt + row * (blocks_pad / 8) + (blk >> 3)) >> (blk & 7)) & 1;
                c.x = codes_to_kernel_layout(c.x);
                c.y = codes_to_kernel_layout(c.y);
                sb = (sb & 0x7fu) | (fbit ? 0x80u : 0u);
            }
            *reinterpret_cast<uint2*>(cptr) = c;
            *sptr = static_cast<uint8_t>(sb);
        } else {
            uint2 c = *reinterpret_cast<const uint2*>(cptr);
            const uint32_t sb = *sptr;
            fbit = (sb >> 7) & 1;
            c.x = codes_from_kernel_layout(c.x);
            c.y = codes_from_kernel_layout(c.y);
            *reinterpret_cast<uint2*>(codes_out + row * blocks_pad * 8 + blk * 8) = c;
            scales_out[row * blocks_pad + blk] = static_cast<uint8_t>(sb & 0x7fu);
        }
    }
    if constexpr (!kToStream) {
        const uint32_t bits = __ballot_sync(0xffffffffu, fbit);
        const int64_t col = (warp - row * groups32) * 4 + lane;
        if (lane < 4 && col < blocks_pad / 8) fmt_out[row * (blocks_pad / 8) + col] = static_cast<uint8_t>(bits >> (8 * lane));
    }
}

__global__ void decode_table_kernel(const float* __restrict__ global_scale, uint4* __restrict__ lut) {
    const int e = threadIdx.x;
    lut[e] = make_lut_entry(e & 127, e >> 7, *global_scale);
}

__global__ void decode_table_wide_kernel(const float* __restrict__ global_scale, uint4* __restrict__ lut) {
    const int e = threadIdx.x;
    const uint4 v = make_lut_entry(e & 127, e >> 7, *global_scale);
    lut[e] = v;
#pragma unroll
    for (int j = 0; j < 8; ++j) lut[256 + e * 8 + j] = v;
}

size_t elem_size(int dtype) { return dtype == MIXFP4_F32 ? 4 : 2; }

bool rows_vectorizable(const void* p, int64_t ld, int dtype) {
    return aligned(p, 16) && (ld * (int64_t)elem_size(dtype)) % 16 == 0;
}

}  // namespace
}  // namespace mixfp4

using namespace mixfp4;

extern "C" int mixfp4_amax(const void* x, int dtype, int64_t rows, int64_t k, int64_t ldx, float* amax,
                           void* stream) {
    if (!x || !amax) return MIXFP4_E_NULL;
    if (rows <= 0 || k <= 0 || ldx < k) return MIXFP4_E_SHAPE;
    if (dtype < MIXFP4_BF16 || dtype > MIXFP4_F32) return MIXFP4_E_DTYPE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    MIXFP4_CUDA_CHECK(cudaMemsetAsync(amax, 0, sizeof(float), st));
    const bool vec = rows_vectorizable(x, ldx, dtype) && (k * (int64_t)elem_size(dtype)) % 16 == 0;
    const int64_t items = vec ? rows * (k * (int64_t)elem_size(dtype) / 16) : rows * k;
    int64_t ctas = (items + kThreads * 8 - 1) / (kThreads * 8);
    if (ctas < 1) ctas = 1;
    if (ctas > 148 * 8) ctas = 148 * 8;   // a few waves of grid-stride CTAs
    unsigned int* out = reinterpret_cast<unsigned int*>(amax);
    switch (dtype) {
        case MIXFP4_BF16:
            amax_kernel<<<(unsigned)ctas, kThreads, 0, st>>>(static_cast<const __nv_bfloat16*>(x), rows, k, ldx, vec, out);
            break;
        case MIXFP4_F16:
            amax_kernel<<<(unsigned)ctas, kThreads, 0, st>>>(static_cast<const __half*>(x), rows, k, ldx, vec, out);
            break;
        default:
            amax_kernel<<<(unsigned)ctas, kThreads, 0, st>>>(static_cast<const float*>(x), rows, k, ldx, vec, out);
    }
    return check_launch("amax_kernel");
}

// One format per region of region_rows x region_groups K16 blocks (project_quant/region.py:73-86
// aggregate_regions + selector.py:28-33 mse_selection): E0M3 iff the region's summed E0M3 error
// is smaller.  The fp32 sums follow the reference's CPU reduction order: inside a row the
// region's blocks left to right, then the rows top to bottom, cells past the tensor's edge
// counting as zero.  Regions one block wide (n8k16, m16k16: region_groups = 1) follow the
// reference's reduction of a strided dimension as PyTorch's CPU kernels run it on an AVX-512
// host: columns inside whole chunks of 32 block columns are added top to bottom, the columns
// left after the last whole chunk go through four accumulators (row i into accumulator i mod 4)
// added 0 + 1 + 2 + 3.  One thread owns one format byte (8 blocks) of one row of regions and
// writes it to every row of the region.
__global__ void __launch_bounds__(kThreads) select_regions_kernel(const float* __restrict__ e2_err,
                                                                  const float* __restrict__ e0_err, int64_t rows,
                                                                  int64_t groups, int64_t fmt_cols, int region_rows,
                                                                  int region_groups, uint8_t* __restrict__ fmt) {
    const int64_t t = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    const int64_t region_row = t / fmt_cols, col = t - region_row * fmt_cols;
    const int64_t r0 = region_row * region_rows;
    if (r0 >= rows) return;
    uint32_t byte = 0;
    for (int sub = 0; sub < 8 / region_groups; ++sub) {
        const int64_t g0 = col * 8 + sub * region_groups;
        if (g0 >= groups) break;
        float sum2 = 0.0f, sum0 = 0.0f;
        if (region_groups == 1 && g0 >= groups / 32 * 32) {
            float a2[4] = {0.0f, 0.0f, 0.0f, 0.0f}, a0[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            for (int r = 0; r < region_rows && r0 + r < rows; r += 4) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const bool in = r + q < region_rows && r0 + r + q < rows;
                    a2[q] = __fadd_rn(a2[q], in ? __ldg(e2_err + (r0 + r + q) * groups + g0) : 0.0f);
                    a0[q] = __fadd_rn(a0[q], in ? __ldg(e0_err + (r0 + r + q) * groups + g0) : 0.0f);
                }
            }
            sum2 = __fadd_rn(__fadd_rn(__fadd_rn(a2[0], a2[1]), a2[2]), a2[3]);
            sum0 = __fadd_rn(__fadd_rn(__fadd_rn(a0[0], a0[1]), a0[2]), a0[3]);
        } else {
            for (int r = 0; r < region_rows; ++r) {
                float t2 = 0.0f, t0 = 0.0f;
                for (int g = 0; g < region_groups; ++g) {
                    const bool in = r0 + r < rows && g0 + g < groups;
                    t2 = __fadd_rn(t2, in ? __ldg(e2_err + (r0 + r) * groups + g0 + g) : 0.0f);
                    t0 = __fadd_rn(t0, in ? __ldg(e0_err + (r0 + r) * groups + g0 + g) : 0.0f);
                }
                sum2 = __fadd_rn(sum2, t2);
                sum0 = __fadd_rn(sum0, t0);
            }
        }
        if (sum0 < sum2) {
            for (int g = 0; g < region_groups; ++g)
                if (g0 + g < groups) byte |= 1u << (sub * region_groups + g);
        }
    }
    for (int r = 0; r < region_rows && r0 + r < rows; ++r) fmt[(r0 + r) * fmt_cols + col] = static_cast<uint8_t>(byte);
}

// "layer" (one format for the whole tensor, project_quant/region.py:44-45): both error sums in double
// precision (one atomic add per warp), then every format byte set or cleared.  The reference's own fp32
// sum of all blocks depends on its host's thread count; the decision does not unless the two sums agree
// to about 1e-7.
__global__ void __launch_bounds__(kThreads) sum_errors_kernel(const float* __restrict__ e2_err,
                                                              const float* __restrict__ e0_err, int64_t count,
                                                              double* __restrict__ sums) {
    double s2 = 0.0, s0 = 0.0;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < count; i += (int64_t)gridDim.x * kThreads) {
        s2 += static_cast<double>(__ldg(e2_err + i));
        s0 += static_cast<double>(__ldg(e0_err + i));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        s2 += __shfl_xor_sync(0xffffffffu, s2, o);
        s0 += __shfl_xor_sync(0xffffffffu, s0, o);
    }
    if ((threadIdx.x & 31) == 0) {
        atomicAdd(sums, s2);
        atomicAdd(sums + 1, s0);
    }
}
__global__ void __launch_bounds__(kThreads) fill_format_kernel(const double* __restrict__ sums, uint8_t* __restrict__ fmt,
                                                               int64_t bytes) {
    const uint8_t value = sums[1] < sums[0] ? 0xff : 0x00;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < bytes; i += (int64_t)gridDim.x * kThreads)
        fmt[i] = value;
}

namespace mixfp4 {
namespace {
int launch_quantize(const void* x, int dtype, int64_t rows, int64_t k, int64_t ldx, int mode, const float* amax,
                    uint8_t* codes, uint8_t* scales, uint8_t* fmt, float* global_scale, float* e2_err, float* e0_err,
                    float* e2_scale, float* e0_scale, void* dequant, int64_t ld_dequant, cudaStream_t st) {
    QuantArgs a;
    a.x = x; a.rows = rows; a.k = k; a.ldx = ldx;
    a.groups = (k + kGroup - 1) / kGroup;
    a.blocks_pad = padded_k(k) / kGroup;
    a.chunks = (a.blocks_pad + 63) / 64;
    a.mode = mode;
    a.vec_in = rows_vectorizable(x, ldx, dtype);
    a.vec_out = dequant && rows_vectorizable(dequant, ld_dequant, dtype);
    a.in_place = dequant == x;
    a.amax = amax; a.codes = codes; a.scales = scales; a.fmt = fmt; a.global_scale = global_scale;
    a.e2_err = e2_err; a.e0_err = e0_err; a.e2_scale = e2_scale; a.e0_scale = e0_scale;
    a.any_stats = e2_err || e0_err || e2_scale || e0_scale;
    a.dequant = dequant; a.ld_dequant = ld_dequant;
    const int64_t warps = rows * a.chunks;
    int64_t ctas = (warps + kWarpsPerCta - 1) / kWarpsPerCta;
    if (ctas > 148 * 6) ctas = 148 * 6;            // the warps stride over the (row, chunk) items
#define MIXFP4_LAUNCH_QUANTIZE(T)                                                                       \
    do {                                                                                                \
        if (codes && dequant) quantize_kernel<T, true, true><<<(unsigned)ctas, kThreads, 0, st>>>(a);    \
        else if (codes) quantize_kernel<T, true, false><<<(unsigned)ctas, kThreads, 0, st>>>(a);         \
        else quantize_kernel<T, false, true><<<(unsigned)ctas, kThreads, 0, st>>>(a);                    \
    } while (0)
    switch (dtype) {
        case MIXFP4_BF16: MIXFP4_LAUNCH_QUANTIZE(__nv_bfloat16); break;
        case MIXFP4_F16: MIXFP4_LAUNCH_QUANTIZE(__half); break;
        default: MIXFP4_LAUNCH_QUANTIZE(float);
    }
#undef MIXFP4_LAUNCH_QUANTIZE
    return check_launch("quantize_kernel");
}
}  // namespace

int fake_quantize_with_amax(const void* x, int dtype, int64_t rows, int64_t k, int64_t ldx, int mode, const float* amax,
                            void* y, int64_t ldy, cudaStream_t st) {
    return launch_quantize(x, dtype, rows, k, ldx, mode, amax, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
                           nullptr, nullptr, y, ldy, st);
}
}  // namespace mixfp4

extern "C" int mixfp4_quantize(const void* x, int dtype, int64_t rows, int64_t k, int64_t ldx, int mode,
                               const float* amax, uint8_t* codes, uint8_t* scales, uint8_t* fmt,
                               float* global_scale, float* e2_err, float* e0_err, float* e2_scale,
                               float* e0_scale, void* dequant, int64_t ld_dequant, void* stream) {
    if (!x || !amax || !codes || !scales || !fmt || !global_scale) return MIXFP4_E_NULL;
    if (rows <= 0 || k <= 0 || ldx < k || (dequant && ld_dequant < k)) return MIXFP4_E_SHAPE;
    if (dtype < MIXFP4_BF16 || dtype > MIXFP4_F32) return MIXFP4_E_DTYPE;
    if (mode < MIXFP4_MODE_ORACLE16 || mode > MIXFP4_MODE_GIVEN) return MIXFP4_E_MODE;
    if (!aligned(codes, 8)) return MIXFP4_E_ALIGN;
    return launch_quantize(x, dtype, rows, k, ldx, mode, amax, codes, scales, fmt, global_scale, e2_err, e0_err,
                           e2_scale, e0_scale, dequant, ld_dequant, static_cast<cudaStream_t>(stream));
}

extern "C" int mixfp4_fake_quantize(const void* x, int dtype, int64_t rows, int64_t k, int64_t ldx, int mode,
                                    float* amax, void* y, int64_t ldy, void* stream) {
    if (!x || !amax || !y) return MIXFP4_E_NULL;
    if (rows <= 0 || k <= 0 || ldx < k || ldy < k) return MIXFP4_E_SHAPE;
    if (dtype < MIXFP4_BF16 || dtype > MIXFP4_F32) return MIXFP4_E_DTYPE;
    if (mode < MIXFP4_MODE_ORACLE16 || mode > MIXFP4_MODE_ALL_E0M3) return MIXFP4_E_MODE;
    // in place is allowed when the two views coincide exactly; any other overlap is not
    if (y == x && ldy != ldx) return MIXFP4_E_SHAPE;
    const int rc = mixfp4_amax(x, dtype, rows, k, ldx, amax, stream);
    if (rc != MIXFP4_OK) return rc;
    return launch_quantize(x, dtype, rows, k, ldx, mode, amax, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
                           nullptr, nullptr, y, ldy, static_cast<cudaStream_t>(stream));
}

extern "C" int mixfp4_dequant(const uint8_t* codes, const uint8_t* scales, const uint8_t* fmt,
                              const float* global_scale, int64_t rows, int64_t k, int layout, void* out,
                              int out_dtype, int64_t ldo, void* stream) {
    if (layout != MIXFP4_LAYOUT_CANONICAL && layout != MIXFP4_LAYOUT_KERNEL && layout != MIXFP4_LAYOUT_STREAM)
        return MIXFP4_E_MODE;
    if (!codes || (!scales && layout != MIXFP4_LAYOUT_STREAM) || (!fmt && layout == MIXFP4_LAYOUT_CANONICAL) ||
        !global_scale || !out)
        return MIXFP4_E_NULL;
    if (rows <= 0 || k <= 0 || ldo < k) return MIXFP4_E_SHAPE;
    if (out_dtype < MIXFP4_BF16 || out_dtype > MIXFP4_F32) return MIXFP4_E_DTYPE;
    if (!aligned(codes, 8)) return MIXFP4_E_ALIGN;
    const int64_t groups = (k + kGroup - 1) / kGroup, blocks_pad = padded_k(k) / kGroup;
    const int64_t ctas = (rows * groups + kThreads - 1) / kThreads;
    if (ctas > 0x7fffffffLL) return MIXFP4_E_SHAPE;
    const bool vec = rows_vectorizable(out, ldo, out_dtype);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
#define MIXFP4_LAUNCH_DEQUANT_L(T, L)                                                                        \
    dequant_kernel<T, L><<<(unsigned)ctas, kThreads, 0, st>>>(codes, scales, fmt, global_scale, rows, k, groups, \
                                                              blocks_pad, static_cast<T*>(out), ldo, vec)
#define MIXFP4_LAUNCH_DEQUANT(T)                                                                             \
    do {                                                                                                    \
        if (layout == MIXFP4_LAYOUT_STREAM) MIXFP4_LAUNCH_DEQUANT_L(T, MIXFP4_LAYOUT_STREAM);               \
        else if (layout == MIXFP4_LAYOUT_KERNEL) MIXFP4_LAUNCH_DEQUANT_L(T, MIXFP4_LAYOUT_KERNEL);          \
        else MIXFP4_LAUNCH_DEQUANT_L(T, MIXFP4_LAYOUT_CANONICAL);                                           \
    } while (0)
    switch (out_dtype) {
        case MIXFP4_BF16: MIXFP4_LAUNCH_DEQUANT(__nv_bfloat16); break;
        case MIXFP4_F16: MIXFP4_LAUNCH_DEQUANT(__half); break;
        default: MIXFP4_LAUNCH_DEQUANT(float);
    }
#undef MIXFP4_LAUNCH_DEQUANT
#undef MIXFP4_LAUNCH_DEQUANT_L
    return check_launch("dequant_kernel");
}

extern "C" int mixfp4_e0_four_over_six(const float* grouped, int64_t nblocks, const float* amax, float* codes,
                                       float* dequant, float* scales, float* errors, uint8_t* expansion_ids,
                                       void* stream) {
    if (!grouped || !amax || !codes || !dequant || !scales || !errors || !expansion_ids) return MIXFP4_E_NULL;
    if (nblocks <= 0 || nblocks > (0x7fffffffLL - 1) * 128) return MIXFP4_E_SHAPE;
    e0_four_over_six_kernel<<<(unsigned)((nblocks + 127) / 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        grouped, nblocks, amax, codes, dequant, scales, errors, expansion_ids);
    return check_launch("e0_four_over_six_kernel");
}

extern "C" int mixfp4_round_codebook(const float* x, float* y, int64_t n, int e0m3, void* stream) {
    if (!x || !y) return MIXFP4_E_NULL;
    if (n <= 0) return MIXFP4_E_SHAPE;
    if (e0m3 != 0 && e0m3 != 1) return MIXFP4_E_MODE;
    const int64_t ctas = (n + kThreads - 1) / kThreads;
    round_codebook_kernel<<<(unsigned)(ctas < 4096 ? ctas : 4096), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        x, y, n, e0m3 != 0);
    return check_launch("round_codebook_kernel");
}

extern "C" int64_t mixfp4_stream_bytes(int64_t rows, int64_t k) {
    return rows > 0 && k > 0 ? stream_bytes(rows, k) : 0;
}

extern "C" int mixfp4_repack_stream(const uint8_t* codes, const uint8_t* scales, const uint8_t* fmt, int64_t rows,
                                    int64_t k, uint8_t* chunks, void* stream) {
    if (!codes || !scales || !fmt || !chunks) return MIXFP4_E_NULL;
    if (rows <= 0 || k <= 0) return MIXFP4_E_SHAPE;
    if (!aligned(codes, 8) || !aligned(chunks, 16)) return MIXFP4_E_ALIGN;
    const int64_t blocks_pad = padded_k(k) / kGroup, groups32 = (blocks_pad + 31) / 32;
    const int64_t rows_pad = stream_tiles(rows) * kChunkRows;
    const int64_t ctas = (rows_pad * groups32 + kWarpsPerCta - 1) / kWarpsPerCta;
    if (ctas > 0x7fffffffLL) return MIXFP4_E_SHAPE;
    repack_stream_kernel<true><<<(unsigned)ctas, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        codes, scales, fmt, chunks, rows, rows_pad, blocks_pad, groups32, nullptr, nullptr, nullptr);
    return check_launch("repack_stream_kernel");
}

extern "C" int mixfp4_repack_from_stream(const uint8_t* chunks, int64_t rows, int64_t k, uint8_t* codes_out,
                                         uint8_t* scales_out, uint8_t* fmt_out, void* stream) {
    if (!chunks || !codes_out || !scales_out || !fmt_out) return MIXFP4_E_NULL;
    if (rows <= 0 || k <= 0) return MIXFP4_E_SHAPE;
    if (!aligned(codes_out, 8) || !aligned(chunks, 16)) return MIXFP4_E_ALIGN;
    const int64_t blocks_pad = padded_k(k) / kGroup, groups32 = (blocks_pad + 31) / 32;
    const int64_t ctas = (rows * groups32 + kWarpsPerCta - 1) / kWarpsPerCta;
    if (ctas > 0x7fffffffLL) return MIXFP4_E_SHAPE;
    repack_stream_kernel<false><<<(unsigned)ctas, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        nullptr, nullptr, nullptr, const_cast<uint8_t*>(chunks), rows, stream_tiles(rows) * kChunkRows, blocks_pad,
        groups32, codes_out, scales_out, fmt_out);
    return check_launch("repack_stream_kernel");
}

extern "C" int mixfp4_repack(const uint8_t* codes, const uint8_t* scales, const uint8_t* fmt, int64_t rows, int64_t k,
                             int to_layout, uint8_t* codes_out, uint8_t* scales_out, uint8_t* fmt_out, void* stream) {
    if (to_layout != MIXFP4_LAYOUT_CANONICAL && to_layout != MIXFP4_LAYOUT_KERNEL) return MIXFP4_E_MODE;
    if (!codes || !scales || !codes_out || !scales_out) return MIXFP4_E_NULL;
    if (to_layout == MIXFP4_LAYOUT_KERNEL ? !fmt : !fmt_out) return MIXFP4_E_NULL;
    if (rows <= 0 || k <= 0) return MIXFP4_E_SHAPE;
    if (!aligned(codes, 8) || !aligned(codes_out, 8)) return MIXFP4_E_ALIGN;
    const int64_t blocks_pad = padded_k(k) / kGroup, chunks = (blocks_pad + 31) / 32;
    const int64_t ctas = (rows * chunks + kWarpsPerCta - 1) / kWarpsPerCta;
    if (ctas > 0x7fffffffLL) return MIXFP4_E_SHAPE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (to_layout == MIXFP4_LAYOUT_KERNEL)
        repack_kernel<true><<<(unsigned)ctas, kThreads, 0, st>>>(codes, scales, fmt, rows, blocks_pad, chunks, codes_out,
                                                                 scales_out, fmt_out);
    else
        repack_kernel<false><<<(unsigned)ctas, kThreads, 0, st>>>(codes, scales, fmt, rows, blocks_pad, chunks, codes_out,
                                                                  scales_out, fmt_out);
    return check_launch("repack_kernel");
}

extern "C" int mixfp4_decode_table(const float* global_scale, void* lut, void* stream) {
    if (!global_scale || !lut) return MIXFP4_E_NULL;
    if (!aligned(lut, 16)) return MIXFP4_E_ALIGN;
    decode_table_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(global_scale, static_cast<uint4*>(lut));
    return check_launch("decode_table_kernel");
}

extern "C" int mixfp4_decode_table_wide(const float* global_scale, void* lut, void* stream) {
    if (!global_scale || !lut) return MIXFP4_E_NULL;
    if (!aligned(lut, 16)) return MIXFP4_E_ALIGN;
    decode_table_wide_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(global_scale, static_cast<uint4*>(lut));
    return check_launch("decode_table_wide_kernel");
}

extern "C" int mixfp4_selftest_division(unsigned long long* mismatches, void* stream) {
    if (!mismatches) return MIXFP4_E_NULL;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    MIXFP4_CUDA_CHECK(cudaMemsetAsync(mismatches, 0, sizeof(unsigned long long), st));
    selftest_division_kernel<<<(1u << 23) / 256, 256, 0, st>>>(mismatches);
    int rc = check_launch("selftest_division_kernel");
    if (rc != MIXFP4_OK) return rc;
    selftest_e2m1_kernel<<<(kE2m1SweepPairs + 255) / 256, 256, 0, st>>>(mismatches);
    rc = check_launch("selftest_e2m1_kernel");
    return rc != MIXFP4_OK ? rc : fwht_selftest_division(mismatches, st);
}

extern "C" int mixfp4_select_regions(const float* e2_err, const float* e0_err, int64_t rows, int64_t k,
                                     int region_rows, int region_groups, uint8_t* fmt, void* stream) {
    if (!e2_err || !e0_err || !fmt) return MIXFP4_E_NULL;
    if (rows <= 0 || k <= 0 || region_rows <= 0) return MIXFP4_E_SHAPE;
    if (region_groups != 1 && region_groups != 2 && region_groups != 4) return MIXFP4_E_MODE;
    if (region_groups == 1 && region_rows < 2) return MIXFP4_E_MODE;         // 1 x 1 is the per-block mode
    const int64_t groups = (k + 15) / 16;
    // with a single region along K the reference's reduction takes another order (not reproduced)
    if (region_rows > 1 && (groups + region_groups - 1) / region_groups == 1) return MIXFP4_E_MODE;
    const int64_t fmt_cols = padded_k(k) / 128;
    const int64_t threads = (rows + region_rows - 1) / region_rows * fmt_cols;
    const int64_t ctas = (threads + kThreads - 1) / kThreads;
    if (ctas > 0x7fffffffLL) return MIXFP4_E_SHAPE;
    select_regions_kernel<<<(unsigned)ctas, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        e2_err, e0_err, rows, groups, fmt_cols, region_rows, region_groups, fmt);
    return check_launch("select_regions_kernel");
}

extern "C" int mixfp4_select_layer(const float* e2_err, const float* e0_err, int64_t rows, int64_t k, double* sums,
                                   uint8_t* fmt, void* stream) {
    if (!e2_err || !e0_err || !sums || !fmt) return MIXFP4_E_NULL;
    if (rows <= 0 || k <= 0) return MIXFP4_E_SHAPE;
    if (!aligned(sums, 8)) return MIXFP4_E_ALIGN;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t count = rows * ((k + 15) / 16), bytes = rows * (padded_k(k) / 128);
    MIXFP4_CUDA_CHECK(cudaMemsetAsync(sums, 0, 2 * sizeof(double), st));
    int64_t ctas = (count + kThreads * 8 - 1) / (kThreads * 8);
    if (ctas > 148 * 4) ctas = 148 * 4;
    sum_errors_kernel<<<(unsigned)ctas, kThreads, 0, st>>>(e2_err, e0_err, count, sums);
    if (const int rc = check_launch("sum_errors_kernel")) return rc;
    int64_t fill = (bytes + kThreads - 1) / kThreads;
    if (fill > 148 * 8) fill = 148 * 8;
    fill_format_kernel<<<(unsigned)fill, kThreads, 0, st>>>(sums, fmt, bytes);
    return check_launch("fill_format_kernel");
}
