// Stand-alone normalised block Hadamard (project_quant/rotation.py:47-75 fwht / apply_transform).
//
// Natural (Sylvester) order: stage with stride s maps every pair (i, i+s) inside a block
// to (l + r, l - r); after log2(size) stages the block is divided by sqrt(size) (IEEE
// division by the fp32 value of sqrt(size), as the reference's CPU path does).  Each
// output of a stage is a single add, so the result does not depend on how the work is
// split across threads.  One lane keeps 16 consecutive elements (32 bytes of bf16 in flight
// per thread): strides 1..8 stay in registers, strides 16..64 are warp shuffles.  A warp
// covers 512 consecutive elements of a row, i.e. whole blocks.  HBM-bound: one read and one
// write of the tensor.

#include <math.h>

#include "common.cuh"

namespace mixfp4 {
namespace {

constexpr int kThreads = 256;
constexpr int kE = 16;                    // elements per lane

template <typename T>
__device__ __forceinline__ float round_to(float v) { return static_cast<float>(Elem<T>::round(v)); }
template <> __device__ __forceinline__ float round_to<__nv_bfloat16>(float v) {
    return __bfloat162float(__float2bfloat16_rn(v));
}
template <> __device__ __forceinline__ float round_to<__half>(float v) { return __half2float(__float2half_rn(v)); }
template <> __device__ __forceinline__ float round_to<float>(float v) { return v; }

// v / root, IEEE round-to-nearest.  Block sizes 16 and 64 have a power-of-two root (an exact
// scaling).  For sqrt(32) and sqrt(128) the quotient comes from the reciprocal and two fused
// corrections, which equals the IEEE quotient for every significand of the dividend (swept
// by mixfp4_selftest_division); dividends outside [2^-100, 2^100] (zeros, subnormals,
// infinities, NaN) take the division instruction sequence.
__device__ __forceinline__ float div_root(float v, float root, float inv, bool pow2) {
    if (pow2) return __fmul_rn(v, inv);
    const float mag = fabsf(v);
    if (mag >= 7.888609e-31f && mag <= 1.2676506e30f) {
        const float q = __fmul_rn(v, inv);
        const float rem = __fmaf_rn(-q, root, v);
        return __fmaf_rn(rem, inv, q);
    }
    return __fdiv_rn(v, root);
}

template <typename T, bool kStagewise>
__global__ void __launch_bounds__(kThreads) fwht_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows,
                                                        int64_t k, int64_t ldx, int64_t ldy, int size, float root,
                                                        const float* __restrict__ signs, bool vec, int64_t chunks) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * (kThreads / 32) + __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);   // provably warp-uniform
    const int64_t row = warp / chunks;
    if (row >= rows) return;
    const int64_t chunk = warp - row * chunks;
    const int64_t col = chunk * (32 * kE) + lane * kE;
    const int64_t full_k = k / size * size;
    const T* xr = x + row * ldx;
    T* yr = y + row * ldy;
    const bool inside = col + kE <= full_k;      // a lane's 16 elements never straddle full_k (size % 16 == 0)

    float v[kE];
    if (col + kE <= k && vec) {
        constexpr int kPerVec = 16 / sizeof(T);
#pragma unroll
        for (int q = 0; q < kE / kPerVec; ++q) {
            const uint4 w = *reinterpret_cast<const uint4*>(xr + col + q * kPerVec);
            const T* e = reinterpret_cast<const T*>(&w);
#pragma unroll
            for (int j = 0; j < kPerVec; ++j) v[q * kPerVec + j] = Elem<T>::load(e + j);
        }
    } else {
#pragma unroll
        for (int j = 0; j < kE; ++j) v[j] = col + j < k ? Elem<T>::load(xr + col + j) : 0.0f;
    }

    if (inside) {
        if (signs) {
            const int e0 = static_cast<int>(col % size);
#pragma unroll
            for (int j = 0; j < kE; ++j) {
                v[j] = __fmul_rn(v[j], signs[e0 + j]);
                if (kStagewise) v[j] = round_to<T>(v[j]);
            }
        }
        // strides 1, 2, 4, 8 inside the lane
#pragma unroll
        for (int s = 1; s < kE; s <<= 1) {
#pragma unroll
            for (int j = 0; j < kE; ++j) {
                if (j & s) continue;
                const float l = v[j], r = v[j | s];
                v[j] = __fadd_rn(l, r);
                v[j | s] = __fsub_rn(l, r);
                if (kStagewise) { v[j] = round_to<T>(v[j]); v[j | s] = round_to<T>(v[j | s]); }
            }
        }
    }
    // strides 16 ... size/2 across lanes; every lane of the warp takes part in the shuffles,
    // lanes outside a whole block simply discard what they receive
    for (int bit = 1; bit * kE < size; bit <<= 1) {
#pragma unroll
        for (int j = 0; j < kE; ++j) {
            const float other = __shfl_xor_sync(0xffffffffu, v[j], bit);
            if (inside) {
                const float r = (lane & bit) ? __fsub_rn(other, v[j]) : __fadd_rn(v[j], other);
                v[j] = kStagewise ? round_to<T>(r) : r;
            }
        }
    }
    if (inside) {
        const bool pow2 = size == 16 || size == 64;
        const float inv = __frcp_rn(root);
#pragma unroll
        for (int j = 0; j < kE; ++j) v[j] = div_root(v[j], root, inv, pow2);
    }

    if (col + kE <= k && vec) {
        constexpr int kPerVec = 16 / sizeof(T);
#pragma unroll
        for (int q = 0; q < kE / kPerVec; ++q) {
            T o[kPerVec];
#pragma unroll
            for (int j = 0; j < kPerVec; ++j) o[j] = Elem<T>::round(v[q * kPerVec + j]);
            *reinterpret_cast<uint4*>(yr + col + q * kPerVec) = *reinterpret_cast<const uint4*>(o);
        }
    } else {
#pragma unroll
        for (int j = 0; j < kE; ++j)
            if (col + j < k) yr[col + j] = Elem<T>::round(v[j]);   // tail values pass through unchanged
    }
}

// Block size 128 on 16-bit inputs, one rounding at the end, no sign vector: what the prefill GEMM
// runs in front of itself.  Same stages, same order and the same single-add outputs as fwht_kernel
// (so the same bits), arranged for fewer instructions: a pair of lanes owns one 128-element block;
// a lane keeps the eight 16-byte chunks h, h+2, ..., h+14 of the block (h = lane parity: the pair reads
// and writes whole 32-byte sectors), so strides 1..4 and 16..64 stay in its registers and only stride 8
// crosses to the neighbouring lane (one shuffle per element instead of three).  Strides above 1 and the division run as packed two-element
// fp32 operations (add/fma .f32x2: each half is the IEEE operation).  The division by sqrt(128)
// takes the reciprocal form for the whole lane when every value lies inside the range for which
// that form was swept; a lane holding a zero, a tiny or an infinite value redoes its 64 divisions one by
// one with div_root (a NaN passes through either form as a NaN).
__device__ __forceinline__ void butterfly2(float2& a, float2& b) {      // (a, b) <- (a + b, a - b), both halves
    const float2 sum = __fadd2_rn(a, b);
    b = __ffma2_rn(b, make_float2(-1.0f, -1.0f), a);
    a = sum;
}

constexpr int kFastThreads = 128;
constexpr int kFastBlocksPerWarp = 16;

template <typename T>
__global__ void __launch_bounds__(kFastThreads) fwht128_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows,
                                                               int64_t ldx, int64_t ldy, int64_t blocks_per_row,
                                                               int64_t total_blocks, float root) {
    // a kernel launched behind this one with programmatic dependent launch (the prefill GEMM) may set itself
    // up once every CTA of this grid is under way; it still waits for this grid's end before it reads y
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int lane = threadIdx.x & 31, h = lane & 1;
    const int64_t warp = (int64_t)blockIdx.x * (kFastThreads / 32) + (threadIdx.x >> 5);
    const int64_t blk = warp * kFastBlocksPerWarp + (lane >> 1);
    const bool live = blk < total_blocks;        // dead lanes still take part in the shuffles
    const int64_t row = live ? blk / blocks_per_row : 0;
    const int64_t col = live ? (blk - row * blocks_per_row) * 128 : 0;
    const T* src = x + row * ldx + col;
    T* dst = y + row * ldy + col;

    float2 v[8][4];                              // [chunk c][pair p]: elements 8 * (2 c + h) + 2 p, + 1
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        uint4 w = make_uint4(0, 0, 0, 0);
        if (live) w = *reinterpret_cast<const uint4*>(src + 8 * (2 * c + h));      // (x may alias y: no read-only path)
        const T* e = reinterpret_cast<const T*>(&w);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float l = Elem<T>::load(e + 2 * q), r = Elem<T>::load(e + 2 * q + 1);
            v[c][q] = make_float2(__fadd_rn(l, r), __fsub_rn(l, r));       // stride 1
        }
        butterfly2(v[c][0], v[c][1]);            // stride 2
        butterfly2(v[c][2], v[c][3]);
        butterfly2(v[c][0], v[c][2]);            // stride 4
        butterfly2(v[c][1], v[c][3]);
    }
    // stride 8: the neighbouring lane holds the partner chunk; the even lane keeps l + r, the odd one l - r
    const float2 sgn = h ? make_float2(-1.0f, -1.0f) : make_float2(1.0f, 1.0f);
#pragma unroll
    for (int c = 0; c < 8; ++c)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            float2 o;
            o.x = __shfl_xor_sync(0xffffffffu, v[c][q].x, 1);
            o.y = __shfl_xor_sync(0xffffffffu, v[c][q].y, 1);
            v[c][q] = __ffma2_rn(v[c][q], sgn, o);       // v + o, or o - v: one rounding either way
        }
    // strides 16, 32, 64: chunks c and c + 1, + 2, + 4
#pragma unroll
    for (int st = 1; st < 8; st <<= 1)
#pragma unroll
        for (int c = 0; c < 8; ++c)
            if (!(c & st))
#pragma unroll
                for (int q = 0; q < 4; ++q) butterfly2(v[c][q], v[c | st][q]);
    // division by sqrt(128)
    const float inv = __frcp_rn(root);
    const float2 inv2 = make_float2(inv, inv), nroot2 = make_float2(-root, -root);
    float hi = 0.0f, lo = 3.0e38f;
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float ax = fabsf(v[i][j].x), ay = fabsf(v[i][j].y);      // |.| folds into the comparisons
            hi = fmaxf(hi, fmaxf(ax, ay));
            lo = fminf(lo, fminf(ax, ay));
        }
    if (lo >= 7.888609e-31f && hi <= 1.2676506e30f) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 t = __fmul2_rn(v[i][j], inv2);
                const float2 rem = __ffma2_rn(t, nroot2, v[i][j]);
                v[i][j] = __ffma2_rn(rem, inv2, t);
            }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
                v[i][j] = make_float2(div_root(v[i][j].x, root, inv, false), div_root(v[i][j].y, root, inv, false));
    }
    if (live) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            T o[8];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                o[2 * q] = Elem<T>::round(v[c][q].x);
                o[2 * q + 1] = Elem<T>::round(v[c][q].y);
            }
            *reinterpret_cast<uint4*>(dst + 8 * (2 * c + h)) = *reinterpret_cast<const uint4*>(o);
        }
    }
}

// The same block size on 16-bit inputs with EVERY stage rounded to the input type -- what the reference's
// activation hook computes on a bf16 tensor (project_quant/rotation.py:51-58 inside modeling.py:662-668) --
// in packed two-element 16-bit arithmetic.  A stage output is RN16(a +- b); the reference rounds the fp32 sum
// of two 16-bit values to 16 bits, and with 24 >= 2 * 11 + 2 significand bits that double rounding equals the
// single one of the packed add / fma.  Layout as in fwht128_kernel (a pair of lanes per block, chunks h, h+2,
// ... per lane), values kept as words of two neighbouring elements: stride 1 pairs the halves of a word
// ((l, l) + (r, r) * (1, -1) in one fma), strides 2 and 4 pair words of a chunk, stride 8 the neighbouring
// lane's word, strides 16 to 64 the chunks.  The final division is the fp32 one of fwht128_kernel, rounded
// once more to the input type.  amax (optional): the largest output magnitude, for the activation
// quantizer that follows (one atomic maximum per CTA on the float's bit pattern).
template <typename T> struct Pair;
template <> struct Pair<__nv_bfloat16> {
    using type = __nv_bfloat162;
    __device__ static type make(float a, float b) { return __floats2bfloat162_rn(a, b); }
    __device__ static type low2(type v) { return __low2bfloat162(v); }
    __device__ static type high2(type v) { return __high2bfloat162(v); }
    __device__ static float2 to_float2(type v) { return __bfloat1622float2(v); }
};
template <> struct Pair<__half> {
    using type = __half2;
    __device__ static type make(float a, float b) { return __floats2half2_rn(a, b); }
    __device__ static type low2(type v) { return __low2half2(v); }
    __device__ static type high2(type v) { return __high2half2(v); }
    __device__ static float2 to_float2(type v) { return __half22float2(v); }
};

template <typename T>
__global__ void __launch_bounds__(kFastThreads) fwht128_stagewise_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                                         int64_t ldx, int64_t ldy, int64_t blocks_per_row,
                                                                         int64_t total_blocks, float root,
                                                                         unsigned int* __restrict__ amax) {
    using P = Pair<T>;
    using T2 = typename P::type;
    const int lane = threadIdx.x & 31, h = lane & 1;
    const int64_t warp = (int64_t)blockIdx.x * (kFastThreads / 32) + (threadIdx.x >> 5);
    const int64_t blk = warp * kFastBlocksPerWarp + (lane >> 1);
    const bool live = blk < total_blocks;        // dead lanes still take part in the shuffles
    const int64_t row = live ? blk / blocks_per_row : 0;
    const int64_t col = live ? (blk - row * blocks_per_row) * 128 : 0;
    const T* src = x + row * ldx + col;
    T* dst = y + row * ldy + col;

    const T2 plus_minus = P::make(1.0f, -1.0f);
    T2 v[8][4];                                  // [chunk c][word p]: elements 8 * (2 c + h) + 2 p, + 1
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        uint4 w = make_uint4(0, 0, 0, 0);
        if (live) w = *reinterpret_cast<const uint4*>(src + 8 * (2 * c + h));      // (x may alias y: no read-only path)
        const T2* e = reinterpret_cast<const T2*>(&w);
#pragma unroll
        for (int q = 0; q < 4; ++q) v[c][q] = __hfma2(P::high2(e[q]), plus_minus, P::low2(e[q]));   // stride 1
#pragma unroll
        for (int st = 1; st < 4; st <<= 1)       // strides 2, 4: word q with word q + 1, + 2
#pragma unroll
            for (int q = 0; q < 4; ++q)
                if (!(q & st)) {
                    const T2 a = v[c][q], b = v[c][q | st];
                    v[c][q] = __hadd2(a, b);
                    v[c][q | st] = __hsub2(a, b);
                }
    }
    // stride 8: the even lane keeps l + r, the odd one l - r
    const T2 sgn = h ? P::make(-1.0f, -1.0f) : P::make(1.0f, 1.0f);
#pragma unroll
    for (int c = 0; c < 8; ++c)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint32_t mine = *reinterpret_cast<const uint32_t*>(&v[c][q]);
            const uint32_t other = __shfl_xor_sync(0xffffffffu, mine, 1);
            v[c][q] = __hfma2(v[c][q], sgn, *reinterpret_cast<const T2*>(&other));
        }
    // strides 16, 32, 64: chunks c and c + 1, + 2, + 4
#pragma unroll
    for (int st = 1; st < 8; st <<= 1)
#pragma unroll
        for (int c = 0; c < 8; ++c)
            if (!(c & st))
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const T2 a = v[c][q], b = v[c | st][q];
                    v[c][q] = __hadd2(a, b);
                    v[c | st][q] = __hsub2(a, b);
                }
    // division by sqrt(128) in fp32, one more rounding to the input type
    const float inv = __frcp_rn(root);
    const float2 inv2 = make_float2(inv, inv), nroot2 = make_float2(-root, -root);
    float2 f[8][4];
    float hi = 0.0f, lo = 3.0e38f;
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            f[i][j] = P::to_float2(v[i][j]);
            const float ax = fabsf(f[i][j].x), ay = fabsf(f[i][j].y);
            hi = fmaxf(hi, fmaxf(ax, ay));
            lo = fminf(lo, fminf(ax, ay));
        }
    if (lo >= 7.888609e-31f && hi <= 1.2676506e30f) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 t = __fmul2_rn(f[i][j], inv2);
                const float2 rem = __ffma2_rn(t, nroot2, f[i][j]);
                f[i][j] = __ffma2_rn(rem, inv2, t);
            }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
                f[i][j] = make_float2(div_root(f[i][j].x, root, inv, false), div_root(f[i][j].y, root, inv, false));
    }
    float top = 0.0f;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        T2 o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            o[q] = P::make(f[c][q].x, f[c][q].y);
            const float2 r = P::to_float2(o[q]);
            top = fmaxf(top, fmaxf(fabsf(r.x), fabsf(r.y)));
        }
        if (live) *reinterpret_cast<uint4*>(dst + 8 * (2 * c + h)) = *reinterpret_cast<const uint4*>(o);
    }
    if (amax) {
        if (!live) top = 0.0f;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, off));
        __shared__ float warp_top[kFastThreads / 32];
        if (lane == 0) warp_top[threadIdx.x >> 5] = top;
        __syncthreads();
        if (threadIdx.x == 0) {
#pragma unroll
            for (int w = 1; w < kFastThreads / 32; ++w) top = fmaxf(top, warp_top[w]);
            if (top > 0.0f) atomicMax(amax, __float_as_uint(top));       // non-negative floats order like their bits
        }
    }
}

// Sweep of div_root's reciprocal form against IEEE division: all 2^23 significands of the
// dividend for both irrational roots.
__global__ void fwht_selftest_kernel(unsigned long long* mismatches) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    const float a = __uint_as_float(0x3f800000u | i);
    unsigned long long bad = 0;
    const float roots[2] = {static_cast<float>(sqrt(32.0)), static_cast<float>(sqrt(128.0))};
#pragma unroll
    for (int d = 0; d < 2; ++d) {
        const float inv = __frcp_rn(roots[d]);
        bad += __float_as_uint(div_root(a, roots[d], inv, false)) != __float_as_uint(__fdiv_rn(a, roots[d]));
        bad += __float_as_uint(div_root(-a * 3.0e-5f, roots[d], inv, false)) != __float_as_uint(__fdiv_rn(-a * 3.0e-5f, roots[d]));
    }
    if (bad) atomicAdd(mismatches, bad);
}

template <typename T>
int launch(const void* x, void* y, int64_t rows, int64_t k, int64_t ldx, int64_t ldy, int size,
           const float* signs, int stagewise, cudaStream_t st, unsigned int* amax = nullptr) {
    const int64_t chunks = (k + 32 * kE - 1) / (32 * kE);
    const int64_t warps = rows * chunks;
    const int64_t ctas = (warps + kThreads / 32 - 1) / (kThreads / 32);
    if (ctas > 0x7fffffffLL) return MIXFP4_E_SHAPE;
    const bool vec = aligned(x, 16) && aligned(y, 16) && (ldx * sizeof(T)) % 16 == 0 && (ldy * sizeof(T)) % 16 == 0;
    const float root = static_cast<float>(sqrt(static_cast<double>(size)));
    if constexpr (sizeof(T) == 2) {
        if (size == 128 && !stagewise && !signs && vec && k % 128 == 0) {
            const int64_t blocks_per_row = k / 128, total = rows * blocks_per_row;
            const int64_t per_cta = (kFastThreads / 32) * kFastBlocksPerWarp;
            const int64_t fast_ctas = (total + per_cta - 1) / per_cta;
            if (fast_ctas > 0x7fffffffLL) return MIXFP4_E_SHAPE;
            fwht128_kernel<T><<<(unsigned)fast_ctas, kFastThreads, 0, st>>>(static_cast<const T*>(x), static_cast<T*>(y), rows,
                                                                           ldx, ldy, blocks_per_row, total, root);
            return check_launch("fwht128_kernel");
        }
    }
    if constexpr (sizeof(T) == 2) {
        if (size == 128 && stagewise && !signs && vec && k % 128 == 0) {
            const int64_t blocks_per_row = k / 128, total = rows * blocks_per_row;
            const int64_t per_cta = (kFastThreads / 32) * kFastBlocksPerWarp;
            const int64_t fast_ctas = (total + per_cta - 1) / per_cta;
            if (fast_ctas > 0x7fffffffLL) return MIXFP4_E_SHAPE;
            fwht128_stagewise_kernel<T><<<(unsigned)fast_ctas, kFastThreads, 0, st>>>(
                static_cast<const T*>(x), static_cast<T*>(y), ldx, ldy, blocks_per_row, total, root, amax);
            return check_launch("fwht128_stagewise_kernel");
        }
    }
    if (amax) return MIXFP4_E_UNSUPPORTED;           // only the kernel above reports the maximum
    if (stagewise && sizeof(T) == 2)
        fwht_kernel<T, true><<<(unsigned)ctas, kThreads, 0, st>>>(static_cast<const T*>(x), static_cast<T*>(y), rows, k,
                                                                  ldx, ldy, size, root, signs, vec, chunks);
    else
        fwht_kernel<T, false><<<(unsigned)ctas, kThreads, 0, st>>>(static_cast<const T*>(x), static_cast<T*>(y), rows, k,
                                                                   ldx, ldy, size, root, signs, vec, chunks);
    return check_launch("fwht_kernel");
}

}  // namespace

// Part of mixfp4_selftest_division: adds this file's mismatches to the counter.
int fwht_selftest_division(unsigned long long* mismatches, cudaStream_t st) {
    fwht_selftest_kernel<<<(1u << 23) / 256, 256, 0, st>>>(mismatches);
    return check_launch("fwht_selftest_kernel");
}

// H128 with every stage rounded (the activation hook's arithmetic) plus the largest output magnitude in
// *amax (zeroed here first), in one pass; MIXFP4_E_UNSUPPORTED when the rows are not whole 16-byte
// aligned blocks of 128 (the caller then runs the two passes separately).
int fwht128_stagewise_amax(const void* x, void* y, int dtype, int64_t rows, int64_t k, int64_t ldx, int64_t ldy,
                           float* amax, cudaStream_t st) {
    if (dtype != MIXFP4_BF16 && dtype != MIXFP4_F16) return MIXFP4_E_UNSUPPORTED;
    const bool vec = aligned(x, 16) && aligned(y, 16) && (ldx * 2) % 16 == 0 && (ldy * 2) % 16 == 0;
    if (!vec || k % 128 != 0) return MIXFP4_E_UNSUPPORTED;
    MIXFP4_CUDA_CHECK(cudaMemsetAsync(amax, 0, sizeof(float), st));
    unsigned int* out = reinterpret_cast<unsigned int*>(amax);
    return dtype == MIXFP4_BF16 ? launch<__nv_bfloat16>(x, y, rows, k, ldx, ldy, 128, nullptr, 1, st, out)
                                : launch<__half>(x, y, rows, k, ldx, ldy, 128, nullptr, 1, st, out);
}

}  // namespace mixfp4

using namespace mixfp4;

extern "C" int mixfp4_fwht(const void* x, void* y, int dtype, int64_t rows, int64_t k, int64_t ldx, int64_t ldy,
                           int size, const float* signs, int stagewise, void* stream) {
    if (!x || !y) return MIXFP4_E_NULL;
    if (rows <= 0 || k <= 0 || ldx < k || ldy < k) return MIXFP4_E_SHAPE;
    if (size != 16 && size != 32 && size != 64 && size != 128) return MIXFP4_E_MODE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case MIXFP4_BF16: return launch<__nv_bfloat16>(x, y, rows, k, ldx, ldy, size, signs, stagewise, st);
        case MIXFP4_F16: return launch<__half>(x, y, rows, k, ldx, ldy, size, signs, stagewise, st);
        case MIXFP4_F32: return launch<float>(x, y, rows, k, ldx, ldy, size, signs, stagewise, st);
        default: return MIXFP4_E_DTYPE;
    }
}
