// Stand-alone normalised block Hadamard (project_quant/rotation.py:47-75 fwht / apply_transform).
//
// Natural (Sylvester) order: stage with stride s maps every pair (i, i+s) inside a block
// to (l + r, l - r); after log2(size) stages the block is divided by sqrt(size) (IEEE
// division by the fp32 value of sqrt(size), as the reference's CPU path does).  Each
// output of a stage is a single add, so the result does not depend on how the work is
// split across threads.  One lane keeps 4 consecutive elements: strides 1 and 2 stay in
// registers, strides 4..64 are warp shuffles.  A warp covers 128 consecutive elements of
// a row, i.e. 128/size whole blocks.  HBM-bound: one read and one write of the tensor.

#include <math.h>

#include "common.cuh"

namespace mixfp4 {
namespace {

constexpr int kThreads = 256;

template <typename T>
__device__ __forceinline__ float round_to(float v) { return static_cast<float>(Elem<T>::round(v)); }
template <> __device__ __forceinline__ float round_to<__nv_bfloat16>(float v) {
    return __bfloat162float(__float2bfloat16_rn(v));
}
template <> __device__ __forceinline__ float round_to<__half>(float v) { return __half2float(__float2half_rn(v)); }
template <> __device__ __forceinline__ float round_to<float>(float v) { return v; }

template <typename T, bool kStagewise>
__global__ void __launch_bounds__(kThreads) fwht_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows,
                                                        int64_t k, int64_t ldx, int64_t ldy, int size, float root,
                                                        const float* __restrict__ signs, bool vec, int64_t chunks) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
    const int64_t row = warp / chunks;
    if (row >= rows) return;
    const int64_t chunk = warp - row * chunks;
    const int64_t col = chunk * 128 + lane * 4;
    const int64_t full_k = k / size * size;
    const T* xr = x + row * ldx;
    T* yr = y + row * ldy;
    const bool inside = col + 4 <= full_k;       // quads never straddle full_k (size % 4 == 0)

    float v[4];
    if (inside && vec) {
        if constexpr (sizeof(T) == 2) {
            const uint2 w = *reinterpret_cast<const uint2*>(xr + col);
            const T* e = reinterpret_cast<const T*>(&w);
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = Elem<T>::load(e + j);
        } else {
            const float4 w = *reinterpret_cast<const float4*>(xr + col);
            v[0] = w.x; v[1] = w.y; v[2] = w.z; v[3] = w.w;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = col + j < k ? Elem<T>::load(xr + col + j) : 0.0f;
    }

    if (inside) {
        if (signs) {
            const int e0 = static_cast<int>(col % size);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                v[j] = __fmul_rn(v[j], signs[e0 + j]);
                if (kStagewise) v[j] = round_to<T>(v[j]);
            }
        }
        // strides 1 and 2 inside the lane
        float a = __fadd_rn(v[0], v[1]), b = __fsub_rn(v[0], v[1]);
        float c = __fadd_rn(v[2], v[3]), d = __fsub_rn(v[2], v[3]);
        if (kStagewise) { a = round_to<T>(a); b = round_to<T>(b); c = round_to<T>(c); d = round_to<T>(d); }
        v[0] = __fadd_rn(a, c); v[2] = __fsub_rn(a, c);
        v[1] = __fadd_rn(b, d); v[3] = __fsub_rn(b, d);
        if (kStagewise) {
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = round_to<T>(v[j]);
        }
    }
    // strides 4, 8, ... size/2 across lanes; every lane of the warp takes part in the
    // shuffles, lanes outside a whole block simply discard what they receive
    for (int bit = 1; bit * 4 < size; bit <<= 1) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float other = __shfl_xor_sync(0xffffffffu, v[j], bit);
            if (inside) {
                float r = (lane & bit) ? __fsub_rn(other, v[j]) : __fadd_rn(v[j], other);
                v[j] = kStagewise ? round_to<T>(r) : r;
            }
        }
    }
    if (inside) {
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = __fdiv_rn(v[j], root);
    }

    if (inside && vec) {
        T o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = Elem<T>::round(v[j]);
        if constexpr (sizeof(T) == 2) *reinterpret_cast<uint2*>(yr + col) = *reinterpret_cast<const uint2*>(o);
        else *reinterpret_cast<float4*>(yr + col) = *reinterpret_cast<const float4*>(o);
    } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (col + j < k) yr[col + j] = Elem<T>::round(v[j]);   // tail values pass through unchanged
    }
}

template <typename T>
int launch(const void* x, void* y, int64_t rows, int64_t k, int64_t ldx, int64_t ldy, int size,
           const float* signs, int stagewise, cudaStream_t st) {
    const int64_t chunks = (k + 127) / 128;
    const int64_t warps = rows * chunks;
    const int64_t ctas = (warps + kThreads / 32 - 1) / (kThreads / 32);
    if (ctas > 0x7fffffffLL) return MIXFP4_E_SHAPE;
    const size_t quad = 4 * sizeof(T);
    const bool vec = aligned(x, quad) && aligned(y, quad) && (ldx * sizeof(T)) % quad == 0 &&
                     (ldy * sizeof(T)) % quad == 0;
    const float root = static_cast<float>(sqrt(static_cast<double>(size)));
    if (stagewise && sizeof(T) == 2)
        fwht_kernel<T, true><<<(unsigned)ctas, kThreads, 0, st>>>(static_cast<const T*>(x), static_cast<T*>(y), rows, k,
                                                                  ldx, ldy, size, root, signs, vec, chunks);
    else
        fwht_kernel<T, false><<<(unsigned)ctas, kThreads, 0, st>>>(static_cast<const T*>(x), static_cast<T*>(y), rows, k,
                                                                   ldx, ldy, size, root, signs, vec, chunks);
    return check_launch("fwht_kernel");
}

}  // namespace
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
