// Shared device/host helpers for the mixfp4_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/mixfp4_b200.h"

namespace mixfp4 {

constexpr int kGroup = 16;          // elements per scale block (project_quant/candidates.py:14)
constexpr int kFmtSpan = 128;       // elements covered by one format byte

// Records a CUDA error for mixfp4_last_cuda_error() and returns MIXFP4_E_CUDA.
int record_cuda_error(cudaError_t err, const char* where);
int record_error_text(const char* text);

#define MIXFP4_CUDA_CHECK(expr)                                         \
    do {                                                                \
        cudaError_t err__ = (expr);                                     \
        if (err__ != cudaSuccess) return ::mixfp4::record_cuda_error(err__, #expr); \
    } while (0)

inline int check_launch(const char* where) {
    cudaError_t err = cudaGetLastError();
    return err == cudaSuccess ? MIXFP4_OK : record_cuda_error(err, where);
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per kernel instantiation AND device: the
// attribute belongs to the device's copy of the function, and a process may drive several GPUs.
// `done` is the instantiation's own bit mask (one bit per device ordinal, up to 64 devices).
template <typename Kernel>
inline int ensure_dynamic_smem(Kernel kernel, int bytes, unsigned long long& done) {
    int dev = 0;
    MIXFP4_CUDA_CHECK(cudaGetDevice(&dev));
    const unsigned long long bit = 1ull << (dev & 63);
    if (!(done & bit)) {
        MIXFP4_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
        done |= bit;
    }
    return MIXFP4_OK;
}

__host__ __device__ inline int64_t padded_k(int64_t k) { return (k + 127) / 128 * 128; }

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// ---- element conversions ---------------------------------------------------------------
__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) { return __uint_as_float(bits16 << 16); }

template <typename T> struct Elem;
template <> struct Elem<__nv_bfloat16> {
    static constexpr int kDtype = MIXFP4_BF16;
    __device__ static float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
    __device__ static __nv_bfloat16 round(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Elem<__half> {
    static constexpr int kDtype = MIXFP4_F16;
    __device__ static float load(const __half* p) { return __half2float(*p); }
    __device__ static __half round(float v) { return __float2half_rn(v); }
};
template <> struct Elem<float> {
    static constexpr int kDtype = MIXFP4_F32;
    __device__ static float load(const float* p) { return *p; }
    __device__ static float round(float v) { return v; }
};

// E4M3 byte -> float (exact; only non-negative finite bytes occur as block scales).
__device__ __forceinline__ float e4m3_to_float(uint32_t byte) {
    __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(byte), __NV_E4M3);
    return __half2float(__half(h));
}

__device__ __forceinline__ float level_value(uint32_t idx, bool e0m3) {
    // E0M3: the index itself.  E2M1: 0,.5,1,1.5,2,3,4,6 -- for idx >= 2 the index is the
    // (exponent, mantissa bit) pair of the float: bits = (idx + 252) << 22.
    if (e0m3) return static_cast<float>(idx);
    return idx >= 2 ? __uint_as_float((idx + 252u) << 22) : 0.5f * static_cast<float>(idx);
}

// fwht.cu: sweep of its reciprocal-form division (called by mixfp4_selftest_division).
int fwht_selftest_division(unsigned long long* mismatches, cudaStream_t st);
// fwht.cu: stage-wise rounded H128 of 16-bit rows plus the output's largest magnitude in one pass
// (MIXFP4_E_UNSUPPORTED unless the rows are whole, 16-byte aligned blocks of 128).
int fwht128_stagewise_amax(const void* x, void* y, int dtype, int64_t rows, int64_t k, int64_t ldx, int64_t ldy,
                           float* amax, cudaStream_t st);
// quantize.cu: the activation fake-quantization with the tensor maximum already in *amax.
int fake_quantize_with_amax(const void* x, int dtype, int64_t rows, int64_t k, int64_t ldx, int mode, const float* amax,
                            void* y, int64_t ldy, cudaStream_t st);

// comm.cu: the parts of a communicator the fused GEMV + all-reduce kernel needs (peers: 8 entries).
int comm_view(const mixfp4_comm* c, int* rank, int* world, int64_t* slot_packets, uint2** recv, uint2** peers,
              uint32_t** words);

}  // namespace mixfp4
