// Status strings, version and the per-thread record of the last CUDA error.
#include <stdio.h>
#include <string.h>

#include "common.cuh"

namespace mixfp4 {
namespace {
thread_local char g_last_error[512] = "";
}

int record_error_text(const char* text) {
    snprintf(g_last_error, sizeof(g_last_error), "%s", text);
    return MIXFP4_E_CUDA;
}

int record_cuda_error(cudaError_t err, const char* where) {
    snprintf(g_last_error, sizeof(g_last_error), "%s: %s (%s)", where, cudaGetErrorString(err),
             cudaGetErrorName(err));
    return MIXFP4_E_CUDA;
}
}  // namespace mixfp4

extern "C" int mixfp4_abi_version(void) { return MIXFP4_ABI_VERSION; }

extern "C" const char* mixfp4_last_cuda_error(void) { return mixfp4::g_last_error; }

extern "C" int64_t mixfp4_padded_k(int64_t k) { return mixfp4::padded_k(k); }

extern "C" const char* mixfp4_status_string(int status) {
    switch (status) {
        case MIXFP4_OK: return "ok";
        case MIXFP4_E_NULL: return "a required pointer is NULL";
        case MIXFP4_E_SHAPE: return "invalid size or stride";
        case MIXFP4_E_ALIGN: return "pointer or stride alignment requirement violated";
        case MIXFP4_E_DTYPE: return "unsupported element type";
        case MIXFP4_E_MODE: return "unknown mode";
        case MIXFP4_E_CUDA: return "CUDA call failed";
        case MIXFP4_E_WORKSPACE: return "workspace missing or too small";
        case MIXFP4_E_UNSUPPORTED: return "not supported by this build";
        case MIXFP4_E_DEVICE_WAIT: return "a bounded device-side wait gave up";
        case MIXFP4_E_TOO_LARGE: return "request exceeds the built-in capacity of this entry point";
        default: return "unknown status";
    }
}
