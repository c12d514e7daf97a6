// Prefill-shape dequant-linear (tcgen05).  Placeholder until the tensor-core kernel lands:
// the entry points exist so that the ABI is complete, and report MIXFP4_E_UNSUPPORTED.
#include "common.cuh"

extern "C" int64_t mixfp4_gemm_workspace_bytes(int64_t, int64_t, int64_t) { return 0; }

extern "C" int mixfp4_gemm(const void*, int64_t, int64_t, const uint8_t*, const uint8_t*, const uint8_t*,
                           const float*, int64_t, int64_t, int, void*, int, int64_t, void*, int64_t, int*, void*) {
    return MIXFP4_E_UNSUPPORTED;
}
