// Packed-code decode shared by the GEMV and GEMM kernels.
//
// A 256-entry table (4 KB, built per launch from the tensor scale) maps
// (format bit << 7 | E4M3 scale byte) to the block's eight magnitudes
// bf16((level * scale) * global) -- bit-identical to the reference's dequantized weight
// (project_quant/scale.py:59 followed by the bf16 cast of core.py:143) -- stored as 8 low
// bytes (x, y) and 8 high bytes (z, w).  Eight 4-bit codes become four bf16x2 registers
// with byte permutes only.
#pragma once

#include "common.cuh"

namespace mixfp4 {

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
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

// Kernel layout ("KL") of the packed weight -- a pure bit permutation of the canonical
// layout that makes the decode cheaper:
//   codes:  inside every 32-bit word (8 elements) the 3-bit magnitudes stay in their
//           nibbles, but bit 3 of nibble 2i+1 holds the sign of element i (i = 0..3) and
//           bit 3 of nibble 2i holds the sign of element 4+i, so one mask (elements 0..3)
//           and one shift+mask (elements 4..7) put the signs on bit 7 of the high bytes;
//   scales: bit 7 of the E4M3 byte (always 0 for a block scale) carries the block's format
//           bit, so the byte is the table index and no format array is read.
__host__ __device__ __forceinline__ uint32_t codes_to_kernel_layout(uint32_t w) {
    uint32_t out = w & 0x77777777u;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        out |= ((w >> (4 * i + 3)) & 1u) << (8 * i + 7);          // sign of element i
        out |= ((w >> (4 * (4 + i) + 3)) & 1u) << (8 * i + 3);    // sign of element 4 + i
    }
    return out;
}
__host__ __device__ __forceinline__ uint32_t codes_from_kernel_layout(uint32_t w) {
    uint32_t out = w & 0x77777777u;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        out |= ((w >> (8 * i + 7)) & 1u) << (4 * i + 3);
        out |= ((w >> (8 * i + 3)) & 1u) << (4 * (4 + i) + 3);
    }
    return out;
}

// Eight kernel-layout codes -> four bf16x2 registers (elements 01, 23, 45, 67).
// (Issuing the two shifts on the FMA pipe as multiplications was measured slower: the longer
// latency of the integer multiply outweighs the relief of the ALU pipe.)
__device__ __forceinline__ void decode8_kl(uint32_t w, const uint4& t, uint32_t (&p)[4]) {
    const uint32_t mag = w & 0x77777777u;
    const uint32_t mag_hi = mag >> 16, w4 = w << 4;
    uint32_t lo_a = prmt(t.x, t.y, mag), hi_a = prmt(t.z, t.w, mag);
    uint32_t lo_b = prmt(t.x, t.y, mag_hi), hi_b = prmt(t.z, t.w, mag_hi);
    hi_a |= w & 0x80808080u;
    hi_b |= w4 & 0x80808080u;
    p[0] = prmt(lo_a, hi_a, 0x5140u);
    p[1] = prmt(lo_a, hi_a, 0x7362u);
    p[2] = prmt(lo_b, hi_b, 0x5140u);
    p[3] = prmt(lo_b, hi_b, 0x7362u);
}

// Stream layout of the packed weight -- what the decode-shape kernels read fastest.  The weight is
// cut into chunks of 16 rows x 128 K elements, each chunk one contiguous run of kChunkBytes:
//   bytes    0 .. 1023   codes, row-major [16 rows][64 B], code words in the kernel-layout bit order;
//   bytes 1024 .. 1151   scale bytes, row-major [16 rows][8 blocks], format bit in bit 7.
// Chunks follow each other along K, then by row tile: chunk (tile, sub) starts at
// (tile * kpad/128 + sub) * kChunkBytes.  Rows past N in the last tile hold zero codes and the
// scale byte 0x01.  One cp.async.bulk moves a chunk; a warp's 16 x 128 step is exactly one chunk.
constexpr uint32_t kChunkBytes = 1152, kChunkCodeBytes = 1024, kChunkRows = 16, kChunkK = 128;
__host__ __device__ inline int64_t stream_tiles(int64_t rows) { return (rows + kChunkRows - 1) / kChunkRows; }
__host__ __device__ inline int64_t stream_bytes(int64_t rows, int64_t k) {
    return stream_tiles(rows) * (padded_k(k) / kChunkK) * kChunkBytes;
}


template <bool kKernelLayout>
__device__ __forceinline__ void decode_word(uint32_t w, const uint4& t, uint32_t (&p)[4]) {
    if constexpr (kKernelLayout) decode8_kl(w, t, p);
    else decode8(w, t, p);
}

}  // namespace mixfp4
