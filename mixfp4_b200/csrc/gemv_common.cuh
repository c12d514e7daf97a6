// Pieces shared by the decode-shape kernels (gemv.cu, gemv_stream.cu): the mma.sync wrapper, the
// cp.async and shared-memory access helpers, and the packet form of the fused all-reduce.
#pragma once

#include "common.cuh"
#include "decode.cuh"

namespace mixfp4 {

constexpr int kRowsPerCta = 16;
constexpr int kStepK = 128;               // K elements one warp consumes per step
// The decode table is kept kLutRep times in shared memory, lane t of a quad reading copy t: lanes
// of a quad then never collide on a bank, which removes most conflicts of the random lookups.
constexpr int kLutRep = 1;
constexpr int kLutBytes = 4096 * kLutRep;

struct GemvArgs {
    const __nv_bfloat16* x;
    int64_t m, ldx;
    const uint8_t* codes;
    const uint8_t* scales;
    const uint8_t* fmt;
    const float* global_scale;
    const uint4* lut;                      // optional prebuilt decode table
    int64_t n, k, kpad;
    void* y;
    int out_dtype;
    int64_t ldy;
    bool x_vec;                            // x rows are 16-byte aligned and K % 8 == 0
    bool stream;                           // stream layout: `codes` is the chunk buffer, `scales` unused
    uint32_t code_step, scale_step;        // bytes from one 128-element step of a row tile to the next
};

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async16_stream(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory"); }

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
// Predicated load: lanes with pred == false keep the previous contents of v.
__device__ __forceinline__ void lds128_if(uint4& v, uint32_t addr, bool pred) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "@p ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n\t}"
        : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)
        : "r"(addr), "r"((uint32_t)pred));
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, const uint4& v) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// One ring stage of a warp: x [chunk 0..3][batch row][t] 16 B (m * 256 bytes), then the codes
// [row half][lane] 16 B, then the scales [row 0..15] 8 B.
__host__ __device__ inline uint32_t stage_bytes(int64_t m, bool x_resident) {
    return (x_resident ? 0u : (uint32_t)m * 256u) + 1024u + 128u;
}
// With x resident in shared memory (small M*K) a row of x takes kpad*2 + 16 bytes (the pad
// staggers the banks of different batch rows).
__host__ __device__ inline uint32_t xres_row_bytes(int64_t kpad) { return (uint32_t)kpad * 2u + 16u; }


// Fused all-reduce of a row-parallel GEMV (every rank holds a K shard of the same N rows): the
// partial sums of a row tile go straight into every peer's receive buffer as 8-byte packets
// {fp32 bits, sequence number}, the tile's owner threads then poll their own buffer and add the
// world partials in rank order (identical bits on every rank).  See comm.cu for the buffers.
struct AllReduceArgs {
    int rank, world;
    int64_t slot_packets;        // packets per source rank and parity
    uint2* recv;                 // this rank's buffer
    uint2* peer[8];              // every rank's buffer as seen from this GPU
    uint32_t* words;             // [0] sequence number, [1] finished-CTA counter
    int* status;                 // optional device word: nonzero after an expired wait
    uint64_t wait_ns;            // limit of a wait for a peer's packet (and at least a few thousand polls)
};


__device__ __forceinline__ void st_packet(uint2* p, uint32_t value, uint32_t flag) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(value), "r"(flag) : "memory");
}
__device__ __forceinline__ uint2 ld_packet(const uint2* p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint64_t gemv_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// gemv_stream.cu: the decode-shape linear on the stream layout (segments[i].codes = the chunk buffer,
// .scales unused); comm != nullptr selects the row-parallel form with the fused all-reduce.
int gemv_stream(const void* x, int64_t m, int64_t ldx, int64_t k, const mixfp4_gemv_segment* segments, int count,
                int out_dtype, int flags, const mixfp4_comm* comm, int* ar_status, cudaStream_t st);
// Limit of the bounded device-side waits (2 s unless mixfp4_set_wait_limit_ns changed it).
uint64_t wait_limit_ns();

}  // namespace mixfp4
