/*
 * mixfp4_b200 -- C ABI of the B200 (sm_100a) mixed-FP4 quantize / dequant-linear path.
 *
 * Plain pointers and sizes only; every pointer is a DEVICE pointer unless a
 * parameter says otherwise.  All work is enqueued on the caller's stream (a
 * cudaStream_t passed as void*) and nothing is synchronised.  Functions return 0
 * on success or a negative MIXFP4_E_* code; no exception crosses the boundary and
 * nothing is allocated behind the caller's back (kernels that need scratch
 * memory take a caller-supplied workspace).
 *
 * The reference (Xrelifen/mixfp4, package project_quant) is PyTorch-only and has
 * no FFI of its own; each entry point below names the reference function whose
 * work it replaces.
 *
 * Packed weight layout (row-major, produced by mixfp4_quantize):
 *   kpad   = mixfp4_padded_k(K)            K rounded up to a multiple of 128
 *   codes  u8 [rows, kpad/2]   element 2j in the low nibble of byte j, element 2j+1 in
 *                              the high nibble; nibble = sign<<3 | level index
 *                              (E2M1 levels 0,.5,1,1.5,2,3,4,6; E0M3 levels 0..7)
 *   scales u8 [rows, kpad/16]  E4M3 bit pattern of the block scale
 *   fmt    u8 [rows, kpad/128] bit b of byte j <-> block 8j+b; 1 = E0M3, 0 = E2M1
 *   global_scale f32 [1]       tensor scale (device memory)
 * Decode contract: w = round_bf16( (level * float(scale)) * global_scale ), two fp32
 * multiplies left to right, sign from nibble bit 3.
 */
#ifndef MIXFP4_B200_H_
#define MIXFP4_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MIXFP4_ABI_VERSION 3

#if defined(__GNUC__)
#define MIXFP4_API __attribute__((visibility("default")))
#else
#define MIXFP4_API
#endif

enum {
    MIXFP4_OK = 0,
    MIXFP4_E_NULL = -1,        /* a required pointer is NULL */
    MIXFP4_E_SHAPE = -2,       /* non-positive or inconsistent sizes / strides */
    MIXFP4_E_ALIGN = -3,       /* pointer or stride alignment requirement violated */
    MIXFP4_E_DTYPE = -4,       /* unknown or unsupported element type */
    MIXFP4_E_MODE = -5,        /* unknown format-selection mode / rotation size */
    MIXFP4_E_CUDA = -6,        /* a CUDA runtime or driver call failed; see mixfp4_last_cuda_error */
    MIXFP4_E_WORKSPACE = -7,   /* workspace missing or too small */
    MIXFP4_E_UNSUPPORTED = -8, /* valid request this build does not implement */
    MIXFP4_E_DEVICE_WAIT = -9, /* a bounded device-side wait gave up (status word non-zero) */
    MIXFP4_E_TOO_LARGE = -10   /* request exceeds a fixed built-in capacity */
};

/* element types */
enum { MIXFP4_BF16 = 0, MIXFP4_F16 = 1, MIXFP4_F32 = 2 };

/* Packed layouts.  CANONICAL is the layout above (what mixfp4_quantize writes and what
 * parity is hashed on).  KERNEL is a bit permutation of it that the linear kernels decode
 * with fewer instructions: same array shapes, but inside every 32-bit word of `codes`
 * (8 elements) bit 3 of nibble 2i+1 holds the sign of element i and bit 3 of nibble 2i the
 * sign of element 4+i (i = 0..3), and bit 7 of every scale byte holds the block's format
 * bit (the `fmt` array is not used).  mixfp4_repack converts either way.
 * STREAM is what the decode kernels stream fastest: one buffer of mixfp4_stream_bytes(rows, k)
 * bytes made of 1152-byte chunks, one per 16 rows x 128 K elements, chunk (tile, j) at
 * (tile * kpad/128 + j) * 1152: first 16 x 64 bytes of codes (row-major, code words in the KERNEL
 * bit order), then 16 x 8 scale bytes (row-major, format bit in bit 7).  Rows that pad the last
 * tile hold zero codes.  Entry points that take a layout accept the chunk buffer as `codes`;
 * `scales` and `fmt` are then unused and may be NULL.  mixfp4_repack_stream /
 * mixfp4_repack_from_stream convert from and to the canonical layout. */
enum { MIXFP4_LAYOUT_CANONICAL = 0, MIXFP4_LAYOUT_KERNEL = 1, MIXFP4_LAYOUT_STREAM = 2 };

/* flags of the linear entry points */
enum {
    /* Programmatic dependent launch: the kernel may start while the previous kernel in the
     * stream is still draining.  It prefetches the packed weight early and reads x only
     * after the previous kernel has completed.  Set it only if the previous kernel in the
     * stream does not write this call's packed weight, decode table or global scale. */
    MIXFP4_FLAG_OVERLAP_PREVIOUS = 1,
    /* Every `lut` of the call points to a table from mixfp4_decode_table_wide (36864 bytes: the
     * 4 KB table followed by its eightfold, bank-interleaved copy).  The stream-layout decode
     * kernel then takes the tables with one bulk copy instead of replicating them in every CTA. */
    MIXFP4_FLAG_WIDE_TABLE = 2
};

/* format selection (project_quant/region.py:22-39 mode names) */
enum { MIXFP4_MODE_ORACLE16 = 0, MIXFP4_MODE_ALL_E2M1 = 1, MIXFP4_MODE_ALL_E0M3 = 2,
       MIXFP4_MODE_GIVEN = 3 /* take every block's format from the bits already in fmt */ };

MIXFP4_API int mixfp4_abi_version(void);
MIXFP4_API const char* mixfp4_status_string(int status);
/* Text of the last CUDA error seen by this library on the calling thread ("" if none). */
MIXFP4_API const char* mixfp4_last_cuda_error(void);
MIXFP4_API int64_t mixfp4_padded_k(int64_t k);

/* Tensor-wide max |x| (first half of project_quant/scale.py:28-36 compute_global_scale).
 * x: [rows, k] with row stride ldx elements.  amax: one float; the call first sets it
 * to 0 on the stream and then reduces into it.  To quantize a shard with the scale of
 * the whole tensor, reduce the shards' amax values (max) before mixfp4_quantize. */
MIXFP4_API int mixfp4_amax(const void* x, int dtype, int64_t rows, int64_t k, int64_t ldx,
                float* amax, void* stream);

/* Block quantizer: replaces project_quant/candidates.py:62-106 build_candidates +
 * scale.py:43-61 _one_scale_candidate (standard rule) + codebook.py:12-25,41-43 +
 * the per-block choice and output cast of core.py:115-143.  Bit-exact with the
 * reference's CPU arithmetic.
 *   amax          device float from mixfp4_amax (global scale = amax / 2688, or 1 if 0)
 *   codes/scales/fmt/global_scale   packed outputs (layout above); padding blocks are
 *                 written too, so the buffers need no initialisation
 *   e2_err, e0_err, e2_scale, e0_scale   optional f32 [rows, ceil(k/16)] per-block
 *                 candidate errors and scales (GranularityResult fields), may be NULL
 *   dequant       optional [rows, k] (row stride ld_dequant) dequantized tensor in the
 *                 source dtype -- the reference's return value -- may be NULL */
MIXFP4_API int mixfp4_quantize(const void* x, int dtype, int64_t rows, int64_t k, int64_t ldx, int mode,
                    const float* amax,
                    uint8_t* codes, uint8_t* scales, uint8_t* fmt, float* global_scale,
                    float* e2_err, float* e0_err, float* e2_scale, float* e0_scale,
                    void* dequant, int64_t ld_dequant, void* stream);

/* Fake-quantization of an activation tensor: y = dequantized mixed-FP4 form of x, in x's dtype
 * (what the reference's forward-pre-hook feeds the linear in its W4A4 modes,
 * project_quant/modeling.py:662-705: quant_mixfp4_granularity(x, operand_role="activation_a")
 * with the global scale taken over the whole tensor of this call, scale.py:28-36).  One call =
 * mixfp4_amax into *amax (device float[1] scratch, left holding max|x|) followed by the
 * quantizer with no packed outputs.  mode: ORACLE16, ALL_E2M1 or ALL_E0M3 (coarse activation
 * regions take the three-pass route: mixfp4_quantize, mixfp4_select_regions, mixfp4_quantize).
 * y may be x itself (same pointer and row stride); any other overlap is not allowed. */
MIXFP4_API int mixfp4_fake_quantize(const void* x, int dtype, int64_t rows, int64_t k, int64_t ldx, int mode,
                         float* amax, void* y, int64_t ldy, void* stream);

/* Coarse format regions (project_quant/region.py:42-86 region_shape / aggregate_regions and
 * selector.py:28-33 mse_selection): one format per region of region_rows x region_groups K16
 * blocks, E0M3 iff the region's summed E0M3 error is smaller (ties keep E2M1), summed in the
 * reference's fp32 order.  e2_err / e0_err: f32 [rows, ceil(k/16)] from mixfp4_quantize; fmt:
 * [rows, kpad/128] format bits out.  Follow with mixfp4_quantize(mode = MIXFP4_MODE_GIVEN) on the
 * same fmt.  region_groups 2 or 4 (k32 / k64 regions), or 1 with region_rows 8 or 16 (n8k16 /
 * m16k16: the column sums follow the order PyTorch's CPU kernels use on an AVX-512 host, see
 * quantize.cu); MIXFP4_E_MODE for other widths and for multi-row regions when K has a single
 * region (the reference's sum order differs there).
 * mixfp4_select_layer: the "layer" region (one format for the whole tensor, region.py:44-45):
 * sets every format bit iff the E0M3 errors of all blocks sum to less than the E2M1 errors.  The
 * sums are taken in double precision in *sums (device double[2] scratch, zeroed by the call); the
 * reference's fp32 sum over the whole tensor depends on its host's thread count, the decision
 * does not unless both sums agree to about 1e-7. */
MIXFP4_API int mixfp4_select_regions(const float* e2_err, const float* e0_err, int64_t rows, int64_t k,
                          int region_rows, int region_groups, uint8_t* fmt, void* stream);
MIXFP4_API int mixfp4_select_layer(const float* e2_err, const float* e0_err, int64_t rows, int64_t k,
                          double* sums, uint8_t* fmt, void* stream);

/* Diagnostic: the quantizer divides by block scales with a reciprocal-and-residual sequence
 * instead of a full IEEE division.  This runs the exhaustive proof that the two agree (all 2^23
 * dividend significands x the 8 significands an E4M3 scale or the constants 6 and 7 can have;
 * likewise for the Hadamard kernel's division by sqrt(32) and sqrt(128)), and the proof that the
 * E2M1 rounding done on the FP4 conversion unit equals the reference's round-half-up
 * (project_quant/codebook.py:12-25) for every fp32 magnitude from 0 to 16, level and code;
 * it leaves the number of disagreements (expected 0) in *mismatches (device memory). */
MIXFP4_API int mixfp4_selftest_division(unsigned long long* mismatches, void* stream);

/* Element-wise rounding to a codebook: y[i] = sign(x[i]) * nearest level of |x[i]| with the
 * reference's tie rules (project_quant/codebook.py:12-25 quantize_e2m1: round half up on the
 * private mantissa, saturate at 6; :41-43 quantize_e0m3: round half even, saturate at 7).
 * x, y: device f32 [n]; e0m3: 0 = E2M1, 1 = E0M3. */
MIXFP4_API int mixfp4_round_codebook(const float* x, float* y, int64_t n, int e0m3, void* stream);

/* The E0M3 candidate of every K16 block under the reference's scale_rule "four_over_six"
 * (project_quant/scale.py:64-103 _four_over_six_scale_candidate with qmax 7 and :207-225: the base
 * and the 1.5x expanded E4M3 scale, the expanded one kept where its squared error is strictly
 * smaller).  Bit-exact with the reference's CPU arithmetic.  The E2M1 side of that rule lives in an
 * upstream package the reference does not vendor and is not provided.
 *   grouped        device f32 [nblocks, 16]: the tensor up-cast, zero-padded and grouped
 *   amax           device float: max |x| of the whole tensor (mixfp4_amax)
 *   codes, dequant f32 [nblocks, 16]: level values with sign, dequantized values
 *   scales, errors f32 [nblocks];  expansion_ids u8 [nblocks] (1 = the expanded scale was kept) */
MIXFP4_API int mixfp4_e0_four_over_six(const float* grouped, int64_t nblocks, const float* amax,
                            float* codes, float* dequant, float* scales, float* errors,
                            uint8_t* expansion_ids, void* stream);

/* Packed -> dense weight in out_dtype (the tensor the reference stores back into
 * nn.Linear.weight, project_quant/modeling.py:629). */
MIXFP4_API int mixfp4_dequant(const uint8_t* codes, const uint8_t* scales, const uint8_t* fmt,
                   const float* global_scale, int64_t rows, int64_t k, int layout,
                   void* out, int out_dtype, int64_t ldo, void* stream);

/* Layout conversion (no reference counterpart: the reference has no packed form).
 * to_layout = MIXFP4_LAYOUT_KERNEL: reads codes/scales/fmt, writes codes_out/scales_out
 * (fmt_out unused).  to_layout = MIXFP4_LAYOUT_CANONICAL: reads codes/scales (fmt unused),
 * writes codes_out/scales_out/fmt_out.  A pure bit permutation; round trip is the identity. */
MIXFP4_API int mixfp4_repack(const uint8_t* codes, const uint8_t* scales, const uint8_t* fmt,
                  int64_t rows, int64_t k, int to_layout,
                  uint8_t* codes_out, uint8_t* scales_out, uint8_t* fmt_out, void* stream);

/* Stream layout (no reference counterpart).  mixfp4_stream_bytes: size of the chunk buffer of a
 * [rows, k] weight.  mixfp4_repack_stream: canonical codes/scales/fmt -> chunks.
 * mixfp4_repack_from_stream: chunks -> canonical codes_out/scales_out/fmt_out.  Pure permutations. */
MIXFP4_API int64_t mixfp4_stream_bytes(int64_t rows, int64_t k);
MIXFP4_API int mixfp4_repack_stream(const uint8_t* codes, const uint8_t* scales, const uint8_t* fmt,
                         int64_t rows, int64_t k, uint8_t* chunks, void* stream);
MIXFP4_API int mixfp4_repack_from_stream(const uint8_t* chunks, int64_t rows, int64_t k,
                              uint8_t* codes_out, uint8_t* scales_out, uint8_t* fmt_out, void* stream);

/* Decode table of a packed weight: 256 entries x 16 B indexed by (format << 7 | E4M3 scale
 * byte) holding the block's eight bf16 magnitudes bf16((level * scale) * global).  Optional
 * input of the linear kernels (they build it per launch when given NULL). */
MIXFP4_API int mixfp4_decode_table(const float* global_scale, void* lut, void* stream);
/* The same table (first 4096 bytes, usable wherever a `lut` is taken) followed by 32768 bytes that
 * hold every entry eight times (entry e, copy j at 4096 + (8 e + j) * 16): the image the
 * stream-layout decode kernel keeps in shared memory, where a quarter-warp's eight look-ups then
 * never share a bank.  lut: 36864 bytes, 16-byte aligned.  See MIXFP4_FLAG_WIDE_TABLE. */
MIXFP4_API int mixfp4_decode_table_wide(const float* global_scale, void* lut, void* stream);

/* Normalised block Hadamard along the last axis (project_quant/rotation.py:47-75
 * fwht / apply_transform).  size in {16,32,64,128}; only whole blocks are transformed,
 * a tail of k % size elements is copied through.  signs: optional device f32 [size]
 * of +-1 applied before the butterflies (rotation.py:41-44).  y may alias x.
 * stagewise != 0 rounds to the element type after every butterfly stage, which is
 * what the reference does when it runs on a bf16/fp16 tensor; 0 keeps fp32 through all
 * stages and rounds once at the end. */
MIXFP4_API int mixfp4_fwht(const void* x, void* y, int dtype, int64_t rows, int64_t k, int64_t ldx,
                int64_t ldy, int size, const float* signs, int stagewise, void* stream);

/* Decode-shape dequant-linear, 1 <= M <= 16: y[M,N] = x[M,K] * W[N,K]^T with W packed
 * (replaces F.linear on the dequantized weight, modeling.py:629 + nn.Linear.forward).
 * x bf16 [M,K] row stride ldx; y in out_dtype (MIXFP4_F32 or MIXFP4_BF16) row stride ldy.
 * fp32 accumulation.  layout: MIXFP4_LAYOUT_*; fmt may be NULL for the kernel layout.
 * lut: optional table from mixfp4_decode_table.  flags: MIXFP4_FLAG_*. */
MIXFP4_API int mixfp4_gemv(const void* x, int64_t m, int64_t ldx,
                const uint8_t* codes, const uint8_t* scales, const uint8_t* fmt,
                const float* global_scale, int64_t n, int64_t k, int layout, const void* lut,
                void* y, int out_dtype, int64_t ldy, int flags, void* stream);

/* Several weights that take the same x in one launch (q/k/v, gate/up of a decoder layer; no
 * single counterpart in the reference, which calls nn.Linear.forward once per projection,
 * modeling.py:629): y_i[M,n_i] = x[M,K] * W_i[n_i,K]^T for i < count, 1 <= count <= 3,
 * 1 <= M <= 16, all weights in the same layout (MIXFP4_LAYOUT_KERNEL or MIXFP4_LAYOUT_STREAM)
 * with the same K.  Saves the per-launch ramp of the small projections.  Returns MIXFP4_E_SHAPE
 * when x (M * (2 * padded K + 16) bytes) or the tables do not fit in shared memory: call
 * mixfp4_gemv per weight then. */
typedef struct mixfp4_gemv_segment {
    const uint8_t* codes;          /* kernel layout [n, kpad/2], or the stream layout's chunk buffer */
    const uint8_t* scales;         /* kernel layout [n, kpad/16]; unused (NULL) for the stream layout */
    const float* global_scale;     /* device f32[1] */
    const void* lut;               /* optional table from mixfp4_decode_table, else NULL */
    void* y;                       /* [M, n] in out_dtype */
    int64_t ldy;
    int64_t n;
} mixfp4_gemv_segment;
/* 1 if the stream-layout decode kernel can keep x resident for `count` weights of this K (the
 * fused all-reduce and the grouped launch need that), else 0.  Host-only arithmetic; ranks of a
 * tensor-parallel group call it with the largest K shard so that all take the same branch. */
MIXFP4_API int mixfp4_gemv_x_fits(int64_t m, int64_t k, int count);
MIXFP4_API int mixfp4_gemv_grouped(const void* x, int64_t m, int64_t ldx, int64_t k,
                        const mixfp4_gemv_segment* segments, int count, int layout,
                        int out_dtype, int flags, void* stream);

/* Row-parallel decode linear with the all-reduce fused into the kernel (tensor parallelism over
 * the GPUs of one node, one process per GPU; replaces F.linear on a K shard of the weight,
 * modeling.py:629, followed by the sum over ranks that a row-parallel split needs -- the reference
 * itself is single-device).  Every rank calls with its own K shard (x [M, k_shard], weight
 * [n, k_shard] in MIXFP4_LAYOUT_KERNEL or MIXFP4_LAYOUT_STREAM) and receives the same y = sum over
 * ranks, added in rank order.  Partial sums travel as 8-byte {value, sequence} packets stored
 * directly into the peers' buffers; every wait is bounded (2 s unless mixfp4_set_wait_limit_ns
 * changed it) and reports through *status (device int, optional: 100 + the rank whose packet did
 * not arrive; the output is then invalid, the kernel still returns and later launches work).
 * 1 <= M <= 8.
 *
 * Communicator: mixfp4_comm_create allocates this rank's receive buffer (slot_floats >= M * n of
 * the largest call) on the current device; mixfp4_comm_handle exports it (mixfp4_comm_handle_bytes
 * bytes); after the ranks have exchanged the handles, mixfp4_comm_open maps the peers' buffers
 * (handles = world entries in rank order).  All ranks must issue the same sequence of
 * mixfp4_gemv_allreduce calls. */
typedef struct mixfp4_comm mixfp4_comm;
MIXFP4_API int mixfp4_comm_create(int rank, int world, int64_t slot_floats, mixfp4_comm** out);
MIXFP4_API int mixfp4_comm_handle_bytes(void);
MIXFP4_API int mixfp4_comm_handle(const mixfp4_comm* comm, void* handle);
MIXFP4_API int mixfp4_comm_open(mixfp4_comm* comm, const void* handles);
/* Same for a process that drives several GPUs itself (or a test): buffers = world device pointers
 * in rank order, each at least mixfp4_comm_buffer_bytes(world, slot_floats) bytes, zeroed, and
 * reachable from this GPU (peer access enabled by the caller); this rank's own entry is ignored. */
MIXFP4_API int64_t mixfp4_comm_buffer_bytes(int world, int64_t slot_floats);
/* This rank's receive buffer (device pointer): [2 parities][world source ranks][slot_floats] packets
 * of {fp32 bits, sequence number + 1}, the pointer the other GPUs' communicators are opened with. */
MIXFP4_API int mixfp4_comm_buffer(const mixfp4_comm* comm, void** buffer);
MIXFP4_API int mixfp4_comm_open_local(mixfp4_comm* comm, void* const* buffers);
MIXFP4_API int mixfp4_comm_destroy(mixfp4_comm* comm);
MIXFP4_API int mixfp4_gemv_allreduce(const mixfp4_comm* comm, const void* x, int64_t m, int64_t ldx,
                          const uint8_t* codes, const uint8_t* scales, const float* global_scale,
                          const void* lut, int64_t n, int64_t k, int layout, void* y, int out_dtype,
                          int64_t ldy, int* status, int flags, void* stream);

/* Bounded device-side waits.  Every spin in the kernels (on a weight chunk, a tensor-core stage, a
 * peer's packet) gives up after a time limit, records a code in a status word and lets the kernel
 * finish.  mixfp4_set_wait_limit_ns changes the limit of the decode kernels' waits for later
 * launches (default 2 s; meant for tests and for hosts with their own watchdog).
 * mixfp4_check_status synchronises `stream`, reads the device word `dev_status` (NULL: the decode
 * kernels' own word for weight chunks on the current device), stores it in *value (optional) and
 * returns MIXFP4_E_DEVICE_WAIT if it is non-zero, else MIXFP4_OK. */
MIXFP4_API int mixfp4_set_wait_limit_ns(uint64_t ns);
MIXFP4_API int mixfp4_check_status(const int* dev_status, int* value, void* stream);

/* Prefill-shape dequant-linear on the tcgen05 tensor cores (any M >= 1, meant for
 * M >= 128).  rotation_block: 0, or 128 to apply the block-Hadamard H128 to x first (the
 * reference's forward-pre-hook, modeling.py:662-668): a rotation kernel of its own writes
 * bf16(FWHT_fp32(x)) into the workspace and the GEMM kernel, launched behind it as a programmatic
 * dependent, reads that (its set-up and weight loads overlap the rotation's tail; the rotation is
 * not part of the GEMM kernel).  workspace: device scratch of at least
 * mixfp4_gemm_workspace_bytes(m, n, k) bytes: a staging area for x (needed with rotation_block =
 * 128 or an x that TMA cannot address: MIXFP4_E_WORKSPACE without it) followed by room for
 * split-K partial sums (problems with few output tiles and a long K run several CTAs per tile;
 * optional: with a smaller or NULL workspace one CTA per tile does the whole K range, the result
 * then differs in fp32 summation order only) and a 256-byte slot used by mixfp4_gemm_a4.
 * status: optional device int[1]; non-zero after completion if a bounded device-side
 * wait gave up (the output is then invalid). */
MIXFP4_API int64_t mixfp4_gemm_workspace_bytes(int64_t m, int64_t n, int64_t k);
MIXFP4_API int mixfp4_gemm(const void* x, int64_t m, int64_t ldx,
                const uint8_t* codes, const uint8_t* scales, const uint8_t* fmt,
                const float* global_scale, int64_t n, int64_t k, int layout, const void* lut,
                int rotation_block, void* y, int out_dtype, int64_t ldy,
                void* workspace, int64_t workspace_bytes, int* status, int flags, void* stream);

/* W4A4 in the reference's sense: the activations are rotated (rotation_block 0 or 128; every
 * butterfly stage rounded to bf16, which is what the reference's hook computes on a bf16 tensor,
 * rotation.py:47-58), fake-quantized with mixfp4_fake_quantize(mode = act_mode) and then multiplied
 * with the packed weight by mixfp4_gemm -- ActivationHooks._hook followed by nn.Linear.forward
 * (modeling.py:662-705, :629).  The operand the tensor cores read is the reference's dequantized
 * bf16 activation, bit for bit; an FP4 x FP4 MMA on the codes would not reproduce the bf16 rounding
 * of either operand.  workspace: at least mixfp4_gemm_workspace_bytes(m, n, k) bytes, required
 * (staging area, split-K partial sums, amax word).  Other arguments as mixfp4_gemm. */
MIXFP4_API int mixfp4_gemm_a4(const void* x, int64_t m, int64_t ldx,
                const uint8_t* codes, const uint8_t* scales, const uint8_t* fmt,
                const float* global_scale, int64_t n, int64_t k, int layout, const void* lut,
                int rotation_block, int act_mode, void* y, int out_dtype, int64_t ldy,
                void* workspace, int64_t workspace_bytes, int* status, int flags, void* stream);

/* Allocation-free form of the H128-rotated prefill linear.  No counterpart in the
 * reference: it exists for hosts that must not (or cannot) allocate device memory around
 * the call -- an inference server that handed its whole memory budget to its own arena at
 * start-up, a plugin running inside another runtime's allocator, a real-time loop where
 * cudaMalloc's implicit synchronisation is unacceptable.  It computes exactly what
 * mixfp4_gemm(..., rotation_block = 128, ...) computes, but the buffer that holds the
 * rotated activations bf16(H128 x) is a fixed array inside the library instead of a
 * caller-supplied workspace (split-K partial sums go into the same array when they fit behind
 * the activations; when they do not, the result differs from the workspace form in fp32
 * summation order only).  The call makes no cudaMalloc/cudaFree and calls no routine
 * that allocates.
 *   Limit: m * round_up(k, 8) * 2 bytes must not exceed
 *   mixfp4_gemm_h128_static_max_bytes() (8 MiB, e.g. 1024 x 4096); larger requests return
 *   MIXFP4_E_TOO_LARGE and do nothing.  Every GPU that loads the library holds those 8 MiB
 *   until the process exits.
 *   The first call on each device looks up the array's device address (the device must be
 *   current); make that first call outside any stream capture.
 *   All calls on a device share the one array and it keeps whatever the last call left in
 *   it.  Each call rewrites every element it later reads, so nothing needs clearing, but
 *   two calls whose kernels can overlap on the GPU (different streams, no ordering) race on
 *   the array and corrupt each other: order them. */
MIXFP4_API int64_t mixfp4_gemm_h128_static_max_bytes(void);
MIXFP4_API int mixfp4_gemm_h128_static(const void* x, int64_t m, int64_t ldx,
                const uint8_t* codes, const uint8_t* scales, const uint8_t* fmt,
                const float* global_scale, int64_t n, int64_t k, int layout, const void* lut,
                void* y, int out_dtype, int64_t ldy, int* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MIXFP4_B200_H_ */
