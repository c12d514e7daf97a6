/*
 * CPU oracle for the mixed-FP4 (E2M1 / E0M3) block quantizer, its packed form,
 * the block-Hadamard rotation and the dequant-linear.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in scalar C, the arithmetic of
 * the reference's PyTorch CPU path so that the CUDA kernels can be compared with
 * it bit for bit.  It is never part of the product path: only the tests, the
 * smoke check and the CPU-baseline leg of the benchmark may build or call it.
 *
 * Parity is PINNED: the fixtures under tests/golden/ were produced by running the
 * reference itself (project_quant, torch CPU) and this file reproduces every one
 * of them exactly (codes, scales, format ids, both candidates' block errors as
 * fp32 bit patterns, dequantized tensors, rotations).
 *
 * Reference functions restated here (paths inside the reference project):
 *   project_quant/candidates.py:62-106   build_candidates  (fp32 up-cast, right zero pad of K to x16)
 *   project_quant/scale.py:28-36         compute_global_scale (amax / (6*448), all-zero -> 1)
 *   project_quant/scale.py:39-61         _e4m3, _one_scale_candidate (standard rule)
 *   project_quant/codebook.py:12-25      quantize_e2m1  (round-half-up on the private mantissa)
 *   project_quant/codebook.py:41-43      quantize_e0m3  (round-half-even, saturate 7)
 *   project_quant/core.py:115-143        oracle16 choice (e0 < e2, ties keep E2M1), select, un-pad, cast
 *   project_quant/rotation.py:47-75      fwht / apply_transform
 *   project_quant/region.py:42-86, selector.py:28-33   coarse format regions (mse selector)
 *   project_quant/scale.py:64-103, 207-225   the E0M3 candidate under scale_rule "four_over_six"
 *
 * All arithmetic is IEEE binary32, round-to-nearest-even, with NO fused
 * multiply-add (compile with -ffp-contract=off, no -ffast-math).
 *
 * Packed layout written by this file (the reference has no packed form; the
 * product defines it and this oracle packs the reference's per-block results):
 *   kpad   = K rounded up to a multiple of 128
 *   codes  u8 [rows, kpad/2]   element 2j in the low nibble of byte j, 2j+1 in the
 *                              high nibble; nibble = sign<<3 | level index
 *   scales u8 [rows, kpad/16]  E4M3 bit pattern of the selected block scale
 *   fmt    u8 [rows, kpad/128] bit b of byte j <-> block 8j+b; 1 = E0M3
 *   global_scale f32
 * Blocks past the last real K16 block are what an all-zero block quantizes to:
 * codes 0, scale byte 0x01 (2^-9), format bit 0.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define MIXFP4_GROUP 16

static const float kE2M1Levels[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

static inline float bits_to_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f32_to_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

static inline float bf16_to_f32(uint16_t h) { return bits_to_f32((uint32_t)h << 16); }

/* fp32 -> bf16, round-to-nearest-even (what torch's .to(bfloat16) does). */
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u = f32_to_bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

static inline float round_to_bf16(float f) { return bf16_to_f32(f32_to_bf16(f)); }

/* scale.py:39-40 on a value already clamped to [2^-9, 448]: nearest E4M3
 * (4 exponent bits, bias 7, 3 mantissa bits, subnormal step 2^-9), ties to even.
 * Returns the byte; *value receives the decoded float. */
static inline uint8_t e4m3_round(float v, float* value) {
    float r;
    if (v < 0.015625f) {                      /* below the smallest normal 2^-6 */
        r = rintf(v * 512.0f);                /* exact scaling, RNE */
        *value = r / 512.0f;
        return (uint8_t)r;                    /* 1..8; 8 is the encoding of 2^-6 */
    }
    int e;
    (void)frexpf(v, &e);                      /* v = m * 2^e, m in [0.5, 1) */
    e -= 1;                                   /* v in [2^e, 2^(e+1)) */
    float quantum = ldexpf(1.0f, e - 3);
    r = rintf(v / quantum) * quantum;         /* both steps exact except the RNE */
    (void)frexpf(r, &e);
    e -= 1;
    int mant = (int)(r / ldexpf(1.0f, e - 3)) - 8;
    *value = r;
    return (uint8_t)(((e + 7) << 3) | mant);
}

static inline float e4m3_decode(uint8_t b) {
    int e = (b >> 3) & 15, m = b & 7;
    float v = e ? ldexpf((float)(8 + m), e - 10) : ldexpf((float)m, -9);
    return (b & 0x80) ? -v : v;
}

/* codebook.py:12-25 replayed for |x|: exponent floor(log2|x|) clamped at 0,
 * mantissa = |x| / 2^e * 2, floor(mantissa + 0.5), back-scale, saturate 6.
 * Returns the level index 0..7 into kE2M1Levels. */
static inline int e2m1_index(float mag) {
    float q;
    if (mag < 2.0f)       q = floorf(mag * 2.0f + 0.5f) * 0.5f;   /* e = 0 */
    else if (mag < 4.0f)  q = floorf(mag + 0.5f);                 /* e = 1 */
    else if (mag < 8.0f)  q = floorf(mag * 0.5f + 0.5f) * 2.0f;   /* e = 2 */
    else                  q = 8.0f;                               /* e >= 3: >= 8 before the clamp */
    if (q > 6.0f) q = 6.0f;
    if (q < 2.0f) return (int)(q * 2.0f);
    if (q < 4.0f) return 2 + (int)q;
    return q == 4.0f ? 6 : 7;
}

/* codebook.py:41-43 for |x|: round-half-even, saturate 7. */
static inline int e0m3_index(float mag) {
    float q = rintf(mag);
    if (q > 7.0f) q = 7.0f;
    return (int)q;
}

/* One candidate of one block (scale.py:43-61).  s[] = x / global.  Fills the
 * 16 nibbles, returns the block error; *scale_byte / *scale_val the E4M3 scale. */
static inline float block_candidate(const float* x, const float* s, float global_scale,
                                    int e0m3, uint8_t* nib, uint8_t* scale_byte, float* scale_val) {
    float amax = 0.0f;
    for (int i = 0; i < MIXFP4_GROUP; ++i) { float a = fabsf(s[i]); if (a > amax) amax = a; }
    float ideal = amax / (e0m3 ? 7.0f : 6.0f) * 1.0f;
    if (ideal < 0.001953125f) ideal = 0.001953125f;
    if (ideal > 448.0f) ideal = 448.0f;
    float sc;
    *scale_byte = e4m3_round(ideal, &sc);
    *scale_val = sc;
    float sq[MIXFP4_GROUP];
    for (int i = 0; i < MIXFP4_GROUP; ++i) {
        float n = s[i] / sc;
        float mag = fabsf(n);
        int idx = e0m3 ? e0m3_index(mag) : e2m1_index(mag);
        float level = e0m3 ? (float)idx : kE2M1Levels[idx];
        int neg = n < 0.0f;
        float code = neg ? -level : level;     /* sign(n) * level; -0.0 when level == 0 */
        nib[i] = (uint8_t)((neg << 3) | idx);
        float d = code * sc;
        d = d * global_scale;
        float e = d - x[i];
        sq[i] = e * e;
    }
    /* torch CPU sums a contiguous row of 16 floats as two 8-lane vectors added
     * lane-wise, then the 8 lanes left to right. */
    float acc = sq[0] + sq[8];
    for (int j = 1; j < 8; ++j) acc = acc + (sq[j] + sq[j + 8]);
    return acc;
}

/* scale.py:28-36 */
float mixfp4_oracle_global_scale(const float* x, int64_t rows, int64_t k, int64_t ldx) {
    float amax = 0.0f;
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t c = 0; c < k; ++c) { float a = fabsf(x[r * ldx + c]); if (a > amax) amax = a; }
    return amax > 0.0f ? amax / 2688.0f : 1.0f;
}

/* mode: 0 = oracle16 (per-block minimum error), 1 = all E2M1, 2 = all E0M3.
 * Optional outputs (may be NULL): per-block candidate errors and scales
 * [rows, G] with G = ceil(k/16); per-element candidate nibbles [rows, G*16].
 * global_scale_in: if > 0 it is used instead of this tensor's own amax (lets a
 * shard of a larger tensor be quantized with the whole tensor's scale). */
int mixfp4_oracle_quantize(const float* x, int64_t rows, int64_t k, int64_t ldx, int mode,
                           float global_scale_in,
                           uint8_t* codes, uint8_t* scales, uint8_t* fmt, float* global_scale_out,
                           float* e2_err, float* e0_err, float* e2_scale, float* e0_scale,
                           uint8_t* e2_nib, uint8_t* e0_nib) {
    if (rows <= 0 || k <= 0 || mode < 0 || mode > 2) return -1;
    const int64_t groups = (k + 15) / 16;
    const int64_t kpad = (k + 127) / 128 * 128;
    const int64_t ld_codes = kpad / 2, ld_scales = kpad / 16, ld_fmt = kpad / 128;
    const float gs = global_scale_in > 0.0f ? global_scale_in
                                            : mixfp4_oracle_global_scale(x, rows, k, ldx);
    if (global_scale_out) *global_scale_out = gs;
    memset(codes, 0, (size_t)(rows * ld_codes));
    memset(scales, 0x01, (size_t)(rows * ld_scales));
    memset(fmt, 0, (size_t)(rows * ld_fmt));
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        for (int64_t g = 0; g < groups; ++g) {
            float xb[MIXFP4_GROUP], sb[MIXFP4_GROUP];
            for (int i = 0; i < MIXFP4_GROUP; ++i) {
                int64_t c = g * 16 + i;
                xb[i] = c < k ? x[r * ldx + c] : 0.0f;
                sb[i] = xb[i] / gs;
            }
            uint8_t n2[MIXFP4_GROUP], n0[MIXFP4_GROUP], b2, b0;
            float s2, s0;
            float err2 = block_candidate(xb, sb, gs, 0, n2, &b2, &s2);
            float err0 = block_candidate(xb, sb, gs, 1, n0, &b0, &s0);
            int use_e0 = mode == 0 ? (err0 < err2) : (mode == 2);
            const uint8_t* nib = use_e0 ? n0 : n2;
            uint8_t* crow = codes + r * ld_codes + g * 8;
            for (int i = 0; i < 8; ++i) crow[i] = (uint8_t)(nib[2 * i] | (nib[2 * i + 1] << 4));
            scales[r * ld_scales + g] = use_e0 ? b0 : b2;
            if (use_e0) fmt[r * ld_fmt + (g >> 3)] |= (uint8_t)(1u << (g & 7));
            if (e2_err) e2_err[r * groups + g] = err2;
            if (e0_err) e0_err[r * groups + g] = err0;
            if (e2_scale) e2_scale[r * groups + g] = s2;
            if (e0_scale) e0_scale[r * groups + g] = s0;
            if (e2_nib) memcpy(e2_nib + (r * groups + g) * 16, n2, 16);
            if (e0_nib) memcpy(e0_nib + (r * groups + g) * 16, n0, 16);
        }
    }
    return 0;
}

/* Coarse format regions (project_quant/region.py:73-86 aggregate_regions,
 * selector.py:28-33 mse_selection): one format per region of region_rows x
 * region_groups K16 blocks, E0M3 iff the region's summed E0M3 error is smaller
 * (ties keep E2M1); every block keeps its own scale of the chosen format.
 * The fp32 sum of a region follows torch's CPU reduction of the padded
 * [R, region_rows, G, region_groups] view over dims (1, 3): inside a row the
 * region's blocks left to right, then the rows top to bottom; cells past the
 * tensor's edge count as zero.  (Checked against the reference for region_groups
 * in {2, 4} and more than one region along K.)
 * region_groups == 1 (n8k16, m16k16: a column of region_rows blocks): torch's
 * reduction of a non-contiguous dimension, as PyTorch 2.11 runs it on an AVX-512
 * host: block columns inside whole chunks of 32 columns are added top to bottom;
 * the columns left over after the last whole chunk go through four accumulators
 * (row i into accumulator i mod 4) that are then added 0 + 1 + 2 + 3.  (Checked
 * against the reference for 8 and 16 rows and 2 to 896 columns, 1 and 8 threads;
 * a single column takes yet another path and is refused.)
 * region_groups == 0 ("layer": one format for the whole tensor): the two sums are
 * taken in double precision; the reference's own fp32 sum of all blocks depends on
 * the host's thread count, the decision does not unless the sums agree to ~1e-7.
 * Inputs: the per-block candidate errors, nibbles and scales written by
 * mixfp4_oracle_quantize.  Outputs: the packed bytes. */
int mixfp4_oracle_apply_regions(const float* e2_err, const float* e0_err,
                                const uint8_t* e2_nib, const uint8_t* e0_nib,
                                const float* e2_scale, const float* e0_scale,
                                int64_t rows, int64_t k, int region_rows, int region_groups,
                                uint8_t* codes, uint8_t* scales, uint8_t* fmt) {
    if (rows <= 0 || k <= 0 || region_rows <= 0 || region_groups < 0) return -1;
    const int64_t groups = (k + 15) / 16;
    const int64_t kpad = (k + 127) / 128 * 128;
    const int64_t ld_codes = kpad / 2, ld_scales = kpad / 16, ld_fmt = kpad / 128;
    int layer_e0 = 0, is_layer = 0;
    if (region_groups == 0) {                       /* "layer" */
        is_layer = 1;
        double d2 = 0.0, d0 = 0.0;
        for (int64_t i = 0; i < rows * groups; ++i) { d2 += e2_err[i]; d0 += e0_err[i]; }
        layer_e0 = d0 < d2;
        region_rows = 1;
        region_groups = 1;
    } else if (region_groups == 1 && region_rows > 1 && groups < 2) {
        return -2;
    }
    const int64_t whole_chunks = region_groups == 1 ? groups / 32 * 32 : 0;
    memset(codes, 0, (size_t)(rows * ld_codes));
    memset(scales, 0x01, (size_t)(rows * ld_scales));
    memset(fmt, 0, (size_t)(rows * ld_fmt));
    for (int64_t r0 = 0; r0 < rows; r0 += region_rows) {
        for (int64_t g0 = 0; g0 < groups; g0 += region_groups) {
            float sum2 = 0.0f, sum0 = 0.0f;
            if (region_groups == 1 && region_rows > 1 && g0 >= whole_chunks) {
                float a2[4] = {0.0f, 0.0f, 0.0f, 0.0f}, a0[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                for (int64_t r = r0; r < r0 + region_rows && r < rows; ++r) {
                    a2[(r - r0) & 3] = a2[(r - r0) & 3] + e2_err[r * groups + g0];
                    a0[(r - r0) & 3] = a0[(r - r0) & 3] + e0_err[r * groups + g0];
                }
                sum2 = ((a2[0] + a2[1]) + a2[2]) + a2[3];
                sum0 = ((a0[0] + a0[1]) + a0[2]) + a0[3];
            } else {
                for (int64_t r = r0; r < r0 + region_rows; ++r) {
                    float t2 = 0.0f, t0 = 0.0f;
                    for (int64_t g = g0; g < g0 + region_groups; ++g) {
                        const int in = r < rows && g < groups;
                        t2 = t2 + (in ? e2_err[r * groups + g] : 0.0f);
                        t0 = t0 + (in ? e0_err[r * groups + g] : 0.0f);
                    }
                    sum2 = sum2 + t2;
                    sum0 = sum0 + t0;
                }
            }
            const int use_e0 = is_layer ? layer_e0 : sum0 < sum2;
            for (int64_t r = r0; r < r0 + region_rows && r < rows; ++r) {
                for (int64_t g = g0; g < g0 + region_groups && g < groups; ++g) {
                    const uint8_t* nib = (use_e0 ? e0_nib : e2_nib) + (r * groups + g) * 16;
                    uint8_t* crow = codes + r * ld_codes + g * 8;
                    for (int i = 0; i < 8; ++i) crow[i] = (uint8_t)(nib[2 * i] | (nib[2 * i + 1] << 4));
                    float back;
                    scales[r * ld_scales + g] = e4m3_round(use_e0 ? e0_scale[r * groups + g] : e2_scale[r * groups + g], &back);
                    if (use_e0) fmt[r * ld_fmt + (g >> 3)] |= (uint8_t)(1u << (g & 7));
                }
            }
        }
    }
    return 0;
}

/* Decode contract of the packed form: value = ((level * scale) * global) in
 * fp32, two multiplies left to right, sign from nibble bit 3 (scale.py:59);
 * out_kind 0 -> fp32, 1 -> bf16 (RNE, core.py:143), written un-padded [rows, k]. */
int mixfp4_oracle_dequant(const uint8_t* codes, const uint8_t* scales, const uint8_t* fmt,
                          float global_scale, int64_t rows, int64_t k, int out_kind, void* out) {
    if (rows <= 0 || k <= 0 || out_kind < 0 || out_kind > 1) return -1;
    const int64_t kpad = (k + 127) / 128 * 128;
    const int64_t ld_codes = kpad / 2, ld_scales = kpad / 16, ld_fmt = kpad / 128;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        for (int64_t c = 0; c < k; ++c) {
            int64_t g = c >> 4;
            uint8_t byte = codes[r * ld_codes + (c >> 1)];
            int nib = (c & 1) ? (byte >> 4) : (byte & 15);
            int e0 = (fmt[r * ld_fmt + (g >> 3)] >> (g & 7)) & 1;
            float level = e0 ? (float)(nib & 7) : kE2M1Levels[nib & 7];
            if (nib & 8) level = -level;
            float sc = e4m3_decode(scales[r * ld_scales + g]);
            float d = level * sc;
            d = d * global_scale;
            if (out_kind == 0) ((float*)out)[r * k + c] = d;
            else ((uint16_t*)out)[r * k + c] = f32_to_bf16(d);
        }
    }
    return 0;
}

/* rotation.py:47-75.  In place on x [rows, k] (row stride ldx): every full
 * block of `size` along k gets (optional +-1 signs, then) the natural-order
 * Walsh-Hadamard butterflies (stride 1, 2, 4, ...) and a division by
 * sqrt(size); a tail shorter than `size` is left untouched.
 * bf16_stages != 0 emulates the reference running on a bfloat16 tensor: every
 * stage's sums, the sign product and the final quotient are rounded to bf16. */
int mixfp4_oracle_fwht(float* x, int64_t rows, int64_t k, int64_t ldx, int size,
                       const float* signs, int bf16_stages) {
    if (size <= 0 || (size & (size - 1)) || size > 1024) return -1;
    const int64_t nblk = k / size;
    const float root = (float)sqrt((double)size);
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        float buf[1024];
        for (int64_t b = 0; b < nblk; ++b) {
            float* p = x + r * ldx + b * size;
            for (int i = 0; i < size; ++i) {
                float v = p[i];
                if (signs) { v = v * signs[i]; if (bf16_stages) v = round_to_bf16(v); }
                buf[i] = v;
            }
            for (int stride = 1; stride < size; stride <<= 1) {
                for (int base = 0; base < size; base += 2 * stride) {
                    for (int j = 0; j < stride; ++j) {
                        float l = buf[base + j], rr = buf[base + stride + j];
                        float s = l + rr, d = l - rr;
                        if (bf16_stages) { s = round_to_bf16(s); d = round_to_bf16(d); }
                        buf[base + j] = s;
                        buf[base + stride + j] = d;
                    }
                }
            }
            for (int i = 0; i < size; ++i) {
                float v = buf[i] / root;
                p[i] = bf16_stages ? round_to_bf16(v) : v;
            }
        }
    }
    return 0;
}

/* Linear oracle: y[m, n] = sum_k x[m, k] * w[n, k], accumulated in double and
 * returned as fp32 (the reference path is F.linear on the dequantized weight,
 * modeling.py:629; double accumulation removes summation-order noise). */
int mixfp4_oracle_linear(const float* x, const float* w, int64_t m, int64_t n, int64_t k, float* y) {
    if (m <= 0 || n <= 0 || k <= 0) return -1;
#pragma omp parallel for schedule(static)
    for (int64_t j = 0; j < n; ++j) {
        for (int64_t i = 0; i < m; ++i) {
            double acc = 0.0;
            const float* xr = x + i * k;
            const float* wr = w + j * k;
            for (int64_t c = 0; c < k; ++c) acc += (double)xr[c] * (double)wr[c];
            y[i * n + j] = (float)acc;
        }
    }
    return 0;
}

/* codebook.py:12-25 quantize_e2m1 / :41-43 quantize_e0m3 element by element: sign(x) * level(|x|),
 * where sign(+-0) = 0 makes the result +0 and a negative x that rounds to zero gives -0. */
int mixfp4_oracle_round_codebook(const float* x, float* y, int64_t n, int e0m3) {
    if (!x || !y || n < 0) return -1;
    for (int64_t i = 0; i < n; ++i) {
        const float v = x[i], mag = fabsf(v);
        const float q = e0m3 ? (float)e0m3_index(mag) : kE2M1Levels[e2m1_index(mag)];
        const float sign = v > 0.0f ? 1.0f : (v < 0.0f ? -1.0f : 0.0f);
        y[i] = sign * q;
    }
    return 0;
}

/* scale.py:64-103 _four_over_six_scale_candidate for the E0M3 codebook (qmax 7), one expansion
 * factor: every operation in the reference's order (the encode scale 1536 / amax, the reciprocal
 * of decode_scale * scale, the left-to-right dequantization).  No clamp before the E4M3 cast:
 * tiny ideals round to a zero scale, which zeroes the block. */
static float e0_four_over_six_block(const float* x, float amax, float expansion, float* codes, float* dequant,
                                    float* scale_out) {
    const float denominator = 1536.0f;
    float bmax = 0.0f;
    for (int i = 0; i < MIXFP4_GROUP; ++i) { float a = fabsf(x[i]); if (a > bmax) bmax = a; }
    float ideal = 0.0f;
    if (amax != 0.0f) {
        const float encode_scale = denominator / amax;
        ideal = bmax / 7.0f * encode_scale;
    }
    ideal = ideal * expansion;
    float scale = 0.0f;
    if (ideal > 0.0f) (void)e4m3_round(ideal, &scale);
    const float decode_scale = amax > 0.0f ? 1.0f / (denominator / amax) : 0.0f;
    float sq[MIXFP4_GROUP];
    for (int i = 0; i < MIXFP4_GROUP; ++i) {
        float n = 0.0f;
        if (scale != 0.0f) n = x[i] * (1.0f / (decode_scale * scale));
        const float level = (float)e0m3_index(fabsf(n));
        const float sign = n > 0.0f ? 1.0f : (n < 0.0f ? -1.0f : 0.0f);
        const float code = sign * level;
        codes[i] = code;
        float d = code * scale;
        d = d * amax;
        d = d / denominator;
        dequant[i] = d;
        const float e = d - x[i];
        sq[i] = e * e;
    }
    float acc = sq[0] + sq[8];
    for (int j = 1; j < 8; ++j) acc = acc + (sq[j] + sq[j + 8]);
    *scale_out = scale;
    return acc;
}

/* scale.py:207-225: the base (x1.0) and the expanded (x1.5) E0M3 candidate of every block, the
 * expanded one kept where its error is strictly smaller.  x: nblocks * 16 floats (the padded,
 * grouped tensor); amax is taken over all of it. */
int mixfp4_oracle_e0_four_over_six(const float* x, int64_t nblocks, float* codes, float* dequant, float* scales,
                                   float* errors, uint8_t* expanded) {
    if (!x || !codes || !dequant || !scales || !errors || !expanded || nblocks < 0) return -1;
    float amax = 0.0f;
    for (int64_t i = 0; i < nblocks * MIXFP4_GROUP; ++i) { float a = fabsf(x[i]); if (a > amax) amax = a; }
    for (int64_t b = 0; b < nblocks; ++b) {
        float c0[MIXFP4_GROUP], d0[MIXFP4_GROUP], c1[MIXFP4_GROUP], d1[MIXFP4_GROUP], s0, s1;
        const float e0 = e0_four_over_six_block(x + b * MIXFP4_GROUP, amax, 1.0f, c0, d0, &s0);
        const float e1 = e0_four_over_six_block(x + b * MIXFP4_GROUP, amax, 1.5f, c1, d1, &s1);
        const int pick = e1 < e0;
        memcpy(codes + b * MIXFP4_GROUP, pick ? c1 : c0, sizeof(c0));
        memcpy(dequant + b * MIXFP4_GROUP, pick ? d1 : d0, sizeof(d0));
        scales[b] = pick ? s1 : s0;
        errors[b] = pick ? e1 : e0;
        expanded[b] = (uint8_t)pick;
    }
    return 0;
}

int mixfp4_oracle_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
