// NVFP4 activation codec for sm_100a: E2M1 codes, E4M3 block scales, tiled scale addressing.
//
// Semantics follow aiis-clef's kernels/nvfp4_quant.h (to_e2m1 :13-33, to_e4m3 :35-57,
// from_e4m3 :59-66) and the per-block recipe of kernels/quantise.cu:22-52, bit for bit, but none
// of the code is taken from there: the encoders below are integer/bit formulations and the E2M1
// path uses Blackwell's packed FP4 converter with a pre-rounding nudge (see e2m1x2_fast).
//
//   amax      = max |v_i| over 16 values (NaN operands ignored)
//   stored    = e4m3_encode((amax / 6) * global_scale)            one byte per block
//   inv_scale = stored > 0 ? global_scale / e4m3_decode(stored) : 0
//   code_i    = e2m1(v_i * inv_scale), byte p of the block = code[2p] | code[2p+1] << 4
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

#include "f32x2.cuh"

namespace clef {

// --------------------------------------------------------------------------------------------
// E4M3 (unsigned, scales only).
// --------------------------------------------------------------------------------------------

// Encode a scale. Reference behaviour (kernels/nvfp4_quant.h:35-57): non-positive and NaN -> 0;
// mantissa rounded half UP to 3 bits; clamp to 0x7E; below 2^-6 the code is
// min(int(v*512 + 0.5f), 7) where the addition rounds in f32. Only finite v may be passed
// (callers route +inf to the literal path, whose answer depends on frexpf's treatment of inf).
//
// Bit form: adding half of the kept mantissa step (1 << 19) to the f32 pattern rounds the
// 3-bit mantissa half up and carries into the exponent by itself; the biased-exponent/mantissa
// field shifted down by 20 and rebased by 120 << 3 is then the E4M3 code.
__device__ __forceinline__ uint32_t e4m3_encode_finite(float v) {
    const uint32_t r = __float_as_uint(v) + 0x00080000u;
    const int code = (int)(r >> 20) - (120 << 3);
    const int sub = min(__float2int_rz(__fmaf_rn(v, 512.0f, 0.5f)), 7);   // v*512 is exact
    const int normal = min(code, 0x7E);
    const int out = (code >= 8) ? normal : sub;
    return (v > 0.0f) ? (uint32_t)out : 0u;
}

// Decode a stored scale byte (kernels/nvfp4_quant.h:59-66): exact in f32.
__device__ __forceinline__ float e4m3_decode(uint32_t b) {
    const uint32_t e = (b >> 3) & 0xFu;
    const float subnormal = (float)(b & 7u) * (1.0f / 512.0f);
    const float normal = __uint_as_float(((b & 0x7Fu) << 20) + 0x3C000000u);
    return e ? normal : subnormal;
}

// inv_scale for a stored byte (kernels/quantise.cu:44-45).
__device__ __forceinline__ float inv_scale_of(uint32_t stored, float global_scale) {
    const float stored_f = e4m3_decode(stored);
    return (stored_f > 0.0f) ? __fdiv_rn(global_scale, stored_f) : 0.0f;
}

// Number of distinct stored scale bytes (0 ..= 0x7E) rounded up; size of the per-CTA inv_scale table.
constexpr int kInvScaleTableSize = 128;

// Fill a shared table t[b] = inv_scale_of(b). Call with all threads of the CTA, then __syncthreads().
__device__ __forceinline__ void fill_inv_scale_table(float* table, float global_scale) {
    for (int b = threadIdx.x; b < kInvScaleTableSize; b += blockDim.x) {
        table[b] = inv_scale_of((uint32_t)b, global_scale);
    }
}

// --------------------------------------------------------------------------------------------
// E2M1.
// --------------------------------------------------------------------------------------------

// Literal semantics of the reference encoder for ONE value (kernels/nvfp4_quant.h:13-33 in its
// default build): the table entry with the smallest |a - entry|, the FIRST such entry when several
// tie (so exact ties go to the smaller magnitude), where the differences are rounded f32 values and
// only differences below 1e30 count. Consequences the fast path must respect: for |v| >= 2^25 the
// rounded differences to 4 and 6 can coincide, so the answer is no longer simply "7", and from 1e30
// up, for infinities and for NaN, the magnitude is 0. The sign nibble is (v < 0): -0.0 and NaN carry
// none. Used on the rare path and by the device-side comparison with the reference header.
__device__ __forceinline__ uint32_t e2m1_exact(float v) {
    const float grid[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    const float a = fabsf(v);
    uint32_t mag = 0;
    float least = 1e30f;
#pragma unroll
    for (uint32_t i = 0; i < 8; ++i) {
        const float d = fabsf(__fsub_rn(a, grid[i]));
        const bool better = d < least;
        least = better ? d : least;
        mag = better ? i : mag;
    }
    return mag | ((v < 0.0f) ? 8u : 0u);
}

// Largest magnitude (exclusive) the fast converter path is used for: below 2^24 every difference
// |a - entry| above is exact or ordered strictly, so "nearest, ties down, saturate at 6" is the
// reference's answer.
constexpr float kE2m1FastLimit = 16777216.0f;

// Two values -> one byte (first value in the low nibble) with the hardware converter
// cvt.rn.satfinite.e2m1x2.f32. The converter rounds ties to even; the reference rounds ties
// toward zero. They differ exactly at |p| = 0.75, 1.75, 3.5 (ties whose even neighbour is the
// larger one). Pre-multiplying by (1 - c), c = 2^-24 / 1.375, moves p down by one ulp precisely
// when its mantissa is above 1.375 (c*p is then between 0.5 and 0.73 ulp) and leaves it alone
// when the mantissa is in (1, 1.375): the three "odd" ties (mantissa 1.5 or 1.75) drop just
// below the tie and round down, the four "even" ties (mantissa 1 or 1.25) and their upper
// neighbours are untouched, so the converter's result equals the reference's for every
// |p| < 2^24. The same FMA turns -0.0 into +0.0 (the reference gives -0.0 no sign nibble).
// NaN, infinities and |p| >= 2^24 must not reach this function (see quantise16).
__device__ __forceinline__ uint32_t e2m1x2_fast(float first, float second) {
    constexpr float kNudge = -4.33488326e-08f;   // -(2^-24 / 1.375)
    const float a = __fmaf_rn(first, kNudge, first);
    const float b = __fmaf_rn(second, kNudge, second);
    uint32_t r;
    asm("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tcvt.u32.u8 %0, t;\n\t}"
        : "=r"(r)
        : "f"(b), "f"(a));   // first source operand lands in the high nibble
    return r;
}

// 8 scaled values -> 32 packed bits (value 0 in the lowest nibble).
__device__ __forceinline__ uint32_t e2m1x8_fast(const float* p) {
    const uint32_t b0 = e2m1x2_fast(p[0], p[1]);
    const uint32_t b1 = e2m1x2_fast(p[2], p[3]);
    const uint32_t b2 = e2m1x2_fast(p[4], p[5]);
    const uint32_t b3 = e2m1x2_fast(p[6], p[7]);
    return b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
}

__device__ __forceinline__ uint32_t e2m1x8_exact(const float* p) {
    uint32_t w = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        w |= e2m1_exact(p[i]) << (4 * i);
    }
    return w;
}

// NaN-propagating max of magnitudes (max.NaN.f32): equals fmaxf when no operand is NaN, and is
// NaN as soon as one is, which is how the fast path notices values it must not handle.
__device__ __forceinline__ float amax_nan(float acc, float v) {
    float r;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(acc), "f"(fabsf(v)));
    return r;
}

// Literal path for one block of 16: the reference recipe with NaN-ignoring fmaxf, the literal
// E2M1 rule and a literal walk of the E4M3 encoder for a non-finite scale argument.
static __device__ __noinline__ void quantise16_rare(const float* v, float global_scale, uint32_t& stored_out,
                                             uint32_t& lo_out, uint32_t& hi_out) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        amax = fmaxf(amax, fabsf(v[i]));
    }
    const float sv = __fmul_rn(__fdiv_rn(amax, 6.0f), global_scale);
    uint32_t stored;
    if (sv == __int_as_float(0x7F800000)) {
        // kernels/nvfp4_quant.h:40-56 with v = +inf: CUDA's frexpf(+inf) returns +inf with
        // exponent 0, the mantissa term converts to INT_MAX, and the code is (6 << 3) | 7.
        stored = (6u << 3) | 7u;
    } else {
        stored = e4m3_encode_finite(sv);
    }
    const float inv = inv_scale_of(stored, global_scale);
    float p[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        p[i] = __fmul_rn(v[i], inv);
    }
    stored_out = stored;
    lo_out = e2m1x8_exact(p);
    hi_out = e2m1x8_exact(p + 8);
}

// One block of 16 f32 values held by one thread -> scale byte + 64 packed bits.
// `inv_table` is the shared table of fill_inv_scale_table (or nullptr to divide in place).
__device__ __forceinline__ void quantise16(const float* v, float global_scale, const float* inv_table,
                                           uint32_t& stored_out, uint32_t& lo_out, uint32_t& hi_out) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        amax = amax_nan(amax, v[i]);
    }
    const float sv = __fmul_rn(__fdiv_rn(amax, 6.0f), global_scale);
    const uint32_t stored = e4m3_encode_finite(sv);
    const float inv = inv_table ? inv_table[stored] : inv_scale_of(stored, global_scale);
    const float pmax = __fmul_rn(amax, inv);
    if (!(fabsf(sv) <= 3.0e38f) || !(pmax < kE2m1FastLimit)) {
        quantise16_rare(v, global_scale, stored_out, lo_out, hi_out);
        return;
    }
    float p[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        p[i] = __fmul_rn(v[i], inv);
    }
    stored_out = stored;
    lo_out = e2m1x8_fast(p);
    hi_out = e2m1x8_fast(p + 8);
}

// Range of global_scale the tuned kernels' block quantiser is built for (quantise16_qp in kernels_hot.cuh);
// launchers send any other scale (zero, negative, NaN, or beyond these) to the shape-general kernels.
constexpr float kHotGlobalScaleMin = 5.42101086e-20f;   // 2^-64
constexpr float kHotGlobalScaleMax = 1.84467441e+19f;   // 2^64

// amax / 6 without the IEEE-division sequence: q0 = x * RN(1/6), one exact-remainder correction.
// Checked against div.rn.f32 for every non-negative finite f32: equal for x = 0 and for every
// x >= 2^-100; smaller non-zero x go to the literal path.
constexpr float kDivSixExactFrom = 7.888609052e-31f;   // 2^-100
__device__ __forceinline__ float div_six_fast(float x) {
    constexpr float kSixth = 0.16666667163372040f;
    const float q0 = __fmul_rn(x, kSixth);
    const float rem = __fmaf_rn(-6.0f, q0, x);
    return __fmaf_rn(rem, kSixth, q0);
}

// Same block quantiser on 8 packed pairs (f32x2.cuh): 3-input NaN-propagating max, the short
// division by six, packed multiply and nudge. Falls back to quantise16_rare exactly when the
// scalar version would, and additionally for 0 < amax < 2^-100.
__device__ __forceinline__ void quantise16_x2(const f32x2* v, float global_scale, const float* inv_table,
                                              uint32_t& stored_out, uint32_t& lo_out, uint32_t& hi_out) {
    float a[16];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        f2_unpack(v[i], a[2 * i], a[2 * i + 1]);
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        amax = max3_abs_nan(amax, a[2 * i], a[2 * i + 1]);
    }
    const float sv = __fmul_rn(div_six_fast(amax), global_scale);
    const uint32_t stored = e4m3_encode_finite(sv);
    const float inv = inv_table[stored];
    const float pmax = __fmul_rn(amax, inv);
    const bool tiny = (amax < kDivSixExactFrom) && (amax > 0.0f);
    if (!(fabsf(sv) <= 3.0e38f) || !(pmax < kE2m1FastLimit) || tiny) {
        quantise16_rare(a, global_scale, stored_out, lo_out, hi_out);
        return;
    }
    constexpr float kNudge = -4.33488326e-08f;   // see e2m1x2_fast
    const f32x2 inv2 = f2_splat(inv);
    const f32x2 nudge2 = f2_splat(kNudge);
    uint32_t bytes[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const f32x2 p = f2_mul(v[i], inv2);
        const f32x2 q = f2_fma(p, nudge2, p);
        float first, second;
        f2_unpack(q, first, second);
        asm("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tcvt.u32.u8 %0, t;\n\t}"
            : "=r"(bytes[i])
            : "f"(second), "f"(first));
    }
    stored_out = stored;
    lo_out = bytes[0] | (bytes[1] << 8) | (bytes[2] << 16) | (bytes[3] << 24);
    hi_out = bytes[4] | (bytes[5] << 8) | (bytes[6] << 16) | (bytes[7] << 24);
}

// --------------------------------------------------------------------------------------------
// Scale addressing (activation side, kernels/quantise.cu:34-41): tiles of [blk_mn rows x 4
// blocks] = `chunk` bytes, ordered (row tile, group of 4 blocks). Inside a tile the reference's
// activation side stores row r at byte 4 r ("conflict-free", src/swizzle.rs:64-65); the standard
// block-scaled layout of a tcgen05 GEMM stores it at 4 ((r % 32) * (blk_mn / 32) + r / 32)
// (src/swizzle.rs:66-68, the weight side's order). Kernels receive the choice folded into their
// `chunk` argument: a NEGATED chunk selects the interleaved order (chunk is always 4 * blk_mn, so
// the sign is free); sf_layout_of undoes the folding.
// --------------------------------------------------------------------------------------------
struct SfLayout {
    int chunk;   // bytes per tile
    int sub;     // blk_mn / 32 for the interleaved order, 0 for the reference's activation-side order
};
__device__ __forceinline__ SfLayout sf_layout_of(int blk_mn, int chunk_arg) {
    return chunk_arg < 0 ? SfLayout{-chunk_arg, blk_mn >> 5} : SfLayout{chunk_arg, 0};
}
__device__ __forceinline__ uint32_t sf_row_slot(uint32_t row_in_tile, const SfLayout& sf) {
    return sf.sub ? (row_in_tile & 31u) * (uint32_t)sf.sub + (row_in_tile >> 5) : row_in_tile;
}

__device__ __forceinline__ size_t scale_offset(int row, int block, int blocks_per_row, int blk_mn, int chunk_arg) {
    const SfLayout sf = sf_layout_of(blk_mn, chunk_arg);
    const int k1_count = blocks_per_row >> 2;
    const int m_rest = row / blk_mn;
    const uint32_t m_atom = sf_row_slot((uint32_t)(row - m_rest * blk_mn), sf);
    return ((size_t)m_rest * k1_count + (size_t)(block >> 2)) * (size_t)sf.chunk + (size_t)m_atom * 4 + (size_t)(block & 3);
}

}  // namespace clef
