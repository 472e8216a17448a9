// NVFP4 quantiser for a GEMM epilogue, as reusable device functions.
//
// What the reference's gated-GEMM epilogue does on its accumulator fragments (aiis-clef kernels/gemm.cu:882-967):
// v = silu(accg * gscale_g) * (accu * gscale_u) per element (the SwiGLU of kernels/elementwise.cu:225-241 with
// the IEEE quotient), then per 16-column block the activation quantiser of kernels/quantise.cu:22-52
// (amax, E4M3 scale byte with the global scale, E2M1 codes) and the scale byte's address in the tiled
// activation-side layout. The bytes equal clef_swiglu_quantise_nvfp4 on the matrices
// accg * gscale_g and accu * gscale_u (the tests compare them, and both with the reference's header).
//
// Two accumulator layouts are served:
//   block16  one thread holds the 16 values of a block: the layout tcgen05.ld 32x32b gives (lane = row,
//            consecutive columns per lane), which is how a tcgen05 GEMM's epilogue warps read TMEM;
//   quad4    the mma.sync m16n8 fragment of gemm.cu: lanes l, l^1, l^2, l^3 of a 4-lane group hold a row's
//            block, lane (l & 3) the columns 8 s + 2 (l & 3) + {0, 1} of its two 8-column slabs s.
// Nothing here touches memory except through the addresses the caller forms with nvfp4_scale_offset().
#pragma once

#include "common.cuh"
#include "nvfp4_codec.cuh"
#include "silu_forms.cuh"

namespace clef {

// Values of the C-ABI's CLEF_SF_* constants (include/clef_fused.h), for device code that does not include that header.
enum Nvfp4ScaleTileOrder { kSfActivation = 0, kSfInterleaved = 1 };

// Byte offset of the scale of (row, block) in the tiled scale buffer of a [rows, 16 * blocks_per_row] operand.
__device__ __forceinline__ size_t nvfp4_scale_offset(int row, int block, int blocks_per_row, int blk_mn, int tile_order) {
    return scale_offset(row, block, blocks_per_row, blk_mn, tile_order == kSfInterleaved ? -4 * blk_mn : 4 * blk_mn);
}

// One activation value of the gated epilogue: (gg / (1 + __expf(-gg))) * gu, gg = accg * gscale_g, gu = accu * gscale_u
// (gemm.cu:909-921). The quotient takes the short exact form for |gg| <= 44 and the literal one beyond.
__device__ __forceinline__ float swiglu_epilogue_value(float accg, float accu, float gscale_g, float gscale_u) {
    const float gg = __fmul_rn(accg, gscale_g), gu = __fmul_rn(accu, gscale_u);
    const float s = fabsf(gg) <= kSiluFastMaxAbs ? silu_ieee_refined_f32(gg) : silu_ieee_div(gg);
    return __fmul_rn(s, gu);
}

// E4M3 scale byte of a scale argument, any input (kernels/nvfp4_quant.h:35-57): e4m3_encode_finite plus the
// reference's answer for +infinity (CUDA's frexpf(+inf) returns +inf with exponent 0: code (6 << 3) | 7).
__device__ __forceinline__ uint32_t e4m3_encode_scale(float sv) {
    return sv == __int_as_float(0x7F800000) ? ((6u << 3) | 7u) : e4m3_encode_finite(sv);
}

// Two scaled values -> one byte (first value in the low nibble), any input.
__device__ __forceinline__ uint32_t e2m1_pair_any(float first, float second) {
    const bool fast = fabsf(first) < kE2m1FastLimit && fabsf(second) < kE2m1FastLimit;   // false for a NaN
    return fast ? e2m1x2_fast(first, second) : (e2m1_exact(first) | (e2m1_exact(second) << 4));
}

struct Nvfp4Block {
    uint32_t stored;   // E4M3 scale byte
    uint32_t lo, hi;   // packed codes of values 0-7 and 8-15 (value 0 in the lowest nibble): 8 bytes at packed[row][8 * block]
};

// ---- block16: the thread holds the block ------------------------------------------------------------------------
// `inv_table` is the per-CTA table of fill_inv_scale_table(out_global) in shared memory, or nullptr to divide in place.
// `row_live` false (a padding row of the M tile): scale byte 0 and zero codes, as the reference stores for them.
__device__ __forceinline__ Nvfp4Block nvfp4_quantise_block16(const float* v, float out_global, const float* inv_table, bool row_live = true) {
    Nvfp4Block b{0u, 0u, 0u};
    if (row_live) {
        quantise16(v, out_global, inv_table, b.stored, b.lo, b.hi);
    }
    return b;
}

__device__ __forceinline__ Nvfp4Block nvfp4_swiglu_epilogue_block16(const float* accg, const float* accu, float gscale_g, float gscale_u,
                                                                   float out_global, const float* inv_table, bool row_live = true) {
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        v[i] = swiglu_epilogue_value(accg[i], accu[i], gscale_g, gscale_u);
    }
    return nvfp4_quantise_block16(v, out_global, inv_table, row_live);
}

// ---- quad4: four lanes hold the block -----------------------------------------------------------------------------
struct Nvfp4Quad {
    uint32_t stored;    // E4M3 scale byte of the block (the same in the four lanes; lane (l & 3) == 0 stores it)
    uint32_t byte[2];   // this lane's codes: byte s belongs at packed[row][8 * block + 4 * s + (l & 3)]
};

// v[2 s + e] = the value at column 8 s + 2 (l & 3) + e of the block. Every lane of the warp must call (two shuffles).
__device__ __forceinline__ Nvfp4Quad nvfp4_quantise_quad4(const float (&v)[4], float out_global, bool row_live) {
    float m0 = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    m0 = fmaxf(m0, __shfl_xor_sync(kFullMask, m0, 1));
    m0 = fmaxf(m0, __shfl_xor_sync(kFullMask, m0, 2));
    Nvfp4Quad out{0u, {0u, 0u}};
    if (row_live) {
        out.stored = e4m3_encode_scale(__fmul_rn(__fdiv_rn(m0, 6.0f), out_global));
        const float inv = inv_scale_of(out.stored, out_global);
        out.byte[0] = e2m1_pair_any(__fmul_rn(v[0], inv), __fmul_rn(v[1], inv));
        out.byte[1] = e2m1_pair_any(__fmul_rn(v[2], inv), __fmul_rn(v[3], inv));
    }
    return out;
}

__device__ __forceinline__ Nvfp4Quad nvfp4_swiglu_epilogue_quad4(const float (&accg)[4], const float (&accu)[4], float gscale_g,
                                                                float gscale_u, float out_global, bool row_live) {
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[i] = swiglu_epilogue_value(accg[i], accu[i], gscale_g, gscale_u);
    }
    return nvfp4_quantise_quad4(v, out_global, row_live);
}

}  // namespace clef
