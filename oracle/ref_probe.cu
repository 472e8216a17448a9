// ref_probe.cu -- TEST INFRASTRUCTURE, not product code.
//
// Device-side comparison of this repo's NVFP4 codec (aiis_clef_b200/csrc/nvfp4_codec.cuh) with the
// reference's own encoder header, which is included from the reference tree where it lies
// (-I<reference>/kernels, see Makefile): to_e2m1, to_e4m3, from_e4m3 of kernels/nvfp4_quant.h.
// Built only into oracle/_ref/ref_probe.cubin and launched only by the GPU tests.
//
// Every kernel walks f32 bit patterns, evaluates both sides and counts disagreements; up to 16
// disagreeing patterns are kept for the test's failure message.
#include <cstdint>
#include <cuda_runtime.h>

#include "nvfp4_quant.h"    // the reference's header (to_e2m1 / to_e4m3 / from_e4m3)
#include "nvfp4_codec.cuh"  // this repo's codec (namespace clef)
#include "kernels_generic.cuh"
#include "kernels_hot.cuh"   // packed-pair quantiser and the short silu forms of the tuned kernels
#include "kernels_fp8.cuh"   // e4m3_encode_any, the FP8 quantisers' element encoder
#include "nvfp4_epilogue.cuh"   // the GEMM-epilogue quantiser as device functions

struct ProbeResult {
    unsigned long long checked;
    unsigned long long mismatches;
    uint32_t first_bad[16];
};

__device__ void report(ProbeResult* r, uint32_t pattern) {
    const unsigned long long slot = atomicAdd(&r->mismatches, 1ull);
    if (slot < 16) {
        r->first_bad[slot] = pattern;
    }
}

__device__ __forceinline__ uint32_t mix(uint32_t x) {
    x ^= x >> 16;
    x *= 0x7feb352du;
    x ^= x >> 15;
    x *= 0x846ca68bu;
    x ^= x >> 16;
    return x;
}

// All 2^32 patterns starting at `base` for `count` patterns (count may be 2^32 = 0 wrapped: pass as u64).
// result[0]: fast pair converter, low nibble, on its domain (|p| < 2^24)
// result[1]: fast pair converter, high nibble, same domain
// result[2]: literal single-value encoder e2m1_exact on every pattern
extern "C" __global__ void probe_e2m1(unsigned long long base, unsigned long long count, ProbeResult* result) {
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    unsigned long long checked_fast = 0, checked_all = 0;
    for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        const uint32_t bits = (uint32_t)(base + i);
        const float p = __uint_as_float(bits);
        const uint32_t want = to_e2m1(p);
        ++checked_all;
        if (clef::e2m1_exact(p) != want) {
            report(&result[2], bits);
        }
        const float a = fabsf(p);
        if (a < clef::kE2m1FastLimit) {   // false for NaN
            ++checked_fast;
            // A partner value that is always inside the fast path's domain (|q| < 2).
            const uint32_t qbits = mix(bits) & 0xBFFFFFFFu;
            const float q = __uint_as_float(qbits);
            const uint32_t want_q = to_e2m1(q);
            const uint32_t lo_first = clef::e2m1x2_fast(p, q);
            const uint32_t hi_first = clef::e2m1x2_fast(q, p);
            if (lo_first != (want | (want_q << 4))) {
                report(&result[0], bits);
            }
            if (hi_first != (want_q | (want << 4))) {
                report(&result[1], bits);
            }
        }
    }
    atomicAdd(&result[0].checked, checked_fast);
    atomicAdd(&result[1].checked, checked_fast);
    atomicAdd(&result[2].checked, checked_all);
}

// result[0] (and result[1], see below): scale encoder on every pattern. +inf goes through the literal branch of the rare path
// (clef::quantise16_rare handles it the same way), everything else through e4m3_encode_finite.
extern "C" __global__ void probe_e4m3(unsigned long long base, unsigned long long count, ProbeResult* result) {
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    unsigned long long checked = 0, checked_fast = 0, checked_hw = 0;
    for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        const uint32_t bits = (uint32_t)(base + i);
        const float v = __uint_as_float(bits);
        const uint32_t want = to_e4m3(v);
        const uint32_t got = (bits == 0x7F800000u) ? ((6u << 3) | 7u) : clef::e4m3_encode_finite(v);
        ++checked;
        if (got != want) {
            report(&result[0], bits);
        }
        if (clef::e4m3_encode_any(v) != want) {   // the FP8 quantisers' element encoder, every pattern
            report(&result[1], bits);
        }
        if (bits < 0x43E80000u) {                 // the tuned FP8 kernels' short encoder on its domain, +0 <= v < 464
            ++checked_fast;
            if (clef::e4m3_mag_fast(v) != want) {
                report(&result[2], bits);
            }
        }
        if (bits < 0x43E80000u) {   // the hardware-converter form on +0 <= v < 464: v in every byte position, both signs,
            ++checked_hw;           // beside a partner of the domain; a byte is either flagged (0 or 8 in its low seven
                                    // bits) or the reference's, and the word test fires exactly when a byte is flagged
            const float q = __uint_as_float(mix(bits) % 0x43E80000u);
            const uint32_t want_q = to_e4m3(q);
            const uint32_t got_w[2] = {clef::e4m3x4_hw(v, -q, q, -v), clef::e4m3x4_hw(-q, v, -v, q)};
            const uint32_t neg_v = want | (bits ? 0x80u : 0u), neg_q = want_q | (q > 0.0f ? 0x80u : 0u);   // (t < 0) is false for -0.0
            const uint32_t want_w[2] = {want | (neg_q << 8) | (want_q << 16) | (neg_v << 24),
                                        neg_q | (want << 8) | (neg_v << 16) | (want_q << 24)};
            bool bad = false;
            for (int k = 0; k < 2; ++k) {
                bool flagged = false;
                for (int byte = 0; byte < 4; ++byte) {
                    const uint32_t g = (got_w[k] >> (8 * byte)) & 0xFFu, w = (want_w[k] >> (8 * byte)) & 0xFFu;
                    if ((g & 0x77u) == 0u) {
                        flagged = true;
                    } else if (g != w) {
                        bad = true;
                    }
                }
                if ((clef::e4m3x4_suspect(got_w[k]) != 0u) != flagged) bad = true;
                // what the kernels do with a flagged word
                if (flagged && clef::fp8_encode4_int(k == 0 ? v : -q, k == 0 ? -q : v, k == 0 ? q : -v, k == 0 ? -v : q, 1.0f) != want_w[k]) {
                    bad = true;
                }
            }
            if (bad) report(&result[3], bits);
        }
    }
    atomicAdd(&result[0].checked, checked);
    atomicAdd(&result[1].checked, checked);
    atomicAdd(&result[2].checked, checked_fast);
    atomicAdd(&result[3].checked, checked_hw);
}

// result[0]: decoder on all 256 bytes (bit-exact f32); result[1]: inv_scale for `global_scale`.
extern "C" __global__ void probe_e4m3_decode(float global_scale, ProbeResult* result) {
    const uint32_t b = threadIdx.x;
    if (b < 256) {
        const float want = from_e4m3((uint8_t)b);
        const float got = clef::e4m3_decode(b);
        atomicAdd(&result[0].checked, 1ull);
        if (__float_as_uint(want) != __float_as_uint(got)) {
            report(&result[0], b);
        }
        const float want_inv = (want > 0.0f) ? global_scale / want : 0.0f;
        atomicAdd(&result[1].checked, 1ull);
        if (__float_as_uint(want_inv) != __float_as_uint(clef::inv_scale_of(b, global_scale))) {
            report(&result[1], b);
        }
    }
}

// Whole 16-value blocks: the reference recipe of kernels/quantise.cu:22-52 spelled with the
// reference's encoder functions, against clef::quantise16. `values` holds n_blocks * 16 floats.
// result[0]: scale byte, result[1]: packed codes (counted per block). first_bad holds block indices.
extern "C" __global__ void probe_blocks(const float* values, unsigned long long n_blocks, float global_scale,
                                        uint8_t* want_scale, uint8_t* want_packed, uint8_t* got_scale,
                                        uint8_t* got_packed, ProbeResult* result, int use_pairs) {
    __shared__ float inv_table[clef::kInvScaleTableSize];
    clef::fill_inv_scale_table(inv_table, global_scale);
    __syncthreads();
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    for (unsigned long long b = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; b < n_blocks; b += stride) {
        const float* src = values + b * 16;
        float amax = 0.0f;
        for (int i = 0; i < 16; ++i) {
            amax = fmaxf(amax, fabsf(src[i]));
        }
        const float block_scale = amax / 6.0f;
        const uint8_t stored = to_e4m3(block_scale * global_scale);
        const float stored_f = from_e4m3(stored);
        const float inv_scale = (stored_f > 0.0f) ? global_scale / stored_f : 0.0f;
        uint8_t want[8];
        for (int pair = 0; pair < 8; ++pair) {
            const uint8_t lo = to_e2m1(src[pair * 2] * inv_scale);
            const uint8_t hi = to_e2m1(src[pair * 2 + 1] * inv_scale);
            want[pair] = (uint8_t)(lo | (hi << 4));
        }
        float v[16];
        for (int i = 0; i < 16; ++i) {
            v[i] = src[i];
        }
        uint32_t got_stored, lo, hi;
        if (use_pairs) {
            // the tuned kernels' path: quad-pair layout, fast quantiser, literal routine when it declines
            clef::f32x2 qp[8];
            for (int q = 0; q < 4; ++q) {
                qp[2 * q] = clef::f2_pack(v[4 * q], v[4 * q + 2]);
                qp[2 * q + 1] = clef::f2_pack(v[4 * q + 1], v[4 * q + 3]);
            }
            if (!clef::quantise16_qp<false>(qp, global_scale, inv_table, got_stored, lo, hi)) {
                clef::quantise16_rare(v, global_scale, got_stored, lo, hi);
            }
        } else {
            clef::quantise16(v, global_scale, nullptr, got_stored, lo, hi);
        }
        const unsigned long long got_bits = (unsigned long long)lo | ((unsigned long long)hi << 32);
        unsigned long long want_bits = 0;
        for (int pair = 0; pair < 8; ++pair) {
            want_bits |= (unsigned long long)want[pair] << (8 * pair);
            want_packed[b * 8 + pair] = want[pair];
            got_packed[b * 8 + pair] = (uint8_t)(got_bits >> (8 * pair));
        }
        want_scale[b] = stored;
        got_scale[b] = (uint8_t)got_stored;
        atomicAdd(&result[0].checked, 1ull);
        atomicAdd(&result[1].checked, 1ull);
        if (got_stored != stored) {
            report(&result[0], (uint32_t)b);
        }
        if (got_bits != want_bits) {
            report(&result[1], (uint32_t)b);
        }
    }
}

// The short silu forms of the tuned kernels against the reference expressions, for every bf16 pattern
// inside their domain (|g| <= 44, NaN excluded). Zero results may differ in sign (the quantiser maps
// both to code 0). result[0]: g / (1 + __expf(-g)); result[1]: __fdividef(g, 1 + __expf(-g)).
extern "C" __global__ void probe_silu_bf16(ProbeResult* result) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= 65536u) {
        return;
    }
    const float g = __uint_as_float(i << 16);
    if (!(fabsf(g) <= clef::kSiluFastMaxAbs)) {
        return;
    }
    const float other = __uint_as_float(((i * 2654435761u) >> 16 & 0x3FFFu) << 16);   // a second in-domain value
    const float want_ieee = g / (1.0f + __expf(-g));
    const float want_fast = __fdividef(g, 1.0f + __expf(-g));
    const clef::f32x2 a = clef::silu_ieee_fast_x2(clef::f2_pack(g, other));
    const clef::f32x2 b = clef::silu_ieee_fast_x2(clef::f2_pack(other, g));
    const clef::f32x2 c = clef::silu_approx_fast_x2(clef::f2_pack(g, other));
    const clef::f32x2 d = clef::silu_approx_fast_x2(clef::f2_pack(other, g));
    auto same = [](float x, float y) { return __float_as_uint(x) == __float_as_uint(y) || (x == 0.0f && y == 0.0f); };
    atomicAdd(&result[0].checked, 1ull);
    atomicAdd(&result[1].checked, 1ull);
    if (!same(a.x, want_ieee) || !same(b.y, want_ieee)) {
        report(&result[0], i);
    }
    if (!same(c.x, want_fast) || !same(d.y, want_fast)) {
        report(&result[1], i);
    }
}

// The short silu forms for f32 accumulators (the causal convolution) against g / (1 + __expf(-g)) for `count` f32
// patterns from `base`, those with |g| <= 44 only, bit for bit including the sign of zero.
// result[0]: silu_ieee_refined_f32_x2 in both lanes; result[1]: silu_ieee_refined_f32. No mismatch allowed.
extern "C" __global__ void probe_silu_f32(unsigned long long base, unsigned long long count, ProbeResult* result) {
    unsigned long long checked = 0;
    for (unsigned long long i = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; i < count;
         i += (unsigned long long)gridDim.x * blockDim.x) {
        const uint32_t bits = (uint32_t)(base + i);
        const float g = __uint_as_float(bits);
        if (!(fabsf(g) <= clef::kSiluFastMaxAbs)) {
            continue;
        }
        const float other = __uint_as_float((mix(bits) & 0x3FFFFFFFu) | (bits & 0x80000000u));   // some |value| < 2
        const float want = g / (1.0f + __expf(-g));
        const clef::f32x2 a = clef::silu_ieee_refined_f32_x2(clef::f2_pack(g, other));
        const clef::f32x2 b = clef::silu_ieee_refined_f32_x2(clef::f2_pack(other, g));
        ++checked;
        if (__float_as_uint(a.x) != __float_as_uint(want) || __float_as_uint(b.y) != __float_as_uint(want)) {
            report(&result[0], bits);
        }
        if (__float_as_uint(clef::silu_ieee_refined_f32(g)) != __float_as_uint(want)) {
            report(&result[1], bits);
        }
        // result[2]: the approximate-quotient form of the gated norm on f32 activations, __fdividef(g, 1 + __expf(-g))
        const float want_fast = __fdividef(g, 1.0f + __expf(-g));
        const clef::f32x2 c = clef::silu_approx_fast_x2(clef::f2_pack(g, other));
        const clef::f32x2 e = clef::silu_approx_fast_x2(clef::f2_pack(other, g));
        if (__float_as_uint(c.x) != __float_as_uint(want_fast) || __float_as_uint(e.y) != __float_as_uint(want_fast)) {
            report(&result[2], bits);
        }
    }
    atomicAdd(&result[0].checked, checked);
    atomicAdd(&result[1].checked, checked);
    atomicAdd(&result[2].checked, checked);
}

// The short form of x * 1.0f / (1.0f + __expf(-g)) (kernels/elementwise.cu:350-353) for every pair of a
// bf16 g with |g| <= 44 and a finite bf16 x: 2^16 threads (one per g) each walk all x. Zero results may
// differ in sign. result[0]: all pairs; result[1]: the pairs of the tuned kernels' domain, x == 0 or |x| >= 2^-60.
extern "C" __global__ void probe_sigmoid_mul_bf16(ProbeResult* result) {
    const uint32_t gi = blockIdx.x * blockDim.x + threadIdx.x;
    if (gi >= 65536u) {
        return;
    }
    const float g = __uint_as_float(gi << 16);
    if (!(fabsf(g) <= clef::kSiluFastMaxAbs)) {
        return;
    }
    const float d = 1.0f + __expf(-g);
    unsigned long long checked = 0, checked_normal = 0;
    for (uint32_t xi = 0; xi < 65536u; ++xi) {
        const float x = __uint_as_float(xi << 16);
        if (!(fabsf(x) < INFINITY)) {
            continue;
        }
        const float want = x * 1.0f / d;
        const clef::f32x2 a = clef::sigmoid_mul_fast_x2(clef::f2_pack(g, 1.0f), clef::f2_pack(x, 2.0f));
        const clef::f32x2 b = clef::sigmoid_mul_fast_x2(clef::f2_pack(1.0f, g), clef::f2_pack(2.0f, x));
        const bool ok = (__float_as_uint(a.x) == __float_as_uint(want) || (a.x == 0.0f && want == 0.0f)) &&
                        (__float_as_uint(b.y) == __float_as_uint(want) || (b.y == 0.0f && want == 0.0f));
        const bool normal = x == 0.0f || fabsf(x) >= clef::kSigmoidMulMinAbs;
        ++checked;
        checked_normal += normal;
        if (!ok) {
            report(&result[0], (gi << 16) | xi);
            if (normal) {
                report(&result[1], (gi << 16) | xi);
            }
        }
    }
    atomicAdd(&result[0].checked, checked);
    atomicAdd(&result[1].checked, checked_normal);
}

// amax / 6.0f (kernels/quantise.cu:29) against the three-operation form, on the patterns the fast
// quantiser uses it for: +0 and every finite x >= 2^-100.
extern "C" __global__ void probe_div_six(ProbeResult* result) {
    const unsigned long long first = __float_as_uint(clef::kDivSixExactFrom), last = 0x7F800000ull;
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    unsigned long long checked = 0;
    for (unsigned long long i = first + (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < last; i += stride) {
        const float x = __uint_as_float((uint32_t)i);
        ++checked;
        if (__float_as_uint(clef::div_six_fast(x)) != __float_as_uint(x / 6.0f)) {
            report(&result[0], (uint32_t)i);
        }
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        ++checked;
        if (__float_as_uint(clef::div_six_fast(0.0f)) != 0u) {
            report(&result[0], 0u);
        }
    }
    atomicAdd(&result[0].checked, checked);
}


// ---------------------------------------------------------------------------------------------------------
// The GEMM-epilogue quantiser (nvfp4_epilogue.cuh) fed with "accumulators" from global memory.
// accg / accu: [rows_padded, cols] f32 (rows >= a_rows are padding of the M tile). Outputs use the layout of
// clef_swiglu_quantise_nvfp4: packed [rows_padded, cols / 2], scales tiled (chunk_arg < 0: interleaved order).
// mode 0: one thread per (row, block) holding the block (the tcgen05.ld 32x32b layout);
// mode 1: the mma.sync m16n8 fragment layout of kernels/gemm.cu through nvfp4_swiglu_epilogue_quad4;
// mode 2: the same fragment walk spelled with the REFERENCE's header (to_e4m3 / to_e2m1 / from_e4m3) and the
//         literal SwiGLU expression, as kernels/gemm.cu:895-958 writes it.
// ---------------------------------------------------------------------------------------------------------
extern "C" __global__ void probe_epilogue(const float* accg, const float* accu, int a_rows, int rows_padded, int cols,
                                          float gscale_g, float gscale_u, float out_global, int blk_mn, int chunk_arg,
                                          uint8_t* packed, uint8_t* scales, int mode) {
    const int blocks = cols / 16;
    const int order = chunk_arg < 0 ? clef::kSfInterleaved : clef::kSfActivation;
    if (mode == 0) {
        const long long total = (long long)rows_padded * blocks;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
            const int row = (int)(i / blocks), b = (int)(i % blocks);
            const clef::Nvfp4Block q = clef::nvfp4_swiglu_epilogue_block16(accg + (size_t)row * cols + b * 16, accu + (size_t)row * cols + b * 16,
                                                                            gscale_g, gscale_u, out_global, nullptr, row < a_rows);
            scales[clef::nvfp4_scale_offset(row, b, blocks, blk_mn, order)] = (uint8_t)q.stored;
            *reinterpret_cast<uint2*>(packed + (size_t)row * (cols / 2) + b * 8) = make_uint2(q.lo, q.hi);
        }
        return;
    }
    // fragment walk: a warp per 16-row x 16-column tile; lane holds rows c_row and c_row + 8, columns 8 s + 2 (lane & 3) + e
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int c_row = lane >> 2, quad = lane & 3;
    const long long tiles = (long long)(rows_padded / 16) * blocks;
    for (long long t = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < tiles; t += warps) {
        const int r0 = (int)(t / blocks) * 16, b = (int)(t % blocks);
        for (int r = 0; r < 2; ++r) {
            const int row = r0 + c_row + 8 * r;
            float g[4], u[4];
            for (int s = 0; s < 2; ++s) {
                for (int e = 0; e < 2; ++e) {
                    const size_t at = (size_t)row * cols + b * 16 + 8 * s + 2 * quad + e;
                    g[2 * s + e] = accg[at];
                    u[2 * s + e] = accu[at];
                }
            }
            uint32_t stored, byte0, byte1;
            if (mode == 1) {
                const clef::Nvfp4Quad q = clef::nvfp4_swiglu_epilogue_quad4(g, u, gscale_g, gscale_u, out_global, row < a_rows);
                stored = q.stored;
                byte0 = q.byte[0];
                byte1 = q.byte[1];
            } else {
                float vv[4];
                float m0 = 0.0f;
                for (int i = 0; i < 4; ++i) {
                    const float gg = g[i] * gscale_g;
                    const float gu = u[i] * gscale_u;
                    vv[i] = (gg / (1.0f + __expf(-gg))) * gu;
                }
                m0 = fmaxf(fmaxf(fabsf(vv[0]), fabsf(vv[1])), fmaxf(fabsf(vv[2]), fabsf(vv[3])));
                m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 1));
                m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 2));
                const uint8_t st = (row < a_rows) ? to_e4m3((m0 / 6.0f) * out_global) : (uint8_t)0;
                const float stored_f = from_e4m3(st);
                const float inv_scale = (stored_f > 0.0f) ? out_global / stored_f : 0.0f;
                stored = st;
                byte0 = byte1 = 0;
                if (row < a_rows) {
                    byte0 = to_e2m1(vv[0] * inv_scale) | (to_e2m1(vv[1] * inv_scale) << 4);
                    byte1 = to_e2m1(vv[2] * inv_scale) | (to_e2m1(vv[3] * inv_scale) << 4);
                }
            }
            if (quad == 0) {
                scales[clef::nvfp4_scale_offset(row, b, blocks, blk_mn, order)] = (uint8_t)stored;
            }
            packed[(size_t)row * (cols / 2) + b * 8 + quad] = (uint8_t)byte0;
            packed[(size_t)row * (cols / 2) + b * 8 + 4 + quad] = (uint8_t)byte1;
        }
    }
}
