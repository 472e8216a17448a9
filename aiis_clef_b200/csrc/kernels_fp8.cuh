// FP8 (E4M3) activation quantisers: the siblings of the NVFP4 kernels that feed the FP8 projections of
// a mixed checkpoint (kernels/quantise.cu:123-191 gated norm, :273-381 RMSNorm with bf16 twin output,
// :390-452 SwiGLU, :454-514 plain).
//
// Recipe, per quantised row (a token row, or the vh head rows of a token for the gated norm):
//   amax   = max |v_i|  (NaN operands ignored, as fmaxf does)
//   scale  = amax / 448                    stored as the UPPER 16 bits of the f32 (bf16 by truncation)
//   inv    = scale > 0 ? 1 / scale : 0     (from the untruncated scale)
//   code_i = e4m3(|v_i| * inv) | sign(v_i < 0)      e4m3 = the reference's own round-half-up encoder
// The maximum is exact in any order, so the row decomposition is free; the sum of squares of the two
// norms keeps the reference order (team_sum_squares / warp tree). One CTA owns one quantised row, keeps
// the row's f32 values in registers between the amax pass and the encode pass, and loops over rows.
#pragma once

#include "kernels_generic.cuh"

namespace clef {

// The reference E4M3 encoder (kernels/nvfp4_quant.h:35-57) for ANY f32 pattern, without a
// float-to-int conversion: e4m3_encode_finite's bit form, the subnormal code
// min(int(v * 512 + 0.5f), 7) taken from the low mantissa bits of (v * 512 + 0.5f) + 2^23 added
// toward zero, and +inf mapped to the reference's own answer for it (0x37).
__device__ __forceinline__ uint32_t e4m3_encode_any(float v) {
    const uint32_t r = __float_as_uint(v) + 0x00080000u;
    const int code = (int)(r >> 20) - (120 << 3);
    const uint32_t sub = min(__float_as_uint(__fadd_rz(__fmaf_rn(v, 512.0f, 0.5f), 8388608.0f)) & 0xFu, 7u);
    uint32_t out = (code >= 8) ? (uint32_t)min(code, 0x7E) : sub;
    out = (v == __int_as_float(0x7F800000)) ? ((6u << 3) | 7u) : out;
    return (v > 0.0f) ? out : 0u;
}

__device__ __forceinline__ uint32_t fp8_code(float t, float inv_scale) {
    return e4m3_encode_any(__fmul_rn(fabsf(t), inv_scale)) | ((t < 0.0f) ? 0x80u : 0u);
}

// 8 consecutive activations widened to f32.
template <typename T>
__device__ __forceinline__ void load8(const typename T::storage* p, float* v);
template <>
__device__ __forceinline__ void load8<Bf16>(const uint16_t* p, float* v) {
    const uint4 d = ldg_stream_v4(p);
    v[0] = bf16_lo(d.x), v[1] = bf16_hi(d.x), v[2] = bf16_lo(d.y), v[3] = bf16_hi(d.y);
    v[4] = bf16_lo(d.z), v[5] = bf16_hi(d.z), v[6] = bf16_lo(d.w), v[7] = bf16_hi(d.w);
}
template <>
__device__ __forceinline__ void load8<F32>(const float* p, float* v) {
    const uint4 a = ldg_stream_v4(p), b = ldg_stream_v4(p + 4);
    v[0] = __uint_as_float(a.x), v[1] = __uint_as_float(a.y), v[2] = __uint_as_float(a.z), v[3] = __uint_as_float(a.w);
    v[4] = __uint_as_float(b.x), v[5] = __uint_as_float(b.y), v[6] = __uint_as_float(b.z), v[7] = __uint_as_float(b.w);
}

// Maximum over the CTA of a non-negative value (exact in any order). All threads call; two barriers.
__device__ __forceinline__ float cta_max(float v, float* s_part) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        v = fmaxf(v, __shfl_xor_sync(kFullMask, v, off));
    }
    if ((threadIdx.x & 31) == 0) {
        s_part[threadIdx.x >> 5] = v;
    }
    __syncthreads();
    float t = s_part[0];
#pragma unroll
    for (int w = 1; w < kCtaThreads / 32; ++w) {
        t = fmaxf(t, s_part[w]);
    }
    __syncthreads();   // s_part is reused by the next row
    return t;
}

enum Fp8Mode { kFp8Plain = 0, kFp8SwiGLU = 1, kFp8RmsNorm = 2 };

// quantise_fp8 (MODE plain: a = x), swiglu_quantise_fp8 (a = gate, b = up), rms_norm_fp8_bf16 (a = x,
// weight; bf_out optional twin output of the normalised row in bf16). cols % 8 == 0, cols <= 2048 * KMAX.
// Thread t holds the 8-value vectors t, t + 256, ... of the row.
template <typename T, int MODE, int KMAX>
__global__ void __launch_bounds__(kCtaThreads)
fp8_rows_kernel(const typename T::storage* __restrict__ a, const typename T::storage* __restrict__ b,
                const float* __restrict__ weight, uint8_t* __restrict__ out, uint16_t* __restrict__ scales,
                uint16_t* __restrict__ bf_out, int rows, int cols, float eps) {
    __shared__ float s_part[kCtaThreads / 32];
    __shared__ float s_total;
    const int vecs = cols >> 3;
    const int tpr = ref_threads_per_row(cols);
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const typename T::storage* arow = a + (size_t)row * cols;
        float inv_norm = 0.0f;
        if (MODE == kFp8RmsNorm) {
            // The reference team of `tpr` threads sums the row (kernels/elementwise.cu:22-52); the rest idle.
            const float total = team_sum_squares<T>(arow, threadIdx.x < tpr, cols, tpr, s_part);
            if (threadIdx.x == 0) {
                s_total = total;
            }
            __syncthreads();
            inv_norm = inv_rms(s_total, cols, eps);
        }
        float v[KMAX][8];
        float amax = 0.0f;
#pragma unroll
        for (int k = 0; k < KMAX; ++k) {
            const int vec = threadIdx.x + k * kCtaThreads;
            if (vec < vecs) {
                load8<T>(arow + vec * 8, v[k]);
                if (MODE == kFp8SwiGLU) {
                    float u[8];
                    load8<T>(b + (size_t)row * cols + vec * 8, u);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        v[k][i] = silu_ieee_div(v[k][i]) * u[i];
                    }
                } else if (MODE == kFp8RmsNorm) {
                    const float4 w0 = *reinterpret_cast<const float4*>(weight + vec * 8);
                    const float4 w1 = *reinterpret_cast<const float4*>(weight + vec * 8 + 4);
                    const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        v[k][i] = v[k][i] * inv_norm * (1.0f + w[i]);
                    }
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    amax = fmaxf(amax, fabsf(v[k][i]));
                }
            }
        }
        amax = cta_max(amax, s_part);
        const float scale = __fdiv_rn(amax, 448.0f);
        if (threadIdx.x == 0) {
            scales[row] = (uint16_t)(__float_as_uint(scale) >> 16);
        }
        const float inv = (scale > 0.0f) ? __fdiv_rn(1.0f, scale) : 0.0f;
#pragma unroll
        for (int k = 0; k < KMAX; ++k) {
            const int vec = threadIdx.x + k * kCtaThreads;
            if (vec < vecs) {
                uint32_t lo = 0, hi = 0;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    lo |= fp8_code(v[k][i], inv) << (8 * i);
                    hi |= fp8_code(v[k][4 + i], inv) << (8 * i);
                }
                stg_v2(out + (size_t)row * cols + vec * 8, make_uint2(lo, hi));
                if (MODE == kFp8RmsNorm && bf_out) {
                    stg_v4(bf_out + (size_t)row * cols + vec * 8,
                           make_uint4(pack_bf16x2(v[k][0], v[k][1]), pack_bf16x2(v[k][2], v[k][3]),
                                      pack_bf16x2(v[k][4], v[k][5]), pack_bf16x2(v[k][6], v[k][7])));
                }
            }
        }
    }
}

// rms_norm_gated_quantise_fp8 (kernels/quantise.cu:123-191): one CTA per token; warp w normalises the
// head rows w, w + 8, ... (< vh) of the token, a lane the quads lane, lane + 32 (cols <= 256) of a head
// row in the reference's order; v = x * inv * weight * __fdividef(g, 1 + __expf(-g)); the token's amax
// spans its vh head rows. Head rows >= rows_live hold no data: they add 0 to the amax and are not written.
template <typename T, int HMAX>
__global__ void __launch_bounds__(kCtaThreads)
fp8_gated_kernel(const typename T::storage* __restrict__ x, const typename T::storage* __restrict__ gate,
                 const float* __restrict__ weight, uint8_t* __restrict__ out, uint16_t* __restrict__ scales,
                 int tokens, int cols, float eps, int vh, int rows_live) {
    __shared__ float s_part[kCtaThreads / 32];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int c4 = cols >> 2;
    for (int token = blockIdx.x; token < tokens; token += gridDim.x) {
        float4 v[HMAX][2];
        float amax = 0.0f;
#pragma unroll
        for (int h = 0; h < HMAX; ++h) {
            const int head = warp + h * (kCtaThreads / 32);
            const int row = token * vh + head;
            const bool live = head < vh && row < rows_live;
            v[h][0] = v[h][1] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (head >= vh) {
                continue;   // warp-uniform
            }
            float acc = 0.0f;
            if (live) {
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int i = lane + 32 * j;
                    if (i < c4) {
                        v[h][j] = load_quad<T>(x + (size_t)row * cols, i);
                        acc = __fadd_rn(acc, quad_sq(v[h][j]));
                    }
                }
            }
            const float total = warp_tree_sum(acc);
            if (live) {
                const float inv = inv_rms(total, cols, eps);
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int i = lane + 32 * j;
                    if (i < c4) {
                        const float4 g = load_quad<T>(gate + (size_t)row * cols, i);
                        const float4 w = *reinterpret_cast<const float4*>(weight + 4 * i);
                        float4& t = v[h][j];
                        t = make_float4(t.x * inv * w.x * silu_fast_div(g.x), t.y * inv * w.y * silu_fast_div(g.y),
                                        t.z * inv * w.z * silu_fast_div(g.z), t.w * inv * w.w * silu_fast_div(g.w));
                        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(t.x), fabsf(t.y)), fmaxf(fabsf(t.z), fabsf(t.w))));
                    }
                }
            }
        }
        amax = cta_max(amax, s_part);
        const float scale = __fdiv_rn(amax, 448.0f);
        if (threadIdx.x == 0) {
            scales[token] = (uint16_t)(__float_as_uint(scale) >> 16);
        }
        const float inv_scale = (scale > 0.0f) ? __fdiv_rn(1.0f, scale) : 0.0f;
#pragma unroll
        for (int h = 0; h < HMAX; ++h) {
            const int head = warp + h * (kCtaThreads / 32);
            const int row = token * vh + head;
            if (head < vh && row < rows_live) {
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int i = lane + 32 * j;
                    if (i < c4) {
                        const float4 t = v[h][j];
                        const uint32_t q = fp8_code(t.x, inv_scale) | (fp8_code(t.y, inv_scale) << 8) |
                                           (fp8_code(t.z, inv_scale) << 16) | (fp8_code(t.w, inv_scale) << 24);
                        *reinterpret_cast<uint32_t*>(out + (size_t)row * cols + 4 * i) = q;
                    }
                }
            }
        }
    }
}

}  // namespace clef
