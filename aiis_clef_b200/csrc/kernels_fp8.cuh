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
#include "kernels_hot.cuh"

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


// =============================================================================================
// Tuned bf16 kernels.
// =============================================================================================

// Magnitude code of p for 0 <= p < 464 (finite), the reference encoder in 6 operations:
//   n = ((bits(p) + half step) >> 20) - 960      the normal-range code; below 8 (even negative) under 2^-6
//   k = floor(min(p * 512 + 0.5, 8 - ulp))       the subnormal code min(int(p*512 + 0.5), 7); 7 for larger p
// and the code is max(n, k): where the normal branch applies n >= 8 > k, and where the subnormal branch
// applies n <= k (n counts eighths of 2^-7 above 2^-7, k halves of them above 4, rounded). Compared with the
// reference encoder for every f32 pattern of the domain (oracle/ref_probe.cu).
__device__ __forceinline__ uint32_t e4m3_mag_fast(float p) {
    const int n = (int)(__float_as_uint(p) + (0x00080000u - (960u << 20))) >> 20;
    const float s = fminf(__fmaf_rn(p, 512.0f, 0.5f), 7.99999952f);
    const int u = __float_as_int(__fadd_rz(s, 8388608.0f));
    return (uint32_t)__viaddmax_s32(u, -0x4B000000, n);
}

// Largest and smallest non-zero row maximum the short encoder is used for: the row scale amax / 448 and its
// reciprocal are then normal numbers and every |t| * inv is finite and below 464.
constexpr float kFp8FastMinAmax = 7.888609052e-31f;   // 2^-100
constexpr float kFp8FastMaxAmax = 3.0e38f;

// The tuned kernels serve bf16 and f32 activations. A lane's 16-value block is one 32-byte load of bf16 (widened into
// the quad-pair layout) or two of f32 (pairs of consecutive values: nothing to widen). With bf16 the next row's raw
// registers are fetched while the current row is processed; with f32 the loaded registers are the row, so it is
// loaded at the top of its iteration and the next one is only named to L2.
template <typename T>
struct RawBlock16 {
    U8x32 r[T::kBytes / 2];
};
template <typename T>
__device__ __forceinline__ RawBlock16<T> ldg_block16(const typename T::storage* p) {
    RawBlock16<T> b;
#pragma unroll
    for (int i = 0; i < T::kBytes / 2; ++i) b.r[i] = ldg_stream_v8(reinterpret_cast<const uint8_t*>(p) + 32 * i);
    return b;
}
template <typename T>
__device__ __forceinline__ void unpack_block16(const RawBlock16<T>& b, f32x2* v) {
    if (T::kBytes == 2) {
        unpack16_quadpairs(b.r[0], v);
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[i] = f2_pack(__uint_as_float(b.r[0].w[2 * i]), __uint_as_float(b.r[0].w[2 * i + 1]));
            v[4 + i] = f2_pack(__uint_as_float(b.r[T::kBytes / 2 - 1].w[2 * i]), __uint_as_float(b.r[T::kBytes / 2 - 1].w[2 * i + 1]));
        }
    }
}
// (x*x + y*y) + (z*z + w*w) per quad with the reference build's contraction, for either pair order.
template <bool NAT>
__device__ __forceinline__ void quad_squares_of(const f32x2* v, float* quad) {
    if (!NAT) {
        quad_squares(v, quad);
    } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            quad[q] = __fadd_rn(__fmaf_rn(v[2 * q].x, v[2 * q].x, __fmul_rn(v[2 * q].y, v[2 * q].y)),
                                __fmaf_rn(v[2 * q + 1].x, v[2 * q + 1].x, __fmul_rn(v[2 * q + 1].y, v[2 * q + 1].y)));
        }
    }
}
// One quad (of weights) in the order the pairs of `NAT` want it: (x, z, y, w) for quad pairs, natural otherwise.
template <bool NAT>
__device__ __forceinline__ float4 quad_order(float4 w) {
    return NAT ? w : make_float4(w.x, w.z, w.y, w.w);
}
template <bool NAT>
__device__ __forceinline__ U8x32 pack16_bf16_of(const f32x2* v) {
    if (!NAT) return pack16_bf16(v);
    U8x32 o;
#pragma unroll
    for (int i = 0; i < 8; ++i) o.w[i] = pack_bf16x2(v[i].x, v[i].y);
    return o;
}

// Four scaled values p = t * inv with |p| < 464 (signs kept) -> their four code bytes, x in the lowest, by the hardware
// converter cvt.rn.satfinite.e4m3x2.f32. From the smallest normal E4M3 value up the reference encoder is round-half-up
// on the 3-bit mantissa (carrying into the exponent) with saturation at 448 = 0x7E, which is also the converter's
// finite maximum. The converter rounds ties to even: an exact tie has zero low mantissa bits, so setting the lowest
// one lifts it just above the tie, and no other value changes its rounding (a value below a tie stays below it, a
// code point stays nearest to itself). The same holds for the subnormal codes 1 to 7. The converter's bytes differ
// from the reference's only where it answers 0 or 8 in the low seven bits: 7.5/512 <= p < 8/512 gives 7 in the
// reference (its subnormal branch clamps) and 8 here, the f32 just below 2^-10 gives 1 there (its p * 512 + 0.5
// rounds up to 1) and 0 here, and -0.0 keeps its sign here. e4m3x4_suspect flags exactly the words that hold such a
// byte; the caller recomputes them with the integer form. Compared with the reference encoder for every f32 pattern
// of [0, 464), both signs, every byte position: each byte is either flagged or equal (oracle/ref_probe.cu).
__device__ __forceinline__ uint32_t e4m3x4_hw(float x, float y, float z, float w) {
    uint32_t r;
    asm("{\n\t.reg .b16 lo, hi;\n\t"
        "cvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\n\t"   // the first source operand lands in the high byte
        "cvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\n\t"
        "mov.b32 %0, {lo, hi};\n\t}"
        : "=r"(r)
        : "f"(__uint_as_float(__float_as_uint(x) | 1u)), "f"(__uint_as_float(__float_as_uint(y) | 1u)),
          "f"(__uint_as_float(__float_as_uint(z) | 1u)), "f"(__uint_as_float(__float_as_uint(w) | 1u)));
    return r;
}
// Non-zero iff one of the four bytes is 0x00, 0x08, 0x80 or 0x88 (a zero byte after the mask, by the borrow test).
__device__ __forceinline__ uint32_t e4m3x4_suspect(uint32_t word) {
    const uint32_t m = word & 0x77777777u;
    return (m - 0x01010101u) & ~m & 0x80808080u;
}

// The four codes of one quad by the integer form, for any magnitudes below 464: signs from t + 0.0f, which turns
// -0.0 into +0.0 (the reference's (t < 0) is false for it) and changes nothing else. Out of line: it runs for the
// few quads the converter form flags.
static __device__ __noinline__ uint32_t fp8_encode4_int(float x, float y, float z, float w, float inv) {
    x = __fadd_rn(x, 0.0f), y = __fadd_rn(y, 0.0f), z = __fadd_rn(z, 0.0f), w = __fadd_rn(w, 0.0f);
    const uint32_t cx = e4m3_mag_fast(__fmul_rn(fabsf(x), inv)), cy = e4m3_mag_fast(__fmul_rn(fabsf(y), inv));
    const uint32_t cz = e4m3_mag_fast(__fmul_rn(fabsf(z), inv)), cw = e4m3_mag_fast(__fmul_rn(fabsf(w), inv));
    const uint32_t mags = cx | (cy << 8) | (cz << 16) | (cw << 24);
    // top bytes of x, y, z, w -> bytes 0..3
    const uint32_t xy = __byte_perm(__float_as_uint(x), __float_as_uint(y), 0x0073);
    const uint32_t zw = __byte_perm(__float_as_uint(z), __float_as_uint(w), 0x0073);
    return mags | (__byte_perm(xy, zw, 0x5410) & 0x80808080u);
}

// 16 values of a row (quad pairs, or consecutive pairs with NAT) -> 16 code bytes in natural order. `inv2` =
// splat(1 / scale). Every quad goes through the hardware converter; one test per block sends the flagged quads
// (a zero, a value that rounds to zero, one at the top of the subnormal codes) through the integer form.
// NaN rows never get here.
template <bool NAT = false>
__device__ __forceinline__ uint4 fp8_encode16_qp(const f32x2* v, f32x2 inv2) {
    uint32_t word[4], suspect[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const f32x2 pa = f2_mul(v[2 * q], inv2), pb = f2_mul(v[2 * q + 1], inv2);   // (x, z), (y, w); NAT: (x, y), (z, w)
        word[q] = e4m3x4_hw(pa.x, NAT ? pa.y : pb.x, NAT ? pb.x : pa.y, pb.y);
        suspect[q] = e4m3x4_suspect(word[q]);
    }
    if ((suspect[0] | suspect[1]) | (suspect[2] | suspect[3])) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            if (suspect[q]) {
                const f32x2 a = v[2 * q], b = v[2 * q + 1];
                word[q] = fp8_encode4_int(a.x, NAT ? a.y : b.x, NAT ? b.x : a.y, b.y, inv2.x);
            }
        }
    }
    return make_uint4(word[0], word[1], word[2], word[3]);
}

// Literal encoder for one block of a row that left the short encoder's domain: values recomputed from global
// memory in natural order. MODE as in fp8_rows_kernel; inv_norm is the row's 1 / rms (RMSNorm only).
template <int MODE, typename T>
static __device__ __noinline__ void fp8_block_cold(const typename T::storage* ablk, const typename T::storage* bblk,
                                                   const float* wblk, float inv_norm, float inv_scale, uint4* dst) {
    uint32_t word[4] = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        float t = load_scalar<T>(ablk + i);
        if (MODE == kFp8SwiGLU) {
            t = silu_ieee_div(t) * load_scalar<T>(bblk + i);
        } else if (MODE == kFp8RmsNorm) {
            t = t * inv_norm * (1.0f + wblk[i]);
        }
        word[i >> 2] |= fp8_code(t, inv_scale) << (8 * (i & 3));
    }
    *dst = make_uint4(word[0], word[1], word[2], word[3]);
}

// max |v| over a block, NaN if any value is NaN (the fast path's detector) / NaN ignored (the recipe's amax).
__device__ __forceinline__ float block_abs_max_ignoring_nan(const f32x2* v) {
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        m = fmaxf(m, fmaxf(fabsf(v[i].x), fabsf(v[i].y)));
    }
    return m;
}

// quantise_fp8 (MODE plain) and rms_norm_fp8_bf16 (MODE RmsNorm, bf_out optional) for cols = NB * 512, one warp
// per row: the row structure, prefetch and summation tree of rms_norm_quant_hot_kernel; the row maximum is a
// 5-step butterfly, the row scale is computed by every lane, each lane encodes its NB blocks (16 bytes each).
template <int NB, int MODE, typename T = Bf16>
__global__ void __launch_bounds__(kCtaThreads, (NB <= 4 ? 2 : 1))
fp8_rows_hot_kernel(const typename T::storage* __restrict__ x, const float* __restrict__ weight, uint8_t* __restrict__ out,
                    uint16_t* __restrict__ scales, uint16_t* __restrict__ bf_out, int rows, float eps) {
    constexpr int COLS = NB * 512;
    constexpr bool NAT = T::kBytes == 4, REGPF = T::kBytes == 2;
    constexpr int LINE = 128 / T::kBytes;   // values per 128-byte line
    extern __shared__ float4 s_w[];   // (1 + w) in the pairs' order, as in rms_norm_quant_hot_kernel
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    pdl_launch_dependents();
    if (MODE == kFp8RmsNorm) {
        for (int idx = threadIdx.x; idx < COLS / 4; idx += kCtaThreads) {
            const int l = idx & 31, q = (idx >> 5) & 3, j = idx >> 7;
            const float4 w = *reinterpret_cast<const float4*>(weight + (l + 32 * j) * 16 + 4 * q);
            s_w[idx] = quad_order<NAT>(make_float4(1.0f + w.x, 1.0f + w.y, 1.0f + w.z, 1.0f + w.w));
        }
    }
    int row = blockIdx.x * 8 + warp;
    auto name_row_to_l2 = [&](int r) {   // a row is NB * 1 KiB (bf16) or NB * 2 KiB (f32): a lane covers 128 bytes per step
#pragma unroll
        for (int h = 0; h < NB * T::kBytes / 8; ++h) {
            prefetch_l2(x + (size_t)r * COLS + (size_t)(lane + 32 * h) * LINE);
        }
    };
    if (row < rows) name_row_to_l2(row);   // this warp's first row towards L2; see prefetch_l2
    pdl_wait_prior_grids();
    RawBlock16<T> d[NB];
    if (REGPF && row < rows) {
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            d[j] = ldg_block16<T>(x + (size_t)row * COLS + (size_t)(lane + 32 * j) * 16);
        }
    }
    __syncthreads();
    for (; row < rows; row += gridDim.x * 8) {
        if (!REGPF) {
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                d[j] = ldg_block16<T>(x + (size_t)row * COLS + (size_t)(lane + 32 * j) * 16);
            }
        }
        f32x2 v[NB][8];
        float p[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            unpack_block16<T>(d[j], v[j]);
            if (MODE == kFp8RmsNorm) {
                float quad[4];
                quad_squares_of<NAT>(v[j], quad);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    p[j & 1][k] = __fadd_rn(p[j & 1][k], quad[k]);
                }
            }
        }
        const int next = row + gridDim.x * 8;
        if (next < rows) {
            if (REGPF) {
#pragma unroll
                for (int j = 0; j < NB; ++j) {
                    d[j] = ldg_block16<T>(x + (size_t)next * COLS + (size_t)(lane + 32 * j) * 16);
                }
            } else {
                name_row_to_l2(next);
            }
        }
        float inv_norm = 0.0f;
        if (MODE == kFp8RmsNorm) {
            inv_norm = (COLS & (COLS - 1)) == 0 ? inv_rms_pow2<COLS>(row_tree_256(p, lane), eps)
                                                : inv_rms(row_tree_256(p, lane), COLS, eps);
            const f32x2 inv2 = f2_splat(inv_norm);
#pragma unroll
            for (int j = 0; j < NB; ++j) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float4 w = s_w[(4 * j + q) * 32 + lane];
                    v[j][2 * q] = f2_mul(f2_mul(v[j][2 * q], inv2), make_float2(w.x, w.y));
                    v[j][2 * q + 1] = f2_mul(f2_mul(v[j][2 * q + 1], inv2), make_float2(w.z, w.w));
                }
            }
        }
        float amax = 0.0f;
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            amax = fmaxf_nan(amax, block_abs_max(v[j]));
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            amax = fmaxf_nan(amax, __shfl_xor_sync(kFullMask, amax, off));
        }
        uint8_t* orow = out + (size_t)row * COLS;
        const bool fast = amax == 0.0f || (amax >= kFp8FastMinAmax && amax <= kFp8FastMaxAmax);   // false for NaN
        if (fast) {
            const float scale = __fdiv_rn(amax, 448.0f);
            if (lane == 0) {
                scales[row] = (uint16_t)(__float_as_uint(scale) >> 16);
            }
            const f32x2 inv2 = f2_splat((scale > 0.0f) ? __frcp_rn(scale) : 0.0f);
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                *reinterpret_cast<uint4*>(orow + (size_t)(lane + 32 * j) * 16) = fp8_encode16_qp<NAT>(v[j], inv2);
            }
        } else {
            // A NaN, an infinity or a tiny maximum in the row: the recipe's own maximum (NaN ignored), literal codes.
            float m = 0.0f;
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                m = fmaxf(m, block_abs_max_ignoring_nan(v[j]));
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                m = fmaxf(m, __shfl_xor_sync(kFullMask, m, off));
            }
            const float scale = __fdiv_rn(m, 448.0f);
            if (lane == 0) {
                scales[row] = (uint16_t)(__float_as_uint(scale) >> 16);
            }
            const float inv_scale = (scale > 0.0f) ? __fdiv_rn(1.0f, scale) : 0.0f;
            for (int j = 0; j < NB; ++j) {
                const int b = lane + 32 * j;
                fp8_block_cold<MODE, T>(x + (size_t)row * COLS + b * 16, nullptr, weight + b * 16, inv_norm, inv_scale,
                                        reinterpret_cast<uint4*>(orow + (size_t)b * 16));
            }
        }
        if (MODE == kFp8RmsNorm && bf_out) {
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                stg_v8(bf_out + (size_t)row * COLS + (size_t)(lane + 32 * j) * 16, pack16_bf16_of<NAT>(v[j]));
            }
        }
    }
}


// A barrier over the WPR warps of one team (named barrier 1 + team; barrier 0 is __syncthreads).
template <int WPR>
__device__ __forceinline__ void team_barrier(int team) {
    if (WPR > 1) {
        asm volatile("bar.sync %0, %1;" ::"r"(1 + team), "r"(WPR * 32) : "memory");
    }
}

// quantise_fp8 (MODE plain) and swiglu_quantise_fp8 for cols = 512 * WPR * BPL: a team of WPR warps owns a row
// (8 / WPR rows per CTA at a time), lane l of team warp w holds the 16-value blocks (32 w + l) + 32 WPR j, j < BPL,
// keeps their f32 values in registers, and the team's row maximum goes through shared memory: one named barrier
// per row, the slots double-buffered by row parity so a fast warp's next row cannot overwrite a slow warp's read.
// f32 activations: the gate's silu is silu_ieee_refined_f32_x2 (the IEEE quotient for every f32 |g| <= 44).
template <int MODE, int BPL, int WPR, typename T = Bf16>
__global__ void __launch_bounds__(kCtaThreads, 2)
fp8_team_hot_kernel(const typename T::storage* __restrict__ a, const typename T::storage* __restrict__ b,
                    uint8_t* __restrict__ out, uint16_t* __restrict__ scales, int rows) {
    constexpr int COLS = 512 * WPR * BPL;
    constexpr int TEAMS = (kCtaThreads / 32) / WPR;
    constexpr bool NAT = T::kBytes == 4, REGPF = T::kBytes == 2;
    constexpr int LPB = 4 * T::kBytes;      // 128-byte lines in the 32 blocks a warp loads at once
    constexpr int LINE = 128 / T::kBytes;   // values per line
    __shared__ float s_max[2][2][kCtaThreads / 32];   // [fast | literal][row parity][warp]
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int team = warp / WPR, wt = warp % WPR;
    const int first_block = wt * 32 + lane;
    pdl_launch_dependents();
    int row = blockIdx.x * TEAMS + team;
    auto name_row_to_l2 = [&](int r) {   // this warp's share of the team's row r: LPB lines per group of 32 blocks
#pragma unroll
        for (int h = 0; h < (BPL * LPB + 31) / 32; ++h) {
            const int idx = lane + 32 * h;
            if (idx < BPL * LPB) {
                const size_t off = (size_t)r * COLS + (size_t)(wt * 32 + 32 * WPR * (idx / LPB)) * 16 + (size_t)(idx % LPB) * LINE;
                prefetch_l2(a + off);
                if (MODE == kFp8SwiGLU) prefetch_l2(b + off);
            }
        }
    };
    if (row < rows) name_row_to_l2(row);   // see prefetch_l2
    pdl_wait_prior_grids();
    RawBlock16<T> da[REGPF ? BPL : 1], db[REGPF && MODE == kFp8SwiGLU ? BPL : 1];
    if (REGPF && row < rows) {
#pragma unroll
        for (int j = 0; j < BPL; ++j) {
            const size_t off = (size_t)row * COLS + (size_t)(first_block + 32 * WPR * j) * 16;
            da[j] = ldg_block16<T>(a + off);
            if (MODE == kFp8SwiGLU) db[j] = ldg_block16<T>(b + off);
        }
    }
    int parity = 0;
    for (; row < rows; row += gridDim.x * TEAMS, parity ^= 1) {
        f32x2 v[BPL][8];
        float amax = 0.0f;
        RawBlock16<T> ub;   // f32: the `b` block of the current j, fetched one block ahead
        if (!REGPF) {
            // all of this lane's `a` blocks at once (they are the values: no raw copies), `b` one block ahead
#pragma unroll
            for (int j = 0; j < BPL; ++j) {
                unpack_block16<T>(ldg_block16<T>(a + (size_t)row * COLS + (size_t)(first_block + 32 * WPR * j) * 16), v[j]);
            }
            if (MODE == kFp8SwiGLU) ub = ldg_block16<T>(b + (size_t)row * COLS + (size_t)first_block * 16);
            const int next = row + gridDim.x * TEAMS;
            if (next < rows) name_row_to_l2(next);
        }
#pragma unroll
        for (int j = 0; j < BPL; ++j) {
            if (REGPF) unpack_block16<T>(da[j], v[j]);
            if (MODE == kFp8SwiGLU) {
                f32x2 u[8];
                unpack_block16<T>(REGPF ? db[j] : ub, u);
                if (!REGPF && j + 1 < BPL) {
                    ub = ldg_block16<T>(b + (size_t)row * COLS + (size_t)(first_block + 32 * WPR * (j + 1)) * 16);
                }
                if (NAT) {
                    if (block_abs_max(v[j]) <= kSiluFastMaxAbs) {   // false for a NaN
#pragma unroll
                        for (int i = 0; i < 8; ++i) v[j][i] = f2_mul(silu_ieee_refined_f32_x2(v[j][i]), u[i]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            v[j][i] = make_float2(gated_literal<kActSwiGLU>(v[j][i].x, u[i].x), gated_literal<kActSwiGLU>(v[j][i].y, u[i].y));
                        }
                    }
                } else if (gated_fast_domain<kActSwiGLU, false>(v[j], u, nullptr)) {
                    gated_fast<kActSwiGLU>(v[j], u);
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        v[j][i] = make_float2(gated_literal<kActSwiGLU>(v[j][i].x, u[i].x), gated_literal<kActSwiGLU>(v[j][i].y, u[i].y));
                    }
                }
            }
            amax = fmaxf_nan(amax, block_abs_max(v[j]));
        }
        const int next = row + gridDim.x * TEAMS;
        if (REGPF && next < rows) {
#pragma unroll
            for (int j = 0; j < BPL; ++j) {
                const size_t off = (size_t)next * COLS + (size_t)(first_block + 32 * WPR * j) * 16;
                da[j] = ldg_block16<T>(a + off);
                if (MODE == kFp8SwiGLU) db[j] = ldg_block16<T>(b + off);
            }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            amax = fmaxf_nan(amax, __shfl_xor_sync(kFullMask, amax, off));
        }
        if (WPR > 1) {
            if (lane == 0) s_max[0][parity][warp] = amax;
            team_barrier<WPR>(team);
            amax = s_max[0][parity][team * WPR];
#pragma unroll
            for (int w = 1; w < WPR; ++w) {
                amax = fmaxf_nan(amax, s_max[0][parity][team * WPR + w]);
            }
        }
        uint8_t* orow = out + (size_t)row * COLS;
        const bool fast = amax == 0.0f || (amax >= kFp8FastMinAmax && amax <= kFp8FastMaxAmax);   // false for NaN
        if (fast) {
            const float scale = __fdiv_rn(amax, 448.0f);
            if (wt == 0 && lane == 0) {
                scales[row] = (uint16_t)(__float_as_uint(scale) >> 16);
            }
            const f32x2 inv2 = f2_splat((scale > 0.0f) ? __frcp_rn(scale) : 0.0f);
#pragma unroll
            for (int j = 0; j < BPL; ++j) {
                *reinterpret_cast<uint4*>(orow + (size_t)(first_block + 32 * WPR * j) * 16) = fp8_encode16_qp<NAT>(v[j], inv2);
            }
        } else {
            float m = 0.0f;
#pragma unroll
            for (int j = 0; j < BPL; ++j) {
                m = fmaxf(m, block_abs_max_ignoring_nan(v[j]));
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                m = fmaxf(m, __shfl_xor_sync(kFullMask, m, off));
            }
            if (WPR > 1) {
                if (lane == 0) s_max[1][parity][warp] = m;
                team_barrier<WPR>(team);
                m = s_max[1][parity][team * WPR];
#pragma unroll
                for (int w = 1; w < WPR; ++w) {
                    m = fmaxf(m, s_max[1][parity][team * WPR + w]);
                }
            }
            const float scale = __fdiv_rn(m, 448.0f);
            if (wt == 0 && lane == 0) {
                scales[row] = (uint16_t)(__float_as_uint(scale) >> 16);
            }
            const float inv_scale = (scale > 0.0f) ? __fdiv_rn(1.0f, scale) : 0.0f;
            for (int j = 0; j < BPL; ++j) {
                const size_t off = (size_t)row * COLS + (size_t)(first_block + 32 * WPR * j) * 16;
                fp8_block_cold<MODE, T>(a + off, MODE == kFp8SwiGLU ? b + off : nullptr, nullptr, 0.0f, inv_scale,
                                        reinterpret_cast<uint4*>(out + off));
            }
        }
    }
}


// Literal values and codes of one 16-value block of the gated norm (kernels/quantise.cu:149-157, 185-190).
template <typename T>
static __device__ __noinline__ void fp8_gated_block_cold(const typename T::storage* xblk, const typename T::storage* gblk,
                                                         const float* wblk, float inv_norm, float inv_scale, uint4* dst) {
    uint32_t word[4] = {0u, 0u, 0u, 0u};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float t = load_scalar<T>(xblk + i) * inv_norm * wblk[i] * silu_fast_div(load_scalar<T>(gblk + i));
        word[i >> 2] |= fp8_code(t, inv_scale) << (8 * (i & 3));
    }
    *dst = make_uint4(word[0], word[1], word[2], word[3]);
}

// rms_norm_gated_quantise_fp8 for 128-wide heads, vh = 8 * STEPS * WPT head rows per token, every head row live:
// WPT warps own a token; in each of its STEPS steps a warp normalises 8 head rows with the lane layout and the
// summation tree of gated_norm_quant_hot_kernel (4 lanes per head row); the values stay in registers until the
// token's maximum is known (butterfly, then the team exchange of fp8_team_hot_kernel).
template <int STEPS, int WPT, typename T = Bf16>
__global__ void __launch_bounds__(kCtaThreads, 2)
fp8_gated_hot_kernel(const typename T::storage* __restrict__ x, const typename T::storage* __restrict__ gate,
                     const float* __restrict__ weight, uint8_t* __restrict__ out, uint16_t* __restrict__ scales,
                     int tokens, float eps) {
    constexpr int COLS = 128;
    constexpr int VH = 8 * STEPS * WPT;
    constexpr int TEAMS = (kCtaThreads / 32) / WPT;
    constexpr bool NAT = T::kBytes == 4, REGPF = T::kBytes == 2;
    constexpr int LINE = 128 / T::kBytes;   // values per 128-byte line
    __shared__ float s_max[2][2][kCtaThreads / 32];
    __shared__ float4 s_w[32];   // plain weight in the pairs' order: s_w[(h * 4 + q) * 4 + m]
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int m = lane & 3;
    const int team = warp / WPT, wt = warp % WPT;
    pdl_launch_dependents();
    if (threadIdx.x < 32) {
        const int mm = threadIdx.x & 3, q = (threadIdx.x >> 2) & 3, h = threadIdx.x >> 4;
        const float4 t = *reinterpret_cast<const float4*>(weight + (mm + 4 * h) * 16 + 4 * q);
        s_w[threadIdx.x] = quad_order<NAT>(t);
    }
    // Head row of this lane group in step s of token t: t * VH + (wt * STEPS + s) * 8 + (lane >> 2).
    auto head_row = [&](int token, int step) { return (size_t)token * VH + (size_t)(wt * STEPS + step) * 8 + (lane >> 2); };
    int token = blockIdx.x * TEAMS + team;
    // the 8 head rows of a step are 16 lines (bf16) or 32 (f32) of x and as many of the gate
    auto name_step_to_l2 = [&](int t, int step) {
        const size_t first = ((size_t)t * VH + (size_t)(wt * STEPS + step) * 8) * COLS;
        if (REGPF) {
            prefetch_l2((lane < 16 ? x : gate) + first + (size_t)(lane & 15) * LINE);
        } else {
            prefetch_l2(x + first + (size_t)lane * LINE);
            prefetch_l2(gate + first + (size_t)lane * LINE);
        }
    };
    if (token < tokens) name_step_to_l2(token, 0);   // see prefetch_l2
    pdl_wait_prior_grids();
    __syncthreads();
    RawBlock16<T> dx[2], dg[2];
    if (REGPF && token < tokens) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            dx[h] = ldg_block16<T>(x + head_row(token, 0) * COLS + (m + 4 * h) * 16);
            dg[h] = ldg_block16<T>(gate + head_row(token, 0) * COLS + (m + 4 * h) * 16);
        }
    }
    int parity = 0;
    for (; token < tokens; token += gridDim.x * TEAMS, parity ^= 1) {
        f32x2 v[STEPS][2][8];
        float inv_norm[STEPS];
        float amax = 0.0f;
#pragma unroll
        for (int step = 0; step < STEPS; ++step) {
            f32x2 gv[2][8];
            float quad[2][4];
            if (!REGPF) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    dx[h] = ldg_block16<T>(x + head_row(token, step) * COLS + (m + 4 * h) * 16);
                    dg[h] = ldg_block16<T>(gate + head_row(token, step) * COLS + (m + 4 * h) * 16);
                }
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                unpack_block16<T>(dx[h], v[step][h]);
                unpack_block16<T>(dg[h], gv[h]);
                quad_squares_of<NAT>(v[step][h], quad[h]);
            }
            // fetch (bf16) or name to L2 (f32) the next step (of this token, or the first of this team's next token)
            const int ntoken = (step + 1 < STEPS) ? token : token + gridDim.x * TEAMS;
            const int nstep = (step + 1 < STEPS) ? step + 1 : 0;
            if (ntoken < tokens) {
                if (REGPF) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        dx[h] = ldg_block16<T>(x + head_row(ntoken, nstep) * COLS + (m + 4 * h) * 16);
                        dg[h] = ldg_block16<T>(gate + head_row(ntoken, nstep) * COLS + (m + 4 * h) * 16);
                    }
                } else {
                    name_step_to_l2(ntoken, nstep);
                }
            }
            inv_norm[step] = inv_rms_pow2<COLS>(head_tree_32(quad[0], quad[1], lane), eps);
            const f32x2 inv2 = f2_splat(inv_norm[step]);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (block_abs_max(gv[h]) <= kSiluFastMaxAbs) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float4 w = s_w[(h * 4 + q) * 4 + m];
                        v[step][h][2 * q] = f2_mul(f2_mul(f2_mul(v[step][h][2 * q], inv2), make_float2(w.x, w.y)),
                                                   silu_approx_fast_x2(gv[h][2 * q]));
                        v[step][h][2 * q + 1] = f2_mul(f2_mul(f2_mul(v[step][h][2 * q + 1], inv2), make_float2(w.z, w.w)),
                                                       silu_approx_fast_x2(gv[h][2 * q + 1]));
                    }
                } else {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float4 w = s_w[(h * 4 + q) * 4 + m];
                        f32x2& a = v[step][h][2 * q];
                        f32x2& b = v[step][h][2 * q + 1];
                        a = make_float2(a.x * inv_norm[step] * w.x * silu_fast_div(gv[h][2 * q].x),
                                        a.y * inv_norm[step] * w.y * silu_fast_div(gv[h][2 * q].y));
                        b = make_float2(b.x * inv_norm[step] * w.z * silu_fast_div(gv[h][2 * q + 1].x),
                                        b.y * inv_norm[step] * w.w * silu_fast_div(gv[h][2 * q + 1].y));
                    }
                }
                amax = fmaxf_nan(amax, block_abs_max(v[step][h]));
            }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            amax = fmaxf_nan(amax, __shfl_xor_sync(kFullMask, amax, off));
        }
        if (WPT > 1) {
            if (lane == 0) s_max[0][parity][warp] = amax;
            team_barrier<WPT>(team);
            amax = s_max[0][parity][team * WPT];
#pragma unroll
            for (int w = 1; w < WPT; ++w) {
                amax = fmaxf_nan(amax, s_max[0][parity][team * WPT + w]);
            }
        }
        const bool fast = amax == 0.0f || (amax >= kFp8FastMinAmax && amax <= kFp8FastMaxAmax);
        if (fast) {
            const float scale = __fdiv_rn(amax, 448.0f);
            if (wt == 0 && lane == 0) {
                scales[token] = (uint16_t)(__float_as_uint(scale) >> 16);
            }
            const f32x2 inv2 = f2_splat((scale > 0.0f) ? __frcp_rn(scale) : 0.0f);
#pragma unroll
            for (int step = 0; step < STEPS; ++step) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    *reinterpret_cast<uint4*>(out + head_row(token, step) * COLS + (m + 4 * h) * 16) =
                        fp8_encode16_qp<NAT>(v[step][h], inv2);
                }
            }
        } else {
            float mx = 0.0f;
#pragma unroll
            for (int step = 0; step < STEPS; ++step) {
                mx = fmaxf(mx, fmaxf(block_abs_max_ignoring_nan(v[step][0]), block_abs_max_ignoring_nan(v[step][1])));
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                mx = fmaxf(mx, __shfl_xor_sync(kFullMask, mx, off));
            }
            if (WPT > 1) {
                if (lane == 0) s_max[1][parity][warp] = mx;
                team_barrier<WPT>(team);
                mx = s_max[1][parity][team * WPT];
#pragma unroll
                for (int w = 1; w < WPT; ++w) {
                    mx = fmaxf(mx, s_max[1][parity][team * WPT + w]);
                }
            }
            const float scale = __fdiv_rn(mx, 448.0f);
            if (wt == 0 && lane == 0) {
                scales[token] = (uint16_t)(__float_as_uint(scale) >> 16);
            }
            const float inv_scale = (scale > 0.0f) ? __fdiv_rn(1.0f, scale) : 0.0f;
#pragma unroll
            for (int step = 0; step < STEPS; ++step) {
                for (int h = 0; h < 2; ++h) {
                    const size_t off = head_row(token, step) * COLS + (m + 4 * h) * 16;
                    fp8_gated_block_cold<T>(x + off, gate + off, weight + (m + 4 * h) * 16, inv_norm[step], inv_scale,
                                         reinterpret_cast<uint4*>(out + off));
                }
            }
        }
    }
}

}  // namespace clef
