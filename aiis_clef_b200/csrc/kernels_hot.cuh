// Tuned sm_100a kernels for bf16 activations at the shapes the fused layer runs at.
//
// Common shape of every kernel here: persistent CTAs (grid = SM count x resident CTAs), each lane
// moves 32 contiguous bytes per access (256-bit ld/st, a warp covers 1 KiB), so one lane owns one
// whole 16-value NVFP4 block; arithmetic runs on packed fp32 pairs (f32x2.cuh) because these
// kernels are bound by instruction issue before they are bound by HBM; row reductions are warp
// shuffles arranged to reproduce the reference's summation tree; no global scratch memory.
//
// Register layout of one 16-value block ("quad pairs"): for quad q (elements 4q..4q+3 = x,y,z,w)
// pair 2q holds (x, z) and pair 2q+1 holds (y, w). That is the layout in which the reference's
// (x*x + y*y) + (z*z + w*w) becomes one packed multiply and one packed FMA, and the quantiser
// accepts it directly.
#pragma once

#include "common.cuh"
#include "f32x2.cuh"
#include "nvfp4_codec.cuh"
#include "silu_forms.cuh"

namespace clef {

// n / d for n < 2^31 by multiply-high (d fixed per launch, prepared on the host).
struct FastDiv {
    uint32_t d, mul, shr;
};
inline FastDiv make_fast_div(uint32_t d) {
    FastDiv f{d, 0u, 0u};
    if (d > 1) {
        uint32_t lg = 0;
        while ((1ull << lg) < d) ++lg;
        const uint32_t p = 31 + lg;
        f.mul = (uint32_t)(((1ull << p) + d - 1) / d);
        f.shr = p - 32;
    }
    return f;
}
__device__ __forceinline__ uint32_t fast_div(uint32_t n, const FastDiv& f) {
    return f.d == 1 ? n : (__umulhi(n, f.mul) >> f.shr);
}

// 32 bytes = 16 bf16 values -> 8 packed pairs in the quad-pair layout.
__device__ __forceinline__ void unpack16_quadpairs(const U8x32& d, f32x2* v) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const uint32_t w0 = d.w[2 * q], w1 = d.w[2 * q + 1];
        v[2 * q] = f2_pack(bf16_lo(w0), bf16_lo(w1));       // (x, z)
        v[2 * q + 1] = f2_pack(bf16_hi(w0), bf16_hi(w1));   // (y, w)
    }
}

// Quad-pair registers of one block -> 32 bytes of bf16 in natural order (round to nearest even).
__device__ __forceinline__ U8x32 pack16_bf16(const f32x2* v) {
    U8x32 o;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        o.w[2 * q] = pack_bf16x2(v[2 * q].x, v[2 * q + 1].x);       // (x, y)
        o.w[2 * q + 1] = pack_bf16x2(v[2 * q].y, v[2 * q + 1].y);   // (z, w)
    }
    return o;
}

// Sum of squares of the 4 quads of a block, reference association and contraction:
// quad = fma(x,x,y*y) + fma(z,z,w*w).
__device__ __forceinline__ void quad_squares(const f32x2* v, float* quad) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const f32x2 t = f2_mul(v[2 * q + 1], v[2 * q + 1]);       // (y*y, w*w)
        const f32x2 s = f2_fma(v[2 * q], v[2 * q], t);            // (fma(x,x,y*y), fma(z,z,w*w))
        float a, b;
        f2_unpack(s, a, b);
        quad[q] = __fadd_rn(a, b);
    }
}

// Eight scaled values -> 32 packed bits (first value in the lowest nibble) with the hardware
// FP4 converter; see e2m1x2_fast in nvfp4_codec.cuh for why the inputs are nudged first.
__device__ __forceinline__ uint32_t e2m1_pack8(float e0, float e1, float e2, float e3, float e4, float e5, float e6,
                                               float e7) {
    uint32_t r;
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
        "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
        : "=r"(r)
        : "f"(e0), "f"(e1), "f"(e2), "f"(e3), "f"(e4), "f"(e5), "f"(e6), "f"(e7));
    return r;
}

// Block quantiser on the quad-pair layout, fast path only. Always writes stored/lo/hi; returns false when
// they are not the block's answer and the caller must run its cold routine (which recomputes the block from
// global memory, literally, and overwrites what was stored). Keeping the literal path out of this function
// keeps address-taken arrays and call set-up out of the hot loop.
//
// Fast domain: the block's scale argument sv = (amax / 6) * global_scale lies in [2^-6, 2^30) (a normal E4M3
// code, clamped to 0x7E from 448 up as the reference clamps it), or the block is all zeros. With
// 2^-64 <= global_scale <= 2^64 (the launchers send other scales to the shape-general kernels) sv >= 2^-6
// implies amax >= 2^-68, where the short division by six is exact; sv < 2^30 keeps the scaled maximum
// amax * inv_scale below 6 * 2^30 / 448 < 2^24, inside the FP4 converter's domain (which saturates at 6 as the
// reference does); a NaN or an infinity in the block makes sv NaN or infinite, whose code is out of range. What
// falls outside is rare in activations: scale arguments below 2^-6 (subnormal codes) and non-finite values.
// For an all-zero block the codes come out as zeros whatever table entry is read, and the scale byte is 0.
// NEG: the pairs hold the NEGATED values (the SwiGLU fast path produces -v); magnitudes are unaffected
// and the sign is restored by scaling with -inv_scale.
// NATURAL: the pairs hold consecutive values, pair i = (value 2i, value 2i + 1), instead of the quad-pair layout
// (f32 activations arrive that way from a 32-byte load and need no widening).
template <bool NEG, bool NATURAL = false>
__device__ __forceinline__ bool quantise16_qp(const f32x2* v, float global_scale, const float* inv_table,
                                              uint32_t& stored_out, uint32_t& lo_out, uint32_t& hi_out) {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        amax = max3_abs_nan(amax, v[i].x, v[i].y);
    }
    const float sv = __fmul_rn(div_six_fast(amax), global_scale);
    // e4m3_encode_finite's normal branch: round the 3-bit mantissa half up by an integer add, rebase the exponent
    const uint32_t code = ((__float_as_uint(sv) + 0x00080000u) >> 20) - (120u << 3);
    const bool normal = (code - 8u) < 288u;          // 2^-6 <= sv < 2^30 (code 296 is the first with exponent 30)
    const uint32_t stored = min(code, 0x7Eu);        // the reference's clamp; also a safe table index for any code
    const float inv = inv_table[stored];
    constexpr float kNudge = -4.33488326e-08f;   // see e2m1x2_fast
    const f32x2 inv2 = f2_splat(NEG ? -inv : inv);
    const f32x2 nudge2 = f2_splat(kNudge);
    f32x2 p[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const f32x2 t = f2_mul(v[i], inv2);
        p[i] = f2_fma(t, nudge2, t);
    }
    // quad q: p[2q] = (x, z), p[2q+1] = (y, w); element order x, y, z, w
    stored_out = normal ? stored : 0u;
    if (NATURAL) {
        lo_out = e2m1_pack8(p[0].x, p[0].y, p[1].x, p[1].y, p[2].x, p[2].y, p[3].x, p[3].y);
        hi_out = e2m1_pack8(p[4].x, p[4].y, p[5].x, p[5].y, p[6].x, p[6].y, p[7].x, p[7].y);
    } else {
        lo_out = e2m1_pack8(p[0].x, p[1].x, p[0].y, p[1].y, p[2].x, p[3].x, p[2].y, p[3].y);
        hi_out = e2m1_pack8(p[4].x, p[5].x, p[4].y, p[5].y, p[6].x, p[7].x, p[6].y, p[7].y);
    }
    return normal || amax == 0.0f;
}

// Cold path shared by the kernels: the caller has the block's 16 f32 values recomputed in natural
// order; quantise them literally and store codes and scale.
static __device__ __noinline__ void quantise16_cold_store(const float* a, float global_scale, uint2* packed_dst,
                                                   uint8_t* scale_dst) {
    uint32_t stored, lo, hi;
    quantise16_rare(a, global_scale, stored, lo, hi);
    *packed_dst = make_uint2(lo, hi);
    *scale_dst = (uint8_t)stored;
}

// ---------------------------------------------------------------------------------------------
// RMSNorm + NVFP4 quantiser, cols = NB * 512 (NB = 4: 2048, NB = 8: 4096), one warp per row.
//
// Reference association (kernels/quantise.cu:207-237 with 256 threads, equal to
// kernels/elementwise.cu:22-52 for cols >= 1793): reference thread `sub` adds quads sub, sub+256, ..;
// warps of 32 consecutive `sub` join by the 16,8,4,2,1 tree; the 8 warp sums join by the 4,2,1 tree.
// Here lane L holds chunks c = L + 32 j (j < NB), i.e. quads 4c + k (k < 4), so
//   sub            = k + 4 L + 128 (j & 1)        reference lane = k + 4 (L & 7)
//   reference warp = (L >> 3) + 4 (j & 1)
// The 8 per-lane partial sums P[j & 1][k] go through the same tree as a reduce-scatter: each of the
// three levels over L bits 2,1,0 halves the values a lane keeps (every tree node is computed once,
// not in every lane), then butterflies over k (k^2, k^1), j & 1, L bit 4, L bit 3. 12 shuffles.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float row_tree_256(const float (&p)[2][4], int lane) {
    const bool l2 = lane & 4, l1 = lane & 2, l0 = lane & 1;
    float s[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {   // level L bit 2: keep j0 == l2
        const float send = l2 ? p[0][k] : p[1][k];
        const float keep = l2 ? p[1][k] : p[0][k];
        s[k] = __fadd_rn(keep, __shfl_xor_sync(kFullMask, send, 4));
    }
    float t[2];
#pragma unroll
    for (int m = 0; m < 2; ++m) {   // level L bit 1: keep k bit 1 == l1
        const float send = l1 ? s[m] : s[2 + m];
        const float keep = l1 ? s[2 + m] : s[m];
        t[m] = __fadd_rn(keep, __shfl_xor_sync(kFullMask, send, 2));
    }
    // level L bit 0: keep k bit 0 == l0
    float u = __fadd_rn(l0 ? t[1] : t[0], __shfl_xor_sync(kFullMask, l0 ? t[0] : t[1], 1));
    u = __fadd_rn(u, __shfl_xor_sync(kFullMask, u, 2));    // k ^ 2
    u = __fadd_rn(u, __shfl_xor_sync(kFullMask, u, 1));    // k ^ 1   -> reference warp sum
    u = __fadd_rn(u, __shfl_xor_sync(kFullMask, u, 4));    // reference warps w, w + 4
    u = __fadd_rn(u, __shfl_xor_sync(kFullMask, u, 16));   // w, w + 2
    u = __fadd_rn(u, __shfl_xor_sync(kFullMask, u, 8));    // w, w + 1
    return u;
}

// 1 / sqrt(total / COLS + eps) for a power-of-two COLS: dividing by 2^k is the same rounding as
// multiplying by 2^-k, and rcp.rn is the correctly rounded 1/x that div.rn(1, x) also returns, so this
// equals the reference expression bit for bit at a fraction of the instructions.
template <int COLS>
__device__ __forceinline__ float inv_rms_pow2(float total, float eps) {
    static_assert((COLS & (COLS - 1)) == 0, "COLS must be a power of two");
    return __frcp_rn(__fsqrt_rn(__fadd_rn(__fmul_rn(total, 1.0f / (float)COLS), eps)));
}

// Cold path of one RMSNorm block: recompute from global memory in natural order, literal quantiser.
static __device__ __noinline__ void rms_block_cold(const uint16_t* xblk, const float* wblk, float inv, float global_scale,
                                            uint2* packed_dst, uint8_t* scale_dst) {
    float a[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        a[i] = __uint_as_float((uint32_t)xblk[i] << 16) * inv * (1.0f + wblk[i]);
    }
    quantise16_cold_store(a, global_scale, packed_dst, scale_dst);
}

#ifndef CLEF_RMS_MIN_CTAS
#define CLEF_RMS_MIN_CTAS 2
#endif
// With ADD the row that is normalised is bf16(x + addend) (the residual add of kernels/head.cu:117-129 fused
// in front); that sum is also written to sum_out, which may be x itself. The sum is rounded to bf16 before
// the norm, so the result equals the add followed by the plain kernel on the stored residual. This variant
// loads at the top of each row instead of one row ahead (two inputs would not fit the register budget).
// With EMBED the row is row ids[row] of the table `x` (the embedding gather of kernels/elementwise.cu:396-407
// fused in front) and is also copied to sum_out (the residual stream the layer goes on with): the first layer's
// gather and norm + quantiser in one pass over the row.
template <int NB, bool ADD, bool EMBED = false>
__global__ void __launch_bounds__(kCtaThreads, (NB <= 4 ? CLEF_RMS_MIN_CTAS : 1))
rms_norm_quant_hot_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ addend, uint16_t* sum_out,
                          const float* __restrict__ weight, uint8_t* __restrict__ packed,
                          uint8_t* __restrict__ scales, int rows, int rows_total, float eps, float global_scale,
                          int blk_mn, int chunk, FastDiv atom_div, const int* __restrict__ ids) {
    static_assert(!(ADD && EMBED), "one fused producer at a time");
    constexpr int COLS = NB * 512;
    constexpr int BLOCKS = COLS / 16;
    __shared__ float s_inv[kInvScaleTableSize];
    const SfLayout sf = sf_layout_of(blk_mn, chunk);   // a negated chunk selects the interleaved tile order
    chunk = sf.chunk;
    // (1 + w) in the quad-pair layout, transposed so lane L reads s_w[(4 j + q) * 32 + L] =
    // (1+w_x, 1+w_z, 1+w_y, 1+w_w) of quad q of chunk L + 32 j.
    extern __shared__ float4 s_w[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;

    pdl_launch_dependents();
    fill_inv_scale_table(s_inv, global_scale);
    for (int idx = threadIdx.x; idx < COLS / 4; idx += kCtaThreads) {
        const int l = idx & 31, q = (idx >> 5) & 3, j = idx >> 7;
        const float4 w = *reinterpret_cast<const float4*>(weight + (l + 32 * j) * 16 + 4 * q);
        s_w[idx] = make_float4(1.0f + w.x, 1.0f + w.z, 1.0f + w.y, 1.0f + w.w);
    }
    int row = blockIdx.x * 8 + warp;
    if (!EMBED && row < rows) {   // this warp's first row towards L2 (a lane covers 128 bytes); see prefetch_l2
#pragma unroll
        for (int h = 0; h < NB / 4; ++h) {
            prefetch_l2(x + (size_t)row * COLS + (size_t)(lane + 32 * h) * 64);
            if (ADD) prefetch_l2(addend + (size_t)row * COLS + (size_t)(lane + 32 * h) * 64);
        }
    }
    pdl_wait_prior_grids();
    // (the token ids are an activation of the pass: they are read after the wait, so there is no early hint for EMBED)
    auto source_row = [&](int r) { return x + (size_t)(EMBED ? __ldg(ids + r) : r) * COLS; };
    // Tail balance (plain form): when the last round of rows would occupy at most half of the grid's warps, its rows
    // are handled by PAIRS of warps, half a row each (see the tail block below), so the round takes about half as long.
    // At 8,192 rows the grid's 2,368 warps run three full rounds and 1,088 rows are left: 9.45 -> 8.74 us.
    constexpr bool PAIR = true;   // every form: the plain one prefetches its half row, the fused producers load it in the tail block
    const int grid_warps = gridDim.x * 8;
    const int tail_base = (rows_total / grid_warps) * grid_warps;
    const bool pair_mode = PAIR && rows_total > tail_base && 2 * (rows_total - tail_base) <= grid_warps;
    const int main_end = pair_mode ? tail_base : rows_total;
    const int live_end = min(rows, main_end);
    const int tail_row = tail_base + ((blockIdx.x * 8 + warp) >> 1);   // pair mode: the row this warp shares with its neighbour
    const int half = warp & 1;
    U8x32 d[NB];
    auto fetch_tail_half = [&]() {   // this warp's half of its tail row: blocks half * NB / 2 + i
        if (tail_row < rows) {
#pragma unroll
            for (int i = 0; i < NB / 2; ++i) {
                d[i] = ldg_stream_v8(x + (size_t)tail_row * COLS + (size_t)(lane + 32 * (half * (NB / 2) + i)) * 16);
            }
        }
    };
    if (!ADD && row < live_end) {
        const uint16_t* src = source_row(row);
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            d[j] = ldg_stream_v8(src + (size_t)(lane + 32 * j) * 16);
        }
    } else if (!ADD && !EMBED && pair_mode && row >= main_end) {
        fetch_tail_half();
    }
    __syncthreads();

    for (; row < main_end; row += gridDim.x * 8) {
        uint8_t* prow = packed + (size_t)row * (COLS / 2);
        const uint32_t m_rest = fast_div((uint32_t)row, atom_div);
        const uint32_t m_atom = sf_row_slot((uint32_t)row - m_rest * (uint32_t)blk_mn, sf);
        uint8_t* srow = scales + (size_t)m_rest * (BLOCKS / 4) * (size_t)chunk + (size_t)m_atom * 4;
        if (row >= rows) {
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                const int b = lane + 32 * j;
                *reinterpret_cast<uint2*>(prow + b * 8) = make_uint2(0u, 0u);
                srow[(size_t)(b >> 2) * chunk + (b & 3)] = 0;
            }
            continue;
        }
        // EMBED: the next row's table row is known one row ahead, so that its loads can go out below.
        const int next = row + gridDim.x * 8;
        const uint16_t* next_src = (!ADD && next < live_end) ? source_row(next) : nullptr;
        // Unpack once; partial sums P[j & 1][k] in-lane over j (stride 2, ascending), as the reference thread does.
        f32x2 v[NB][8];
        float p[2][4];
#pragma unroll
        for (int j0 = 0; j0 < 2; ++j0) {
#pragma unroll
            for (int k = 0; k < 4; ++k) p[j0][k] = 0.0f;
        }
        U8x32 e[ADD ? NB : 1];
        if (ADD) {
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                d[j] = ldg_stream_v8(x + (size_t)row * COLS + (size_t)(lane + 32 * j) * 16);
                e[j] = ldg_stream_v8(addend + (size_t)row * COLS + (size_t)(lane + 32 * j) * 16);
            }
        }
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            float quad[4];
            if (EMBED) stg_v8(sum_out + (size_t)row * COLS + (size_t)(lane + 32 * j) * 16, d[j]);   // the gathered row
            unpack16_quadpairs(d[j], v[j]);
            if (ADD) {
                f32x2 t[8];
                unpack16_quadpairs(e[j], t);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    v[j][i] = f2_add(v[j][i], t[i]);
                }
                const U8x32 sum = pack16_bf16(v[j]);
                stg_v8(sum_out + (size_t)row * COLS + (size_t)(lane + 32 * j) * 16, sum);
                unpack16_quadpairs(sum, v[j]);
            }
            quad_squares(v[j], quad);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                p[j & 1][k] = __fadd_rn(p[j & 1][k], quad[k]);
            }
        }
        // The raw registers are free now: fetch this warp's next row while the current one is processed.
        if (!ADD && next < live_end) {
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                d[j] = ldg_stream_v8(next_src + (size_t)(lane + 32 * j) * 16);
            }
        } else if (!ADD && !EMBED && pair_mode && next >= main_end) {
            fetch_tail_half();
        }
        const float inv = (COLS & (COLS - 1)) == 0 ? inv_rms_pow2<COLS>(row_tree_256(p, lane), eps)
                                                   : inv_rms(row_tree_256(p, lane), COLS, eps);
        const f32x2 inv2 = f2_splat(inv);
        uint32_t bad = 0u;   // bit j: block j is outside the fast domain
#pragma unroll
        for (int j = 0; j < NB; ++j) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 w = s_w[(4 * j + q) * 32 + lane];
                v[j][2 * q] = f2_mul(f2_mul(v[j][2 * q], inv2), make_float2(w.x, w.y));
                v[j][2 * q + 1] = f2_mul(f2_mul(v[j][2 * q + 1], inv2), make_float2(w.z, w.w));
            }
            uint32_t stored, lo, hi;
            const bool ok = quantise16_qp<false>(v[j], global_scale, s_inv, stored, lo, hi);
            const int b = lane + 32 * j;
            *reinterpret_cast<uint2*>(prow + b * 8) = make_uint2(lo, hi);
            srow[(size_t)(b >> 2) * chunk + (b & 3)] = (uint8_t)stored;
            bad |= ok ? 0u : (1u << j);
        }
        if (bad) {   // rare: the literal path overwrites what the fast path stored
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                if (bad & (1u << j)) {
                    const int b = lane + 32 * j;
                    // ADD, EMBED: this lane stored the block's row above, so it reads its own bytes back.
                    rms_block_cold(((ADD || EMBED) ? (const uint16_t*)sum_out : x) + (size_t)row * COLS + b * 16, weight + b * 16, inv,
                                   global_scale, reinterpret_cast<uint2*>(prow + b * 8),
                                   srow + (size_t)(b >> 2) * chunk + (b & 3));
                }
            }
        }
    }
    if (PAIR && pair_mode && tail_row < rows_total) {
        // The tail round: warps 2i and 2i + 1 of a CTA share row tail_row, blocks half * NB / 2 + i each. The sums of
        // squares of a lane's quads cross through shared memory, after which both warps add all NB of them in the
        // order of the one-warp form (ascending j into P[j & 1][k]) and walk the same tree: the same bits.
        constexpr int HB = NB / 2;
        __shared__ float s_quads[4][2][HB * 4][32];
        uint8_t* prow = packed + (size_t)tail_row * (COLS / 2);
        const uint32_t m_rest = fast_div((uint32_t)tail_row, atom_div);
        const uint32_t m_atom = sf_row_slot((uint32_t)tail_row - m_rest * (uint32_t)blk_mn, sf);
        uint8_t* srow = scales + (size_t)m_rest * (BLOCKS / 4) * (size_t)chunk + (size_t)m_atom * 4;
        if (tail_row >= rows) {   // a pad row: both warps zero their halves
#pragma unroll
            for (int i = 0; i < HB; ++i) {
                const int b = lane + 32 * (half * HB + i);
                *reinterpret_cast<uint2*>(prow + b * 8) = make_uint2(0u, 0u);
                srow[(size_t)(b >> 2) * chunk + (b & 3)] = 0;
            }
        } else {
            f32x2 v[HB][8];
            float quad[HB][4];
            if (ADD || EMBED) {   // no row-ahead prefetch in these forms: this warp's half row is loaded here
                const uint16_t* src = source_row(tail_row);
#pragma unroll
                for (int i = 0; i < HB; ++i) d[i] = ldg_stream_v8(src + (size_t)(lane + 32 * (half * HB + i)) * 16);
            }
#pragma unroll
            for (int i = 0; i < HB; ++i) {
                const size_t off = (size_t)tail_row * COLS + (size_t)(lane + 32 * (half * HB + i)) * 16;
                if (EMBED) stg_v8(sum_out + off, d[i]);   // the gathered row
                unpack16_quadpairs(d[i], v[i]);
                if (ADD) {   // the stored (rounded) sum is what the norm sees, as in the main loop
                    f32x2 t[8];
                    unpack16_quadpairs(ldg_stream_v8(addend + off), t);
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[i][e] = f2_add(v[i][e], t[e]);
                    const U8x32 sum = pack16_bf16(v[i]);
                    stg_v8(sum_out + off, sum);
                    unpack16_quadpairs(sum, v[i]);
                }
                quad_squares(v[i], quad[i]);
#pragma unroll
                for (int k = 0; k < 4; ++k) s_quads[warp >> 1][half][i * 4 + k][lane] = quad[i][k];
            }
            switch (warp >> 1) {   // the two warps of the pair meet at a barrier of their own (a constant id each)
                case 0: asm volatile("bar.sync 1, 64;" ::: "memory"); break;
                case 1: asm volatile("bar.sync 2, 64;" ::: "memory"); break;
                case 2: asm volatile("bar.sync 3, 64;" ::: "memory"); break;
                default: asm volatile("bar.sync 4, 64;" ::: "memory"); break;
            }
            float p[2][4];
#pragma unroll
            for (int j0 = 0; j0 < 2; ++j0) {
#pragma unroll
                for (int k = 0; k < 4; ++k) p[j0][k] = 0.0f;
            }
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                const int i = j % HB;
                const bool mine = (j / HB) == half;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float other = s_quads[warp >> 1][half ^ 1][i * 4 + k][lane];
                    p[j & 1][k] = __fadd_rn(p[j & 1][k], mine ? quad[i][k] : other);
                }
            }
            const float inv = (COLS & (COLS - 1)) == 0 ? inv_rms_pow2<COLS>(row_tree_256(p, lane), eps)
                                                       : inv_rms(row_tree_256(p, lane), COLS, eps);
            const f32x2 inv2 = f2_splat(inv);
#pragma unroll
            for (int i = 0; i < HB; ++i) {
                const int j = half * HB + i;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float4 w = s_w[(4 * j + q) * 32 + lane];
                    v[i][2 * q] = f2_mul(f2_mul(v[i][2 * q], inv2), make_float2(w.x, w.y));
                    v[i][2 * q + 1] = f2_mul(f2_mul(v[i][2 * q + 1], inv2), make_float2(w.z, w.w));
                }
                uint32_t stored, lo, hi;
                const bool ok = quantise16_qp<false>(v[i], global_scale, s_inv, stored, lo, hi);
                const int b = lane + 32 * j;
                *reinterpret_cast<uint2*>(prow + b * 8) = make_uint2(lo, hi);
                srow[(size_t)(b >> 2) * chunk + (b & 3)] = (uint8_t)stored;
                if (!ok) {   // rare: the literal path overwrites what the fast path stored
                    // ADD, EMBED: this lane stored the block's row above, so it reads its own bytes back.
                    rms_block_cold(((ADD || EMBED) ? (const uint16_t*)sum_out : x) + (size_t)tail_row * COLS + b * 16, weight + b * 16,
                                   inv, global_scale, reinterpret_cast<uint2*>(prow + b * 8), srow + (size_t)(b >> 2) * chunk + (b & 3));
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// The same kernel for f32 activations (the reference engine's own residual-stream type), cols = NB * 512.
// A lane's 16-value block is 64 bytes (two 256-bit loads) and arrives as f32, so there is nothing to widen and the
// loaded registers ARE the row: pairs hold consecutive values (NATURAL), the sum of squares is scalar
// (fma(x, x, y * y) + fma(z, z, w * w), the reference's association; the quad-pair trick would cost the moves it saves),
// the summation tree is row_tree_256. Without raw registers to prefetch into, a row is loaded at the top of its
// iteration (as in the residual-add form) and the NEXT row is only named to L2 one row ahead.
// ---------------------------------------------------------------------------------------------
static __device__ __noinline__ void rms_block_cold_f32(const float* xblk, const float* wblk, float inv, float global_scale,
                                                       uint2* packed_dst, uint8_t* scale_dst) {
    float a[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        a[i] = xblk[i] * inv * (1.0f + wblk[i]);
    }
    quantise16_cold_store(a, global_scale, packed_dst, scale_dst);
}

// ADD and EMBED as in the bf16 kernel: the row is x + addend (f32 sum, also stored to sum_out, which may be x), or
// row ids[row] of the table x (also copied to sum_out).
template <int NB, bool ADD = false, bool EMBED = false>
__global__ void __launch_bounds__(kCtaThreads, (NB <= 4 ? 2 : 1))
rms_norm_quant_f32_hot_kernel(const float* __restrict__ x, const float* __restrict__ addend, float* sum_out,
                              const float* __restrict__ weight, uint8_t* __restrict__ packed,
                              uint8_t* __restrict__ scales, int rows, int rows_total, float eps, float global_scale,
                              int blk_mn, int chunk, FastDiv atom_div, const int* __restrict__ ids) {
    static_assert(!(ADD && EMBED), "one fused producer at a time");
    constexpr int COLS = NB * 512;
    constexpr int BLOCKS = COLS / 16;
    __shared__ float s_inv[kInvScaleTableSize];
    const SfLayout sf = sf_layout_of(blk_mn, chunk);   // a negated chunk selects the interleaved tile order
    chunk = sf.chunk;
    extern __shared__ float4 s_w[];   // (1 + w) of quad q of chunk L + 32 j at s_w[(4 j + q) * 32 + L], natural order
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;

    pdl_launch_dependents();
    fill_inv_scale_table(s_inv, global_scale);
    for (int idx = threadIdx.x; idx < COLS / 4; idx += kCtaThreads) {
        const int l = idx & 31, q = (idx >> 5) & 3, j = idx >> 7;
        const float4 w = *reinterpret_cast<const float4*>(weight + (l + 32 * j) * 16 + 4 * q);
        s_w[idx] = make_float4(1.0f + w.x, 1.0f + w.y, 1.0f + w.z, 1.0f + w.w);
    }
    int row = blockIdx.x * 8 + warp;
    // a row is COLS * 4 bytes = NB * 16 lines of 128 bytes: NB / 2 per lane
    auto name_row_to_l2 = [&](const float* src) {
#pragma unroll
        for (int h = 0; h < NB / 2; ++h) {
            prefetch_l2(src + (size_t)(lane + 32 * h) * 32);
        }
    };
    if (!EMBED && row < rows) {   // under the previous kernel's tail; see prefetch_l2
        name_row_to_l2(x + (size_t)row * COLS);
        if (ADD) name_row_to_l2(addend + (size_t)row * COLS);
    }
    pdl_wait_prior_grids();
    // (the token ids are an activation of the pass: they are read after the wait)
    auto source_row = [&](int r) { return x + (size_t)(EMBED ? __ldg(ids + r) : r) * COLS; };
    if (EMBED && row < rows) name_row_to_l2(source_row(row));
    // Tail balance as in the bf16 kernel: a last round for at most half of the grid's warps is shared by warp pairs.
    constexpr bool PAIR = !ADD && !EMBED;
    const int grid_warps = gridDim.x * 8;
    const int tail_base = (rows_total / grid_warps) * grid_warps;
    const bool pair_mode = PAIR && rows_total > tail_base && 2 * (rows_total - tail_base) <= grid_warps;
    const int main_end = pair_mode ? tail_base : rows_total;
    const int tail_row = tail_base + ((blockIdx.x * 8 + warp) >> 1);
    const int half_id = warp & 1;
    __syncthreads();

    for (; row < main_end; row += gridDim.x * 8) {
        uint8_t* prow = packed + (size_t)row * (COLS / 2);
        const uint32_t m_rest = fast_div((uint32_t)row, atom_div);
        const uint32_t m_atom = sf_row_slot((uint32_t)row - m_rest * (uint32_t)blk_mn, sf);
        uint8_t* srow = scales + (size_t)m_rest * (BLOCKS / 4) * (size_t)chunk + (size_t)m_atom * 4;
        if (row >= rows) {
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                const int b = lane + 32 * j;
                *reinterpret_cast<uint2*>(prow + b * 8) = make_uint2(0u, 0u);
                srow[(size_t)(b >> 2) * chunk + (b & 3)] = 0;
            }
            continue;
        }
        const float* xrow = source_row(row);
        U8x32 d[NB][2];
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            d[j][0] = ldg_stream_v8(xrow + (size_t)(lane + 32 * j) * 16);
            d[j][1] = ldg_stream_v8(xrow + (size_t)(lane + 32 * j) * 16 + 8);
        }
        const int next = row + gridDim.x * 8;
        if (next < min(rows, main_end)) {
            name_row_to_l2(source_row(next));
            if (ADD) name_row_to_l2(addend + (size_t)next * COLS);
        } else if (PAIR && pair_mode && next >= main_end && tail_row < rows) {
            // this warp's half of its tail row: NB / 2 blocks of 64 bytes per lane = NB * 8 lines, NB / 4 per lane
#pragma unroll
            for (int h = 0; h < NB / 4; ++h) {
                prefetch_l2(x + (size_t)tail_row * COLS + (size_t)half_id * (COLS / 2) + (size_t)(lane + 32 * h) * 32);
            }
        }
        if (ADD) {   // the addend arrives block by block, one block ahead of the sum
            const float* arow = addend + (size_t)row * COLS;
            float* srow_out = sum_out + (size_t)row * COLS;
            U8x32 e[2][2];
            e[0][0] = ldg_stream_v8(arow + (size_t)lane * 16);
            e[0][1] = ldg_stream_v8(arow + (size_t)lane * 16 + 8);
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                if (j + 1 < NB) {
                    e[(j + 1) & 1][0] = ldg_stream_v8(arow + (size_t)(lane + 32 * (j + 1)) * 16);
                    e[(j + 1) & 1][1] = ldg_stream_v8(arow + (size_t)(lane + 32 * (j + 1)) * 16 + 8);
                }
#pragma unroll
                for (int half = 0; half < 2; ++half) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        d[j][half].w[i] = __float_as_uint(__fadd_rn(__uint_as_float(d[j][half].w[i]), __uint_as_float(e[j & 1][half].w[i])));
                    }
                    stg_v8(srow_out + (size_t)(lane + 32 * j) * 16 + 8 * half, d[j][half]);
                }
            }
        }
        if (EMBED) {   // the gathered row, for the residual stream
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                stg_v8(sum_out + (size_t)row * COLS + (size_t)(lane + 32 * j) * 16, d[j][0]);
                stg_v8(sum_out + (size_t)row * COLS + (size_t)(lane + 32 * j) * 16 + 8, d[j][1]);
            }
        }
        f32x2 v[NB][8];
        float p[2][4];
#pragma unroll
        for (int a = 0; a < 2; ++a) {
#pragma unroll
            for (int k = 0; k < 4; ++k) p[a][k] = 0.0f;
        }
#pragma unroll
        for (int j = 0; j < NB; ++j) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {   // quad q = words 4q .. 4q + 3 of the block
                const U8x32& half = d[j][q >> 1];
                const int o = (q & 1) * 4;
                const float vx = __uint_as_float(half.w[o]), vy = __uint_as_float(half.w[o + 1]);
                const float vz = __uint_as_float(half.w[o + 2]), vw = __uint_as_float(half.w[o + 3]);
                v[j][2 * q] = f2_pack(vx, vy);
                v[j][2 * q + 1] = f2_pack(vz, vw);
                const float quad = __fadd_rn(__fmaf_rn(vx, vx, __fmul_rn(vy, vy)), __fmaf_rn(vz, vz, __fmul_rn(vw, vw)));
                p[j & 1][q] = __fadd_rn(p[j & 1][q], quad);
            }
        }
        const float inv = (COLS & (COLS - 1)) == 0 ? inv_rms_pow2<COLS>(row_tree_256(p, lane), eps)
                                                   : inv_rms(row_tree_256(p, lane), COLS, eps);
        const f32x2 inv2 = f2_splat(inv);
        uint32_t bad = 0u;   // bit j: block j is outside the fast domain
#pragma unroll
        for (int j = 0; j < NB; ++j) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 w = s_w[(4 * j + q) * 32 + lane];
                v[j][2 * q] = f2_mul(f2_mul(v[j][2 * q], inv2), make_float2(w.x, w.y));
                v[j][2 * q + 1] = f2_mul(f2_mul(v[j][2 * q + 1], inv2), make_float2(w.z, w.w));
            }
            uint32_t stored, lo, hi;
            const bool ok = quantise16_qp<false, true>(v[j], global_scale, s_inv, stored, lo, hi);
            const int b = lane + 32 * j;
            *reinterpret_cast<uint2*>(prow + b * 8) = make_uint2(lo, hi);
            srow[(size_t)(b >> 2) * chunk + (b & 3)] = (uint8_t)stored;
            bad |= ok ? 0u : (1u << j);
        }
        if (bad) {   // rare: the literal path overwrites what the fast path stored
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                if (bad & (1u << j)) {
                    const int b = lane + 32 * j;
                    // ADD: this lane stored the block's sum above, so it reads its own values back.
                    rms_block_cold_f32((ADD ? (const float*)sum_out + (size_t)row * COLS : xrow) + b * 16, weight + b * 16, inv, global_scale,
                                       reinterpret_cast<uint2*>(prow + b * 8), srow + (size_t)(b >> 2) * chunk + (b & 3));
                }
            }
        }
    }
    if (PAIR && pair_mode && tail_row < rows_total) {
        // The tail round, as in the bf16 kernel: two warps per row, the quads' sums of squares cross through shared
        // memory and are added in the one-warp order.
        constexpr int HB = NB / 2;
        __shared__ float s_quads[4][2][HB * 4][32];
        uint8_t* prow = packed + (size_t)tail_row * (COLS / 2);
        const uint32_t m_rest = fast_div((uint32_t)tail_row, atom_div);
        const uint32_t m_atom = sf_row_slot((uint32_t)tail_row - m_rest * (uint32_t)blk_mn, sf);
        uint8_t* srow = scales + (size_t)m_rest * (BLOCKS / 4) * (size_t)chunk + (size_t)m_atom * 4;
        if (tail_row >= rows) {   // a pad row: both warps zero their halves
#pragma unroll
            for (int i = 0; i < HB; ++i) {
                const int b = lane + 32 * (half_id * HB + i);
                *reinterpret_cast<uint2*>(prow + b * 8) = make_uint2(0u, 0u);
                srow[(size_t)(b >> 2) * chunk + (b & 3)] = 0;
            }
        } else {
            const float* xrow = x + (size_t)tail_row * COLS;
            U8x32 d[HB][2];
#pragma unroll
            for (int i = 0; i < HB; ++i) {
                d[i][0] = ldg_stream_v8(xrow + (size_t)(lane + 32 * (half_id * HB + i)) * 16);
                d[i][1] = ldg_stream_v8(xrow + (size_t)(lane + 32 * (half_id * HB + i)) * 16 + 8);
            }
            f32x2 v[HB][8];
            float quad[HB][4];
#pragma unroll
            for (int i = 0; i < HB; ++i) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const U8x32& hw = d[i][q >> 1];
                    const int o = (q & 1) * 4;
                    const float vx = __uint_as_float(hw.w[o]), vy = __uint_as_float(hw.w[o + 1]);
                    const float vz = __uint_as_float(hw.w[o + 2]), vw = __uint_as_float(hw.w[o + 3]);
                    v[i][2 * q] = f2_pack(vx, vy);
                    v[i][2 * q + 1] = f2_pack(vz, vw);
                    quad[i][q] = __fadd_rn(__fmaf_rn(vx, vx, __fmul_rn(vy, vy)), __fmaf_rn(vz, vz, __fmul_rn(vw, vw)));
                    s_quads[warp >> 1][half_id][i * 4 + q][lane] = quad[i][q];
                }
            }
            switch (warp >> 1) {   // the two warps of the pair meet at a barrier of their own (a constant id each)
                case 0: asm volatile("bar.sync 1, 64;" ::: "memory"); break;
                case 1: asm volatile("bar.sync 2, 64;" ::: "memory"); break;
                case 2: asm volatile("bar.sync 3, 64;" ::: "memory"); break;
                default: asm volatile("bar.sync 4, 64;" ::: "memory"); break;
            }
            float p[2][4];
#pragma unroll
            for (int a = 0; a < 2; ++a) {
#pragma unroll
                for (int k = 0; k < 4; ++k) p[a][k] = 0.0f;
            }
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                const int i = j % HB;
                const bool mine = (j / HB) == half_id;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float other = s_quads[warp >> 1][half_id ^ 1][i * 4 + k][lane];
                    p[j & 1][k] = __fadd_rn(p[j & 1][k], mine ? quad[i][k] : other);
                }
            }
            const float inv = (COLS & (COLS - 1)) == 0 ? inv_rms_pow2<COLS>(row_tree_256(p, lane), eps)
                                                       : inv_rms(row_tree_256(p, lane), COLS, eps);
            const f32x2 inv2 = f2_splat(inv);
#pragma unroll
            for (int i = 0; i < HB; ++i) {
                const int j = half_id * HB + i;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float4 w = s_w[(4 * j + q) * 32 + lane];
                    v[i][2 * q] = f2_mul(f2_mul(v[i][2 * q], inv2), make_float2(w.x, w.y));
                    v[i][2 * q + 1] = f2_mul(f2_mul(v[i][2 * q + 1], inv2), make_float2(w.z, w.w));
                }
                uint32_t stored, lo, hi;
                const bool ok = quantise16_qp<false, true>(v[i], global_scale, s_inv, stored, lo, hi);
                const int b = lane + 32 * j;
                *reinterpret_cast<uint2*>(prow + b * 8) = make_uint2(lo, hi);
                srow[(size_t)(b >> 2) * chunk + (b & 3)] = (uint8_t)stored;
                if (!ok) {   // rare: the literal path overwrites what the fast path stored
                    rms_block_cold_f32(xrow + b * 16, weight + b * 16, inv, global_scale, reinterpret_cast<uint2*>(prow + b * 8),
                                       srow + (size_t)(b >> 2) * chunk + (b & 3));
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// SwiGLU + NVFP4 quantiser (kernels/quantise.cu:523-591) for cols % 512 == 0.
// A warp handles "units" of 32 consecutive blocks (1 KiB of gate, 1 KiB of up); unit u covers
// elements [512 u, 512 u + 512) of the dense [rows, cols] matrices, so only the scale address needs
// the row. UNITS units are in flight per warp.
//
// silu(g) = g / (1 + __expf(-g)). For bf16 g with |g| <= 44 the block takes a short form:
//   e = ex2.approx(g * -log2(e))     the intrinsic's range fix-ups cannot trigger for |g| <= 44
//   d = 1 + e,  r = rcp.approx(d),  q0 = g * r,  rem = fma(-d, q0, g),  q = fma(rem, r, q0)
// and q equals div.rn.f32(g, d) for every such g (all 65536 bf16 patterns are compared on the device
// by the tests; -0.0 gives +0.0, which the quantiser cannot tell apart). Blocks holding a larger |g|,
// an infinity or a NaN take the literal expression.
// ---------------------------------------------------------------------------------------------
// (g0, g1) -> (silu(g0), silu(g1)) with the IEEE quotient, short form; domain above.
__device__ __forceinline__ f32x2 silu_ieee_fast_x2(f32x2 g2) {
    const f32x2 t2 = f2_mul(g2, f2_splat(kNegLog2e));
    const f32x2 d2 = f2_add(f2_splat(1.0f), make_float2(ex2_approx(t2.x), ex2_approx(t2.y)));
    const f32x2 r2 = make_float2(rcp_approx(d2.x), rcp_approx(d2.y));
    const f32x2 q0 = f2_mul(g2, r2);
    const f32x2 rem = f2_fma(make_float2(-d2.x, -d2.y), q0, g2);   // exact remainder
    return f2_fma(rem, r2, q0);
}

// silu for ANY f32 g with |g| <= 44 (accumulators, not bf16 values): the short form above misses div.rn by one ulp
// for two f32 patterns (0x3E609AF2, 0x3E24A9BF), so the reciprocal takes one Newton step first; after it the
// quotient equals div.rn for EVERY f32 g of the range (all patterns are compared on the device by the tests).
// The sign of g is copied onto the result: d > 0, so the exact quotient has the sign of g, and the short form
// loses the sign of a zero.
__device__ __forceinline__ f32x2 silu_ieee_refined_f32_x2(f32x2 g2) {
    // Steps with a constant or a negated operand stay scalar (immediates and operand negation are free there; a
    // packed operation would need the constant moved into a register pair); the others are packed.
    const float dx = __fadd_rn(1.0f, ex2_approx(__fmul_rn(g2.x, kNegLog2e)));
    const float dy = __fadd_rn(1.0f, ex2_approx(__fmul_rn(g2.y, kNegLog2e)));
    const float rx = rcp_approx(dx), ry = rcp_approx(dy);
    const f32x2 r0 = make_float2(rx, ry);
    const f32x2 r2 = f2_fma(make_float2(__fmaf_rn(-dx, rx, 1.0f), __fmaf_rn(-dy, ry, 1.0f)), r0, r0);
    const f32x2 q0 = f2_mul(g2, r2);
    const f32x2 q = f2_fma(make_float2(__fmaf_rn(-dx, q0.x, g2.x), __fmaf_rn(-dy, q0.y, g2.y)), r2, q0);
    return make_float2(__uint_as_float((__float_as_uint(q.x) & 0x7fffffffu) | (__float_as_uint(g2.x) & 0x80000000u)),
                       __uint_as_float((__float_as_uint(q.y) & 0x7fffffffu) | (__float_as_uint(g2.y) & 0x80000000u)));
}
template <int NP>
__device__ __forceinline__ bool silu_f32_magnitude_domain_x2(const f32x2* g) {
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < NP; ++i) m = max3_abs_nan(m, g[i].x, g[i].y);
    return m <= kSiluFastMaxAbs;   // false for a NaN
}
// (g0, g1) -> __fdividef(g, 1 + __expf(-g)) per lane, short form for |g| <= 44: g * rcp.approx(d).
__device__ __forceinline__ f32x2 silu_approx_fast_x2(f32x2 g2) {
    const f32x2 t2 = f2_mul(g2, f2_splat(kNegLog2e));
    const f32x2 d2 = f2_add(f2_splat(1.0f), make_float2(ex2_approx(t2.x), ex2_approx(t2.y)));
    return f2_mul(g2, make_float2(rcp_approx(d2.x), rcp_approx(d2.y)));
}

// (g, x) -> x / (1 + __expf(-g)) per lane with the IEEE quotient (kernels/elementwise.cu:344-353, the
// vector path), short form: the construction of silu_ieee_fast_x2 with numerator x. Domain: bf16 g
// with |g| <= 44 and bf16 x that is zero or has 2^-60 <= |x| < inf, which keeps the quotient and the
// remainder normal numbers (all such pairs are compared on the device by the tests).
constexpr float kSigmoidMulMinAbs = 8.67361738e-19f;   // 2^-60
__device__ __forceinline__ f32x2 sigmoid_mul_fast_x2(f32x2 g2, f32x2 x2) {
    const f32x2 t2 = f2_mul(g2, f2_splat(kNegLog2e));
    const f32x2 d2 = f2_add(f2_splat(1.0f), make_float2(ex2_approx(t2.x), ex2_approx(t2.y)));
    const f32x2 r2 = make_float2(rcp_approx(d2.x), rcp_approx(d2.y));
    const f32x2 q0 = f2_mul(x2, r2);
    const f32x2 rem = f2_fma(make_float2(-d2.x, -d2.y), q0, x2);
    return f2_fma(rem, r2, q0);
}

// max |g| over a block in the quad-pair layout, NaN if any value is NaN.
__device__ __forceinline__ float block_abs_max(const f32x2* g) {
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        m = max3_abs_nan(m, g[i].x, g[i].y);
    }
    return m;
}

__device__ __forceinline__ float block_abs_min(const f32x2* x) {
    float m = INFINITY;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        m = min3_abs(m, x[i].x, x[i].y);
    }
    return m;
}

// True if a block of 16 bf16 values holds a non-zero value of magnitude below kSigmoidMulMinAbs. Rarely
// evaluated, so it re-reads the block from global memory instead of tying up the caller's registers.
static __device__ __noinline__ bool block_has_tiny_nonzero(const uint16_t* xblk) {
    constexpr uint32_t kMinBits = 0x2180u;   // bf16 pattern of 2^-60
    bool bad = false;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const uint32_t m = xblk[i] & 0x7fffu;
        bad |= (m - 1u) < (kMinBits - 1u);
    }
    return bad;
}

// Whether a block may take the short form; xblk addresses the block's x values in global memory.
// FINITE_X: also require finite x (kernels whose result is not checked by the quantiser afterwards).
template <int ACT, bool FINITE_X>
__device__ __forceinline__ bool gated_fast_domain(const f32x2* g, const f32x2* x, const uint16_t* xblk) {
    bool ok = block_abs_max(g) <= kSiluFastMaxAbs;
    if (ACT == kActSigmoidMul) {
        if (FINITE_X) {
            ok = ok && block_abs_max(x) < INFINITY;
        }
        if (ok && block_abs_min(x) < kSigmoidMulMinAbs) {
            ok = !block_has_tiny_nonzero(xblk);
        }
    }
    return ok;
}

// g <- act(g, x) for a block inside the short form's domain.
template <int ACT>
__device__ __forceinline__ void gated_fast(f32x2* g, const f32x2* x) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        g[i] = ACT == kActSwiGLU ? f2_mul(silu_ieee_fast_x2(g[i]), x[i]) : sigmoid_mul_fast_x2(g[i], x[i]);
    }
}

template <int ACT>
__device__ __noinline__ void gated_act_block_cold(const uint16_t* gblk, const uint16_t* xblk, float global_scale,
                                                  uint2* packed_dst, uint8_t* scale_dst) {
    float a[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        a[i] = gated_literal<ACT>(__uint_as_float((uint32_t)gblk[i] << 16), __uint_as_float((uint32_t)xblk[i] << 16));
    }
    quantise16_cold_store(a, global_scale, packed_dst, scale_dst);
}

template <int UNITS, int MIN_CTAS, int ACT>
__global__ void __launch_bounds__(kCtaThreads, MIN_CTAS)
swiglu_quant_hot_kernel(const uint16_t* __restrict__ gate, const uint16_t* __restrict__ up,
                        uint8_t* __restrict__ packed, uint8_t* __restrict__ scales, uint32_t live_units,
                        uint32_t total_units, int cols, float global_scale, int blk_mn, int chunk, FastDiv seg_div,
                        FastDiv atom_div) {
    __shared__ float s_inv[kInvScaleTableSize];
    const SfLayout sf = sf_layout_of(blk_mn, chunk);   // a negated chunk selects the interleaved tile order
    chunk = sf.chunk;
    const int lane = threadIdx.x & 31;
    const uint32_t warps = gridDim.x * (kCtaThreads / 32);
    uint32_t unit0 = blockIdx.x * (kCtaThreads / 32) + (threadIdx.x >> 5);
    const int k1_count = cols >> 6;

    pdl_launch_dependents();
    fill_inv_scale_table(s_inv, global_scale);
    if (unit0 < live_units && lane < 16) {   // this warp's first unit towards L2 (8 lines of gate, 8 of up); see prefetch_l2
        prefetch_l2((lane < 8 ? gate : up) + (size_t)unit0 * 512 + (size_t)(lane & 7) * 64);
    }
    pdl_wait_prior_grids();
    U8x32 g[UNITS], u[UNITS];
#pragma unroll
    for (int k = 0; k < UNITS; ++k) {
        const uint32_t unit = unit0 + k * warps;
        if (unit < live_units) {
            g[k] = ldg_stream_v8(gate + (size_t)unit * 512 + lane * 16);
            u[k] = ldg_stream_v8(up + (size_t)unit * 512 + lane * 16);
        }
    }
    __syncthreads();

    for (; unit0 < total_units; unit0 += UNITS * warps) {
#pragma unroll
        for (int k = 0; k < UNITS; ++k) {
            const uint32_t unit = unit0 + k * warps;
            if (unit >= total_units) {
                break;
            }
            const uint32_t row = fast_div(unit, seg_div);
            const uint32_t block = (unit - row * seg_div.d) * 32 + lane;
            const uint32_t m_rest = fast_div(row, atom_div);
            const uint32_t m_atom = sf_row_slot(row - m_rest * (uint32_t)blk_mn, sf);
            uint8_t* sdst = scales + ((size_t)m_rest * k1_count + (block >> 2)) * (size_t)chunk + m_atom * 4 + (block & 3);
            uint2* pdst = reinterpret_cast<uint2*>(packed + (size_t)unit * 256 + lane * 8);
            if (unit >= live_units) {
                *pdst = make_uint2(0u, 0u);
                *sdst = 0;
                continue;
            }
            f32x2 gv[8], uv[8];
            unpack16_quadpairs(g[k], gv);
            unpack16_quadpairs(u[k], uv);
            // The raw registers of this slot are free: fetch the unit this slot handles next.
            const uint32_t next = unit + UNITS * warps;
            if (next < live_units) {
                g[k] = ldg_stream_v8(gate + (size_t)next * 512 + lane * 16);
                u[k] = ldg_stream_v8(up + (size_t)next * 512 + lane * 16);
            }
            // The short forms sit behind the domain test: measured faster here than running them unconditionally.
            uint32_t stored, lo, hi;
            bool ok = false;
            if (gated_fast_domain<ACT, false>(gv, uv, up + (size_t)unit * 512 + lane * 16)) {
                gated_fast<ACT>(gv, uv);
                ok = quantise16_qp<false>(gv, global_scale, s_inv, stored, lo, hi);
            }
            if (ok) {
                *pdst = make_uint2(lo, hi);
                *sdst = (uint8_t)stored;
            } else {
                gated_act_block_cold<ACT>(gate + (size_t)unit * 512 + lane * 16, up + (size_t)unit * 512 + lane * 16, global_scale,
                                  pdst, sdst);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Gated RMSNorm + NVFP4 quantiser for 128-wide heads (kernels/quantise.cu:57-121).
// Four lanes own one head row: lane m holds chunks m and m + 4 (quads 4m + k and 16 + 4m + k), a warp
// handles 8 head rows per step, and the next step's rows are fetched while the current ones are
// processed. Reference association: lane l of a warp holds quad l; tree 16,8,4,2,1 over l. Here the
// first level (l, l + 16) is in-lane; levels 8 and 4 (m bits 1, 0) are a reduce-scatter that keeps
// k bit 1, then k bit 0; levels 2 and 1 (k bits) are butterflies over lane bits 1 and 0. 5 shuffles.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float head_tree_32(const float* quad_a, const float* quad_b, int lane) {
    const bool m1 = lane & 2, m0 = lane & 1;
    float p[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        p[k] = __fadd_rn(quad_a[k], quad_b[k]);            // reference lanes l, l + 16
    }
    float s[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {                          // l, l + 8: keep k bit 1 == m1
        const float send = m1 ? p[i] : p[2 + i];
        const float keep = m1 ? p[2 + i] : p[i];
        s[i] = __fadd_rn(keep, __shfl_xor_sync(kFullMask, send, 2));
    }
    // l, l + 4: keep k bit 0 == m0
    float u = __fadd_rn(m0 ? s[1] : s[0], __shfl_xor_sync(kFullMask, m0 ? s[0] : s[1], 1));
    u = __fadd_rn(u, __shfl_xor_sync(kFullMask, u, 2));   // l, l + 2 (k bit 1 lives in lane bit 1 now)
    u = __fadd_rn(u, __shfl_xor_sync(kFullMask, u, 1));   // l, l + 1
    return u;
}

static __device__ __noinline__ void gated_block_cold(const uint16_t* xblk, const uint16_t* gblk, const float* wblk, float inv,
                                              float global_scale, uint2* packed_dst, uint8_t* scale_dst) {
    float a[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        a[i] = __uint_as_float((uint32_t)xblk[i] << 16) * inv * wblk[i] *
               silu_fast_div(__uint_as_float((uint32_t)gblk[i] << 16));
    }
    quantise16_cold_store(a, global_scale, packed_dst, scale_dst);
}

static __global__ void __launch_bounds__(kCtaThreads, 2)
gated_norm_quant_hot_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ gate,
                            const float* __restrict__ weight, uint8_t* __restrict__ packed,
                            uint8_t* __restrict__ scales, int rows_live, int rows_total, float eps,
                            float global_scale, int blk_mn, int chunk, int vh, FastDiv vh_div, FastDiv atom_div) {
    constexpr int COLS = 128;
    __shared__ float s_inv[kInvScaleTableSize];
    const SfLayout sf = sf_layout_of(blk_mn, chunk);   // a negated chunk selects the interleaved tile order
    chunk = sf.chunk;
    // plain weight in the quad-pair layout: s_w[(h * 4 + q) * 4 + m] = (w_x, w_z, w_y, w_w) of quad q of chunk m + 4h
    __shared__ float4 s_w[32];
    const int lane = threadIdx.x & 31;
    const int m = lane & 3;
    const int k1_count = (vh * (COLS / 16)) >> 2;

    // Head row handled by this lane group in step s: (global group index) + s * (groups in grid).
    const uint32_t groups_in_grid = gridDim.x * (kCtaThreads / 4);
    uint32_t hrow = blockIdx.x * (kCtaThreads / 4) + (threadIdx.x >> 2);

    pdl_launch_dependents();
    if (threadIdx.x < 32) {
        const int mm = threadIdx.x & 3, q = (threadIdx.x >> 2) & 3, h = threadIdx.x >> 4;
        const float4 t = *reinterpret_cast<const float4*>(weight + (mm + 4 * h) * 16 + 4 * q);
        s_w[threadIdx.x] = make_float4(t.x, t.z, t.y, t.w);
    }
    fill_inv_scale_table(s_inv, global_scale);
    {   // the CTA's first 64 head rows towards L2: 128 lines of x, 128 of gate; see prefetch_l2
        const uint32_t first = blockIdx.x * (kCtaThreads / 4);
        const uint32_t line = threadIdx.x & 127;   // 2 lines per head row
        if (first + (line >> 1) < (uint32_t)rows_live) {
            prefetch_l2((threadIdx.x < 128 ? x : gate) + (size_t)first * COLS + (size_t)line * 64);
        }
    }
    pdl_wait_prior_grids();
    U8x32 dx[2], dg[2];
    if (hrow < (uint32_t)rows_live) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            dx[h] = ldg_stream_v8(x + (size_t)hrow * COLS + (m + 4 * h) * 16);
            dg[h] = ldg_stream_v8(gate + (size_t)hrow * COLS + (m + 4 * h) * 16);
        }
    }
    __syncthreads();

    // Every lane of a warp runs the same number of steps (the shuffles need the full warp).
    for (uint32_t base = hrow - (uint32_t)(lane >> 2); base < (uint32_t)rows_total; base += groups_in_grid, hrow += groups_in_grid) {
        const bool in_range = hrow < (uint32_t)rows_total;
        const bool live = hrow < (uint32_t)rows_live;
        f32x2 v[2][8], gv[2][8];
        float quad[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        if (live) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                unpack16_quadpairs(dx[h], v[h]);
                unpack16_quadpairs(dg[h], gv[h]);
                quad_squares(v[h], quad[h]);
            }
        }
        const uint32_t next = hrow + groups_in_grid;
        if (next < (uint32_t)rows_live) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                dx[h] = ldg_stream_v8(x + (size_t)next * COLS + (m + 4 * h) * 16);
                dg[h] = ldg_stream_v8(gate + (size_t)next * COLS + (m + 4 * h) * 16);
            }
        }
        const float total = head_tree_32(quad[0], quad[1], lane);
        if (!in_range) {
            continue;
        }
        const uint32_t token = fast_div(hrow, vh_div);
        const uint32_t head_block = (hrow - token * (uint32_t)vh) * (COLS / 16);
        const uint32_t m_rest = fast_div(token, atom_div);
        const uint32_t m_atom = sf_row_slot(token - m_rest * (uint32_t)blk_mn, sf);
        const float inv = inv_rms_pow2<COLS>(total, eps);
        const f32x2 inv2 = f2_splat(inv);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t block = head_block + m + 4 * h;
            uint2* pdst = reinterpret_cast<uint2*>(packed + (size_t)hrow * (COLS / 2) + (m + 4 * h) * 8);
            uint8_t* sdst = scales + ((size_t)m_rest * k1_count + (block >> 2)) * (size_t)chunk + m_atom * 4 + (block & 3);
            if (!live) {
                *pdst = make_uint2(0u, 0u);
                *sdst = 0;
                continue;
            }
            uint32_t stored, lo, hi;
            const bool in_domain = block_abs_max(gv[h]) <= kSiluFastMaxAbs;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 w = s_w[(h * 4 + q) * 4 + m];
                // ((x * inv) * w) * silu(g), left to right as the reference writes it
                v[h][2 * q] = f2_mul(f2_mul(f2_mul(v[h][2 * q], inv2), make_float2(w.x, w.y)), silu_approx_fast_x2(gv[h][2 * q]));
                v[h][2 * q + 1] = f2_mul(f2_mul(f2_mul(v[h][2 * q + 1], inv2), make_float2(w.z, w.w)), silu_approx_fast_x2(gv[h][2 * q + 1]));
            }
            const bool done = quantise16_qp<false>(v[h], global_scale, s_inv, stored, lo, hi) && in_domain;
            if (done) {
                *pdst = make_uint2(lo, hi);
                *sdst = (uint8_t)stored;
            } else {
                const size_t off = (size_t)hrow * COLS + (m + 4 * h) * 16;
                gated_block_cold(x + off, gate + off, weight + (m + 4 * h) * 16, inv, global_scale, pdst, sdst);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// The same kernel for f32 activations (the reference engine's own type): a lane's two chunks of x and of the gate
// are 64 bytes each and arrive as f32, pairs hold consecutive values (NATURAL), the sum of squares is scalar, the
// tree is head_tree_32; rows are loaded at the top of a step and the next step's rows are only named to L2.
// silu_approx_fast_x2 equals __fdividef(g, 1 + __expf(-g)) for every f32 |g| <= 44 (all patterns are compared on
// the device by the tests), so the short form serves f32 gates as it serves bf16 ones.
// ---------------------------------------------------------------------------------------------
static __device__ __noinline__ void gated_block_cold_f32(const float* xblk, const float* gblk, const float* wblk, float inv,
                                                         float global_scale, uint2* packed_dst, uint8_t* scale_dst) {
    float a[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        a[i] = xblk[i] * inv * wblk[i] * silu_fast_div(gblk[i]);
    }
    quantise16_cold_store(a, global_scale, packed_dst, scale_dst);
}

static __global__ void __launch_bounds__(kCtaThreads, 2)
gated_norm_quant_f32_hot_kernel(const float* __restrict__ x, const float* __restrict__ gate, const float* __restrict__ weight,
                                uint8_t* __restrict__ packed, uint8_t* __restrict__ scales, int rows_live, int rows_total,
                                float eps, float global_scale, int blk_mn, int chunk, int vh, FastDiv vh_div, FastDiv atom_div) {
    constexpr int COLS = 128;
    __shared__ float s_inv[kInvScaleTableSize];
    const SfLayout sf = sf_layout_of(blk_mn, chunk);   // a negated chunk selects the interleaved tile order
    chunk = sf.chunk;
    __shared__ float4 s_w[32];   // plain weight, natural order: s_w[(h * 4 + q) * 4 + m] = quad q of chunk m + 4h
    const int lane = threadIdx.x & 31;
    const int m = lane & 3;
    const int k1_count = (vh * (COLS / 16)) >> 2;
    const uint32_t groups_in_grid = gridDim.x * (kCtaThreads / 4);
    uint32_t hrow = blockIdx.x * (kCtaThreads / 4) + (threadIdx.x >> 2);

    pdl_launch_dependents();
    if (threadIdx.x < 32) {
        const int mm = threadIdx.x & 3, q = (threadIdx.x >> 2) & 3, h = threadIdx.x >> 4;
        s_w[threadIdx.x] = *reinterpret_cast<const float4*>(weight + (mm + 4 * h) * 16 + 4 * q);
    }
    fill_inv_scale_table(s_inv, global_scale);
    // a CTA step covers 64 head rows of 512 bytes: 256 lines of x and 256 of the gate, two of each per thread
    auto name_step_to_l2 = [&](uint32_t first) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t line = threadIdx.x + 256 * h;   // 4 lines per head row
            if (first + (line >> 2) < (uint32_t)rows_live) {
                prefetch_l2(x + (size_t)first * COLS + (size_t)line * 32);
                prefetch_l2(gate + (size_t)first * COLS + (size_t)line * 32);
            }
        }
    };
    name_step_to_l2(blockIdx.x * (kCtaThreads / 4));   // under the previous kernel's tail; see prefetch_l2
    pdl_wait_prior_grids();
    __syncthreads();

    // Every lane of a warp runs the same number of steps (the shuffles need the full warp).
    uint32_t cta_first = blockIdx.x * (kCtaThreads / 4);
    for (uint32_t base = hrow - (uint32_t)(lane >> 2); base < (uint32_t)rows_total;
         base += groups_in_grid, hrow += groups_in_grid, cta_first += groups_in_grid) {
        const bool in_range = hrow < (uint32_t)rows_total;
        const bool live = hrow < (uint32_t)rows_live;
        U8x32 dx[2][2], dg[2][2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
#pragma unroll
                for (int i = 0; i < 8; ++i) dx[h][half].w[i] = dg[h][half].w[i] = 0u;
            }
        }
        if (live) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const size_t off = (size_t)hrow * COLS + (m + 4 * h) * 16;
                dx[h][0] = ldg_stream_v8(x + off);
                dx[h][1] = ldg_stream_v8(x + off + 8);
                dg[h][0] = ldg_stream_v8(gate + off);
                dg[h][1] = ldg_stream_v8(gate + off + 8);
            }
        }
        if (cta_first + groups_in_grid < (uint32_t)rows_live) name_step_to_l2(cta_first + groups_in_grid);
        f32x2 v[2][8], gv[2][8];
        float quad[2][4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const U8x32& hx = dx[h][q >> 1];
                const U8x32& hg = dg[h][q >> 1];
                const int o = (q & 1) * 4;
                const float vx = __uint_as_float(hx.w[o]), vy = __uint_as_float(hx.w[o + 1]);
                const float vz = __uint_as_float(hx.w[o + 2]), vw = __uint_as_float(hx.w[o + 3]);
                v[h][2 * q] = f2_pack(vx, vy);
                v[h][2 * q + 1] = f2_pack(vz, vw);
                gv[h][2 * q] = f2_pack(__uint_as_float(hg.w[o]), __uint_as_float(hg.w[o + 1]));
                gv[h][2 * q + 1] = f2_pack(__uint_as_float(hg.w[o + 2]), __uint_as_float(hg.w[o + 3]));
                quad[h][q] = __fadd_rn(__fmaf_rn(vx, vx, __fmul_rn(vy, vy)), __fmaf_rn(vz, vz, __fmul_rn(vw, vw)));
            }
        }
        const float total = head_tree_32(quad[0], quad[1], lane);
        if (!in_range) {
            continue;
        }
        const uint32_t token = fast_div(hrow, vh_div);
        const uint32_t head_block = (hrow - token * (uint32_t)vh) * (COLS / 16);
        const uint32_t m_rest = fast_div(token, atom_div);
        const uint32_t m_atom = sf_row_slot(token - m_rest * (uint32_t)blk_mn, sf);
        const float inv = inv_rms_pow2<COLS>(total, eps);
        const f32x2 inv2 = f2_splat(inv);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t block = head_block + m + 4 * h;
            uint2* pdst = reinterpret_cast<uint2*>(packed + (size_t)hrow * (COLS / 2) + (m + 4 * h) * 8);
            uint8_t* sdst = scales + ((size_t)m_rest * k1_count + (block >> 2)) * (size_t)chunk + m_atom * 4 + (block & 3);
            if (!live) {
                *pdst = make_uint2(0u, 0u);
                *sdst = 0;
                continue;
            }
            uint32_t stored, lo, hi;
            const bool in_domain = block_abs_max(gv[h]) <= kSiluFastMaxAbs;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 w = s_w[(h * 4 + q) * 4 + m];
                // ((x * inv) * w) * silu(g), left to right as the reference writes it
                v[h][2 * q] = f2_mul(f2_mul(f2_mul(v[h][2 * q], inv2), make_float2(w.x, w.y)), silu_approx_fast_x2(gv[h][2 * q]));
                v[h][2 * q + 1] = f2_mul(f2_mul(f2_mul(v[h][2 * q + 1], inv2), make_float2(w.z, w.w)), silu_approx_fast_x2(gv[h][2 * q + 1]));
            }
            const bool done = quantise16_qp<false, true>(v[h], global_scale, s_inv, stored, lo, hi) && in_domain;
            if (done) {
                *pdst = make_uint2(lo, hi);
                *sdst = (uint8_t)stored;
            } else {
                const size_t off = (size_t)hrow * COLS + (m + 4 * h) * 16;
                gated_block_cold_f32(x + off, gate + off, weight + (m + 4 * h) * 16, inv, global_scale, pdst, sdst);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Plain NVFP4 quantiser (kernels/quantise.cu:6-53) for cols % 512 == 0: the SwiGLU kernel's unit
// structure with one input.
// ---------------------------------------------------------------------------------------------
static __device__ __noinline__ void quantise_block_cold(const uint16_t* xblk, float global_scale, uint2* packed_dst,
                                                 uint8_t* scale_dst) {
    float a[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        a[i] = __uint_as_float((uint32_t)xblk[i] << 16);
    }
    quantise16_cold_store(a, global_scale, packed_dst, scale_dst);
}

template <int UNITS>
__global__ void __launch_bounds__(kCtaThreads, 4)
quantise_hot_kernel(const uint16_t* __restrict__ x, uint8_t* __restrict__ packed, uint8_t* __restrict__ scales,
                    uint32_t live_units, uint32_t total_units, int cols, float global_scale, int blk_mn, int chunk,
                    FastDiv seg_div, FastDiv atom_div) {
    __shared__ float s_inv[kInvScaleTableSize];
    const SfLayout sf = sf_layout_of(blk_mn, chunk);   // a negated chunk selects the interleaved tile order
    chunk = sf.chunk;
    const int lane = threadIdx.x & 31;
    const uint32_t warps = gridDim.x * (kCtaThreads / 32);
    uint32_t unit0 = blockIdx.x * (kCtaThreads / 32) + (threadIdx.x >> 5);
    const int k1_count = cols >> 6;
    pdl_launch_dependents();
    fill_inv_scale_table(s_inv, global_scale);
    if (unit0 < live_units && lane < 8) {   // this warp's first unit towards L2 (8 lines); see prefetch_l2
        prefetch_l2(x + (size_t)unit0 * 512 + (size_t)lane * 64);
    }
    pdl_wait_prior_grids();
    U8x32 d[UNITS];
#pragma unroll
    for (int k = 0; k < UNITS; ++k) {
        const uint32_t unit = unit0 + k * warps;
        if (unit < live_units) {
            d[k] = ldg_stream_v8(x + (size_t)unit * 512 + lane * 16);
        }
    }
    __syncthreads();
    for (; unit0 < total_units; unit0 += UNITS * warps) {
#pragma unroll
        for (int k = 0; k < UNITS; ++k) {
            const uint32_t unit = unit0 + k * warps;
            if (unit >= total_units) {
                break;
            }
            const uint32_t row = fast_div(unit, seg_div);
            const uint32_t block = (unit - row * seg_div.d) * 32 + lane;
            const uint32_t m_rest = fast_div(row, atom_div);
            const uint32_t m_atom = sf_row_slot(row - m_rest * (uint32_t)blk_mn, sf);
            uint8_t* sdst = scales + ((size_t)m_rest * k1_count + (block >> 2)) * (size_t)chunk + m_atom * 4 + (block & 3);
            uint2* pdst = reinterpret_cast<uint2*>(packed + (size_t)unit * 256 + lane * 8);
            if (unit >= live_units) {
                *pdst = make_uint2(0u, 0u);
                *sdst = 0;
                continue;
            }
            f32x2 v[8];
            unpack16_quadpairs(d[k], v);
            const uint32_t next = unit + UNITS * warps;
            if (next < live_units) {
                d[k] = ldg_stream_v8(x + (size_t)next * 512 + lane * 16);
            }
            uint32_t stored, lo, hi;
            const bool ok = quantise16_qp<false>(v, global_scale, s_inv, stored, lo, hi);
            *pdst = make_uint2(lo, hi);
            *sdst = (uint8_t)stored;
            if (!ok) {   // rare: the literal path overwrites what the fast path stored
                quantise_block_cold(x + (size_t)unit * 512 + lane * 16, global_scale, pdst, sdst);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// The unit-structured quantisers for f32 activations: a lane owns one block of 16 f32 values (two
// 32-byte loads), values stay in natural pair order, and the unit a warp handles next is named to L2
// while the current one is processed (no raw registers are held across units: the values alone take
// 32 registers per input).
// MODE 0: plain quantiser (kernels/quantise.cu:6-53). MODE 1: SwiGLU first (kernels/quantise.cu:523-591),
// silu through silu_ieee_refined_f32_x2, which equals the IEEE quotient for every f32 gate of |g| <= 44.
// MODE 2: x * sigmoid(gate) first (kernels/elementwise.cu:344-353), `gate` the gate and `up` the x rows; the
// quotient has two free f32 operands, so it is the literal IEEE division (the kernel stays memory-bound with it).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void load16_f32_natural(const float* p, f32x2* v) {
    const U8x32 a = ldg_stream_v8(p), b = ldg_stream_v8(p + 8);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[i] = f2_pack(__uint_as_float(a.w[2 * i]), __uint_as_float(a.w[2 * i + 1]));
        v[4 + i] = f2_pack(__uint_as_float(b.w[2 * i]), __uint_as_float(b.w[2 * i + 1]));
    }
}

template <int MODE>
static __device__ __noinline__ void unit_block_cold_f32(const float* gblk, const float* xblk, float global_scale,
                                                        uint2* packed_dst, uint8_t* scale_dst) {
    float a[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        a[i] = MODE == 1 ? gated_literal<kActSwiGLU>(gblk[i], xblk[i])
                         : (MODE == 2 ? gated_literal<kActSigmoidMul>(gblk[i], xblk[i]) : gblk[i]);
    }
    quantise16_cold_store(a, global_scale, packed_dst, scale_dst);
}

template <int MODE, int MIN_CTAS>
__global__ void __launch_bounds__(kCtaThreads, MIN_CTAS)
unit_quant_f32_hot_kernel(const float* __restrict__ gate, const float* __restrict__ up, uint8_t* __restrict__ packed,
                          uint8_t* __restrict__ scales, uint32_t live_units, uint32_t total_units, int cols,
                          float global_scale, int blk_mn, int chunk, FastDiv seg_div, FastDiv atom_div) {
    __shared__ float s_inv[kInvScaleTableSize];
    const SfLayout sf = sf_layout_of(blk_mn, chunk);   // a negated chunk selects the interleaved tile order
    chunk = sf.chunk;
    const int lane = threadIdx.x & 31;
    const uint32_t warps = gridDim.x * (kCtaThreads / 32);
    uint32_t unit = blockIdx.x * (kCtaThreads / 32) + (threadIdx.x >> 5);
    const int k1_count = cols >> 6;
    // a unit is 2 KiB per input = 16 lines of 128 bytes: lanes 0-15 name the gate's, lanes 16-31 the up's
    auto name_unit_to_l2 = [&](uint32_t u) {
        if (MODE != 0) {
            prefetch_l2((lane < 16 ? gate : up) + (size_t)u * 512 + (size_t)(lane & 15) * 32);
        } else if (lane < 16) {
            prefetch_l2(gate + (size_t)u * 512 + (size_t)lane * 32);
        }
    };
    pdl_launch_dependents();
    fill_inv_scale_table(s_inv, global_scale);
    if (unit < live_units) name_unit_to_l2(unit);   // under the previous kernel's tail; see prefetch_l2
    pdl_wait_prior_grids();
    __syncthreads();

    for (; unit < total_units; unit += warps) {
        const uint32_t row = fast_div(unit, seg_div);
        const uint32_t block = (unit - row * seg_div.d) * 32 + lane;
        const uint32_t m_rest = fast_div(row, atom_div);
        const uint32_t m_atom = sf_row_slot(row - m_rest * (uint32_t)blk_mn, sf);
        uint8_t* sdst = scales + ((size_t)m_rest * k1_count + (block >> 2)) * (size_t)chunk + m_atom * 4 + (block & 3);
        uint2* pdst = reinterpret_cast<uint2*>(packed + (size_t)unit * 256 + lane * 8);
        if (unit >= live_units) {
            *pdst = make_uint2(0u, 0u);
            *sdst = 0;
            continue;
        }
        const float* gblk = gate + (size_t)unit * 512 + lane * 16;
        const float* ublk = MODE != 0 ? up + (size_t)unit * 512 + lane * 16 : nullptr;
        f32x2 gv[8], uv[8];
        load16_f32_natural(gblk, gv);
        if (MODE != 0) load16_f32_natural(ublk, uv);
        const uint32_t next = unit + warps;
        if (next < live_units) name_unit_to_l2(next);
        uint32_t stored, lo, hi;
        bool ok = true;
        if (MODE == 1) {
            ok = block_abs_max(gv) <= kSiluFastMaxAbs;   // false for a NaN
            if (ok) {
#pragma unroll
                for (int i = 0; i < 8; ++i) gv[i] = f2_mul(silu_ieee_refined_f32_x2(gv[i]), uv[i]);
            }
        }
        if (MODE == 2) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                gv[i] = make_float2(gated_literal<kActSigmoidMul>(gv[i].x, uv[i].x), gated_literal<kActSigmoidMul>(gv[i].y, uv[i].y));
            }
        }
        if (ok) ok = quantise16_qp<false, true>(gv, global_scale, s_inv, stored, lo, hi);
        if (ok) {
            *pdst = make_uint2(lo, hi);
            *sdst = (uint8_t)stored;
        } else {
            unit_block_cold_f32<MODE>(gblk, ublk, global_scale, pdst, sdst);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// RMSNorm with bf16 output (kernels/elementwise.cu:4-68), cols = NB * 512: the quantising kernel's
// row structure and summation tree, the normalised row rounded to bf16 instead of quantised, so the
// result is the reference's f32 result rounded to nearest even.
// ---------------------------------------------------------------------------------------------
template <int NB>
__global__ void __launch_bounds__(kCtaThreads, (NB <= 4 ? 2 : 1))
rms_norm_hot_kernel(const uint16_t* __restrict__ x, const float* __restrict__ weight, uint16_t* __restrict__ out,
                    int rows, float eps) {
    constexpr int COLS = NB * 512;
    extern __shared__ float4 s_w[];   // (1 + w) or 1, quad-pair layout, transposed (see the quantising kernel)
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    pdl_launch_dependents();
    for (int idx = threadIdx.x; idx < COLS / 4; idx += kCtaThreads) {
        const int l = idx & 31, q = (idx >> 5) & 3, j = idx >> 7;
        float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
        if (weight) {
            w = *reinterpret_cast<const float4*>(weight + (l + 32 * j) * 16 + 4 * q);
        }
        s_w[idx] = make_float4(1.0f + w.x, 1.0f + w.z, 1.0f + w.y, 1.0f + w.w);
    }
    int row = blockIdx.x * 8 + warp;
    if (row < rows) {   // this warp's first row towards L2; see prefetch_l2
#pragma unroll
        for (int h = 0; h < NB / 4; ++h) {
            prefetch_l2(x + (size_t)row * COLS + (size_t)(lane + 32 * h) * 64);
        }
    }
    pdl_wait_prior_grids();
    U8x32 d[NB];
    if (row < rows) {
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            d[j] = ldg_stream_v8(x + (size_t)row * COLS + (size_t)(lane + 32 * j) * 16);
        }
    }
    __syncthreads();
    for (; row < rows; row += gridDim.x * 8) {
        f32x2 v[NB][8];
        float p[2][4];
#pragma unroll
        for (int j0 = 0; j0 < 2; ++j0) {
#pragma unroll
            for (int k = 0; k < 4; ++k) p[j0][k] = 0.0f;
        }
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            float quad[4];
            unpack16_quadpairs(d[j], v[j]);
            quad_squares(v[j], quad);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                p[j & 1][k] = __fadd_rn(p[j & 1][k], quad[k]);
            }
        }
        const int next = row + gridDim.x * 8;
        if (next < rows) {
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                d[j] = ldg_stream_v8(x + (size_t)next * COLS + (size_t)(lane + 32 * j) * 16);
            }
        }
        const f32x2 inv2 = f2_splat(inv_rms_pow2<COLS>(row_tree_256(p, lane), eps));
        uint16_t* orow = out + (size_t)row * COLS;
#pragma unroll
        for (int j = 0; j < NB; ++j) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                if (weight) {   // without a weight the reference computes x * inv only (no multiply by 1)
                    const float4 w = s_w[(4 * j + q) * 32 + lane];
                    v[j][2 * q] = f2_mul(f2_mul(v[j][2 * q], inv2), make_float2(w.x, w.y));
                    v[j][2 * q + 1] = f2_mul(f2_mul(v[j][2 * q + 1], inv2), make_float2(w.z, w.w));
                } else {
                    v[j][2 * q] = f2_mul(v[j][2 * q], inv2);
                    v[j][2 * q + 1] = f2_mul(v[j][2 * q + 1], inv2);
                }
            }
            stg_v8(orow + (size_t)(lane + 32 * j) * 16, pack16_bf16(v[j]));
        }
    }
}

// The same for f32 activations (the reference's own arithmetic type, so the result is the reference's bit for bit):
// the f32 quantising kernel's row structure (natural pair order, loads at the top of a row, the next row named to
// L2), the normalised row stored as f32.
template <int NB>
__global__ void __launch_bounds__(kCtaThreads, (NB <= 4 ? 2 : 1))
rms_norm_f32_hot_kernel(const float* __restrict__ x, const float* __restrict__ weight, float* __restrict__ out, int rows,
                        float eps) {
    constexpr int COLS = NB * 512;
    extern __shared__ float4 s_w[];   // (1 + w) of quad q of chunk L + 32 j at s_w[(4 j + q) * 32 + L], natural order
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    pdl_launch_dependents();
    if (weight) {
        for (int idx = threadIdx.x; idx < COLS / 4; idx += kCtaThreads) {
            const int l = idx & 31, q = (idx >> 5) & 3, j = idx >> 7;
            const float4 w = *reinterpret_cast<const float4*>(weight + (l + 32 * j) * 16 + 4 * q);
            s_w[idx] = make_float4(1.0f + w.x, 1.0f + w.y, 1.0f + w.z, 1.0f + w.w);
        }
    }
    int row = blockIdx.x * 8 + warp;
    auto name_row_to_l2 = [&](int r) {   // a row is NB * 16 lines of 128 bytes: NB / 2 per lane
#pragma unroll
        for (int h = 0; h < NB / 2; ++h) {
            prefetch_l2(x + (size_t)r * COLS + (size_t)(lane + 32 * h) * 32);
        }
    };
    if (row < rows) name_row_to_l2(row);   // under the previous kernel's tail; see prefetch_l2
    pdl_wait_prior_grids();
    __syncthreads();
    for (; row < rows; row += gridDim.x * 8) {
        const float* xrow = x + (size_t)row * COLS;
        U8x32 d[NB][2];
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            d[j][0] = ldg_stream_v8(xrow + (size_t)(lane + 32 * j) * 16);
            d[j][1] = ldg_stream_v8(xrow + (size_t)(lane + 32 * j) * 16 + 8);
        }
        const int next = row + gridDim.x * 8;
        if (next < rows) name_row_to_l2(next);
        float p[2][4];
#pragma unroll
        for (int a = 0; a < 2; ++a) {
#pragma unroll
            for (int k = 0; k < 4; ++k) p[a][k] = 0.0f;
        }
#pragma unroll
        for (int j = 0; j < NB; ++j) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const U8x32& half = d[j][q >> 1];
                const int o = (q & 1) * 4;
                const float vx = __uint_as_float(half.w[o]), vy = __uint_as_float(half.w[o + 1]);
                const float vz = __uint_as_float(half.w[o + 2]), vw = __uint_as_float(half.w[o + 3]);
                const float quad = __fadd_rn(__fmaf_rn(vx, vx, __fmul_rn(vy, vy)), __fmaf_rn(vz, vz, __fmul_rn(vw, vw)));
                p[j & 1][q] = __fadd_rn(p[j & 1][q], quad);
            }
        }
        const f32x2 inv2 = f2_splat(inv_rms_pow2<COLS>(row_tree_256(p, lane), eps));
        float* orow = out + (size_t)row * COLS;
#pragma unroll
        for (int j = 0; j < NB; ++j) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                U8x32 o;
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int q = 2 * half + e;
                    f32x2 a = f2_mul(f2_pack(__uint_as_float(d[j][half].w[4 * e]), __uint_as_float(d[j][half].w[4 * e + 1])), inv2);
                    f32x2 b = f2_mul(f2_pack(__uint_as_float(d[j][half].w[4 * e + 2]), __uint_as_float(d[j][half].w[4 * e + 3])), inv2);
                    if (weight) {   // without a weight the reference computes x * inv only
                        const float4 w = s_w[(4 * j + q) * 32 + lane];
                        a = f2_mul(a, make_float2(w.x, w.y));
                        b = f2_mul(b, make_float2(w.z, w.w));
                    }
                    o.w[4 * e] = __float_as_uint(a.x);
                    o.w[4 * e + 1] = __float_as_uint(a.y);
                    o.w[4 * e + 2] = __float_as_uint(b.x);
                    o.w[4 * e + 3] = __float_as_uint(b.y);
                }
                stg_v8(orow + (size_t)(lane + 32 * j) * 16 + 8 * half, o);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// SwiGLU with bf16 output (kernels/elementwise.cu:225-241) over a flat array, 16 values per lane.
// Blocks with max|g| <= 44 use the short exact quotient (see the quantising kernel); others the
// literal expression. `blocks` = total / 16; a tail of total % 16 values is left to the caller
// (the launcher runs the shape-general kernel on it).
// ---------------------------------------------------------------------------------------------
template <int ACT>
__global__ void __launch_bounds__(kCtaThreads, 4)
swiglu_hot_kernel(const uint16_t* __restrict__ gate, const uint16_t* __restrict__ up, uint16_t* __restrict__ out,
                  uint32_t blocks) {
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    const uint32_t stride = gridDim.x * kCtaThreads;
    uint32_t b = blockIdx.x * kCtaThreads + threadIdx.x;
    U8x32 g, u;
    if (b < blocks) {
        g = ldg_stream_v8(gate + (size_t)b * 16);
        u = ldg_stream_v8(up + (size_t)b * 16);
    }
    for (; b < blocks; b += stride) {
        f32x2 gv[8], uv[8];
        unpack16_quadpairs(g, gv);
        unpack16_quadpairs(u, uv);
        const uint32_t next = b + stride;
        if (next < blocks) {
            g = ldg_stream_v8(gate + (size_t)next * 16);
            u = ldg_stream_v8(up + (size_t)next * 16);
        }
        if (gated_fast_domain<ACT, true>(gv, uv, up + (size_t)b * 16)) {
            gated_fast<ACT>(gv, uv);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                gv[i] = make_float2(gated_literal<ACT>(gv[i].x, uv[i].x), gated_literal<ACT>(gv[i].y, uv[i].y));
            }
        }
        stg_v8(out + (size_t)b * 16, pack16_bf16(gv));
    }
}

// ---------------------------------------------------------------------------------------------
// Gated RMSNorm with bf16 output for 128-wide rows (kernels/elementwise.cu:144-223): the quantising
// kernel's layout (4 lanes per row) and tree; weight and gate are both present on this path.
// ---------------------------------------------------------------------------------------------
static __global__ void __launch_bounds__(kCtaThreads, 2)
gated_norm_hot_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ gate,
                      const float* __restrict__ weight, uint16_t* __restrict__ out, int rows, float eps) {
    constexpr int COLS = 128;
    __shared__ float4 s_w[32];
    const int lane = threadIdx.x & 31;
    const int m = lane & 3;
    const uint32_t groups_in_grid = gridDim.x * (kCtaThreads / 4);
    uint32_t hrow = blockIdx.x * (kCtaThreads / 4) + (threadIdx.x >> 2);
    pdl_launch_dependents();
    if (threadIdx.x < 32) {
        const int mm = threadIdx.x & 3, q = (threadIdx.x >> 2) & 3, h = threadIdx.x >> 4;
        const float4 t = *reinterpret_cast<const float4*>(weight + (mm + 4 * h) * 16 + 4 * q);
        s_w[threadIdx.x] = make_float4(t.x, t.z, t.y, t.w);
    }
    {   // the CTA's first 64 head rows towards L2: 128 lines of x, 128 of gate; see prefetch_l2
        const uint32_t first = blockIdx.x * (kCtaThreads / 4);
        const uint32_t line = threadIdx.x & 127;   // 2 lines per head row
        if (first + (line >> 1) < (uint32_t)rows) {
            prefetch_l2((threadIdx.x < 128 ? x : gate) + (size_t)first * COLS + (size_t)line * 64);
        }
    }
    pdl_wait_prior_grids();
    U8x32 dx[2], dg[2];
    if (hrow < (uint32_t)rows) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            dx[h] = ldg_stream_v8(x + (size_t)hrow * COLS + (m + 4 * h) * 16);
            dg[h] = ldg_stream_v8(gate + (size_t)hrow * COLS + (m + 4 * h) * 16);
        }
    }
    __syncthreads();
    for (uint32_t base = hrow - (uint32_t)(lane >> 2); base < (uint32_t)rows; base += groups_in_grid, hrow += groups_in_grid) {
        const bool live = hrow < (uint32_t)rows;
        f32x2 v[2][8], gv[2][8];
        float quad[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        if (live) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                unpack16_quadpairs(dx[h], v[h]);
                unpack16_quadpairs(dg[h], gv[h]);
                quad_squares(v[h], quad[h]);
            }
        }
        const uint32_t next = hrow + groups_in_grid;
        if (next < (uint32_t)rows) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                dx[h] = ldg_stream_v8(x + (size_t)next * COLS + (m + 4 * h) * 16);
                dg[h] = ldg_stream_v8(gate + (size_t)next * COLS + (m + 4 * h) * 16);
            }
        }
        const float total = head_tree_32(quad[0], quad[1], lane);
        if (!live) {
            continue;
        }
        const f32x2 inv2 = f2_splat(inv_rms_pow2<COLS>(total, eps));
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const bool fast = block_abs_max(gv[h]) <= kSiluFastMaxAbs;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 w = s_w[(h * 4 + q) * 4 + m];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int i = 2 * q + e;
                    const f32x2 wp = e == 0 ? make_float2(w.x, w.y) : make_float2(w.z, w.w);
                    const f32x2 sl = fast ? silu_approx_fast_x2(gv[h][i])
                                          : make_float2(silu_fast_div(gv[h][i].x), silu_fast_div(gv[h][i].y));
                    v[h][i] = f2_mul(f2_mul(f2_mul(v[h][i], inv2), wp), sl);
                }
            }
            stg_v8(out + (size_t)hrow * COLS + (m + 4 * h) * 16, pack16_bf16(v[h]));
        }
    }
}

// The same for f32 activations: the f32 quantising kernel's step structure, the result stored as f32. Gates of
// |g| <= 44 take the short form of __fdividef(g, 1 + __expf(-g)), equal to it for every f32 of that range.
static __global__ void __launch_bounds__(kCtaThreads, 2)
gated_norm_f32_hot_kernel(const float* __restrict__ x, const float* __restrict__ gate, const float* __restrict__ weight,
                          float* __restrict__ out, int rows, float eps) {
    constexpr int COLS = 128;
    __shared__ float4 s_w[32];   // plain weight, natural order: s_w[(h * 4 + q) * 4 + m] = quad q of chunk m + 4h
    const int lane = threadIdx.x & 31;
    const int m = lane & 3;
    const uint32_t groups_in_grid = gridDim.x * (kCtaThreads / 4);
    uint32_t hrow = blockIdx.x * (kCtaThreads / 4) + (threadIdx.x >> 2);
    pdl_launch_dependents();
    if (threadIdx.x < 32) {
        const int mm = threadIdx.x & 3, q = (threadIdx.x >> 2) & 3, h = threadIdx.x >> 4;
        s_w[threadIdx.x] = *reinterpret_cast<const float4*>(weight + (mm + 4 * h) * 16 + 4 * q);
    }
    // a CTA step covers 64 head rows of 512 bytes: 256 lines of x and 256 of the gate, two of each per thread
    auto name_step_to_l2 = [&](uint32_t first) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t line = threadIdx.x + 256 * h;   // 4 lines per head row
            if (first + (line >> 2) < (uint32_t)rows) {
                prefetch_l2(x + (size_t)first * COLS + (size_t)line * 32);
                prefetch_l2(gate + (size_t)first * COLS + (size_t)line * 32);
            }
        }
    };
    name_step_to_l2(blockIdx.x * (kCtaThreads / 4));   // under the previous kernel's tail; see prefetch_l2
    pdl_wait_prior_grids();
    __syncthreads();
    // Every lane of a warp runs the same number of steps (the shuffles need the full warp).
    uint32_t cta_first = blockIdx.x * (kCtaThreads / 4);
    for (uint32_t base = hrow - (uint32_t)(lane >> 2); base < (uint32_t)rows;
         base += groups_in_grid, hrow += groups_in_grid, cta_first += groups_in_grid) {
        const bool live = hrow < (uint32_t)rows;
        U8x32 dx[2][2], dg[2][2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
#pragma unroll
                for (int i = 0; i < 8; ++i) dx[h][half].w[i] = dg[h][half].w[i] = 0u;
            }
        }
        if (live) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const size_t off = (size_t)hrow * COLS + (m + 4 * h) * 16;
                dx[h][0] = ldg_stream_v8(x + off);
                dx[h][1] = ldg_stream_v8(x + off + 8);
                dg[h][0] = ldg_stream_v8(gate + off);
                dg[h][1] = ldg_stream_v8(gate + off + 8);
            }
        }
        if (cta_first + groups_in_grid < (uint32_t)rows) name_step_to_l2(cta_first + groups_in_grid);
        f32x2 v[2][8], gv[2][8];
        float quad[2][4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const U8x32& hx = dx[h][q >> 1];
                const U8x32& hg = dg[h][q >> 1];
                const int o = (q & 1) * 4;
                const float vx = __uint_as_float(hx.w[o]), vy = __uint_as_float(hx.w[o + 1]);
                const float vz = __uint_as_float(hx.w[o + 2]), vw = __uint_as_float(hx.w[o + 3]);
                v[h][2 * q] = f2_pack(vx, vy);
                v[h][2 * q + 1] = f2_pack(vz, vw);
                gv[h][2 * q] = f2_pack(__uint_as_float(hg.w[o]), __uint_as_float(hg.w[o + 1]));
                gv[h][2 * q + 1] = f2_pack(__uint_as_float(hg.w[o + 2]), __uint_as_float(hg.w[o + 3]));
                quad[h][q] = __fadd_rn(__fmaf_rn(vx, vx, __fmul_rn(vy, vy)), __fmaf_rn(vz, vz, __fmul_rn(vw, vw)));
            }
        }
        const float total = head_tree_32(quad[0], quad[1], lane);
        if (!live) {
            continue;
        }
        const f32x2 inv2 = f2_splat(inv_rms_pow2<COLS>(total, eps));
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const bool fast = block_abs_max(gv[h]) <= kSiluFastMaxAbs;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                U8x32 o;
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float4 w = s_w[(h * 4 + 2 * half + e) * 4 + m];
#pragma unroll
                    for (int t = 0; t < 2; ++t) {
                        const int i = 4 * half + 2 * e + t;
                        const f32x2 wp = t == 0 ? make_float2(w.x, w.y) : make_float2(w.z, w.w);
                        const f32x2 sl = fast ? silu_approx_fast_x2(gv[h][i])
                                              : make_float2(silu_fast_div(gv[h][i].x), silu_fast_div(gv[h][i].y));
                        // ((x * inv) * w) * silu(g), left to right as the reference writes it
                        const f32x2 r = f2_mul(f2_mul(f2_mul(v[h][i], inv2), wp), sl);
                        o.w[4 * e + 2 * t] = __float_as_uint(r.x);
                        o.w[4 * e + 2 * t + 1] = __float_as_uint(r.y);
                    }
                }
                stg_v8(out + (size_t)hrow * COLS + (m + 4 * h) * 16 + 8 * half, o);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Partial RoPE (kernels/elementwise.cu:276-315) for head_dim % 32 == 0, rotary_dim % 32 == 0.
// A head row is head_dim/16 chunks of 32 bytes. Work items per head row: rotary_dim/32 "rotating"
// items (chunk i of the lower half together with its partner chunk i + rotary_dim/32) followed by
// (head_dim - rotary_dim)/32 "copy" items (two pass-through chunks each); one lane per item, so
// every lane moves 64 bytes in and 64 bytes out.
// ---------------------------------------------------------------------------------------------
// Where a token's key / value row goes in a KV cache of bf16 rows (kernels/attention_mma.cu:118-171): row
// cache_map[token] when a map is given, else token + *cache_len (0 without a length).
struct KvCacheDest {
    const int* cache_map;
    const int* cache_len;
    const uint16_t* v;    // value rows, same [tokens, heads, head_dim] shape as the keys
    uint16_t* cache_v;
};
__device__ __forceinline__ size_t kv_cache_row(int token, const int* cache_map, const int* cache_len) {
    return cache_map ? (size_t)cache_map[token] : (size_t)token + (size_t)(cache_len ? cache_len[0] : 0);
}

// With KV: `out` is the key cache; total_items counts the items of the key rows followed by as many items of
// the value rows kv.v (every item of a value row is a copy item), and both land at the token's cache row.
// HOIST (plain output only): both chunks of an item are requested before the code splits into rotating and copy
// items. A warp holds both kinds, and loads issued inside the branches wait for each other's round trip; with few
// rounds per thread that latency is the kernel's time (13.0 against 14.0 us at 8,192 rows x 16 heads). With many
// rounds the staggered form streams better (it reaches the copy bandwidth at 130,712 rows, the hoisted one 0.9 of
// it), so the launchers hoist only short launches. The cache-writing form does not fit the hoisted loads into
// the registers of its resident CTAs.
template <bool KV, bool HOIST = false>
__global__ void __launch_bounds__(kCtaThreads, KV ? 4 : 6)
rope_hot_kernel(uint16_t* __restrict__ out, const uint16_t* __restrict__ x, const float* __restrict__ cos_t,
                const float* __restrict__ sin_t, uint32_t total_items, int heads, int head_dim, int rotary_dim,
                const int* __restrict__ seq_start, const int* __restrict__ pos_base,
                const int* __restrict__ pos_map, FastDiv items_div, FastDiv heads_div, KvCacheDest kv) {
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    const uint32_t rot_items = rotary_dim >> 5;
    const uint32_t stride = gridDim.x * blockDim.x;
    const uint32_t key_head_rows = KV ? fast_div(total_items >> 1, items_div) : 0u;
    for (uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total_items; idx += stride) {
        uint32_t head_row = fast_div(idx, items_div);
        uint32_t item = idx - head_row * items_div.d;
        const bool is_value = KV && head_row >= key_head_rows;
        if (is_value) {
            head_row -= key_head_rows;
            item += rot_items;   // a copy item; its column offset is corrected below
        }
        const uint16_t* xr = (is_value ? kv.v : x) + (size_t)head_row * head_dim;
        uint16_t* orow = out + (size_t)head_row * head_dim;
        int row = 0;
        if (KV) {
            row = (int)fast_div(head_row, heads_div);
            orow = (is_value ? kv.cache_v : out) +
                   (kv_cache_row(row, kv.cache_map, kv.cache_len) * (size_t)heads + (head_row - (uint32_t)row * heads)) * head_dim;
        }
        if (HOIST && !KV) {
            const bool rotates = item < rot_items;
            const int half = rotary_dim >> 1;
            const int c0 = rotates ? (int)item * 16 : rotary_dim + (int)(item - rot_items) * 32;
            const int c1 = rotates ? half + (int)item * 16 : c0 + 16;
            int pos = 0;
            if (rotates) pos = rope_position((int)fast_div(head_row, heads_div), seq_start, pos_base, pos_map);
            U8x32 a = ldg_stream_v8(xr + c0);
            U8x32 b = ldg_stream_v8(xr + c1);
            if (rotates) {
                const float* cp = cos_t + (size_t)pos * rotary_dim + item * 16;
                const float* sp = sin_t + (size_t)pos * rotary_dim + item * 16;
#pragma unroll
                for (int q = 0; q < 4; ++q) {   // in place, quad by quad
                    const float4 c = __ldg(reinterpret_cast<const float4*>(cp) + q);
                    const float4 s = __ldg(reinterpret_cast<const float4*>(sp) + q);
                    const uint32_t l0 = a.w[2 * q], l1 = a.w[2 * q + 1], h0 = b.w[2 * q], h1 = b.w[2 * q + 1];
                    float a0, b0, a1, b1, a2, b2, a3, b3;
                    rope_pair(bf16_lo(l0), bf16_lo(h0), c.x, s.x, a0, b0);
                    rope_pair(bf16_hi(l0), bf16_hi(h0), c.y, s.y, a1, b1);
                    rope_pair(bf16_lo(l1), bf16_lo(h1), c.z, s.z, a2, b2);
                    rope_pair(bf16_hi(l1), bf16_hi(h1), c.w, s.w, a3, b3);
                    a.w[2 * q] = pack_bf16x2(a0, a1);
                    a.w[2 * q + 1] = pack_bf16x2(a2, a3);
                    b.w[2 * q] = pack_bf16x2(b0, b1);
                    b.w[2 * q + 1] = pack_bf16x2(b2, b3);
                }
            }
            stg_v8(orow + c0, a);
            stg_v8(orow + c1, b);
        } else if (item < rot_items) {
            if (!KV) row = (int)fast_div(head_row, heads_div);
            const int pos = rope_position(row, seq_start, pos_base, pos_map);
            const int half = rotary_dim >> 1;
            const U8x32 dlo = ldg_stream_v8(xr + item * 16);
            const U8x32 dhi = ldg_stream_v8(xr + half + item * 16);
            const float* cp = cos_t + (size_t)pos * rotary_dim + item * 16;
            const float* sp = sin_t + (size_t)pos * rotary_dim + item * 16;
            U8x32 olo, ohi;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 c = __ldg(reinterpret_cast<const float4*>(cp) + q);
                const float4 s = __ldg(reinterpret_cast<const float4*>(sp) + q);
                const uint32_t l0 = dlo.w[2 * q], l1 = dlo.w[2 * q + 1], h0 = dhi.w[2 * q], h1 = dhi.w[2 * q + 1];
                float a0, b0, a1, b1, a2, b2, a3, b3;
                rope_pair(bf16_lo(l0), bf16_lo(h0), c.x, s.x, a0, b0);
                rope_pair(bf16_hi(l0), bf16_hi(h0), c.y, s.y, a1, b1);
                rope_pair(bf16_lo(l1), bf16_lo(h1), c.z, s.z, a2, b2);
                rope_pair(bf16_hi(l1), bf16_hi(h1), c.w, s.w, a3, b3);
                olo.w[2 * q] = pack_bf16x2(a0, a1);
                olo.w[2 * q + 1] = pack_bf16x2(a2, a3);
                ohi.w[2 * q] = pack_bf16x2(b0, b1);
                ohi.w[2 * q + 1] = pack_bf16x2(b2, b3);
            }
            stg_v8(orow + item * 16, olo);
            stg_v8(orow + half + item * 16, ohi);
        } else {
            const int c0 = (is_value ? 0 : rotary_dim) + (int)(item - rot_items) * 32;
            const U8x32 a = ldg_stream_v8(xr + c0);
            const U8x32 b = ldg_stream_v8(xr + c0 + 16);
            stg_v8(orow + c0, a);
            stg_v8(orow + c0 + 16, b);
        }
    }
}

// Several [rows, heads_i, head_dim] tensors of one token set in ONE launch of the RoPE item structure above: q and k
// rotated with the same positions (the reference's two rope_kernel launches, src/gpu.rs:1722-1725), optionally with
// k going to its bf16 cache rows and v copied to its cache rows (the three conversion launches of attention_dev,
// src/cuda/mod.rs:3201-3227). Work items of the segments follow each other; an item finds its segment by comparing
// with the segments' end items.
struct RopeSegment {
    const uint16_t* x;
    uint16_t* out;
    uint32_t end_item;    // one past this segment's last item in the launch's item numbering
    int heads;
    FastDiv heads_div;
    int rotate;           // 0: every item is a copy item (value rows)
    int to_cache;         // 1: token t's rows are written at cache row kv_cache_row(t)
};
struct RopeSegments {
    RopeSegment seg[3];
};
__device__ __forceinline__ void rope_segment_item(const RopeSegment& sg, uint32_t local, const float* __restrict__ cos_t,
                                                  const float* __restrict__ sin_t, int head_dim, int rotary_dim,
                                                  const int* seq_start, const int* pos_base, const int* pos_map,
                                                  const int* cache_map, const int* cache_len, const FastDiv& items_div) {
    const int half = rotary_dim >> 1;
    const uint32_t head_row = fast_div(local, items_div);
    const uint32_t item = local - head_row * items_div.d;
    const uint32_t rot_items = sg.rotate ? (uint32_t)rotary_dim >> 5 : 0u;
    const int row = (int)fast_div(head_row, sg.heads_div);
    const uint16_t* xr = sg.x + (size_t)head_row * head_dim;
    uint16_t* orow = sg.out + (sg.to_cache ? (kv_cache_row(row, cache_map, cache_len) * (size_t)sg.heads +
                                              (head_row - (uint32_t)row * sg.heads)) * head_dim
                                           : (size_t)head_row * head_dim);
    if (item < rot_items) {
        const int pos = rope_position(row, seq_start, pos_base, pos_map);
        const U8x32 dlo = ldg_stream_v8(xr + item * 16);
        const U8x32 dhi = ldg_stream_v8(xr + half + item * 16);
        const float* cp = cos_t + (size_t)pos * rotary_dim + item * 16;
        const float* sp = sin_t + (size_t)pos * rotary_dim + item * 16;
        U8x32 olo, ohi;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float4 c = __ldg(reinterpret_cast<const float4*>(cp) + q);
            const float4 s = __ldg(reinterpret_cast<const float4*>(sp) + q);
            const uint32_t l0 = dlo.w[2 * q], l1 = dlo.w[2 * q + 1], h0 = dhi.w[2 * q], h1 = dhi.w[2 * q + 1];
            float a0, b0, a1, b1, a2, b2, a3, b3;
            rope_pair(bf16_lo(l0), bf16_lo(h0), c.x, s.x, a0, b0);
            rope_pair(bf16_hi(l0), bf16_hi(h0), c.y, s.y, a1, b1);
            rope_pair(bf16_lo(l1), bf16_lo(h1), c.z, s.z, a2, b2);
            rope_pair(bf16_hi(l1), bf16_hi(h1), c.w, s.w, a3, b3);
            olo.w[2 * q] = pack_bf16x2(a0, a1);
            olo.w[2 * q + 1] = pack_bf16x2(a2, a3);
            ohi.w[2 * q] = pack_bf16x2(b0, b1);
            ohi.w[2 * q + 1] = pack_bf16x2(b2, b3);
        }
        stg_v8(orow + item * 16, olo);
        stg_v8(orow + half + item * 16, ohi);
    } else {
        // copy item: two 32-byte chunks past the rotary span (or anywhere in a value row)
        const int c0 = (sg.rotate ? rotary_dim : 0) + (int)(item - rot_items) * 32;
        const U8x32 a = ldg_stream_v8(xr + c0);
        const U8x32 b = ldg_stream_v8(xr + c0 + 16);
        stg_v8(orow + c0, a);
        stg_v8(orow + c0 + 16, b);
    }
}

#ifndef CLEF_ROPE_MIN_CTAS
#define CLEF_ROPE_MIN_CTAS 6
#endif
template <int NSEG>
__global__ void __launch_bounds__(kCtaThreads, CLEF_ROPE_MIN_CTAS)
rope_multi_hot_kernel(RopeSegments segs, const float* __restrict__ cos_t, const float* __restrict__ sin_t, int head_dim,
                      int rotary_dim, const int* __restrict__ seq_start, const int* __restrict__ pos_base,
                      const int* __restrict__ pos_map, const int* __restrict__ cache_map,
                      const int* __restrict__ cache_len, FastDiv items_div) {
    pdl_launch_dependents();
    const uint32_t total_items = segs.seg[NSEG - 1].end_item;
    const uint32_t stride = gridDim.x * blockDim.x;
    pdl_wait_prior_grids();
    for (uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total_items; idx += stride) {
        // (the segments are addressed with constant indices: kernel parameters cannot be indexed dynamically)
        if (idx < segs.seg[0].end_item) {
            rope_segment_item(segs.seg[0], idx, cos_t, sin_t, head_dim, rotary_dim, seq_start, pos_base, pos_map, cache_map,
                              cache_len, items_div);
        } else if (NSEG == 2 || idx < segs.seg[1].end_item) {
            rope_segment_item(segs.seg[1], idx - segs.seg[0].end_item, cos_t, sin_t, head_dim, rotary_dim, seq_start, pos_base,
                              pos_map, cache_map, cache_len, items_div);
        } else {
            rope_segment_item(segs.seg[NSEG - 1], idx - segs.seg[1].end_item, cos_t, sin_t, head_dim, rotary_dim, seq_start,
                              pos_base, pos_map, cache_map, cache_len, items_div);
        }
    }
}

// The q + k launch in its common short form: positions from a per-token map, results to plain [rows, heads, head_dim]
// tensors (no cache rows), few rounds per thread. Same items as rope_multi_hot_kernel<2> with the loads hoisted
// above the split into rotating and copy items (see rope_hot_kernel); with fewer options to carry it fits 40
// registers (six CTAs per SM), which the general kernel with hoisted loads does not: 13.5 us against 14.3 us at
// 8,192 rows. Long launches go to the general kernel, which streams better.
static __global__ void __launch_bounds__(kCtaThreads, 6)
rope_qk_map_hot_kernel(RopeSegments segs, const float* __restrict__ cos_t, const float* __restrict__ sin_t, int head_dim,
                       int rotary_dim, const int* __restrict__ pos_map, FastDiv items_div) {
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    const uint32_t q_items = segs.seg[0].end_item, total_items = segs.seg[1].end_item;
    const uint32_t stride = gridDim.x * blockDim.x;
    const uint32_t rot_items = (uint32_t)rotary_dim >> 5;
    const int half = rotary_dim >> 1;
    for (uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total_items; idx += stride) {
        const bool is_q = idx < q_items;
        const uint32_t local = is_q ? idx : idx - q_items;
        const uint32_t head_row = fast_div(local, items_div);
        const uint32_t item = local - head_row * items_div.d;
        const uint16_t* xr = (is_q ? segs.seg[0].x : segs.seg[1].x) + (size_t)head_row * head_dim;
        uint16_t* orow = (is_q ? segs.seg[0].out : segs.seg[1].out) + (size_t)head_row * head_dim;
        const bool rotates = item < rot_items;
        const int c0 = rotates ? (int)item * 16 : rotary_dim + (int)(item - rot_items) * 32;
        const int c1 = rotates ? half + (int)item * 16 : c0 + 16;
        int pos = 0;
        if (rotates) {
            const int row = (int)(is_q ? fast_div(head_row, segs.seg[0].heads_div) : fast_div(head_row, segs.seg[1].heads_div));
            pos = __ldg(pos_map + row);
        }
        U8x32 a = ldg_stream_v8(xr + c0);
        U8x32 b = ldg_stream_v8(xr + c1);
        if (rotates) {
            const float* cp = cos_t + (size_t)pos * rotary_dim + item * 16;
            const float* sp = sin_t + (size_t)pos * rotary_dim + item * 16;
#pragma unroll
            for (int q = 0; q < 4; ++q) {   // in place, quad by quad: the results take the registers of their inputs
                const float4 c = __ldg(reinterpret_cast<const float4*>(cp) + q);
                const float4 s = __ldg(reinterpret_cast<const float4*>(sp) + q);
                const uint32_t l0 = a.w[2 * q], l1 = a.w[2 * q + 1], h0 = b.w[2 * q], h1 = b.w[2 * q + 1];
                float a0, b0, a1, b1, a2, b2, a3, b3;
                rope_pair(bf16_lo(l0), bf16_lo(h0), c.x, s.x, a0, b0);
                rope_pair(bf16_hi(l0), bf16_hi(h0), c.y, s.y, a1, b1);
                rope_pair(bf16_lo(l1), bf16_lo(h1), c.z, s.z, a2, b2);
                rope_pair(bf16_hi(l1), bf16_hi(h1), c.w, s.w, a3, b3);
                a.w[2 * q] = pack_bf16x2(a0, a1);
                a.w[2 * q + 1] = pack_bf16x2(a2, a3);
                b.w[2 * q] = pack_bf16x2(b0, b1);
                b.w[2 * q + 1] = pack_bf16x2(b2, b3);
            }
        }
        stg_v8(orow + c0, a);
        stg_v8(orow + c1, b);
    }
}

// The item structure for f32 activations (the reference's own type): a 32-byte chunk is 8 values, so a head row has
// rotary_dim / 16 rotating items and (head_dim - rotary_dim) / 16 copy items; one or two tensors (q, or q and k)
// per launch, plain output rows, loads hoisted above the split. head_dim % 16 == 0, rotary_dim % 16 == 0.
struct RopeSegmentsF32 {
    const float* x[2];
    float* out[2];
    uint32_t end_item[2];
    FastDiv heads_div[2];
};
template <int NSEG>
__global__ void __launch_bounds__(kCtaThreads, 6)
rope_f32_hot_kernel(RopeSegmentsF32 segs, const float* __restrict__ cos_t, const float* __restrict__ sin_t, int head_dim,
                    int rotary_dim, const int* __restrict__ seq_start, const int* __restrict__ pos_base,
                    const int* __restrict__ pos_map, FastDiv items_div) {
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    const uint32_t q_items = segs.end_item[0], total_items = segs.end_item[NSEG - 1];
    const uint32_t stride = gridDim.x * blockDim.x;
    const uint32_t rot_items = (uint32_t)rotary_dim >> 4;
    const int half = rotary_dim >> 1;
    for (uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total_items; idx += stride) {
        const bool is_q = NSEG == 1 || idx < q_items;
        const uint32_t local = is_q ? idx : idx - q_items;
        const uint32_t head_row = fast_div(local, items_div);
        const uint32_t item = local - head_row * items_div.d;
        const float* xr = (is_q ? segs.x[0] : segs.x[1]) + (size_t)head_row * head_dim;
        float* orow = (is_q ? segs.out[0] : segs.out[1]) + (size_t)head_row * head_dim;
        const bool rotates = item < rot_items;
        const int c0 = rotates ? (int)item * 8 : rotary_dim + (int)(item - rot_items) * 16;
        const int c1 = rotates ? half + (int)item * 8 : c0 + 8;
        int pos = 0;
        if (rotates) {
            const int row = (int)(is_q ? fast_div(head_row, segs.heads_div[0]) : fast_div(head_row, segs.heads_div[1]));
            pos = rope_position(row, seq_start, pos_base, pos_map);
        }
        U8x32 a = ldg_stream_v8(xr + c0);
        U8x32 b = ldg_stream_v8(xr + c1);
        if (rotates) {
            const float* cp = cos_t + (size_t)pos * rotary_dim + item * 8;
            const float* sp = sin_t + (size_t)pos * rotary_dim + item * 8;
#pragma unroll
            for (int q = 0; q < 2; ++q) {   // in place, quad by quad
                const float4 c = __ldg(reinterpret_cast<const float4*>(cp) + q);
                const float4 s = __ldg(reinterpret_cast<const float4*>(sp) + q);
                const float cv[4] = {c.x, c.y, c.z, c.w}, sv[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float lo, hi;
                    rope_pair(__uint_as_float(a.w[4 * q + e]), __uint_as_float(b.w[4 * q + e]), cv[e], sv[e], lo, hi);
                    a.w[4 * q + e] = __float_as_uint(lo);
                    b.w[4 * q + e] = __float_as_uint(hi);
                }
            }
        }
        stg_v8(orow + c0, a);
        stg_v8(orow + c1, b);
    }
}

// ---------------------------------------------------------------------------------------------
// Per-head RMSNorm + partial RoPE (kernels/elementwise.cu:70-142) for head_dim 128, rotary_dim 64.
// Four lanes own one head row, a warp 8 head rows. Lane m holds the four 8-value pieces at dims 8m, 32 + 8m,
// 64 + 8m and 96 + 8m (16-byte loads), i.e. quads i, i + 8, i + 16 and i + 24 for i = 2m and 2m + 1. That
// puts both members of every rotation pair (dims j and j + 32) and the first two levels of the norm tree in one
// lane: the reference association (lane l of a warp holds quad l; tree 16, 8, 4, 2, 1 over l) adds quads
// (i, i + 16), then (i, i + 8) in-lane, levels 4 and 2 cross lane bits 1 and 0 (two shuffles each, the pair of
// partial sums a lane keeps), and the last level adds the lane's two sums. 4 shuffles per 8 head rows, no value
// crosses lanes for the rotation. With `gate_out` the input row is [q | gate] and the gate half is copied.
// ---------------------------------------------------------------------------------------------
// With KV (GATE must be false, rows % 8 == 0): `out` is the key cache, the head rows of token t are written at
// cache row kv_cache_row(t), and the value rows ride along as head rows [rows, 2 rows) that are copied to the
// value cache at the same cache row, so one launch fills both caches.
__device__ __forceinline__ void unpack8_quadpairs(const uint4& d, f32x2* v) {
    v[0] = f2_pack(bf16_lo(d.x), bf16_lo(d.y)), v[1] = f2_pack(bf16_hi(d.x), bf16_hi(d.y));   // (x, z), (y, w)
    v[2] = f2_pack(bf16_lo(d.z), bf16_lo(d.w)), v[3] = f2_pack(bf16_hi(d.z), bf16_hi(d.w));
}
__device__ __forceinline__ uint4 pack8_bf16(const f32x2* v) {
    return make_uint4(pack_bf16x2(v[0].x, v[1].x), pack_bf16x2(v[0].y, v[1].y), pack_bf16x2(v[2].x, v[3].x),
                      pack_bf16x2(v[2].y, v[3].y));
}

template <bool GATE, bool KV>
__global__ void __launch_bounds__(kCtaThreads, ((GATE || KV) ? 2 : 3))
qk_norm_rope_hot_kernel(const uint16_t* __restrict__ x, const float* __restrict__ weight,
                        const float* __restrict__ cos_t, const float* __restrict__ sin_t, uint16_t* __restrict__ out,
                        uint16_t* __restrict__ gate_out, uint32_t rows, float eps, const int* __restrict__ seq_start,
                        const int* __restrict__ pos_base, const int* __restrict__ pos_map, FastDiv heads_div,
                        KvCacheDest kv) {
    static_assert(!(GATE && KV), "the key side has no gate half");
    constexpr int HD = 128, ROT = 64, STRIDE = GATE ? 2 * HD : HD;
    const uint32_t key_rows = rows;
    if (KV) rows *= 2;
    __shared__ float4 s_w[32];   // (1 + w) of quad i in the quad-pair order (x, z, y, w)
    const int lane = threadIdx.x & 31;
    const int m = lane & 3;
    const uint32_t groups_in_grid = gridDim.x * (kCtaThreads / 4);
    uint32_t hrow = blockIdx.x * (kCtaThreads / 4) + (threadIdx.x >> 2);
    pdl_launch_dependents();
    if (threadIdx.x < 32) {
        const float4 t = *reinterpret_cast<const float4*>(weight + threadIdx.x * 4);
        s_w[threadIdx.x] = make_float4(1.0f + t.x, 1.0f + t.z, 1.0f + t.y, 1.0f + t.w);
    }
    if (!KV) {   // the warp's first 8 head rows towards L2 (contiguous: 16 lines, 32 with the gate halves); see prefetch_l2
        const uint32_t first = hrow - (uint32_t)(lane >> 2);
        constexpr int LINES = 8 * STRIDE / 64;
        if (lane < LINES && first + (uint32_t)(lane * 64 / STRIDE) < rows) {
            prefetch_l2(x + (size_t)first * STRIDE + (size_t)lane * 64);
        }
    }
    pdl_wait_prior_grids();
    auto row_ptr = [&](uint32_t r) {
        return (KV && r >= key_rows) ? kv.v + (size_t)(r - key_rows) * HD : x + (size_t)r * STRIDE;
    };
    uint4 d[4];   // piece h: dims 32 h + 8 m .. + 7
    U8x32 dgate[2];
    auto fetch = [&](uint32_t r) {
        const uint16_t* src = row_ptr(r) + 8 * m;
#pragma unroll
        for (int h = 0; h < 4; ++h) d[h] = ldg_stream_v4(src + 32 * h);
        if (GATE) {
            dgate[0] = ldg_stream_v8(x + (size_t)r * STRIDE + HD + m * 16);
            dgate[1] = ldg_stream_v8(x + (size_t)r * STRIDE + HD + (m + 4) * 16);
        }
    };
    if (hrow < rows) fetch(hrow);
    __syncthreads();
    for (uint32_t base = hrow - (uint32_t)(lane >> 2); base < rows; base += groups_in_grid, hrow += groups_in_grid) {
        const bool live = hrow < rows;
        if (KV && base >= key_rows) {   // a warp of value rows (warp-uniform: key_rows % 8 == 0): copy and go on
            if (live) {
                const uint32_t vrow = hrow - key_rows;
                const int token = (int)fast_div(vrow, heads_div);
                const size_t dst = (kv_cache_row(token, kv.cache_map, kv.cache_len) * heads_div.d + (vrow - (uint32_t)token * heads_div.d)) * HD;
#pragma unroll
                for (int h = 0; h < 4; ++h) stg_v4(kv.cache_v + dst + 32 * h + 8 * m, d[h]);
            }
            const uint32_t next_v = hrow + groups_in_grid;
            if (next_v < rows) fetch(next_v);
            continue;
        }
        f32x2 v[4][4];
        float quad[4][2] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
        if (live) {
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                unpack8_quadpairs(d[h], v[h]);
#pragma unroll
                for (int e = 0; e < 2; ++e) {   // quad = fma(x,x,y*y) + fma(z,z,w*w), the reference build's contraction
                    const f32x2 t = f2_mul(v[h][2 * e + 1], v[h][2 * e + 1]);
                    const f32x2 sq = f2_fma(v[h][2 * e], v[h][2 * e], t);
                    quad[h][e] = __fadd_rn(sq.x, sq.y);
                }
            }
            if (GATE) {
                stg_v8(gate_out + (size_t)hrow * HD + m * 16, dgate[0]);
                stg_v8(gate_out + (size_t)hrow * HD + (m + 4) * 16, dgate[1]);
            }
        }
        const uint32_t next = hrow + groups_in_grid;
        if (next < rows) fetch(next);
        float s[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            // quads (i, i + 16) and (i + 8, i + 24), then the two sums: reference lanes l, l + 16 and l, l + 8
            s[e] = __fadd_rn(__fadd_rn(quad[0][e], quad[2][e]), __fadd_rn(quad[1][e], quad[3][e]));
            s[e] = __fadd_rn(s[e], __shfl_xor_sync(kFullMask, s[e], 2));   // l, l + 4
            s[e] = __fadd_rn(s[e], __shfl_xor_sync(kFullMask, s[e], 1));   // l, l + 2
        }
        const float total = __fadd_rn(s[0], s[1]);                         // l, l + 1
        if (!live) {
            continue;
        }
        const f32x2 inv2 = f2_splat(inv_rms_pow2<HD>(total, eps));
#pragma unroll
        for (int h = 0; h < 4; ++h) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const float4 w = s_w[8 * h + 2 * m + e];
                v[h][2 * e] = f2_mul(f2_mul(v[h][2 * e], inv2), make_float2(w.x, w.y));
                v[h][2 * e + 1] = f2_mul(f2_mul(v[h][2 * e + 1], inv2), make_float2(w.z, w.w));
            }
        }
        const int token = (int)fast_div(hrow, heads_div);
        const int pos = rope_position(token, seq_start, pos_base, pos_map);
        const float* cp = cos_t + (size_t)pos * ROT + m * 8;
        const float* sp = sin_t + (size_t)pos * ROT + m * 8;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const float4 c = __ldg(reinterpret_cast<const float4*>(cp) + e);
            const float4 sn = __ldg(reinterpret_cast<const float4*>(sp) + e);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const f32x2 c2 = i == 0 ? make_float2(c.x, c.z) : make_float2(c.y, c.w);
                const f32x2 s2 = i == 0 ? make_float2(sn.x, sn.z) : make_float2(sn.y, sn.w);
                // lo' = fma(lo, c, -(hi * s));  hi' = fma(lo, s, hi * c)   (the reference build's contraction)
                const f32x2 lo = v[0][2 * e + i], hi = v[1][2 * e + i];
                v[0][2 * e + i] = f2_fma(lo, c2, f2_mul(hi, make_float2(-s2.x, -s2.y)));
                v[1][2 * e + i] = f2_fma(lo, s2, f2_mul(hi, c2));
            }
        }
        const size_t orow = KV ? (kv_cache_row(token, kv.cache_map, kv.cache_len) * heads_div.d + (hrow - (uint32_t)token * heads_div.d)) * HD
                               : (size_t)hrow * HD;
#pragma unroll
        for (int h = 0; h < 4; ++h) stg_v4(out + orow + 32 * h + 8 * m, pack8_bf16(v[h]));
    }
}

// ---------------------------------------------------------------------------------------------
// The same step for head_dim 256, rotary_dim 64 (the head shape src/cuda/mod.rs:6743 serves). Four lanes own one
// head row again: lane m holds chunks m (rotary), m + 4, m + 8 and m + 12. The reference's norm team for 256
// columns is one warp whose thread l adds quad l and then quad l + 32, so the halves are added quad by quad
// before the head_tree_32 tree. The raw words of a row stay in registers across the tree and are unpacked chunk
// by chunk afterwards; rows that are only copied are items of their own. No software prefetch: two resident CTAs
// of independent row loads cover the latency.
// ---------------------------------------------------------------------------------------------
template <bool GATE, bool KV>
__global__ void __launch_bounds__(kCtaThreads, 2)
qk_norm_rope_hd256_hot_kernel(const uint16_t* __restrict__ x, const float* __restrict__ weight,
                              const float* __restrict__ cos_t, const float* __restrict__ sin_t, uint16_t* __restrict__ out,
                              uint16_t* __restrict__ gate_out, uint32_t rows, float eps, const int* __restrict__ seq_start,
                              const int* __restrict__ pos_base, const int* __restrict__ pos_map, FastDiv heads_div,
                              KvCacheDest kv) {
    static_assert(!(GATE && KV), "the key side has no gate half");
    constexpr int HD = 256, ROT = 64, NCH = 4, STRIDE = GATE ? 2 * HD : HD;
    constexpr bool COPIES = GATE || KV;
    // Rows that are only copied (the gate halves, or the value rows of a KV write) follow the normed rows as
    // items of their own, from the next multiple of 8 so that a warp holds one kind.
    const uint32_t copy_base = (rows + 7u) & ~7u;
    const uint32_t items = COPIES ? copy_base + rows : rows;
    __shared__ float4 s_w[HD / 4];   // (1 + w), quad-pair layout: s_w[c * 4 + q] for chunk c, quad q
    const int lane = threadIdx.x & 31;
    const int m = lane & 3;
    const uint32_t groups_in_grid = gridDim.x * (kCtaThreads / 4);
    uint32_t item = blockIdx.x * (kCtaThreads / 4) + (threadIdx.x >> 2);
    pdl_launch_dependents();
    if (threadIdx.x < HD / 4) {
        const float4 t = *reinterpret_cast<const float4*>(weight + threadIdx.x * 4);
        s_w[threadIdx.x] = make_float4(1.0f + t.x, 1.0f + t.z, 1.0f + t.y, 1.0f + t.w);
    }
    pdl_wait_prior_grids();
    __syncthreads();
    for (uint32_t base = item - (uint32_t)(lane >> 2); base < items; base += groups_in_grid, item += groups_in_grid) {
        if (COPIES && base >= copy_base) {
            const uint32_t crow = item - copy_base;
            if (crow < rows) {
                const uint16_t* src = GATE ? x + (size_t)crow * STRIDE + HD : kv.v + (size_t)crow * HD;
                U8x32 c[NCH];
#pragma unroll
                for (int h = 0; h < NCH; ++h) c[h] = ldg_stream_v8(src + (m + 4 * h) * 16);
                uint16_t* dst;
                if (GATE) {
                    dst = gate_out + (size_t)crow * HD;
                } else {
                    const int token = (int)fast_div(crow, heads_div);
                    dst = kv.cache_v + (kv_cache_row(token, kv.cache_map, kv.cache_len) * heads_div.d + (crow - (uint32_t)token * heads_div.d)) * HD;
                }
#pragma unroll
                for (int h = 0; h < NCH; ++h) stg_v8(dst + (m + 4 * h) * 16, c[h]);
            }
            continue;
        }
        const uint32_t hrow = item;
        const bool live = hrow < rows;
        U8x32 d[NCH];
#pragma unroll
        for (int h = 0; h < NCH; ++h) {
#pragma unroll
            for (int i = 0; i < 8; ++i) d[h].w[i] = 0u;
        }
        if (live) {
#pragma unroll
            for (int h = 0; h < NCH; ++h) d[h] = ldg_stream_v8(x + (size_t)hrow * STRIDE + (m + 4 * h) * 16);
        }
        f32x2 v[8], pv[8];
        float quad[NCH][4];
#pragma unroll
        for (int h = 0; h < NCH; ++h) {
            unpack16_quadpairs(d[h], v);
            quad_squares(v, quad[h]);
        }
        U8x32 praw;
#pragma unroll
        for (int i = 0; i < 8; ++i) {   // partner's raw rotary chunk (lane m ^ 2)
            praw.w[i] = __shfl_xor_sync(kFullMask, d[0].w[i], 2);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {   // reference thread l adds quad l, then quad l + 32 (dims + 128), before the tree
            quad[0][k] = __fadd_rn(quad[0][k], quad[2][k]);
            quad[1][k] = __fadd_rn(quad[1][k], quad[3][k]);
        }
        const float total = head_tree_32(quad[0], quad[1], lane);
        if (!live) {
            continue;
        }
        const f32x2 inv2 = f2_splat(inv_rms_pow2<HD>(total, eps));
        const int token = (int)fast_div(hrow, heads_div);
        uint16_t* orow = out + (KV ? (kv_cache_row(token, kv.cache_map, kv.cache_len) * heads_div.d + (hrow - (uint32_t)token * heads_div.d)) * HD
                                   : (size_t)hrow * HD);
#pragma unroll
        for (int h = 1; h < NCH; ++h) {   // pass-through chunks
            unpack16_quadpairs(d[h], v);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 w = s_w[(m + 4 * h) * 4 + q];
                v[2 * q] = f2_mul(f2_mul(v[2 * q], inv2), make_float2(w.x, w.y));
                v[2 * q + 1] = f2_mul(f2_mul(v[2 * q + 1], inv2), make_float2(w.z, w.w));
            }
            stg_v8(orow + (m + 4 * h) * 16, pack16_bf16(v));
        }
        unpack16_quadpairs(d[0], v);
        unpack16_quadpairs(praw, pv);
        const int pm = m ^ 2;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float4 wa = s_w[m * 4 + q], wp = s_w[pm * 4 + q];
            v[2 * q] = f2_mul(f2_mul(v[2 * q], inv2), make_float2(wa.x, wa.y));
            v[2 * q + 1] = f2_mul(f2_mul(v[2 * q + 1], inv2), make_float2(wa.z, wa.w));
            pv[2 * q] = f2_mul(f2_mul(pv[2 * q], inv2), make_float2(wp.x, wp.y));
            pv[2 * q + 1] = f2_mul(f2_mul(pv[2 * q + 1], inv2), make_float2(wp.z, wp.w));
        }
        const int pos = rope_position(token, seq_start, pos_base, pos_map);
        const float* cp = cos_t + (size_t)pos * ROT + (m & 1) * 16;
        const float* sp = sin_t + (size_t)pos * ROT + (m & 1) * 16;
        const bool holds_lo = m < 2;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float4 c = __ldg(reinterpret_cast<const float4*>(cp) + q);
            const float4 sn = __ldg(reinterpret_cast<const float4*>(sp) + q);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int i = 2 * q + e;
                const f32x2 c2 = e == 0 ? make_float2(c.x, c.z) : make_float2(c.y, c.w);
                const f32x2 s2 = e == 0 ? make_float2(sn.x, sn.z) : make_float2(sn.y, sn.w);
                // lo' = fma(lo, c, -(hi * s));  hi' = fma(lo, s, hi * c)   (the reference build's contraction)
                const f32x2 lo = holds_lo ? v[i] : pv[i];
                const f32x2 hi = holds_lo ? pv[i] : v[i];
                const f32x2 t = f2_mul(hi, holds_lo ? make_float2(-s2.x, -s2.y) : c2);
                v[i] = f2_fma(lo, holds_lo ? c2 : s2, t);
            }
        }
        stg_v8(orow + m * 16, pack16_bf16(v));
    }
}

// ---------------------------------------------------------------------------------------------
// Per-head RMSNorm + partial RoPE for f32 activations (kernels/elementwise.cu:70-142), head_dim HD of 128 or 256,
// rotary_dim 64. One warp per head row exactly as the reference's norm team (32 threads for up to 256 columns:
// thread l adds quad l, then quad l + 32, then the 16..1 tree), two rows in flight per warp; the whole row stays in
// registers. The rotation pairs dims j and j + 32, i.e. quad l of lanes l and l ^ 8 (l < 16): the partner's
// normalised quad crosses by shuffle. With GATE the input row is [q | gate] and the gate half is copied.
// ---------------------------------------------------------------------------------------------
template <int HD, bool GATE>
__global__ void __launch_bounds__(kCtaThreads, 4)
qk_norm_rope_f32_hot_kernel(const float* __restrict__ x, const float* __restrict__ weight, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, float* __restrict__ out, float* __restrict__ gate_out,
                            uint32_t rows, float eps, const int* __restrict__ seq_start, const int* __restrict__ pos_base,
                            const int* __restrict__ pos_map, FastDiv heads_div) {
    constexpr int ROT = 64, NQ = HD / 128, STRIDE = GATE ? 2 * HD : HD, R = 2;
    const int lane = threadIdx.x & 31;
    const uint32_t warps = gridDim.x * (kCtaThreads / 32);
    pdl_launch_dependents();
    float4 w1[NQ];   // (1 + w) of this lane's quads
#pragma unroll
    for (int k = 0; k < NQ; ++k) {
        const float4 t = __ldg(reinterpret_cast<const float4*>(weight) + lane + 32 * k);
        w1[k] = make_float4(1.0f + t.x, 1.0f + t.y, 1.0f + t.z, 1.0f + t.w);
    }
    pdl_wait_prior_grids();
    const bool rotates = lane < 16, holds_lo = lane < 8;
    for (uint32_t row0 = blockIdx.x * (kCtaThreads / 32) + (threadIdx.x >> 5); row0 < rows; row0 += R * warps) {
        float4 v[R][NQ];
        float4 c[R], sn[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint32_t row = row0 + r * warps;
            c[r] = sn[r] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int k = 0; k < NQ; ++k) v[r][k] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (row < rows) {
#pragma unroll
                for (int k = 0; k < NQ; ++k) {
                    const uint4 t = ldg_stream_v4(x + (size_t)row * STRIDE + 4 * (lane + 32 * k));
                    v[r][k] = make_float4(__uint_as_float(t.x), __uint_as_float(t.y), __uint_as_float(t.z), __uint_as_float(t.w));
                }
                if (rotates) {
                    const int pos = rope_position((int)fast_div(row, heads_div), seq_start, pos_base, pos_map);
                    c[r] = __ldg(reinterpret_cast<const float4*>(cos_t + (size_t)pos * ROT) + (lane & 7));
                    sn[r] = __ldg(reinterpret_cast<const float4*>(sin_t + (size_t)pos * ROT) + (lane & 7));
                }
            }
        }
        if (GATE) {   // the gate halves ride along: loaded with the rows, stored straight away
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const uint32_t row = row0 + r * warps;
                if (row < rows) {
#pragma unroll
                    for (int k = 0; k < NQ; ++k) {
                        const uint4 t = ldg_stream_v4(x + (size_t)row * STRIDE + HD + 4 * (lane + 32 * k));
                        stg_v4(gate_out + (size_t)row * HD + 4 * (lane + 32 * k), t);
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint32_t row = row0 + r * warps;
            float acc = 0.0f;
#pragma unroll
            for (int k = 0; k < NQ; ++k) acc = __fadd_rn(acc, quad_sq(v[r][k]));
            const float inv = inv_rms(warp_tree_sum(acc), HD, eps);
#pragma unroll
            for (int k = 0; k < NQ; ++k) {
                v[r][k] = make_float4(v[r][k].x * inv * w1[k].x, v[r][k].y * inv * w1[k].y, v[r][k].z * inv * w1[k].z,
                                      v[r][k].w * inv * w1[k].w);
            }
            float4 p;   // the partner's normalised rotary quad
            p.x = __shfl_xor_sync(kFullMask, v[r][0].x, 8);
            p.y = __shfl_xor_sync(kFullMask, v[r][0].y, 8);
            p.z = __shfl_xor_sync(kFullMask, v[r][0].z, 8);
            p.w = __shfl_xor_sync(kFullMask, v[r][0].w, 8);
            if (rotates) {
                const float4 lo = holds_lo ? v[r][0] : p, hi = holds_lo ? p : v[r][0];
                float4 olo, ohi;
                rope_pair(lo.x, hi.x, c[r].x, sn[r].x, olo.x, ohi.x);
                rope_pair(lo.y, hi.y, c[r].y, sn[r].y, olo.y, ohi.y);
                rope_pair(lo.z, hi.z, c[r].z, sn[r].z, olo.z, ohi.z);
                rope_pair(lo.w, hi.w, c[r].w, sn[r].w, olo.w, ohi.w);
                v[r][0] = holds_lo ? olo : ohi;
            }
            if (row < rows) {
#pragma unroll
                for (int k = 0; k < NQ; ++k) {
                    stg_v4(out + (size_t)row * HD + 4 * (lane + 32 * k),
                           make_uint4(__float_as_uint(v[r][k].x), __float_as_uint(v[r][k].y), __float_as_uint(v[r][k].z),
                                      __float_as_uint(v[r][k].w)));
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Embedding gather (kernels/elementwise.cu:396-407) for rows of a multiple of 1 KiB: one warp per
// token row, every lane moves CH chunks of 32 bytes.
// ---------------------------------------------------------------------------------------------
template <int CH>
__global__ void __launch_bounds__(kCtaThreads)
embed_gather_hot_kernel(const uint8_t* __restrict__ table, const int* __restrict__ ids, uint8_t* __restrict__ out,
                        int tokens) {
    constexpr size_t ROW_BYTES = (size_t)CH * 1024;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    for (int t = blockIdx.x * 8 + warp; t < tokens; t += gridDim.x * 8) {
        const uint8_t* src = table + (size_t)__ldg(ids + t) * ROW_BYTES;
        uint8_t* dst = out + (size_t)t * ROW_BYTES;
        U8x32 d[CH];
#pragma unroll
        for (int j = 0; j < CH; ++j) {
            d[j] = ldg_stream_v8(src + (size_t)(lane + 32 * j) * 32);
        }
#pragma unroll
        for (int j = 0; j < CH; ++j) {
            stg_v8(dst + (size_t)(lane + 32 * j) * 32, d[j]);
        }
    }
}

}  // namespace clef
