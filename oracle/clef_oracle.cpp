// clef_oracle.cpp -- TEST INFRASTRUCTURE, not product code.
//
// A CPU (C++17 + OpenMP) restatement of the arithmetic of aiis-clef's fused per-layer
// elementwise kernels, used only as the checker in tests, in the smoke check and as the timed
// CPU baseline of the benchmark. Nothing in the shipped library links or calls this file.
//
// Every routine names the reference source it follows (paths inside the aiis-clef tree):
//   kernels/nvfp4_quant.h        E2M1 / E4M3 encoders and the E4M3 decoder
//   kernels/quantise.cu          NVFP4 activation quantisers (plain, RMSNorm, gated RMSNorm, SwiGLU)
//   kernels/elementwise.cu       rms_norm, rms_norm_gated, swiglu, rope, qk_norm_rope, embed_gather,
//                                rope_tables
//   src/dequant.rs               NVFP4 dequantiser (the NVFP4 oracle of the reference's own tests)
//   src/swizzle.rs               tiled scale layouts and their index maps
//   src/model/gemm_ref.rs        e4m3_one (signed E4M3 decode)
//   src/model/norm.rs            f64-accumulating RMSNorm / gated RMSNorm (tolerance reference)
//   src/model/attention.rs       rope_tables / apply_rope on the CPU
//
// Parity status: pinned. The scalar encoders/decoders, the layouts and the model routines are
// checked against the known answers in the reference's own unit tests (see tests/), and the
// kernel restatements are checked byte-for-byte against the reference's own CUDA kernels built
// for sm_100a (oracle/_ref) on the GPU. Two reference kernels use GPU-only approximate
// intrinsics (__expf, __fdividef); for those this file uses expf and IEEE division, so the
// comparison with a GPU result is exact only away from rounding boundaries (tests say how far).
//
// Floating-point contract: built with -ffp-contract=off; every fused multiply-add is explicit.
// The reference kernels are built with nvcc's default -fmad=true, so the compiler chose where
// a*b+c became one FMA. Those choices are parameters here (`fma_mode`), fixed by comparing with
// the reference cubin on the GPU; the defaults below are the ones that matched.

#include <cmath>
#include <cstdint>
#include <cstring>
#include <cstdlib>
#include <vector>
#include <algorithm>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API extern "C" __attribute__((visibility("default")))

namespace {

// ---------------------------------------------------------------------------------------------
// bf16 <-> f32. Widening is exact; narrowing is round-to-nearest-even on the bit pattern, the
// same integer formula as kernels/quantise.cu:375-378 (NaN is kept a NaN here).
// ---------------------------------------------------------------------------------------------
inline float bf16_bits_to_f32(uint16_t b) {
    uint32_t u = (uint32_t)b << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
inline uint16_t f32_to_bf16_bits(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) {
        return (uint16_t)0x7FFFu;   // cvt.rn.bf16.f32 / __float2bfloat16 return the canonical NaN
    }
    return (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}

// ---------------------------------------------------------------------------------------------
// kernels/nvfp4_quant.h:13-33  to_e2m1 (CLEF_E2M1_FAST == 0, the build default): nearest of
// {0,.5,1,1.5,2,3,4,6} by a first-minimum search with a strict '<', so ties go to the smaller
// magnitude, anything whose distance to every entry is >= 1e30 (or NaN) maps to magnitude 0,
// and the sign nibble is (v < 0), which is false for -0.0 and for NaN.
// ---------------------------------------------------------------------------------------------
const float kE2M1[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

inline uint8_t to_e2m1(float v) {
    const uint8_t sign = (v < 0.0f) ? 0x8u : 0x0u;
    const float a = std::fabs(v);
    uint8_t best = 0;
    float best_err = 1e30f;
    for (int i = 0; i < 8; ++i) {
        const float err = std::fabs(a - kE2M1[i]);
        if (err < best_err) {
            best_err = err;
            best = (uint8_t)i;
        }
    }
    return (uint8_t)(sign | best);
}

// float -> int conversion with the GPU's semantics (cvt.rzi.s32.f32 saturates, NaN -> 0).
inline int f2i_rz_sat(float f) {
    if (std::isnan(f)) return 0;
    if (f >= 2147483648.0f) return 2147483647;
    if (f <= -2147483648.0f) return (int)(-2147483647 - 1);
    return (int)f;
}

// kernels/nvfp4_quant.h:35-57  to_e4m3: positive values only, mantissa rounded half up,
// clamped to 0x7E, and below the normal range `min(int(v*512 + 0.5), 7)`.
inline uint8_t to_e4m3(float v) {
    if (!(v > 0.0f)) {
        return 0;
    }
    if (std::isinf(v)) {
        // frexpf(+inf) leaves the exponent unspecified in C; CUDA's returns exp = 0 and m = +inf,
        // which walks the code below to (6 << 3) | (INT_MAX & 7). Restated literally.
        return (uint8_t)((6 << 3) | 7);
    }
    int exp = 0;
    float m = std::frexp(v, &exp);
    int e4 = exp + 6;
    float mant = (m * 2.0f - 1.0f) * 8.0f;
    int mi = f2i_rz_sat(mant + 0.5f);
    if (mi == 8) {
        mi = 0;
        ++e4;
    }
    if (e4 <= 0) {
        const int sub = f2i_rz_sat(v * 512.0f + 0.5f);
        return (uint8_t)(sub > 7 ? 7 : sub);
    }
    if (e4 > 15 || (e4 == 15 && mi > 6)) {
        return 0x7E;
    }
    return (uint8_t)((e4 << 3) | (mi & 0x7));
}

// kernels/nvfp4_quant.h:59-66  from_e4m3 (unsigned decode used by the quantisers).
inline float from_e4m3(uint8_t b) {
    const int e = (b >> 3) & 0x0F;
    const float mant = (float)(b & 0x07);
    if (e == 0) {
        return mant * (1.0f / 512.0f);
    }
    return (1.0f + mant / 8.0f) * std::ldexp(1.0f, e - 7);
}

// src/model/gemm_ref.rs:101-111  e4m3_one (signed decode used by the CPU GEMM reference).
inline float e4m3_one(uint8_t b) {
    const float sign = (b & 0x80) ? -1.0f : 1.0f;
    const int exp = (b >> 3) & 0x0F;
    const float mant = (float)(b & 0x07);
    if (exp == 0) {
        return sign * mant * std::ldexp(1.0f, -9);
    }
    return sign * (1.0f + mant / 8.0f) * std::ldexp(1.0f, exp - 7);
}

// ---------------------------------------------------------------------------------------------
// Scale address of the activation-side ("conflict-free") layout:
// kernels/quantise.cu:34-41 (and :103-112, :252-259, :568-575).
// ---------------------------------------------------------------------------------------------
inline size_t scale_index(int row, int block, int blocks_per_row, int blk_mn, int chunk) {
    const int k1_count = blocks_per_row / 4;
    const int m_rest = row / blk_mn;
    const int k1 = block / 4;
    const int k2 = block % 4;
    const int m_atom = row % blk_mn;
    return (size_t)(m_rest * k1_count + k1) * (size_t)chunk + (size_t)m_atom * 4 + (size_t)k2;
}

// One 16-value block: kernels/quantise.cu:22-52. `v` holds the 16 f32 values of a LIVE row.
// Writes one scale byte and 8 packed bytes.
inline void quantise_block(const float* v, float global_scale, uint8_t* scale_out, uint8_t* packed_out) {
    float amax = 0.0f;
    for (int i = 0; i < 16; ++i) {
        amax = std::fmax(amax, std::fabs(v[i]));   // fmaxf ignores a NaN operand, like CUDA's
    }
    const float block_scale = amax / 6.0f;
    const uint8_t stored = to_e4m3(block_scale * global_scale);
    *scale_out = stored;
    const float stored_f = from_e4m3(stored);
    const float inv_scale = (stored_f > 0.0f) ? global_scale / stored_f : 0.0f;
    for (int pair = 0; pair < 8; ++pair) {
        const uint8_t lo = to_e2m1(v[pair * 2] * inv_scale);
        const uint8_t hi = to_e2m1(v[pair * 2 + 1] * inv_scale);
        packed_out[pair] = (uint8_t)(lo | (hi << 4));
    }
}

// One live row of `cols` f32 values -> packed row + its scale bytes in the tiled layout.
inline void quantise_row(const float* v, int row, int cols, float global_scale, int blk_mn, int chunk,
                         uint8_t* packed, uint8_t* scales) {
    const int blocks = cols / 16;
    uint8_t* prow = packed + (size_t)row * (cols / 2);
    for (int b = 0; b < blocks; ++b) {
        quantise_block(v + b * 16, global_scale, &scales[scale_index(row, b, blocks, blk_mn, chunk)],
                       prow + b * 8);
    }
}

// A pad row (row >= rows): scale bytes 0 (kernels/quantise.cu:32) and packed bytes 0 (the
// reference allocates them zeroed, src/cuda/mod.rs:2186-2187).
inline void zero_pad_row(int row, int cols, int blk_mn, int chunk, uint8_t* packed, uint8_t* scales) {
    const int blocks = cols / 16;
    std::memset(packed + (size_t)row * (cols / 2), 0, (size_t)cols / 2);
    for (int b = 0; b < blocks; ++b) {
        scales[scale_index(row, b, blocks, blk_mn, chunk)] = 0;
    }
}

inline int round_up_i(int v, int n) { return (v + n - 1) / n * n; }

// ---------------------------------------------------------------------------------------------
// Sum of squares in the reference's order. kernels/elementwise.cu:8-52 (rms_norm_kernel),
// :148-191 (gated), kernels/quantise.cu:207-237 (fused norm+quant, stride 256 == tpr for 4096).
//   thread `sub` of `tpr`:  acc = 0; for i = sub, sub+tpr, ... < cols/4: acc += quad(i)
//   quad(i) = (x*x + y*y) + (z*z + w*w) over float4 #i   (FMA contraction: fma_mode)
//   warp: shfl_down tree 16,8,4,2,1; lane 0 of each warp -> s_part
//   row:  t = s_part[lane] (lane < wpr, else 0); shfl_down tree 4,2,1
// fma_mode: 0 = no contraction, 1 = fma(a,a,b*b) for each pair, 2 = fma(b,b,a*a).
// ---------------------------------------------------------------------------------------------
inline float pair_sq(float a, float b, int fma_mode) {
    if (fma_mode == 1) return std::fma(a, a, b * b);
    if (fma_mode == 2) return std::fma(b, b, a * a);
    return a * a + b * b;
}
inline float quad_sq(const float* p, int fma_mode) {
    return pair_sq(p[0], p[1], fma_mode) + pair_sq(p[2], p[3], fma_mode);
}
inline int threads_per_row(int cols) {
    return std::min(256, std::max(32, ((cols + 255) / 256) * 32));
}
inline float sum_squares_ref_order(const float* x, int cols, int fma_mode) {
    const int tpr = threads_per_row(cols);
    const int wpr = tpr >> 5;
    const int c4 = cols >> 2;
    float part[256];
    for (int sub = 0; sub < tpr; ++sub) {
        float acc = 0.0f;
        for (int i = sub; i < c4; i += tpr) {
            acc += quad_sq(x + 4 * i, fma_mode);
        }
        part[sub] = acc;
    }
    float warp_sum[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int w = 0; w < wpr; ++w) {
        float* a = part + 32 * w;
        for (int off = 16; off > 0; off >>= 1) {
            for (int l = 0; l < off; ++l) a[l] += a[l + off];
        }
        warp_sum[w] = a[0];
    }
    if (wpr == 1) {
        // elementwise.cu:176-190 skips the cross-warp tree when a row is one warp; the plain
        // rms_norm_kernel runs it with zeros in the unused lanes, which adds exact zeros.
        return warp_sum[0];
    }
    for (int off = 4; off > 0; off >>= 1) {
        for (int l = 0; l < off; ++l) warp_sum[l] += warp_sum[l + off];
    }
    return warp_sum[0];
}
inline float inv_rms(float total, int cols, float eps) {
    return 1.0f / std::sqrt(total / (float)cols + eps);
}

// silu pieces. The reference uses __expf (ex2.approx of x*log2e) and, in the gated norm,
// __fdividef (approximate divide). The CPU restatement uses expf and IEEE division.
inline float silu_div_ieee(float g) { return g / (1.0f + std::exp(-g)); }

// kernels/elementwise.cu:53-66: out = x*inv*(1+w)  (left-associated), or x*inv without weight.
inline void rms_norm_row(const float* x, const float* w, int cols, float eps, int fma_mode, float* out) {
    const float inv = inv_rms(sum_squares_ref_order(x, cols, fma_mode), cols, eps);
    if (w) {
        for (int i = 0; i < cols; ++i) out[i] = x[i] * inv * (1.0f + w[i]);
    } else {
        for (int i = 0; i < cols; ++i) out[i] = x[i] * inv;
    }
}

// kernels/elementwise.cu:192-221 and quantise.cu:84-95: out = x*inv*w*silu(g), plain weight.
inline void rms_norm_gated_row(const float* x, const float* g, const float* w, int cols, float eps,
                               int fma_mode, float* out) {
    const float inv = inv_rms(sum_squares_ref_order(x, cols, fma_mode), cols, eps);
    for (int i = 0; i < cols; ++i) {
        const float gv = g ? g[i] : 0.0f;
        const float s = silu_div_ieee(gv);
        out[i] = w ? (x[i] * inv * w[i] * s) : (x[i] * inv * s);
    }
}

// kernels/elementwise.cu:276-315 rope_kernel, one (row, head): pairs (j, j+half), j < half;
// dims >= rotary_dim are copied. rope_fma = lo_mode + 3 * hi_mode picks the contraction of each
// expression independently:
//   lo_mode (lo*c - hi*s): 0 none, 1 fma(lo,c,-(hi*s)), 2 fma(-hi,s,lo*c)
//   hi_mode (hi*c + lo*s): 0 none, 1 fma(hi,c,lo*s),    2 fma(lo,s,hi*c)
inline void rope_head(const float* x, float* out, const float* cos_row, const float* sin_row,
                      int head_dim, int rotary_dim, int rope_fma) {
    const int half = rotary_dim / 2;
    const int lo_mode = rope_fma % 3, hi_mode = rope_fma / 3;
    for (int j = 0; j < half; ++j) {
        const float c = cos_row[j], s = sin_row[j];
        const float lo = x[j], hi = x[j + half];
        float a, b;
        if (lo_mode == 1) {
            a = std::fma(lo, c, -(hi * s));
        } else if (lo_mode == 2) {
            a = std::fma(-hi, s, lo * c);
        } else {
            a = lo * c - hi * s;
        }
        if (hi_mode == 1) {
            b = std::fma(hi, c, lo * s);
        } else if (hi_mode == 2) {
            b = std::fma(lo, s, hi * c);
        } else {
            b = hi * c + lo * s;
        }
        out[j] = a;
        out[j + half] = b;
    }
    for (int d = rotary_dim; d < head_dim; ++d) out[d] = x[d];
}

inline int rope_position(int row, const int32_t* seq_start, const int32_t* pos_base, const int32_t* pos_map) {
    // elementwise.cu:300-303
    return pos_map ? pos_map[row]
                   : (seq_start ? row - seq_start[row] : row) + (pos_base ? pos_base[0] : 0);
}

inline void widen_row(const void* src, size_t offset_elems, int n, int dtype, float* dst) {
    if (dtype == 0) {
        const uint16_t* p = (const uint16_t*)src + offset_elems;
        for (int i = 0; i < n; ++i) dst[i] = bf16_bits_to_f32(p[i]);
    } else {
        std::memcpy(dst, (const float*)src + offset_elems, (size_t)n * 4);
    }
}
inline void narrow_row(const float* src, int n, int dtype, void* dst, size_t offset_elems) {
    if (dtype == 0) {
        uint16_t* p = (uint16_t*)dst + offset_elems;
        for (int i = 0; i < n; ++i) p[i] = f32_to_bf16_bits(src[i]);
    } else {
        std::memcpy((float*)dst + offset_elems, src, (size_t)n * 4);
    }
}

inline int pick_threads(int nthreads) {
#ifdef _OPENMP
    return nthreads > 0 ? nthreads : omp_get_max_threads();
#else
    (void)nthreads;
    return 1;
#endif
}

}  // namespace

// =================================================================================================
// Exported C interface (ctypes). dtype: 0 = bf16 (uint16 bit patterns), 1 = f32, for activations;
// weights and RoPE tables are always f32. `nthreads` <= 0 means all OpenMP threads.
// =================================================================================================

ORACLE_API int oracle_max_threads(void) { return pick_threads(0); }

ORACLE_API uint8_t oracle_to_e2m1(float v) { return to_e2m1(v); }
ORACLE_API uint8_t oracle_to_e4m3(float v) { return to_e4m3(v); }
ORACLE_API float oracle_from_e4m3(uint8_t b) { return from_e4m3(b); }
ORACLE_API float oracle_e4m3_one(uint8_t b) { return e4m3_one(b); }

ORACLE_API void oracle_to_e2m1_many(const float* v, size_t n, uint8_t* out) {
    for (size_t i = 0; i < n; ++i) out[i] = to_e2m1(v[i]);
}
ORACLE_API void oracle_to_e4m3_many(const float* v, size_t n, uint8_t* out) {
    for (size_t i = 0; i < n; ++i) out[i] = to_e4m3(v[i]);
}

ORACLE_API void oracle_bf16_to_f32(const uint16_t* src, size_t n, float* dst) {
    for (size_t i = 0; i < n; ++i) dst[i] = bf16_bits_to_f32(src[i]);
}
ORACLE_API void oracle_f32_to_bf16(const float* src, size_t n, uint16_t* dst) {
    for (size_t i = 0; i < n; ++i) dst[i] = f32_to_bf16_bits(src[i]);
}

// src/swizzle.rs:16-30 blk_mn_for_tile_m / sf_chunk_stride_for_tile_m.
ORACLE_API int oracle_blk_mn_for_tile_m(int tile_m) {
    if (tile_m < 128) return 128;
    const int cands[4] = {128, 96, 64, 32};
    for (int c : cands) {
        if (tile_m % c == 0) return c;
    }
    return -1;
}

// src/swizzle.rs:324-344 swizzled_index_of.
ORACLE_API size_t oracle_swizzled_index_of(size_t row, size_t block, size_t blocks, int tile_m, int conflict_free) {
    const size_t blk_mn = (size_t)oracle_blk_mn_for_tile_m(tile_m);
    const size_t blk_sub = blk_mn / 32;
    const size_t chunk = blk_mn * 4;
    const size_t k1_count = blocks / 4;
    const size_t m1 = row / blk_mn, k1 = block / 4, k2 = block % 4;
    if (conflict_free) {
        return (m1 * k1_count + k1) * chunk + (row % blk_mn) * 4 + k2;
    }
    const size_t m_atom = (row % 32) * blk_sub + ((row / 32) % blk_sub);
    return (m1 * k1_count + k1) * chunk + m_atom * 4 + k2;
}

ORACLE_API size_t oracle_swizzled_len_tiled(size_t rows, size_t cols, int tile_m) {
    const size_t blk_mn = (size_t)oracle_blk_mn_for_tile_m(tile_m);
    const size_t rows_padded = (rows + blk_mn - 1) / blk_mn * blk_mn;
    const size_t cols_padded = (cols + 3) / 4 * 4;
    return rows_padded * cols_padded;
}

// src/swizzle.rs:40-74 swizzle_tiled. `out` has oracle_swizzled_len_tiled bytes and is zero-filled here.
ORACLE_API void oracle_swizzle_tiled(const uint8_t* scales, size_t rows, size_t cols, int tile_m,
                                     int conflict_free, uint8_t* out) {
    const size_t blk_mn = (size_t)oracle_blk_mn_for_tile_m(tile_m);
    const size_t blk_sub = blk_mn / 32;
    const size_t chunk = blk_mn * 4;
    const size_t cols_padded = (cols + 3) / 4 * 4;
    std::memset(out, 0, oracle_swizzled_len_tiled(rows, cols, tile_m));
    const size_t k1_count = cols_padded / 4;
    for (size_t m = 0; m < rows; ++m) {
        const size_t m1 = m / blk_mn;
        for (size_t k = 0; k < cols; ++k) {
            const size_t k1 = k / 4, k2 = k % 4;
            size_t index;
            if (conflict_free) {
                index = ((m1 * k1_count + k1) * blk_mn + (m % blk_mn)) * 4 + k2;
            } else {
                const size_t m_atom = (m % 32) * blk_sub + ((m / 32) % blk_sub);
                index = (m1 * k1_count + k1) * chunk + m_atom * 4 + k2;
            }
            out[index] = scales[m * cols + k];
        }
    }
}

// src/swizzle.rs:84-104 unswizzle_tiled_conflict_free and :106-126 unswizzle_tiled.
ORACLE_API void oracle_unswizzle_tiled(const uint8_t* swizzled, size_t rows, size_t cols, int tile_m,
                                       int conflict_free, uint8_t* out) {
    const size_t blk_mn = (size_t)oracle_blk_mn_for_tile_m(tile_m);
    const size_t blk_sub = blk_mn / 32;
    const size_t chunk = blk_mn * 4;
    const size_t cols_padded = (cols + 3) / 4 * 4;
    const size_t k1_count = cols_padded / 4;
    for (size_t m = 0; m < rows; ++m) {
        const size_t m1 = m / blk_mn;
        const size_t m_atom = conflict_free ? (m % blk_mn) : ((m % 32) * blk_sub + ((m / 32) % blk_sub));
        for (size_t k = 0; k < cols; ++k) {
            const size_t k1 = k / 4, k2 = k % 4;
            out[m * cols + k] = swizzled[(m1 * k1_count + k1) * chunk + m_atom * 4 + k2];
        }
    }
}

// src/dequant.rs:20-43 dequantise: low nibble first, value * scale / global_scale.
ORACLE_API void oracle_dequantise(const uint8_t* packed, const float* scales, float global_scale,
                                  size_t cols, size_t rows, float* out) {
    const size_t scales_per_row = cols / 16;
    for (size_t row = 0; row < rows; ++row) {
        const uint8_t* prow = packed + row * (cols / 2);
        const float* srow = scales + row * scales_per_row;
        for (size_t index = 0; index < cols / 2; ++index) {
            const uint8_t byte = prow[index];
            const uint8_t lo = byte & 0x0F, hi = (byte >> 4) & 0x0F;
            const float low = (lo & 0x8) ? -kE2M1[lo & 7] : kE2M1[lo & 7];
            const float high = (hi & 0x8) ? -kE2M1[hi & 7] : kE2M1[hi & 7];
            const float scale_low = srow[(index * 2) / 16];
            const float scale_high = srow[(index * 2 + 1) / 16];
            out[row * cols + index * 2] = low * scale_low / global_scale;
            out[row * cols + index * 2 + 1] = high * scale_high / global_scale;
        }
    }
}

// src/model/norm.rs:1-12 and :14-27 (f64 accumulation; tolerance reference of the reference's tests).
ORACLE_API void oracle_model_rms_norm(const float* x, const float* weight, size_t n, float eps, float* out) {
    double ss = 0.0;
    for (size_t i = 0; i < n; ++i) ss += (double)x[i] * (double)x[i];
    const double scale = 1.0 / std::sqrt(ss / (double)n + (double)eps);
    for (size_t i = 0; i < n; ++i) out[i] = (float)((double)x[i] * scale) * (1.0f + weight[i]);
}
ORACLE_API void oracle_model_rms_norm_gated(const float* x, const float* gate, const float* weight,
                                            size_t n, float eps, float* out) {
    double ss = 0.0;
    for (size_t i = 0; i < n; ++i) ss += (double)x[i] * (double)x[i];
    const double scale = 1.0 / std::sqrt(ss / (double)n + (double)eps);
    for (size_t i = 0; i < n; ++i) {
        const float normalised = (float)((double)x[i] * scale) * weight[i];
        out[i] = normalised * (gate[i] / (1.0f + std::exp(-gate[i])));
    }
}

// src/model/attention.rs:64-80 rope_tables and kernels/elementwise.cu:446-462 rope_tables_kernel
// (same formula; libm here, libdevice there).
ORACLE_API void oracle_rope_tables(const int32_t* positions, int rows, int rotary_dim, float theta,
                                   float* cos_out, float* sin_out) {
    const int half = rotary_dim / 2;
    for (int row = 0; row < rows; ++row) {
        for (int j = 0; j < rotary_dim; ++j) {
            const int i = j % half;
            const float inv_freq = 1.0f / std::pow(theta, 2.0f * (float)i / (float)rotary_dim);
            const float f = (float)positions[row] * inv_freq;
            cos_out[(size_t)row * rotary_dim + j] = std::cos(f);
            sin_out[(size_t)row * rotary_dim + j] = std::sin(f);
        }
    }
}

// src/model/attention.rs:82-97 apply_rope via rotate_half: v[j] = v[j]*cos[j] + rot[j]*sin[j].
ORACLE_API void oracle_model_apply_rope(float* vec, const float* cos_row, const float* sin_row, int rot) {
    const int half = rot / 2;
    std::vector<float> rotated(rot);
    for (int j = 0; j < half; ++j) rotated[j] = -vec[j + half];
    for (int j = 0; j < half; ++j) rotated[j + half] = vec[j];
    for (int j = 0; j < rot; ++j) vec[j] = vec[j] * cos_row[j] + rotated[j] * sin_row[j];
}

// -------------------------------------------------------------------------------------------------
// Kernel restatements. All take activations as bf16 bit patterns (dtype 0) or f32 (dtype 1), widen
// exactly to f32, run the reference kernel's f32 arithmetic and either return f32 (out_f32), narrow
// to the activation dtype, or quantise. Rows are independent and run under `omp parallel for`.
// -------------------------------------------------------------------------------------------------

// kernels/elementwise.cu:396-407 embed_gather_kernel: out[t, :] = table[ids[t], :].
ORACLE_API void oracle_embed_gather(const void* table, const int32_t* ids, void* out, int tokens, int hidden,
                                    int dtype, int nthreads) {
    const size_t esz = dtype == 0 ? 2 : 4;
    const int nt = pick_threads(nthreads);
#pragma omp parallel for num_threads(nt) schedule(static)
    for (int t = 0; t < tokens; ++t) {
        std::memcpy((uint8_t*)out + (size_t)t * hidden * esz,
                    (const uint8_t*)table + (size_t)ids[t] * hidden * esz, (size_t)hidden * esz);
    }
}

// kernels/elementwise.cu:4-68 rms_norm_kernel. out_f32 (optional) gets the f32 result; out (optional)
// gets it narrowed to the activation dtype.
ORACLE_API void oracle_rms_norm(const void* x, const float* weight, int rows, int cols, float eps, int dtype,
                                int fma_mode, float* out_f32, void* out, int nthreads) {
    const int nt = pick_threads(nthreads);
#pragma omp parallel num_threads(nt)
    {
        std::vector<float> xin(cols), y(cols);
#pragma omp for schedule(static)
        for (int r = 0; r < rows; ++r) {
            widen_row(x, (size_t)r * cols, cols, dtype, xin.data());
            rms_norm_row(xin.data(), weight, cols, eps, fma_mode, y.data());
            if (out_f32) std::memcpy(out_f32 + (size_t)r * cols, y.data(), (size_t)cols * 4);
            if (out) narrow_row(y.data(), cols, dtype, out, (size_t)r * cols);
        }
    }
}

// kernels/elementwise.cu:144-223 rms_norm_gated_kernel (plain weight, silu(gate) multiplier).
ORACLE_API void oracle_rms_norm_gated(const void* x, const void* gate, const float* weight, int rows, int cols,
                                      float eps, int dtype, int fma_mode, float* out_f32, void* out, int nthreads) {
    const int nt = pick_threads(nthreads);
#pragma omp parallel num_threads(nt)
    {
        std::vector<float> xin(cols), gin(cols), y(cols);
#pragma omp for schedule(static)
        for (int r = 0; r < rows; ++r) {
            widen_row(x, (size_t)r * cols, cols, dtype, xin.data());
            if (gate) widen_row(gate, (size_t)r * cols, cols, dtype, gin.data());
            rms_norm_gated_row(xin.data(), gate ? gin.data() : nullptr, weight, cols, eps, fma_mode, y.data());
            if (out_f32) std::memcpy(out_f32 + (size_t)r * cols, y.data(), (size_t)cols * 4);
            if (out) narrow_row(y.data(), cols, dtype, out, (size_t)r * cols);
        }
    }
}

// kernels/elementwise.cu:225-241 swiglu_kernel: (g / (1 + exp(-g))) * u over a flat array.
ORACLE_API void oracle_swiglu(const void* gate, const void* up, size_t total, int dtype, float* out_f32, void* out,
                              int nthreads) {
    const int nt = pick_threads(nthreads);
    const size_t step = 4096;
    const long nchunks = (long)((total + step - 1) / step);
#pragma omp parallel num_threads(nt)
    {
        std::vector<float> g(step), u(step), y(step);
#pragma omp for schedule(static)
        for (long c = 0; c < nchunks; ++c) {
            const size_t off = (size_t)c * step;
            const int n = (int)std::min(step, total - off);
            widen_row(gate, off, n, dtype, g.data());
            widen_row(up, off, n, dtype, u.data());
            for (int i = 0; i < n; ++i) y[i] = silu_div_ieee(g[i]) * u[i];
            if (out_f32) std::memcpy(out_f32 + off, y.data(), (size_t)n * 4);
            if (out) narrow_row(y.data(), n, dtype, out, off);
        }
    }
}

// kernels/elementwise.cu:276-315 rope_kernel over [rows, heads, head_dim].
ORACLE_API void oracle_rope(void* out, float* out_f32, const void* x, const float* cos_t, const float* sin_t,
                            int rows, int heads, int head_dim, int rotary_dim, const int32_t* seq_start,
                            const int32_t* pos_base, const int32_t* pos_map, int dtype, int rope_fma, int nthreads) {
    const int nt = pick_threads(nthreads);
#pragma omp parallel num_threads(nt)
    {
        std::vector<float> xin(head_dim), y(head_dim);
#pragma omp for schedule(static)
        for (int r = 0; r < rows; ++r) {
            const int pos = rope_position(r, seq_start, pos_base, pos_map);
            const float* c = cos_t + (size_t)pos * rotary_dim;
            const float* s = sin_t + (size_t)pos * rotary_dim;
            for (int h = 0; h < heads; ++h) {
                const size_t base = ((size_t)r * heads + h) * head_dim;
                widen_row(x, base, head_dim, dtype, xin.data());
                rope_head(xin.data(), y.data(), c, s, head_dim, rotary_dim, rope_fma);
                if (out_f32) std::memcpy(out_f32 + base, y.data(), (size_t)head_dim * 4);
                if (out) narrow_row(y.data(), head_dim, dtype, out, base);
            }
        }
    }
}

// kernels/elementwise.cu:70-142 qk_norm_rope_kernel, generalised from head_dim 256 to any multiple
// of 4 by the unfused chain it replaces (rms_norm_kernel per head row, then rope_kernel, then the
// [q, gate] split of elementwise.cu:379-394). x rows are `rows = tokens*heads` head rows of width
// head_dim, or 2*head_dim when gate_out is wanted (q first, gate second).
ORACLE_API void oracle_qk_norm_rope(const void* x, const float* weight, const float* cos_t, const float* sin_t,
                                    void* out, float* out_f32, void* gate_out, int rows, int heads, int head_dim,
                                    int rotary_dim, float eps, const int32_t* seq_start, const int32_t* pos_base,
                                    const int32_t* pos_map, int dtype, int fma_mode, int rope_fma, int nthreads) {
    const int nt = pick_threads(nthreads);
    const size_t esz = dtype == 0 ? 2 : 4;
    const int stride = gate_out ? 2 * head_dim : head_dim;
#pragma omp parallel num_threads(nt)
    {
        std::vector<float> xin(head_dim), n(head_dim), y(head_dim);
#pragma omp for schedule(static)
        for (int row = 0; row < rows; ++row) {
            const int t = row / heads;
            widen_row(x, (size_t)row * stride, head_dim, dtype, xin.data());
            rms_norm_row(xin.data(), weight, head_dim, eps, fma_mode, n.data());
            const int pos = rope_position(t, seq_start, pos_base, pos_map);
            rope_head(n.data(), y.data(), cos_t + (size_t)pos * rotary_dim, sin_t + (size_t)pos * rotary_dim,
                      head_dim, rotary_dim, rope_fma);
            if (out_f32) std::memcpy(out_f32 + (size_t)row * head_dim, y.data(), (size_t)head_dim * 4);
            if (out) narrow_row(y.data(), head_dim, dtype, out, (size_t)row * head_dim);
            if (gate_out) {
                std::memcpy((uint8_t*)gate_out + (size_t)row * head_dim * esz,
                            (const uint8_t*)x + ((size_t)row * stride + head_dim) * esz, (size_t)head_dim * esz);
            }
        }
    }
}

// kernels/quantise.cu:6-53 quantise_nvfp4_kernel. packed: rows_padded*cols/2 bytes, scales:
// rows_padded*cols/16 bytes, rows_padded = rows rounded up to blk_mn; both fully written.
ORACLE_API void oracle_quantise_nvfp4(const void* x, uint8_t* packed, uint8_t* scales, int rows, int cols,
                                      float global_scale, int blk_mn, int chunk, int dtype, int nthreads) {
    const int nt = pick_threads(nthreads);
    const int rows_padded = round_up_i(rows, blk_mn);
#pragma omp parallel num_threads(nt)
    {
        std::vector<float> v(cols);
#pragma omp for schedule(static)
        for (int r = 0; r < rows_padded; ++r) {
            if (r < rows) {
                widen_row(x, (size_t)r * cols, cols, dtype, v.data());
                quantise_row(v.data(), r, cols, global_scale, blk_mn, chunk, packed, scales);
            } else {
                zero_pad_row(r, cols, blk_mn, chunk, packed, scales);
            }
        }
    }
}

// kernels/quantise.cu:193-271 rms_norm_quantise_nvfp4_kernel == rms_norm_kernel then
// quantise_nvfp4_kernel on the f32 result (same expressions, same summation order).
ORACLE_API void oracle_rms_norm_quantise_nvfp4(const void* x, const float* weight, uint8_t* packed, uint8_t* scales,
                                               int rows, int cols, float eps, float global_scale, int blk_mn,
                                               int chunk, int dtype, int fma_mode, int nthreads) {
    const int nt = pick_threads(nthreads);
    const int rows_padded = round_up_i(rows, blk_mn);
#pragma omp parallel num_threads(nt)
    {
        std::vector<float> xin(cols), y(cols);
#pragma omp for schedule(static)
        for (int r = 0; r < rows_padded; ++r) {
            if (r < rows) {
                widen_row(x, (size_t)r * cols, cols, dtype, xin.data());
                rms_norm_row(xin.data(), weight, cols, eps, fma_mode, y.data());
                quantise_row(y.data(), r, cols, global_scale, blk_mn, chunk, packed, scales);
            } else {
                zero_pad_row(r, cols, blk_mn, chunk, packed, scales);
            }
        }
    }
}

// kernels/quantise.cu:57-121 rms_norm_gated_quantise_nvfp4_kernel. `rows` counts head rows including
// padding (tokens_padded*vh), `rows_live` the live head rows; a token's vh head rows of width `cols`
// form one flat quantised row of width vh*cols. packed: rows*cols/2 bytes, scales: (rows/vh)*vh*cols/16.
// pre_f32 (optional, rows_live*cols) receives the f32 values before quantisation.
ORACLE_API void oracle_rms_norm_gated_quantise_nvfp4(const void* x, const void* gate, const float* weight,
                                                     uint8_t* packed, uint8_t* scales, int rows, int cols, float eps,
                                                     float global_scale, int blk_mn, int chunk, int vh,
                                                     int rows_live, int dtype, int fma_mode, float* pre_f32,
                                                     int nthreads) {
    const int nt = pick_threads(nthreads);
    const int tokens = rows / vh;
    const int flat = vh * cols;
    const int blocks = flat / 16;
#pragma omp parallel num_threads(nt)
    {
        std::vector<float> xin(cols), gin(cols), y(cols);
#pragma omp for schedule(static)
        for (int t = 0; t < tokens; ++t) {
            for (int h = 0; h < vh; ++h) {
                const int row = t * vh + h;
                uint8_t* prow = packed + (size_t)row * (cols / 2);
                if (row < rows_live) {
                    widen_row(x, (size_t)row * cols, cols, dtype, xin.data());
                    widen_row(gate, (size_t)row * cols, cols, dtype, gin.data());
                    rms_norm_gated_row(xin.data(), gin.data(), weight, cols, eps, fma_mode, y.data());
                    if (pre_f32) std::memcpy(pre_f32 + (size_t)row * cols, y.data(), (size_t)cols * 4);
                    for (int b = 0; b < cols / 16; ++b) {
                        const int block = h * (cols / 16) + b;
                        quantise_block(y.data() + b * 16, global_scale,
                                       &scales[scale_index(t, block, blocks, blk_mn, chunk)], prow + b * 8);
                    }
                } else {
                    std::memset(prow, 0, (size_t)cols / 2);
                    for (int b = 0; b < cols / 16; ++b) {
                        scales[scale_index(t, h * (cols / 16) + b, blocks, blk_mn, chunk)] = 0;
                    }
                }
            }
        }
    }
}

// kernels/quantise.cu:523-591 swiglu_quantise_nvfp4_kernel == swiglu_kernel then quantise_nvfp4_kernel.
// pre_f32 (optional, rows*cols) receives the f32 values before quantisation.
ORACLE_API void oracle_swiglu_quantise_nvfp4(const void* gate, const void* up, uint8_t* packed, uint8_t* scales,
                                             int rows, int cols, float global_scale, int blk_mn, int chunk,
                                             int dtype, float* pre_f32, int nthreads) {
    const int nt = pick_threads(nthreads);
    const int rows_padded = round_up_i(rows, blk_mn);
#pragma omp parallel num_threads(nt)
    {
        std::vector<float> g(cols), u(cols), y(cols);
#pragma omp for schedule(static)
        for (int r = 0; r < rows_padded; ++r) {
            if (r < rows) {
                widen_row(gate, (size_t)r * cols, cols, dtype, g.data());
                widen_row(up, (size_t)r * cols, cols, dtype, u.data());
                for (int i = 0; i < cols; ++i) y[i] = silu_div_ieee(g[i]) * u[i];
                if (pre_f32) std::memcpy(pre_f32 + (size_t)r * cols, y.data(), (size_t)cols * 4);
                quantise_row(y.data(), r, cols, global_scale, blk_mn, chunk, packed, scales);
            } else {
                zero_pad_row(r, cols, blk_mn, chunk, packed, scales);
            }
        }
    }
}

// kernels/attention_mma.cu:118-171 to_bf16_kernel / to_bf16_scatter_kernel: token t = i / stride of x goes to
// cache row pos_map[t], or (no map) to t + *off_tokens; out is bf16 (round to nearest even).
ORACLE_API void oracle_to_bf16_rows(const void* x, uint16_t* out, size_t n, const int32_t* pos_map,
                                    const int32_t* off_tokens, int stride, int dtype) {
    const size_t base = (!pos_map && off_tokens) ? (size_t)off_tokens[0] * (size_t)stride : 0;
    for (size_t i = 0; i < n; ++i) {
        float v;
        widen_row(x, i, 1, dtype, &v);
        size_t dst = base + i;
        if (pos_map) {
            const size_t t = i / (size_t)stride;
            dst = (size_t)pos_map[t] * (size_t)stride + (i - t * (size_t)stride);
        }
        out[dst] = f32_to_bf16_bits(v);
    }
}

// kernels/elementwise.cu:344-359 sigmoid_mul_kernel: x * 1.0f / (1.0f + exp(-g)) for whole quads and
// x * (1.0f / (1.0f + exp(-g))) for the total % 4 tail (exp stands in for __expf, see the header).
inline float sigmoid_mul_main(float x, float g) { return x * 1.0f / (1.0f + std::exp(-g)); }
inline float sigmoid_mul_tail(float x, float g) { return x * (1.0f / (1.0f + std::exp(-g))); }

ORACLE_API void oracle_sigmoid_mul(const void* x, const void* gate, size_t total, int dtype, float* out_f32, void* out,
                                   int nthreads) {
    const int nt = pick_threads(nthreads);
    const size_t step = 4096;
    const long nchunks = (long)((total + step - 1) / step);
    const size_t whole = total & ~(size_t)3;
#pragma omp parallel num_threads(nt)
    {
        std::vector<float> g(step), v(step), y(step);
#pragma omp for schedule(static)
        for (long c = 0; c < nchunks; ++c) {
            const size_t off = (size_t)c * step;
            const int n = (int)std::min(step, total - off);
            widen_row(gate, off, n, dtype, g.data());
            widen_row(x, off, n, dtype, v.data());
            for (int i = 0; i < n; ++i) {
                y[i] = (off + i < whole) ? sigmoid_mul_main(v[i], g[i]) : sigmoid_mul_tail(v[i], g[i]);
            }
            if (out_f32) std::memcpy(out_f32 + off, y.data(), (size_t)n * 4);
            if (out) narrow_row(y.data(), n, dtype, out, off);
        }
    }
}

// sigmoid_mul_kernel then quantise_nvfp4_kernel (kernels/quantise.cu:6-53) on dense [rows, cols].
ORACLE_API void oracle_sigmoid_mul_quantise_nvfp4(const void* x, const void* gate, uint8_t* packed, uint8_t* scales,
                                                  int rows, int cols, float global_scale, int blk_mn, int chunk,
                                                  int dtype, float* pre_f32, int nthreads) {
    const int nt = pick_threads(nthreads);
    const int rows_padded = round_up_i(rows, blk_mn);
#pragma omp parallel num_threads(nt)
    {
        std::vector<float> g(cols), v(cols), y(cols);
#pragma omp for schedule(static)
        for (int r = 0; r < rows_padded; ++r) {
            if (r < rows) {
                widen_row(gate, (size_t)r * cols, cols, dtype, g.data());
                widen_row(x, (size_t)r * cols, cols, dtype, v.data());
                for (int i = 0; i < cols; ++i) y[i] = sigmoid_mul_main(v[i], g[i]);
                if (pre_f32) std::memcpy(pre_f32 + (size_t)r * cols, y.data(), (size_t)cols * 4);
                quantise_row(y.data(), r, cols, global_scale, blk_mn, chunk, packed, scales);
            } else {
                zero_pad_row(r, cols, blk_mn, chunk, packed, scales);
            }
        }
    }
}

// kernels/head.cu:117-129 add_kernel.
ORACLE_API void oracle_add(const void* a, const void* b, size_t total, int dtype, float* out_f32, void* out) {
    for (size_t i = 0; i < total; ++i) {
        float x, y;
        widen_row(a, i, 1, dtype, &x);
        widen_row(b, i, 1, dtype, &y);
        const float s = x + y;
        if (out_f32) out_f32[i] = s;
        if (out) narrow_row(&s, 1, dtype, out, i);
    }
}

// ---------------------------------------------------------------------------------------------
// FP8 (E4M3) activation quantisers (kernels/quantise.cu:123-191, 273-514). Shared row recipe:
// scale = amax / 448 (amax with fmaxf semantics), the row's scale word is the upper half of that f32,
// code = to_e4m3(|v| * inv) | sign with inv = scale > 0 ? 1 / scale : 0.
// ---------------------------------------------------------------------------------------------
inline void fp8_quantise_span(const float* const* parts, const int* lens, int nparts, uint8_t* const* outs,
                              uint16_t* scale_word) {
    float amax = 0.0f;
    for (int p = 0; p < nparts; ++p) {
        for (int i = 0; i < lens[p]; ++i) amax = std::fmax(amax, std::fabs(parts[p][i]));
    }
    const float scale = amax / 448.0f;
    uint32_t bits;
    std::memcpy(&bits, &scale, 4);
    *scale_word = (uint16_t)(bits >> 16);
    const float inv = (scale > 0.0f) ? 1.0f / scale : 0.0f;
    for (int p = 0; p < nparts; ++p) {
        if (!outs[p]) continue;
        for (int i = 0; i < lens[p]; ++i) {
            const float t = parts[p][i];
            outs[p][i] = (uint8_t)(to_e4m3(std::fabs(t) * inv) | ((t < 0.0f) ? 0x80u : 0x00u));
        }
    }
}

// mode 0: quantise_fp8_kernel (:454-514, every row from its own values); 1: swiglu_quantise_fp8_kernel
// (:390-452, a = gate, b = up); 2: rms_norm_fp8_bf16_kernel (:273-381, bf_out optional bf16 twin).
ORACLE_API void oracle_fp8_rows(int mode, const void* a, const void* b, const float* weight, uint8_t* out,
                                uint16_t* scales, uint16_t* bf_out, int rows, int cols, float eps, int dtype,
                                int fma_mode, int nthreads) {
    const int nt = pick_threads(nthreads);
#pragma omp parallel num_threads(nt)
    {
        std::vector<float> x(cols), u(cols), y(cols);
#pragma omp for schedule(static)
        for (int r = 0; r < rows; ++r) {
            widen_row(a, (size_t)r * cols, cols, dtype, x.data());
            if (mode == 1) {
                widen_row(b, (size_t)r * cols, cols, dtype, u.data());
                for (int i = 0; i < cols; ++i) y[i] = silu_div_ieee(x[i]) * u[i];
            } else if (mode == 2) {
                rms_norm_row(x.data(), weight, cols, eps, fma_mode, y.data());
                if (bf_out) {
                    for (int i = 0; i < cols; ++i) bf_out[(size_t)r * cols + i] = f32_to_bf16_bits(y[i]);
                }
            } else {
                y = x;
            }
            const float* parts[1] = {y.data()};
            uint8_t* outs[1] = {out + (size_t)r * cols};
            fp8_quantise_span(parts, &cols, 1, outs, scales + r);
        }
    }
}

// rms_norm_gated_quantise_fp8_kernel (:123-191): one scale per token over its vh head rows; head rows
// >= rows_live hold no data (they add 0 to the amax and are not written).
ORACLE_API void oracle_rms_norm_gated_quantise_fp8(const void* x, const void* gate, const float* weight, uint8_t* out,
                                                   uint16_t* scales, int rows, int cols, float eps, int vh,
                                                   int rows_live, int dtype, int fma_mode, int nthreads) {
    const int nt = pick_threads(nthreads);
    const int tokens = rows / vh;
#pragma omp parallel num_threads(nt)
    {
        std::vector<float> xin(cols), gin(cols), y((size_t)vh * cols);
        std::vector<const float*> parts(vh);
        std::vector<uint8_t*> outs(vh);
        std::vector<int> lens(vh);
#pragma omp for schedule(static)
        for (int t = 0; t < tokens; ++t) {
            for (int h = 0; h < vh; ++h) {
                const int row = t * vh + h;
                float* yh = y.data() + (size_t)h * cols;
                parts[h] = yh;
                lens[h] = cols;
                if (row < rows_live) {
                    widen_row(x, (size_t)row * cols, cols, dtype, xin.data());
                    widen_row(gate, (size_t)row * cols, cols, dtype, gin.data());
                    rms_norm_gated_row(xin.data(), gin.data(), weight, cols, eps, fma_mode, yh);
                    outs[h] = out + (size_t)row * cols;
                } else {
                    std::fill(yh, yh + cols, 0.0f);
                    outs[h] = nullptr;
                }
            }
            fp8_quantise_span(parts.data(), lens.data(), vh, outs.data(), scales + t);
        }
    }
}

// kernels/elementwise.cu:243-274 causal_conv_silu_kernel: taps in ascending order, each added by a fused multiply-add
// (the reference build contracts `acc += w * x`), taps before the token's sequence start taken from the slot's history
// when there is one and skipped otherwise; silu with exp and the IEEE quotient (exp stands in for __expf).
ORACLE_API void oracle_causal_conv_silu(const void* x, const float* w, float* out_f32, void* out, int rows, int channels,
                                        int k, const int32_t* seq_start, const void* history, const int32_t* slot_map,
                                        int dtype, float* acc_f32, int nthreads) {
    const int nt = pick_threads(nthreads);
#pragma omp parallel for schedule(static) num_threads(nt)
    for (int t = 0; t < rows; ++t) {
        const int lo = seq_start ? seq_start[t] : 0;
        for (int ch = 0; ch < channels; ++ch) {
            float acc = 0.0f;
            for (int tap = 0; tap < k; ++tap) {
                const int src = t - (k - 1) + tap;
                float v;
                if (src >= lo) {
                    widen_row(x, (size_t)src * channels + ch, 1, dtype, &v);
                } else if (history && src >= lo - (k - 1)) {
                    const int slot = slot_map ? slot_map[t] : 0;
                    widen_row(history, ((size_t)slot * (k - 1) + (size_t)(src - lo + (k - 1))) * channels + ch, 1, dtype, &v);
                } else {
                    continue;
                }
                acc = std::fmaf(w[(size_t)ch * k + tap], v, acc);
            }
            const size_t i = (size_t)t * channels + ch;
            if (acc_f32) acc_f32[i] = acc;
            const float y = silu_div_ieee(acc);
            if (out_f32) out_f32[i] = y;
            if (out) narrow_row(&y, 1, dtype, out, i);
        }
    }
}

// kernels/elementwise.cu:361-377 gdn_gates_kernel (exp / log1p stand in for the device's __expf / log1pf).
ORACLE_API void oracle_gdn_gates(const void* a, const void* b, const float* a_log, const float* dt_bias, float* decay,
                                 float* beta, int tokens, int heads, int dtype) {
    for (int i = 0; i < tokens * heads; ++i) {
        const int h = i % heads;
        float av, bv;
        widen_row(a, (size_t)i, 1, dtype, &av);
        widen_row(b, (size_t)i, 1, dtype, &bv);
        beta[i] = 1.0f / (1.0f + std::exp(-bv));
        const float xv = av + dt_bias[h];
        const float sp = (xv > 20.0f) ? xv : std::log1p(std::exp(xv));
        decay[i] = -std::exp(a_log[h]) * sp;
    }
}

// kernels/gdn_chunk.cu:1176-1239 gdn_prep_kernel (and the second half of gdn_conv_prep_kernel, :1109-1172): the
// convolved row [q | k | v] of each token becomes the chunked scan's operands. Per head: lane l of 32 adds the
// squares of p = l, l + 32, ... by fused multiply-add, the 32 partial sums go through the xor tree 16 .. 1;
// value = x * rsqrt(sum + 1e-6) (q also times q_scale), split as hi = rn_bf16(value), lo = rn_bf16(value - hi)
// (split_bf16, :13-17) and stored at the swizzled offset of :1211-1216; k heads repeat heads / kh times; kn is the
// normalised k in f32, v_out the v part of the row. 1 / sqrtf stands in for the device's rsqrtf (within 2 ulp).
ORACLE_API void oracle_gdn_prep(const void* mixed, float* v_out, uint16_t* q_hi, uint16_t* q_lo, uint16_t* k_hi,
                                uint16_t* k_lo, float* kn, int seq_len, int heads, int kh, int kd, int conv_dim,
                                float q_scale, int dtype) {
    const int nchunks = (seq_len + 63) / 64;
    const int ratio = heads / kh;
    std::vector<float> row((size_t)conv_dim);
    for (int t = 0; t < seq_len; ++t) {
        widen_row(mixed, (size_t)t * conv_dim, conv_dim, dtype, row.data());
        for (int h = 0; h < kh; ++h) {
            for (int which = 0; which < 2; ++which) {   // 0: q, 1: k
                const float* x = row.data() + (size_t)which * kh * kd + (size_t)h * kd;
                float lane[32];
                for (int l = 0; l < 32; ++l) {
                    float s = 0.0f;
                    for (int p = l; p < kd; p += 32) s = std::fmaf(x[p], x[p], s);
                    lane[l] = s;
                }
                for (int off = 16; off > 0; off >>= 1) {
                    float next[32];
                    for (int l = 0; l < 32; ++l) next[l] = lane[l] + lane[l ^ off];
                    std::memcpy(lane, next, sizeof(lane));
                }
                float r = 1.0f / std::sqrt(lane[0] + 1e-6f);
                if (which == 0) r = r * q_scale;
                for (int rep = 0; rep < ratio; ++rep) {
                    const int he = h * ratio + rep;
                    const size_t idx = (size_t)he * nchunks + (size_t)(t / 64);
                    const int rr = t % 64;
                    for (int p = 0; p < kd; ++p) {
                        const int tile = p / 64, c = p % 64, seg = c / 8, e = c % 8;
                        const size_t off = ((idx * (size_t)(kd / 64) + tile) * (64 * 128) + (size_t)rr * 128 +
                                            (size_t)((seg ^ (rr % 8)) * 16 + e * 2)) / 2;   // in bf16 units
                        const float val = x[p] * r;
                        const uint16_t hi = f32_to_bf16_bits(val);
                        const uint16_t lo = f32_to_bf16_bits(val - bf16_bits_to_f32(hi));
                        (which == 0 ? q_hi : k_hi)[off] = hi;
                        (which == 0 ? q_lo : k_lo)[off] = lo;
                        if (which == 1) kn[((size_t)t * heads + he) * kd + p] = val;
                    }
                }
            }
        }
        std::memcpy(v_out + (size_t)t * heads * kd, row.data() + (size_t)2 * kh * kd, sizeof(float) * (size_t)heads * kd);
    }
}

// Quantise rows of f32 values that were produced elsewhere (for instance a GPU f32 result), so a
// test can separate "same pre-quantisation values" from "same quantiser".
ORACLE_API void oracle_quantise_rows_f32(const float* v, uint8_t* packed, uint8_t* scales, int rows, int cols,
                                         float global_scale, int blk_mn, int chunk, int nthreads) {
    oracle_quantise_nvfp4(v, packed, scales, rows, cols, global_scale, blk_mn, chunk, 1, nthreads);
}
