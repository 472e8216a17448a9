// Elementwise kernels in front of the Gated-DeltaNet scan: the causal depthwise convolution + silu driven by
// the per-token maps (seq_start, slot_map) and the convolution history, the history save, the gate transform,
// and the q/k/v splitting copies (kernels/elementwise.cu:243-274, 361-445, 463-485). T = Bf16 or F32 is the
// storage type of the activations; weights, biases and the two gate outputs are f32.
#pragma once

#include "kernels_fp8.cuh"   // load8<T>

namespace clef {

template <typename T>
__device__ __forceinline__ void store8(typename T::storage* p, const float* v);
template <>
__device__ __forceinline__ void store8<Bf16>(uint16_t* p, const float* v) {
    stg_v4(p, make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7])));
}
template <>
__device__ __forceinline__ void store8<F32>(float* p, const float* v) {
    stg_v4(p, make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3])));
    stg_v4(p + 4, make_uint4(__float_as_uint(v[4]), __float_as_uint(v[5]), __float_as_uint(v[6]), __float_as_uint(v[7])));
}

// 8 consecutive activations as loaded (16 or 32 bytes), widened later.
template <typename T>
struct Raw8;
template <>
struct Raw8<Bf16> {
    uint4 a = make_uint4(0u, 0u, 0u, 0u);
};
template <>
struct Raw8<F32> {
    uint4 a = make_uint4(0u, 0u, 0u, 0u), b = make_uint4(0u, 0u, 0u, 0u);
};
template <typename T>
__device__ __forceinline__ Raw8<T> load8_raw(const typename T::storage* p);
template <>
__device__ __forceinline__ Raw8<Bf16> load8_raw<Bf16>(const uint16_t* p) {
    Raw8<Bf16> r;
    r.a = ldg_stream_v4(p);
    return r;
}
template <>
__device__ __forceinline__ Raw8<F32> load8_raw<F32>(const float* p) {
    Raw8<F32> r;
    r.a = ldg_stream_v4(p);
    r.b = ldg_stream_v4(p + 4);
    return r;
}
template <typename T>
__device__ __forceinline__ void unpack8(const Raw8<T>& r, float* v);
template <>
__device__ __forceinline__ void unpack8<Bf16>(const Raw8<Bf16>& r, float* v) {
    v[0] = bf16_lo(r.a.x), v[1] = bf16_hi(r.a.x), v[2] = bf16_lo(r.a.y), v[3] = bf16_hi(r.a.y);
    v[4] = bf16_lo(r.a.z), v[5] = bf16_hi(r.a.z), v[6] = bf16_lo(r.a.w), v[7] = bf16_hi(r.a.w);
}
template <>
__device__ __forceinline__ void unpack8<F32>(const Raw8<F32>& r, float* v) {
    v[0] = __uint_as_float(r.a.x), v[1] = __uint_as_float(r.a.y), v[2] = __uint_as_float(r.a.z), v[3] = __uint_as_float(r.a.w);
    v[4] = __uint_as_float(r.b.x), v[5] = __uint_as_float(r.b.y), v[6] = __uint_as_float(r.b.z), v[7] = __uint_as_float(r.b.w);
}

// ---------------------------------------------------------------------------------------------
// causal_conv_silu (kernels/elementwise.cu:243-274): out[t, c] = silu(sum over taps of w[c, tap] * x[t - (K-1) + tap, c]),
// the taps added in ascending order by fused multiply-add (the reference build contracts `acc += w * x`), a tap
// whose source row lies before the token's sequence start (seq_start[t]) taken from the convolution history of
// the token's slot (history[slot_map[t]], K - 1 rows per slot) when there is one and skipped otherwise;
// silu(a) = a / (1 + __expf(-a)) with the IEEE quotient.
// A thread owns 4 channels and R consecutive rows (plus the K - 1 rows above them), so every x value is loaded
// once per strip. channels % 8 == 0.
// ---------------------------------------------------------------------------------------------
// One output value by the literal expression, reading its taps from global memory: the general kernel's element and
// the tuned kernel's path for strips that touch a sequence start.
template <typename T>
__device__ __forceinline__ float causal_conv_silu_element(const typename T::storage* __restrict__ x, const float* __restrict__ w,
                                                          int t, int ch, int channels, int k, const int* __restrict__ seq_start,
                                                          const typename T::storage* __restrict__ history,
                                                          const int* __restrict__ slot_map) {
    const int lo = seq_start ? seq_start[t] : 0;
    float acc = 0.0f;
    for (int tap = 0; tap < k; ++tap) {
        const int src = t - (k - 1) + tap;
        float v;
        if (src >= lo) {
            v = load_scalar<T>(x + (size_t)src * channels + ch);
        } else if (history && src >= lo - (k - 1)) {
            const int slot = slot_map ? slot_map[t] : 0;
            v = load_scalar<T>(history + ((size_t)slot * (k - 1) + (size_t)(src - lo + (k - 1))) * channels + ch);
        } else {
            continue;
        }
        acc = __fmaf_rn(w[(size_t)ch * k + tap], v, acc);
    }
    return silu_ieee_div(acc);
}

// Rows [t0, t1) of 8 channels with every tap tested against the row's sequence start, out of line; a tap's 8
// values are one vector load from x or from the history.
template <typename T, int K>
static __device__ __noinline__ void causal_conv_silu_strip_literal(typename T::storage* __restrict__ out,
                                                                   const typename T::storage* __restrict__ x,
                                                                   const float* __restrict__ w, int t0, int t1, int c0,
                                                                   int channels, const int* __restrict__ seq_start,
                                                                   const typename T::storage* __restrict__ history,
                                                                   const int* __restrict__ slot_map) {
#pragma unroll 2
    for (int t = t0; t < t1; ++t) {
        const int lo = seq_start ? seq_start[t] : 0;
        constexpr int k = K;
        const int slot = (history && slot_map) ? slot_map[t] : 0;
        Raw8<T> raw[K];   // the K taps are requested together
        bool live[K];
#pragma unroll
        for (int tap = 0; tap < K; ++tap) {
            const int src = t - (k - 1) + tap;
            const typename T::storage* p = nullptr;
            if (src >= lo) {
                p = x + (size_t)src * channels + c0;
            } else if (history && src >= lo - (k - 1)) {
                p = history + ((size_t)slot * (k - 1) + (size_t)(src - lo + (k - 1))) * channels + c0;
            }
            live[tap] = p != nullptr;
            if (live[tap]) raw[tap] = load8_raw<T>(p);
        }
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int tap = 0; tap < K; ++tap) {
            if (live[tap]) {
                float v[8];
                unpack8<T>(raw[tap], v);
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = __fmaf_rn(__ldg(w + (size_t)(c0 + j) * k + tap), v[j], acc[j]);
            }
        }
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = silu_ieee_div(acc[j]);
        store8<T>(out + (size_t)t * channels + c0, o);
    }
}

// 4 channels of a row as loaded (8 bytes of bf16, 16 of f32), widened, and stored.
template <typename T>
struct Raw4;
template <>
struct Raw4<Bf16> {
    uint2 d;
};
template <>
struct Raw4<F32> {
    uint4 d;
};
__device__ __forceinline__ Raw4<Bf16> load4_raw(const uint16_t* p) { return Raw4<Bf16>{ldg_stream_v2(p)}; }
__device__ __forceinline__ Raw4<F32> load4_raw(const float* p) { return Raw4<F32>{ldg_stream_v4(p)}; }
__device__ __forceinline__ void unpack4(const Raw4<Bf16>& r, float* v) {
    v[0] = bf16_lo(r.d.x), v[1] = bf16_hi(r.d.x), v[2] = bf16_lo(r.d.y), v[3] = bf16_hi(r.d.y);
}
__device__ __forceinline__ void unpack4(const Raw4<F32>& r, float* v) {
    v[0] = __uint_as_float(r.d.x), v[1] = __uint_as_float(r.d.y), v[2] = __uint_as_float(r.d.z), v[3] = __uint_as_float(r.d.w);
}
__device__ __forceinline__ void store4(uint16_t* p, const float* v) {
    stg_v2(p, make_uint2(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3])));
}
__device__ __forceinline__ void store4(float* p, const float* v) {
    stg_v4(p, make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3])));
}

// 4 channels per thread (8-byte loads and stores of bf16, 16-byte ones of f32): half the registers of an 8-channel
// form, so more warps are resident to overlap one thread's load phase with another's arithmetic. A strip that lies inside the
// matrix with its halo and has no tap before a sequence start runs without any per-row or per-tap test; every
// other strip (the first, a ragged last one, one holding a sequence start) takes the literal path. The arithmetic
// is scalar on purpose: packed multiply-adds cost more register-pair moves here than they save (measured: 105
// against 99 instructions per row of 4 values).
// CH: the channel count when it is known at compile time (0: the `channels` argument). With a constant row stride the
// 19 row addresses of a strip are immediate offsets from one base register instead of a multiply-add each.
template <int K, int R, int MIN_CTAS, int CH = 0, typename T = Bf16>
__global__ void __launch_bounds__(kCtaThreads, MIN_CTAS)
causal_conv_silu_c4_kernel(typename T::storage* __restrict__ out, const typename T::storage* __restrict__ x,
                           const float* __restrict__ w, int rows, int channels_arg, const int* __restrict__ seq_start,
                           const typename T::storage* __restrict__ history, const int* __restrict__ slot_map,
                           FastDiv cvecs_div) {
    constexpr int kLineThreads = 32 / T::kBytes;   // threads whose 4 channels share a 128-byte line
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    const int channels = CH ? CH : channels_arg;
    const uint32_t cvecs = CH ? (uint32_t)(CH / 4) : cvecs_div.d;   // channels / 4
    const uint32_t strips = ((uint32_t)rows + R - 1) / R;
    const uint32_t total = strips * cvecs;
    const uint32_t step = gridDim.x * kCtaThreads;
    const bool starts_vector = R == 8 && (reinterpret_cast<uintptr_t>(seq_start) & 15) == 0;
    for (uint32_t idx = blockIdx.x * kCtaThreads + threadIdx.x; idx < total; idx += step) {
        const uint32_t strip = CH ? idx / (uint32_t)(CH / 4) : fast_div(idx, cvecs_div);
        const int c0 = (int)(idx - strip * cvecs) * 4;
        const int t0 = (int)strip * R;
        bool plain = t0 >= K - 1 && t0 + R <= rows;   // every row of the strip and of its halo exists
        Raw4<T> raw[R + K - 1];
        float wt[4][K];
        if (plain) {
            const typename T::storage* base = x + (size_t)(t0 - (K - 1)) * channels + c0;
#pragma unroll
            for (int i = 0; i < R + K - 1; ++i) raw[i] = load4_raw(base + (size_t)i * channels);
            {   // the strip this thread handles next, named to L2 (one thread per 128-byte line): 70.5 -> 68.9 us with bf16
                const uint32_t nidx = idx + step;
                if (nidx < total && (threadIdx.x & (kLineThreads - 1)) == 0) {
                    const uint32_t nstrip = CH ? nidx / (uint32_t)(CH / 4) : fast_div(nidx, cvecs_div);
                    const typename T::storage* nb = x + (size_t)(nstrip * R) * channels + (nidx - nstrip * cvecs) * 4;
#pragma unroll
                    for (int i = 0; i < R; ++i) prefetch_l2(nb + (size_t)i * channels);
                }
            }
            if (K == 4) {   // a channel's four taps are one 16-byte load
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float4 t4 = __ldg(reinterpret_cast<const float4*>(w) + (c0 + j));
                    wt[j][0] = t4.x, wt[j][1] = t4.y, wt[j][2 % K] = t4.z, wt[j][3 % K] = t4.w;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
#pragma unroll
                    for (int tap = 0; tap < K; ++tap) wt[j][tap] = __ldg(w + (size_t)(c0 + j) * K + tap);
                }
            }
            if (seq_start) {
                const int lim = t0 - (K - 1);
                if (starts_vector) {   // the 8 sequence starts as two 16-byte loads
                    const int4 a = __ldg(reinterpret_cast<const int4*>(seq_start + t0));
                    const int4 b = __ldg(reinterpret_cast<const int4*>(seq_start + t0) + 1);
                    plain = a.x <= lim && a.y <= lim + 1 && a.z <= lim + 2 && a.w <= lim + 3 && b.x <= lim + 4 &&
                            b.y <= lim + 5 && b.z <= lim + 6 && b.w <= lim + 7;
                } else {
#pragma unroll
                    for (int r = 0; r < R; ++r) plain &= __ldg(seq_start + t0 + r) <= lim + r;
                }
            }
        }
        if (!plain) {
            if ((c0 & 4) == 0) {   // the literal path works on 8 channels: the even thread of a pair does both halves
                causal_conv_silu_strip_literal<T, K>(out, x, w, t0, min(t0 + R, rows), c0, channels, seq_start, history, slot_map);
            }
            continue;
        }
        float xs[R + K - 1][4];   // every row of the strip widened once; row r reads xs[r .. r + K - 1]
#pragma unroll
        for (int i = 0; i < R + K - 1; ++i) unpack4(raw[i], xs[i]);
        typename T::storage* orow = out + (size_t)t0 * channels + c0;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            float a4[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                a4[j] = 0.0f;
#pragma unroll
                for (int tap = 0; tap < K; ++tap) a4[j] = __fmaf_rn(wt[j][tap], xs[r + tap][j], a4[j]);
            }
            const float m = fmaxf_nan(max3_abs_nan(fabsf(a4[0]), a4[1], a4[2]), fabsf(a4[3]));
            float o4[4];
            if (m <= kSiluFastMaxAbs) {   // false for a NaN too
#pragma unroll
                for (int j = 0; j < 4; ++j) o4[j] = silu_ieee_refined_f32(a4[j]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) o4[j] = silu_ieee_div(a4[j]);
            }
            store4(orow + (size_t)r * channels, o4);
        }
    }
}

// The same arithmetic for any tap count and any channel count: one thread per (row, channel).
template <typename T>
__global__ void __launch_bounds__(kCtaThreads)
causal_conv_silu_generic_kernel(typename T::storage* __restrict__ out, const typename T::storage* __restrict__ x,
                                const float* __restrict__ w, int rows, int channels, int k,
                                const int* __restrict__ seq_start, const typename T::storage* __restrict__ history,
                                const int* __restrict__ slot_map) {
    const size_t total = (size_t)rows * channels;
    const size_t step = (size_t)gridDim.x * kCtaThreads;
    for (size_t idx = (size_t)blockIdx.x * kCtaThreads + threadIdx.x; idx < total; idx += step) {
        const int t = (int)(idx / channels);
        const int ch = (int)(idx - (size_t)t * channels);
        store_scalar<T>(out + idx, causal_conv_silu_element<T>(x, w, t, ch, channels, k, seq_start, history, slot_map));
    }
}

// conv_hist_save (kernels/elementwise.cu:463-485): for each (row, slot) pair of `saves`, the K - 1 rows ending at
// `row` become the history of `slot`. One CTA per pair, 16 bytes per thread per step.
template <typename T>
__global__ void __launch_bounds__(kCtaThreads)
conv_hist_save_kernel(const typename T::storage* __restrict__ src, typename T::storage* __restrict__ hist,
                      const int* __restrict__ saves, int n_saves, int rows, int k, int channels) {
    const int i = blockIdx.x;
    if (i >= n_saves) return;
    const int row = saves[2 * i], slot = saves[2 * i + 1];
    const int hist_rows = k - 1;
    const size_t per_slot = (size_t)hist_rows * channels;
    const int first = row + 1 - hist_rows;
    if (row < 0 || first < 0 || row >= rows) return;
    const typename T::storage* s = src + (size_t)first * channels;
    typename T::storage* d = hist + (size_t)slot * per_slot;
    constexpr int kPer = 16 / T::kBytes;
    const size_t vecs = per_slot / kPer;
    for (size_t v = threadIdx.x; v < vecs; v += kCtaThreads) {
        stg_v4(d + v * kPer, ldg_stream_v4(s + v * kPer));
    }
    for (size_t c = vecs * kPer + threadIdx.x; c < per_slot; c += kCtaThreads) {
        d[c] = s[c];
    }
}

// ---------------------------------------------------------------------------------------------
// gdn_prep (kernels/gdn_chunk.cu:1176-1239): the convolved row [q | k | v] of a token becomes the operands of the
// chunked GDN scan. Every q and k head (kd = 128) is L2-normalised, rsqrtf(sum of squares + 1e-6), q additionally
// scaled by q_scale; the sum is the reference's: lane l adds p = l, l + 32, l + 64, l + 96 in order by fused
// multiply-add, then the xor tree 16 .. 1. Each value v is stored as the bf16 pair hi = rn(v), lo = rn(v - hi) in
// the scan's layout: per (expanded head, 64-token chunk) two 64-column tiles of 64 rows x 128 bytes, the 16-byte
// segment index xor-ed with row % 8 (kernels/gdn_chunk.cu:35-40); k heads are repeated heads / kh times
// (repeat_interleave), normalised k also goes out as f32 (kn), v is copied as f32. One warp per (token, k head).
// Rows of the last chunk past seq_len are written as zeros, so the caller need not clear the hi / lo buffers
// (the reference allocates them zeroed, src/cuda/mod.rs:3615-3618).
// ---------------------------------------------------------------------------------------------
constexpr int kGdnChunk = 64, kGdnKd = 128, kGdnTileCols = 64, kGdnRowBytes = 128;

__device__ __forceinline__ size_t gdn_operand_offset(size_t chunk_index, int row_in_chunk, int p) {
    const int tile = p / kGdnTileCols, c = p - tile * kGdnTileCols;
    const int seg = c >> 3, e = c & 7;
    return (chunk_index * (kGdnKd / kGdnTileCols) + tile) * (size_t)(kGdnChunk * kGdnRowBytes) +
           (size_t)row_in_chunk * kGdnRowBytes + (size_t)((seg ^ (row_in_chunk & 7)) * 16 + e * 2);
}

__device__ __forceinline__ void store_bf16_hi_lo(float v, uint8_t* hi, uint8_t* lo, size_t off) {
    const uint32_t h = pack_bf16x2(v, 0.0f) & 0xffffu;
    *reinterpret_cast<uint16_t*>(hi + off) = (uint16_t)h;
    *reinterpret_cast<uint16_t*>(lo + off) = (uint16_t)(pack_bf16x2(__fsub_rn(v, __uint_as_float(h << 16)), 0.0f) & 0xffffu);
}

template <typename T>
__device__ __forceinline__ void load4_as_f32(const typename T::storage* p, float* v);
template <>
__device__ __forceinline__ void load4_as_f32<Bf16>(const uint16_t* p, float* v) {
    const uint2 raw = ldg_stream_v2(p);
    v[0] = bf16_lo(raw.x), v[1] = bf16_hi(raw.x), v[2] = bf16_lo(raw.y), v[3] = bf16_hi(raw.y);
}
template <>
__device__ __forceinline__ void load4_as_f32<F32>(const float* p, float* v) {
    const uint4 raw = ldg_stream_v4(p);
    v[0] = __uint_as_float(raw.x), v[1] = __uint_as_float(raw.y), v[2] = __uint_as_float(raw.z), v[3] = __uint_as_float(raw.w);
}

// All index arithmetic is 32-bit with multiply-high divisions (the launcher refuses sizes beyond 2^31 items): a
// 64-bit division by a run-time value per item cost more instructions than the item's own work.
template <typename T>
__global__ void __launch_bounds__(kCtaThreads)
gdn_prep_kernel(const typename T::storage* __restrict__ mixed, float* __restrict__ v_out, uint8_t* __restrict__ q_hi,
                uint8_t* __restrict__ q_lo, uint8_t* __restrict__ k_hi, uint8_t* __restrict__ k_lo, float* __restrict__ kn,
                int seq_len, int heads, int kh, int nchunks, int conv_dim, float q_scale, FastDiv kh_div, FastDiv vvec_div) {
    const int lane = threadIdx.x & 31;
    const uint32_t warp0 = (blockIdx.x * kCtaThreads + threadIdx.x) >> 5;
    const uint32_t warps = gridDim.x * (kCtaThreads / 32);
    const int ratio = heads / kh;
    const uint32_t head_items = (uint32_t)nchunks * kGdnChunk * (uint32_t)kh;   // pad rows of the last chunk included
    for (uint32_t item = warp0; item < head_items; item += warps) {
        const uint32_t t = fast_div(item, kh_div);
        const int h = (int)(item - t * (uint32_t)kh);
        const bool live = t < (uint32_t)seq_len;
        // Each lane reads its head rows twice: strided (p = lane + 32 i) for the sum in the reference's order, and
        // its 4 adjacent values (p = 4 lane ..) for the outputs, so that every store is 8 or 16 bytes wide. The
        // second read hits L1.
        float q[4] = {0.f, 0.f, 0.f, 0.f}, k[4] = {0.f, 0.f, 0.f, 0.f};
        float qa[4] = {0.f, 0.f, 0.f, 0.f}, ka[4] = {0.f, 0.f, 0.f, 0.f};
        if (live) {
            const typename T::storage* qr = mixed + (size_t)t * conv_dim + h * kGdnKd;
            const typename T::storage* kr = qr + kh * kGdnKd;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                q[i] = load_scalar<T>(qr + lane + 32 * i);
                k[i] = load_scalar<T>(kr + lane + 32 * i);
            }
            load4_as_f32<T>(qr + lane * 4, qa);
            load4_as_f32<T>(kr + lane * 4, ka);
        }
        float sq = 0.0f, sk = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            sq = __fmaf_rn(q[i], q[i], sq);
            sk = __fmaf_rn(k[i], k[i], sk);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            sq = __fadd_rn(sq, __shfl_xor_sync(kFullMask, sq, off));
            sk = __fadd_rn(sk, __shfl_xor_sync(kFullMask, sk, off));
        }
        const float rq = __fmul_rn(rsqrtf(__fadd_rn(sq, 1e-6f)), q_scale);
        const float rk = rsqrtf(__fadd_rn(sk, 1e-6f));
        uint32_t qw[4], kw[4];   // hi words 0, 1 and lo words 0, 1
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            qa[j] = __fmul_rn(qa[j], rq);
            ka[j] = __fmul_rn(ka[j], rk);
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            qw[j] = pack_bf16x2(qa[2 * j], qa[2 * j + 1]);
            qw[2 + j] = pack_bf16x2(__fsub_rn(qa[2 * j], bf16_lo(qw[j])), __fsub_rn(qa[2 * j + 1], bf16_hi(qw[j])));
            kw[j] = pack_bf16x2(ka[2 * j], ka[2 * j + 1]);
            kw[2 + j] = pack_bf16x2(__fsub_rn(ka[2 * j], bf16_lo(kw[j])), __fsub_rn(ka[2 * j + 1], bf16_hi(kw[j])));
        }
        const uint32_t chunk = t / kGdnChunk;
        const int r = (int)(t - chunk * kGdnChunk);
        // within an operand tile: row r, the lane's 8 bytes (p = 4 lane .. 4 lane + 3) in their xor-ed 16-byte segment
        const uint32_t in_tile = (uint32_t)r * kGdnRowBytes + (uint32_t)(((((lane & 15) >> 1) ^ (r & 7)) << 4) + (lane & 1) * 8);
        for (int rep = 0; rep < ratio; ++rep) {
            const uint32_t he = (uint32_t)(h * ratio + rep);
            const size_t off = (((size_t)he * nchunks + chunk) * (kGdnKd / kGdnTileCols) + (lane >> 4)) * (size_t)(kGdnChunk * kGdnRowBytes) + in_tile;
            stg_v2(q_hi + off, make_uint2(qw[0], qw[1]));
            stg_v2(q_lo + off, make_uint2(qw[2], qw[3]));
            stg_v2(k_hi + off, make_uint2(kw[0], kw[1]));
            stg_v2(k_lo + off, make_uint2(kw[2], kw[3]));
            if (live) {
                *reinterpret_cast<float4*>(kn + ((size_t)t * heads + he) * kGdnKd + lane * 4) = make_float4(ka[0], ka[1], ka[2], ka[3]);
            }
        }
    }
    // v as f32: a flat conversion of each token's heads x 128 values, 8 per thread
    const uint32_t vvec = vvec_div.d;   // heads * 16 vectors of 8 per token
    const uint32_t v_total = (uint32_t)seq_len * vvec;
    const typename T::storage* vsrc = mixed + 2 * kh * kGdnKd;
    for (uint32_t idx = blockIdx.x * kCtaThreads + threadIdx.x; idx < v_total; idx += gridDim.x * kCtaThreads) {
        const uint32_t t = fast_div(idx, vvec_div);
        const typename T::storage* src = vsrc + (size_t)t * conv_dim + (idx - t * vvec) * 8;
        float* dst = v_out + (size_t)idx * 8;
        if (T::kBytes == 2) {
            const uint4 raw = ldg_stream_v4(src);
            stg_v4(dst, make_uint4(raw.x << 16, raw.x & 0xffff0000u, raw.y << 16, raw.y & 0xffff0000u));
            stg_v4(dst + 4, make_uint4(raw.z << 16, raw.z & 0xffff0000u, raw.w << 16, raw.w & 0xffff0000u));
        } else {
            stg_v4(dst, ldg_stream_v4(src));
            stg_v4(dst + 4, ldg_stream_v4(src + 4));
        }
    }
}

// ---------------------------------------------------------------------------------------------
// gdn_conv_prep (kernels/gdn_chunk.cu:1008-1172): the causal convolution + silu and gdn_prep above in one launch, the
// convolved row staying in f32 (as in the reference, whose stage is shared memory) instead of going through memory.
// One warp owns a strip of R tokens x one 128-channel group: a q head, a k head or a 128-value piece of v. A lane
// convolves 4 adjacent channels exactly as causal_conv_silu_c4_kernel does; a q or k head row is then parked in the
// warp's 4 KiB stage of shared memory so that lane l can add the squares of p = l, l + 32, l + 64, l + 96 in the
// reference's order, and each lane reads its own 4 adjacent values back to scale, split and store them (8-byte
// stores into the operand tiles). Tokens of the last chunk past `rows` are written as zeros.
// The strip's values are NOT carried in registers between the phases (a first version did: 126 registers, two CTAs
// per SM, and with the literal path inlined into the unrolled row loop 100 M warp instructions and 214 us at 8,192
// tokens x 8,192 channels, no faster than the two separate launches). In this form: 80 registers, three CTAs per SM,
// 63 M instructions, 143.5 us against 69.0 + 134.5 us for the two launches.
// ---------------------------------------------------------------------------------------------
// A strip that is not plain (it holds a sequence start, the first rows, or pad tokens of the last chunk), out of line:
// every tap tested, the literal silu; a q or k row goes to the stage, a v row straight out.
template <typename T, int K, int R>
static __device__ __noinline__ void gdn_strip_literal(const typename T::storage* __restrict__ x, const float* __restrict__ w,
                                                      float* st, float* v_row0, size_t v_row_stride, int t0, int rows, int c0,
                                                      int channels, const int* __restrict__ seq_start,
                                                      const typename T::storage* __restrict__ history,
                                                      const int* __restrict__ slot_map, int lane) {
#pragma unroll 1
    for (int r = 0; r < R; ++r) {
        const int t = t0 + r;
        float o4[4] = {0.f, 0.f, 0.f, 0.f};   // a pad token of the last chunk: zero operands
        if (t < rows) {
#pragma unroll 1
            for (int j = 0; j < 4; ++j) o4[j] = causal_conv_silu_element<T>(x, w, t, c0 + j, channels, K, seq_start, history, slot_map);
        }
        if (v_row0) {
            if (t < rows) *reinterpret_cast<float4*>(v_row0 + (size_t)r * v_row_stride) = make_float4(o4[0], o4[1], o4[2], o4[3]);
        } else {
            *reinterpret_cast<float4*>(st + r * kGdnKd + lane * 4) = make_float4(o4[0], o4[1], o4[2], o4[3]);
        }
    }
}

// RATIO = heads / kh (value heads per key head), compiled in so that the repeated stores are straight-line code.
template <typename T, int K, int R, int MIN_CTAS, int RATIO>
__global__ void __launch_bounds__(kCtaThreads, MIN_CTAS)
gdn_conv_prep_kernel(const typename T::storage* __restrict__ x, const float* __restrict__ w, float* __restrict__ v_out,
                     uint8_t* __restrict__ q_hi, uint8_t* __restrict__ q_lo, uint8_t* __restrict__ k_hi,
                     uint8_t* __restrict__ k_lo, float* __restrict__ kn, int rows, int channels,
                     const int* __restrict__ seq_start, const typename T::storage* __restrict__ history,
                     const int* __restrict__ slot_map, int heads, int kh, int nchunks, float q_scale, FastDiv groups_div) {
    static_assert(kGdnChunk % R == 0, "a strip must not straddle two chunks");
    static_assert(R == 8, "the reduce-scatter below is written for 8 rows");
    __shared__ float stage[kCtaThreads / 32][R * kGdnKd];
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    float* st = &stage[warp][0];
    const uint32_t groups = groups_div.d;                              // channels / 128
    const uint32_t strips = (uint32_t)nchunks * (kGdnChunk / R);       // pad tokens of the last chunk included
    const uint32_t total = strips * groups;
    const bool starts_vector = (reinterpret_cast<uintptr_t>(seq_start) & 15) == 0;
    const size_t v_row_stride = (size_t)heads * kGdnKd;
    // within an operand tile: the lane's 8 bytes of row r sit in 16-byte segment ((lane & 15) >> 1) ^ (r & 7); a strip
    // starts at a multiple of 8 rows of its chunk, so r & 7 is the row's index in the strip
    const uint32_t seg16 = (uint32_t)((lane & 15) >> 1) << 4, in_seg = (uint32_t)(lane & 1) * 8;
    const size_t tile_bytes = (size_t)kGdnChunk * kGdnRowBytes;
    const size_t head_stride = (size_t)nchunks * (kGdnKd / kGdnTileCols) * tile_bytes;   // between expanded heads
    for (uint32_t item = blockIdx.x * (kCtaThreads / 32) + warp; item < total; item += gridDim.x * (kCtaThreads / 32)) {
        const uint32_t strip = fast_div(item, groups_div);
        const int g = (int)(item - strip * groups);
        const int c0 = g * kGdnKd + lane * 4;
        const int t0 = (int)strip * R;
        const bool is_v = g >= 2 * kh;
        if (t0 >= rows && is_v) {
            continue;
        }
        float* v_row0 = is_v ? v_out + (size_t)t0 * v_row_stride + (size_t)(g - 2 * kh) * kGdnKd + lane * 4 : nullptr;
        bool plain = t0 >= K - 1 && t0 + R <= rows;   // every row of the strip and of its halo exists
        if (plain && seq_start) {
            const int lim = t0 - (K - 1);
            if (starts_vector) {   // the 8 sequence starts as two 16-byte loads
                const int4 a = __ldg(reinterpret_cast<const int4*>(seq_start + t0));
                const int4 b = __ldg(reinterpret_cast<const int4*>(seq_start + t0) + 1);
                plain = a.x <= lim && a.y <= lim + 1 && a.z <= lim + 2 && a.w <= lim + 3 && b.x <= lim + 4 && b.y <= lim + 5 &&
                        b.z <= lim + 6 && b.w <= lim + 7;
            } else {
#pragma unroll
                for (int r = 0; r < R; ++r) plain &= __ldg(seq_start + t0 + r) <= lim + r;
            }
        }
        if (!plain) {
            gdn_strip_literal<T, K, R>(x, w, st, v_row0, v_row_stride, t0, rows, c0, channels, seq_start, history, slot_map, lane);
        } else {
            // Phase 1: convolution + silu of the strip, row by row: a v row goes straight out as f32, a q or k row is
            // parked in the warp's stage (not carried in registers between the phases).
            float xs[R + K - 1][4];
            float wt[4][K];
            const typename T::storage* base = x + (size_t)(t0 - (K - 1)) * channels + c0;
#pragma unroll
            for (int i = 0; i < R + K - 1; ++i) load4_as_f32<T>(base + (size_t)i * channels, xs[i]);
            if (K == 4) {   // a channel's four taps are one 16-byte load
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float4 t4 = __ldg(reinterpret_cast<const float4*>(w) + (c0 + j));
                    wt[j][0] = t4.x, wt[j][1] = t4.y, wt[j][2 % K] = t4.z, wt[j][3 % K] = t4.w;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
#pragma unroll
                    for (int tap = 0; tap < K; ++tap) wt[j][tap] = __ldg(w + (size_t)(c0 + j) * K + tap);
                }
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
                float a4[4], o4[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    a4[j] = 0.0f;
#pragma unroll
                    for (int tap = 0; tap < K; ++tap) a4[j] = __fmaf_rn(wt[j][tap], xs[r + tap][j], a4[j]);
                }
                const float m = fmaxf_nan(max3_abs_nan(fabsf(a4[0]), a4[1], a4[2]), fabsf(a4[3]));
                if (m <= kSiluFastMaxAbs) {   // false for a NaN too
#pragma unroll
                    for (int j = 0; j < 4; ++j) o4[j] = silu_ieee_refined_f32(a4[j]);
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) o4[j] = silu_ieee_div(a4[j]);
                }
                if (is_v) {
                    *reinterpret_cast<float4*>(v_row0 + (size_t)r * v_row_stride) = make_float4(o4[0], o4[1], o4[2], o4[3]);
                } else {
                    *reinterpret_cast<float4*>(st + r * kGdnKd + lane * 4) = make_float4(o4[0], o4[1], o4[2], o4[3]);
                }
            }
        }
        if (is_v) {
            continue;
        }
        // Phase 2: the R sums of squares. Lane l adds p = l, l + 32, l + 64, l + 96 of a row in order; the R xor trees
        // run as one reduce-scatter (same pairs, same order: the sums are bit-identical to R butterflies), after which
        // lanes 4 r .. 4 r + 3 hold the total of row r.
        __syncwarp();
        float s8[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            s8[r] = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float v = st[r * kGdnKd + lane + 32 * i];
                s8[r] = __fmaf_rn(v, v, s8[r]);
            }
        }
        __syncwarp();
        float s4[4], s2[2];
        const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            s4[j] = __fadd_rn(b4 ? s8[4 + j] : s8[j], __shfl_xor_sync(kFullMask, b4 ? s8[j] : s8[4 + j], 16));
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            s2[j] = __fadd_rn(b3 ? s4[2 + j] : s4[j], __shfl_xor_sync(kFullMask, b3 ? s4[j] : s4[2 + j], 8));
        }
        float total_sq = __fadd_rn(b2 ? s2[1] : s2[0], __shfl_xor_sync(kFullMask, b2 ? s2[0] : s2[1], 4));
        total_sq = __fadd_rn(total_sq, __shfl_xor_sync(kFullMask, total_sq, 2));
        total_sq = __fadd_rn(total_sq, __shfl_xor_sync(kFullMask, total_sq, 1));
        const bool is_q = g < kh;
        float my_scale = rsqrtf(__fadd_rn(total_sq, 1e-6f));   // of row (lane >> 2)
        if (is_q) my_scale = __fmul_rn(my_scale, q_scale);
        // Phase 3: each lane scales its own 4 adjacent values of a row, stores kn, splits into hi + lo and stores
        // 8 bytes into each operand tile, once per repeated head.
        const int h = is_q ? g : g - kh;
        const uint32_t chunk = (uint32_t)t0 / kGdnChunk;
        const uint32_t rr0 = (uint32_t)t0 - chunk * kGdnChunk;
        const size_t base = ((((size_t)(h * RATIO) * nchunks + chunk) * (kGdnKd / kGdnTileCols) + (size_t)(lane >> 4)) * kGdnChunk + rr0) *
                                kGdnRowBytes + in_seg;
        uint8_t* hp = (is_q ? q_hi : k_hi) + base;
        uint8_t* lp = (is_q ? q_lo : k_lo) + base;
        float* kp = kn + ((size_t)t0 * heads + (size_t)(h * RATIO)) * kGdnKd + lane * 4;
        const int live_rows = is_q ? 0 : min(R, rows - t0);   // rows whose normalised k also goes out as f32
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const float scale = __shfl_sync(kFullMask, my_scale, 4 * r);
            const float4 raw4 = *reinterpret_cast<const float4*>(st + r * kGdnKd + lane * 4);   // this lane's own values
            const float o0 = __fmul_rn(raw4.x, scale), o1 = __fmul_rn(raw4.y, scale), o2 = __fmul_rn(raw4.z, scale),
                        o3 = __fmul_rn(raw4.w, scale);
            const uint32_t hi0 = pack_bf16x2(o0, o1), hi1 = pack_bf16x2(o2, o3);
            const uint32_t lo0 = pack_bf16x2(__fsub_rn(o0, bf16_lo(hi0)), __fsub_rn(o1, bf16_hi(hi0)));
            const uint32_t lo1 = pack_bf16x2(__fsub_rn(o2, bf16_lo(hi1)), __fsub_rn(o3, bf16_hi(hi1)));
            const uint32_t off = (uint32_t)r * kGdnRowBytes + (seg16 ^ ((uint32_t)r << 4));
#pragma unroll
            for (int rep = 0; rep < RATIO; ++rep) {
                if (r < live_rows) {
                    *reinterpret_cast<float4*>(kp + (size_t)r * v_row_stride + rep * kGdnKd) = make_float4(o0, o1, o2, o3);
                }
                stg_v2(hp + rep * head_stride + off, make_uint2(hi0, hi1));
                stg_v2(lp + rep * head_stride + off, make_uint2(lo0, lo1));
            }
        }
    }
}

// gdn_gates (kernels/elementwise.cu:361-377): beta = 1 / (1 + __expf(-b)); decay = -__expf(a_log[h]) * softplus(a + dt_bias[h])
// with softplus(x) = x above 20 and log1pf(__expf(x)) otherwise. Outputs are f32.
template <typename T>
__global__ void __launch_bounds__(kCtaThreads)
gdn_gates_kernel(const typename T::storage* __restrict__ a, const typename T::storage* __restrict__ b,
                 const float* __restrict__ a_log, const float* __restrict__ dt_bias, float* __restrict__ decay,
                 float* __restrict__ beta, int total, int heads) {
    const int step = gridDim.x * kCtaThreads;
    for (int i = blockIdx.x * kCtaThreads + threadIdx.x; i < total; i += step) {
        const int h = i % heads;
        beta[i] = __fdiv_rn(1.0f, __fadd_rn(1.0f, __expf(-load_scalar<T>(b + i))));
        const float xv = __fadd_rn(load_scalar<T>(a + i), dt_bias[h]);
        const float sp = (xv > 20.0f) ? xv : log1pf(__expf(xv));
        decay[i] = __fmul_rn(-__expf(a_log[h]), sp);
    }
}

// The three splitting copies (kernels/elementwise.cu:378-445), 16 bytes per thread. `segs` describes, per input
// row of `in_width` values, up to three consecutive column ranges and where each goes.
struct SplitPlan {
    int in_width;        // values per input row
    int n_out;           // outputs in use
    int start[3];        // first input column of each range
    int width[3];        // its width (also the output's row width)
};
template <typename T>
__global__ void __launch_bounds__(kCtaThreads)
split_rows_kernel(const typename T::storage* __restrict__ in, typename T::storage* __restrict__ out0,
                  typename T::storage* __restrict__ out1, typename T::storage* __restrict__ out2, size_t rows,
                  SplitPlan plan) {
    constexpr int kPer = 16 / T::kBytes;
    const size_t vec_per_row = (size_t)plan.in_width / kPer;
    const size_t total = rows * vec_per_row;
    const size_t step = (size_t)gridDim.x * kCtaThreads;
    for (size_t idx = (size_t)blockIdx.x * kCtaThreads + threadIdx.x; idx < total; idx += step) {
        const size_t row = idx / vec_per_row;
        const int col = (int)(idx - row * vec_per_row) * kPer;
        const uint4 v = ldg_stream_v4(in + row * plan.in_width + col);
        typename T::storage* dst = out0;
        int which = 0;
        if (plan.n_out > 1 && col >= plan.start[1]) { dst = out1; which = 1; }
        if (plan.n_out > 2 && col >= plan.start[2]) { dst = out2; which = 2; }
        stg_v4(dst + row * plan.width[which] + (col - plan.start[which]), v);
    }
}

// repeat_interleave (kernels/elementwise.cu:429-445): out[t, h * ratio + r, :] = src[t, h, :].
template <typename T>
__global__ void __launch_bounds__(kCtaThreads)
repeat_interleave_kernel(const typename T::storage* __restrict__ src, typename T::storage* __restrict__ out,
                         size_t head_rows_out, int ratio, int dim) {
    constexpr int kPer = 16 / T::kBytes;
    const size_t vec_per_row = (size_t)dim / kPer;
    const size_t total = head_rows_out * vec_per_row;
    const size_t step = (size_t)gridDim.x * kCtaThreads;
    for (size_t idx = (size_t)blockIdx.x * kCtaThreads + threadIdx.x; idx < total; idx += step) {
        const size_t orow = idx / vec_per_row;                  // t * (kh * ratio) + oh
        const size_t v = idx - orow * vec_per_row;
        stg_v4(out + orow * dim + v * kPer, ldg_stream_v4(src + (orow / ratio) * dim + v * kPer));
    }
}

}  // namespace clef
