// C-ABI of the steps either side of the fused quantisers in a layer: the bf16 KV-cache write (alone
// and fused behind the key-side RoPE), attention-output gating with and without the NVFP4
// quantiser, the residual add. Declarations and the reference interfaces: include/clef_fused.h.
// Same contract as the other entry points: asynchronous on the caller's stream, no allocation, no
// synchronisation, grids that depend on the shape arguments only.

#include "../../include/clef_fused.h"

#include <atomic>

#include "abi_support.cuh"
#include "kernels_hot.cuh"
#include "unit_quant_f32_launch.cuh"
#include "kernels_layer.cuh"

using namespace clef;
using namespace clef::abi;

namespace {

template <typename T>
void launch_to_bf16_rows(cudaStream_t s, const DeviceInfo& dev, void* out, const void* x, size_t n, const int32_t* pos_map,
                         const int32_t* off_tokens, int stride) {
    static std::atomic<int> occ{0};
    const int per_sm = ctas_per_sm(to_bf16_rows_kernel<T>, 0, occ);
    const uint32_t vecs = (uint32_t)(n / 8), tail = pos_map ? 0u : (uint32_t)(n % 8);
    const size_t ctas = ((size_t)vecs + kCtaThreads - 1) / kCtaThreads;
    launch_hot(to_bf16_rows_kernel<T>, clamp_grid(ctas, (size_t)dev.sms * per_sm), 0, s, (const Storage<T>*)x,
               (uint16_t*)out, vecs, tail, (const int*)pos_map, (const int*)off_tokens, stride,
               make_fast_div((uint32_t)(stride >= 8 ? stride / 8 : 1)));
}

int to_bf16_impl(const char* what, clef_stream_t stream, void* out, const void* x, size_t n, const int32_t* pos_map,
                 const int32_t* off_tokens, int stride, int dtype) {
    if (int r = check_dtype(dtype, what)) return r;
    if (!out || !x) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (!aligned(out, 16) || !aligned(x, 16)) return fail(CLEF_ERR_INVALID, "%s: pointers must be 16-byte aligned", what);
    if (n / 8 >= 0x7fffffffull) return fail(CLEF_ERR_TOO_LARGE, "%s: %zu values", what, n);
    if (pos_map) {
        if (stride <= 0 || stride % 8 != 0 || n % (size_t)stride != 0) {
            return fail(CLEF_ERR_INVALID, "%s: stride %d must be a positive multiple of 8 that divides n = %zu", what,
                        stride, n);
        }
    } else if (off_tokens && (stride < 0 || stride % 8 != 0)) {
        return fail(CLEF_ERR_INVALID, "%s: off_stride %d must be a non-negative multiple of 8 (16-byte stores)", what,
                    stride);
    }
    if (n == 0) return CLEF_OK;
    DeviceInfo dev;
    if (int r = device_info(dev)) return r;
    if (dtype == CLEF_BF16) {
        launch_to_bf16_rows<Bf16>(as_stream(stream), dev, out, x, n, pos_map, off_tokens, stride);
    } else {
        launch_to_bf16_rows<F32>(as_stream(stream), dev, out, x, n, pos_map, off_tokens, stride);
    }
    return check_launch(what);
}

int check_kv_shape(const char* what, int tokens, int kv_heads, int head_dim, int rotary_dim) {
    if (tokens < 0 || kv_heads <= 0 || head_dim <= 0 || rotary_dim < 0) {
        return fail(CLEF_ERR_INVALID, "%s: tokens %d kv_heads %d head_dim %d rotary_dim %d", what, tokens, kv_heads,
                    head_dim, rotary_dim);
    }
    if (head_dim % 8 != 0 || rotary_dim % 8 != 0 || rotary_dim > head_dim) {
        return fail(CLEF_ERR_INVALID,
                    "%s: head_dim %d and rotary_dim %d must be multiples of 8, rotary_dim not above head_dim", what,
                    head_dim, rotary_dim);
    }
    return CLEF_OK;
}

}  // namespace

extern "C" {

int clef_to_bf16(clef_stream_t stream, void* out, const void* x, size_t n, const int32_t* off_tokens_dev,
                 int off_stride, int dtype) {
    return to_bf16_impl("clef_to_bf16", stream, out, x, n, nullptr, off_tokens_dev, off_tokens_dev ? off_stride : 0,
                        dtype);
}

int clef_to_bf16_scatter(clef_stream_t stream, void* out, const void* x, size_t n, const int32_t* pos_map, int stride,
                         int dtype) {
    if (!pos_map) return fail(CLEF_ERR_INVALID, "clef_to_bf16_scatter: null position map");
    return to_bf16_impl("clef_to_bf16_scatter", stream, out, x, n, pos_map, nullptr, stride, dtype);
}

int clef_rope_kv_write(clef_stream_t stream, void* cache_k, void* cache_v, const void* k, const void* v,
                       const float* cos_table, const float* sin_table, int tokens, int kv_heads, int head_dim,
                       int rotary_dim, const int32_t* seq_start, const int32_t* pos_base, const int32_t* pos_map,
                       const int32_t* cache_map, const int32_t* cache_len, int dtype) {
    const char* what = "clef_rope_kv_write";
    if (int r = check_dtype(dtype, what)) return r;
    if (!cache_k || !cache_v || !k || !v || !cos_table || !sin_table) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (int r = check_kv_shape(what, tokens, kv_heads, head_dim, rotary_dim)) return r;
    if (!aligned(cache_k, 16) || !aligned(cache_v, 16) || !aligned(k, 16) || !aligned(v, 16) || !aligned(cos_table, 16) ||
        !aligned(sin_table, 16)) {
        return fail(CLEF_ERR_INVALID, "%s: pointers must be 16-byte aligned", what);
    }
    if (tokens == 0) return CLEF_OK;
    DeviceInfo dev;
    if (int r = device_info(dev)) return r;
    cudaStream_t s = as_stream(stream);
    const size_t key_items_hot = (size_t)tokens * kv_heads * (head_dim / 32);
    if (dtype == CLEF_BF16 && use_hot() && head_dim % 32 == 0 && rotary_dim % 32 == 0 && 2 * key_items_hot < 0x7fffffffull &&
        aligned(k, 32) && aligned(v, 32) && aligned(cache_k, 32) && aligned(cache_v, 32)) {
        static std::atomic<int> occ{0};
        const int per_sm = ctas_per_sm(rope_hot_kernel<true>, 0, occ);
        const size_t items = 2 * key_items_hot;
        launch_hot(rope_hot_kernel<true>, clamp_grid((items + kCtaThreads - 1) / kCtaThreads, (size_t)dev.sms * per_sm), 0,
                   s, (uint16_t*)cache_k, (const uint16_t*)k, cos_table, sin_table, (uint32_t)items, kv_heads, head_dim,
                   rotary_dim, (const int*)seq_start, (const int*)pos_base, (const int*)pos_map,
                   make_fast_div((uint32_t)(head_dim / 32)), make_fast_div((uint32_t)kv_heads),
                   KvCacheDest{(const int*)cache_map, (const int*)cache_len, (const uint16_t*)v, (uint16_t*)cache_v});
        return check_launch(what);
    }
    const size_t items =
        (size_t)tokens * kv_heads * ((size_t)(rotary_dim / 8) + (head_dim - rotary_dim) / 4 + head_dim / 4);
    if (dtype == CLEF_BF16) {
        static std::atomic<int> occ{0};
        const int per_sm = ctas_per_sm(rope_kv_write_generic_kernel<Bf16>, 0, occ);
        rope_kv_write_generic_kernel<Bf16><<<clamp_grid((items + kCtaThreads - 1) / kCtaThreads, (size_t)dev.sms * per_sm),
                                             kCtaThreads, 0, s>>>(
            (uint16_t*)cache_k, (uint16_t*)cache_v, (const uint16_t*)k, (const uint16_t*)v, cos_table, sin_table, tokens,
            kv_heads, head_dim, rotary_dim, seq_start, pos_base, pos_map, cache_map, cache_len);
    } else {
        static std::atomic<int> occ{0};
        const int per_sm = ctas_per_sm(rope_kv_write_generic_kernel<F32>, 0, occ);
        rope_kv_write_generic_kernel<F32><<<clamp_grid((items + kCtaThreads - 1) / kCtaThreads, (size_t)dev.sms * per_sm),
                                            kCtaThreads, 0, s>>>(
            (uint16_t*)cache_k, (uint16_t*)cache_v, (const float*)k, (const float*)v, cos_table, sin_table, tokens,
            kv_heads, head_dim, rotary_dim, seq_start, pos_base, pos_map, cache_map, cache_len);
    }
    return check_launch(what);
}

// q and k rotated in one launch; with caches, k goes to its cache rows and v is copied to its own.
static int rope_qkv_impl(const char* what, clef_stream_t stream, void* q_out, const void* q, int q_heads, void* k_dst,
                         void* cache_v, const void* k, const void* v, int kv_heads, const float* cos_table,
                         const float* sin_table, int rows, int head_dim, int rotary_dim, const int32_t* seq_start,
                         const int32_t* pos_base, const int32_t* pos_map, const int32_t* cache_map,
                         const int32_t* cache_len, bool to_cache, int dtype) {
    if (int r = check_dtype(dtype, what)) return r;
    if (!q_out || !q || !k_dst || !k || !cos_table || !sin_table || (to_cache && (!cache_v || !v))) {
        return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    }
    if (q_heads <= 0) return fail(CLEF_ERR_INVALID, "%s: q_heads %d", what, q_heads);
    if (int r = check_kv_shape(what, rows, kv_heads, head_dim, rotary_dim)) return r;
    if (q_out == q || (!to_cache && k_dst == k)) return fail(CLEF_ERR_INVALID, "%s: an output must not alias its input", what);
    if (rows == 0) return CLEF_OK;
    DeviceInfo dev;
    if (int r = device_info(dev)) return r;
    const size_t per_row = (size_t)(head_dim / 32);
    const size_t q_items = (size_t)rows * q_heads * per_row, k_items = (size_t)rows * kv_heads * per_row;
    const size_t items = q_items + k_items * (to_cache ? 2 : 1);
    const bool all32 = aligned(q, 32) && aligned(q_out, 32) && aligned(k, 32) && aligned(k_dst, 32) &&
                       (!to_cache || (aligned(v, 32) && aligned(cache_v, 32)));
    if (dtype == CLEF_BF16 && use_hot() && head_dim % 32 == 0 && rotary_dim % 32 == 0 && items < 0x7fffffffull && all32) {
        RopeSegments segs{};
        segs.seg[0] = RopeSegment{(const uint16_t*)q, (uint16_t*)q_out, (uint32_t)q_items, q_heads,
                                  make_fast_div((uint32_t)q_heads), 1, 0};
        segs.seg[1] = RopeSegment{(const uint16_t*)k, (uint16_t*)k_dst, (uint32_t)(q_items + k_items), kv_heads,
                                  make_fast_div((uint32_t)kv_heads), 1, to_cache ? 1 : 0};
        segs.seg[2] = RopeSegment{(const uint16_t*)v, (uint16_t*)cache_v, (uint32_t)items, kv_heads,
                                  make_fast_div((uint32_t)kv_heads), 0, 1};
        const size_t ctas = (items + kCtaThreads - 1) / kCtaThreads;
        if (to_cache) {
            static std::atomic<int> occ{0};
            const int per_sm = ctas_per_sm(rope_multi_hot_kernel<3>, 0, occ);
            launch_hot(rope_multi_hot_kernel<3>, clamp_grid(ctas, (size_t)dev.sms * per_sm), 0, as_stream(stream), segs, cos_table,
                       sin_table, head_dim, rotary_dim, (const int*)seq_start, (const int*)pos_base, (const int*)pos_map,
                       (const int*)cache_map, (const int*)cache_len, make_fast_div((uint32_t)per_row));
        } else if (pos_map && !seq_start && !pos_base &&
                   rope_launch_is_short(ctas, (size_t)dev.sms * 6)) {   // the engine's case: a pass of at most 8,192 rows, positions from its map
            static std::atomic<int> occ{0};
            const int per_sm = ctas_per_sm(rope_qk_map_hot_kernel, 0, occ);
            launch_hot(rope_qk_map_hot_kernel, balanced_grid(ctas, (size_t)dev.sms * per_sm), 0, as_stream(stream), segs, cos_table,
                       sin_table, head_dim, rotary_dim, (const int*)pos_map, make_fast_div((uint32_t)per_row));
        } else {
            static std::atomic<int> occ{0};
            const int per_sm = ctas_per_sm(rope_multi_hot_kernel<2>, 0, occ);
            launch_hot(rope_multi_hot_kernel<2>, clamp_grid(ctas, (size_t)dev.sms * per_sm), 0, as_stream(stream), segs, cos_table,
                       sin_table, head_dim, rotary_dim, (const int*)seq_start, (const int*)pos_base, (const int*)pos_map,
                       (const int*)nullptr, (const int*)nullptr, make_fast_div((uint32_t)per_row));
        }
        return check_launch(what);
    }
    const size_t q_items32 = (size_t)rows * q_heads * (head_dim / 16), k_items32 = (size_t)rows * kv_heads * (head_dim / 16);
    if (dtype == CLEF_F32 && !to_cache && use_hot() && head_dim % 16 == 0 && rotary_dim % 16 == 0 &&
        q_items32 + k_items32 < 0x7fffffffull && all32) {
        RopeSegmentsF32 segs{};
        segs.x[0] = (const float*)q;
        segs.out[0] = (float*)q_out;
        segs.end_item[0] = (uint32_t)q_items32;
        segs.heads_div[0] = make_fast_div((uint32_t)q_heads);
        segs.x[1] = (const float*)k;
        segs.out[1] = (float*)k_dst;
        segs.end_item[1] = (uint32_t)(q_items32 + k_items32);
        segs.heads_div[1] = make_fast_div((uint32_t)kv_heads);
        static std::atomic<int> occ{0};
        const int per_sm = ctas_per_sm(rope_f32_hot_kernel<2>, 0, occ);
        launch_hot(rope_f32_hot_kernel<2>, clamp_grid((q_items32 + k_items32 + kCtaThreads - 1) / kCtaThreads, (size_t)dev.sms * per_sm),
                   0, as_stream(stream), segs, cos_table, sin_table, head_dim, rotary_dim, (const int*)seq_start,
                   (const int*)pos_base, (const int*)pos_map, make_fast_div((uint32_t)(head_dim / 16)));
        return check_launch(what);
    }
    // Other shapes, and f32 with cache rows: the calls this entry point stands for.
    if (int r = clef_rope(stream, q_out, q, cos_table, sin_table, rows, q_heads, head_dim, rotary_dim, seq_start, pos_base,
                          pos_map, dtype)) return r;
    if (to_cache) {
        return clef_rope_kv_write(stream, k_dst, cache_v, k, v, cos_table, sin_table, rows, kv_heads, head_dim, rotary_dim,
                                  seq_start, pos_base, pos_map, cache_map, cache_len, dtype);
    }
    return clef_rope(stream, k_dst, k, cos_table, sin_table, rows, kv_heads, head_dim, rotary_dim, seq_start, pos_base,
                     pos_map, dtype);
}

int clef_rope_qk(clef_stream_t stream, void* q_out, const void* q, int q_heads, void* k_out, const void* k, int kv_heads,
                 const float* cos_table, const float* sin_table, int rows, int head_dim, int rotary_dim,
                 const int32_t* seq_start, const int32_t* pos_base, const int32_t* pos_map, int dtype) {
    return rope_qkv_impl("clef_rope_qk", stream, q_out, q, q_heads, k_out, nullptr, k, nullptr, kv_heads, cos_table, sin_table,
                         rows, head_dim, rotary_dim, seq_start, pos_base, pos_map, nullptr, nullptr, false, dtype);
}

int clef_rope_qkv_write(clef_stream_t stream, void* q_out, const void* q, int q_heads, void* cache_k, void* cache_v,
                        const void* k, const void* v, int kv_heads, const float* cos_table, const float* sin_table,
                        int tokens, int head_dim, int rotary_dim, const int32_t* seq_start, const int32_t* pos_base,
                        const int32_t* pos_map, const int32_t* cache_map, const int32_t* cache_len, int dtype) {
    return rope_qkv_impl("clef_rope_qkv_write", stream, q_out, q, q_heads, cache_k, cache_v, k, v, kv_heads, cos_table, sin_table,
                         tokens, head_dim, rotary_dim, seq_start, pos_base, pos_map, cache_map, cache_len, true, dtype);
}

int clef_qk_norm_rope_kv_write(clef_stream_t stream, void* cache_k, void* cache_v, const void* k_raw, const void* v,
                               const float* weight, const float* cos_table, const float* sin_table, int tokens,
                               int kv_heads, int head_dim, int rotary_dim, float eps, const int32_t* seq_start,
                               const int32_t* pos_base, const int32_t* pos_map, const int32_t* cache_map,
                               const int32_t* cache_len, int dtype) {
    const char* what = "clef_qk_norm_rope_kv_write";
    if (int r = check_dtype(dtype, what)) return r;
    if (!cache_k || !cache_v || !k_raw || !v || !weight || !cos_table || !sin_table) {
        return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    }
    if (int r = check_kv_shape(what, tokens, kv_heads, head_dim, rotary_dim)) return r;
    if (head_dim > 1024) return fail(CLEF_ERR_TOO_LARGE, "%s: head_dim %d above 1024", what, head_dim);
    if (!aligned(cache_k, 16) || !aligned(cache_v, 16) || !aligned(k_raw, 16) || !aligned(v, 16) || !aligned(weight, 16)) {
        return fail(CLEF_ERR_INVALID, "%s: pointers must be 16-byte aligned", what);
    }
    if (tokens == 0) return CLEF_OK;
    const size_t rows = (size_t)tokens * kv_heads;
    if (rows >= 0x3fffffffull) return fail(CLEF_ERR_TOO_LARGE, "%s: %zu head rows", what, rows);
    DeviceInfo dev;
    if (int r = device_info(dev)) return r;
    cudaStream_t s = as_stream(stream);
    if (dtype == CLEF_BF16 && use_hot() && (head_dim == 128 || head_dim == 256) && rotary_dim == 64 && rows % 8 == 0 &&
        aligned(k_raw, 32) && aligned(v, 32) && aligned(cache_k, 32) && aligned(cache_v, 32)) {
        const size_t groups = (2 * rows + 63) / 64;
        auto launch = [&](auto kernel, std::atomic<int>& occ) {
            const int per_sm = ctas_per_sm(kernel, 0, occ);
            launch_hot(kernel, balanced_grid(groups, (size_t)dev.sms * per_sm), 0, s, (const uint16_t*)k_raw, weight, cos_table,
                       sin_table, (uint16_t*)cache_k, (uint16_t*)nullptr, (uint32_t)rows, eps, (const int*)seq_start,
                       (const int*)pos_base, (const int*)pos_map, make_fast_div((uint32_t)kv_heads),
                       KvCacheDest{(const int*)cache_map, (const int*)cache_len, (const uint16_t*)v, (uint16_t*)cache_v});
        };
        static std::atomic<int> occ[2];
        if (head_dim == 128) launch(qk_norm_rope_hot_kernel<false, true>, occ[0]);
        else launch(qk_norm_rope_hd256_hot_kernel<false, true>, occ[1]);
        return check_launch(what);
    }
    // Shape-general path: the value rows as a cache write of their own, then the fused key kernel.
    const int stride = kv_heads * head_dim;
    if (cache_map) {
        if (int r = to_bf16_impl(what, stream, cache_v, v, rows * head_dim, cache_map, nullptr, stride, dtype)) return r;
    } else {
        if (int r = to_bf16_impl(what, stream, cache_v, v, rows * head_dim, nullptr, cache_len, cache_len ? stride : 0, dtype)) return r;
    }
    const size_t smem = (size_t)8 * head_dim * sizeof(float);
    const size_t groups = (rows + 7) / 8;
    if (dtype == CLEF_BF16) {
        static std::atomic<int> occ{0};
        auto kernel = qk_norm_rope_generic_kernel<Bf16, Bf16, true>;
        const int per_sm = ctas_per_sm(kernel, smem, occ);
        kernel<<<clamp_grid(groups, (size_t)dev.sms * per_sm), kCtaThreads, smem, s>>>(
            (const uint16_t*)k_raw, weight, cos_table, sin_table, (uint16_t*)cache_k, (uint16_t*)nullptr, (int)rows, kv_heads,
            head_dim, rotary_dim, eps, seq_start, pos_base, pos_map, cache_map, cache_len);
    } else {
        static std::atomic<int> occ{0};
        auto kernel = qk_norm_rope_generic_kernel<F32, Bf16, true>;
        const int per_sm = ctas_per_sm(kernel, smem, occ);
        kernel<<<clamp_grid(groups, (size_t)dev.sms * per_sm), kCtaThreads, smem, s>>>(
            (const float*)k_raw, weight, cos_table, sin_table, (uint16_t*)cache_k, (float*)nullptr, (int)rows, kv_heads,
            head_dim, rotary_dim, eps, seq_start, pos_base, pos_map, cache_map, cache_len);
    }
    return check_launch(what);
}

int clef_sigmoid_mul(clef_stream_t stream, void* out, const void* x, const void* gate, size_t total, int dtype) {
    const char* what = "clef_sigmoid_mul";
    if (int r = check_dtype(dtype, what)) return r;
    if (!out || !x || !gate) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (!aligned(out, 16) || !aligned(x, 16) || !aligned(gate, 16)) {
        return fail(CLEF_ERR_INVALID, "%s: pointers must be 16-byte aligned", what);
    }
    if (total == 0) return CLEF_OK;
    DeviceInfo dev;
    if (int r = device_info(dev)) return r;
    cudaStream_t s = as_stream(stream);
    if (dtype == CLEF_BF16 && use_hot() && total >= 16 && total / 16 < 0xffffffffull && aligned(out, 32) && aligned(x, 32) &&
        aligned(gate, 32)) {
        static std::atomic<int> occ{0};
        const int per_sm = ctas_per_sm(swiglu_hot_kernel<kActSigmoidMul>, 0, occ);
        const size_t blocks = total / 16;
        launch_hot(swiglu_hot_kernel<kActSigmoidMul>, clamp_grid((blocks + kCtaThreads - 1) / kCtaThreads, (size_t)dev.sms * per_sm),
                   0, s, (const uint16_t*)gate, (const uint16_t*)x, (uint16_t*)out, (uint32_t)blocks);
        if (int r = check_launch(what)) return r;
        const size_t done = blocks * 16;
        if (done == total) return CLEF_OK;
        // The last total % 16 values go through the shape-general kernel. Its quad / tail split is taken
        // relative to its own start; done % 4 == 0, so the split falls where the whole-array call puts it.
        x = (const uint16_t*)x + done;
        gate = (const uint16_t*)gate + done;
        out = (uint16_t*)out + done;
        total -= done;
    }
    const size_t quads = (total + 3) / 4;
    if (dtype == CLEF_BF16) {
        static std::atomic<int> occ{0};
        const int per_sm = ctas_per_sm(sigmoid_mul_generic_kernel<Bf16>, 0, occ);
        sigmoid_mul_generic_kernel<Bf16><<<clamp_grid((quads + kCtaThreads - 1) / kCtaThreads, (size_t)dev.sms * per_sm),
                                           kCtaThreads, 0, s>>>((uint16_t*)out, (const uint16_t*)x, (const uint16_t*)gate, total);
    } else {
        static std::atomic<int> occ{0};
        const int per_sm = ctas_per_sm(sigmoid_mul_generic_kernel<F32>, 0, occ);
        sigmoid_mul_generic_kernel<F32><<<clamp_grid((quads + kCtaThreads - 1) / kCtaThreads, (size_t)dev.sms * per_sm),
                                          kCtaThreads, 0, s>>>((float*)out, (const float*)x, (const float*)gate, total);
    }
    return check_launch(what);
}

static int clef_sigmoid_mul_quantise_nvfp4_impl(clef_stream_t stream, const void* x, const void* gate, uint8_t* packed,
                                    uint8_t* scales, int rows, int cols, float global_scale, int blk_mn, int chunk,
                                    int dtype, int sf_layout) {
    const char* what = "clef_sigmoid_mul_quantise_nvfp4";
    if (int r = check_dtype(dtype, what)) return r;
    if (!x || !gate || !packed || !scales) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (int r = check_scale_layout(what, rows, cols, blk_mn, &chunk, sf_layout)) return r;   // folds the tile order into chunk
    if (!aligned(x, 16) || !aligned(gate, 16) || !aligned(packed, 8)) {
        return fail(CLEF_ERR_INVALID, "%s: x and gate must be 16-byte aligned, packed 8-byte aligned", what);
    }
    int rows_total = 0;
    if (int r = clef_nvfp4_sizes(rows, cols, blk_mn, &rows_total, nullptr, nullptr)) return r;
    if (rows_total == 0) return CLEF_OK;
    DeviceInfo dev;
    if (int r = device_info(dev)) return r;
    cudaStream_t s = as_stream(stream);
    const size_t total_blocks = (size_t)rows_total * (cols / 16);
    if (dtype == CLEF_BF16 && use_hot() && hot_scale_ok(global_scale) && cols % 512 == 0 && total_blocks / 32 < 0x7fffffffull && aligned(x, 32) &&
        aligned(gate, 32)) {
        const uint32_t segs = (uint32_t)(cols / 512);
        const uint32_t live_units = (uint32_t)rows * segs, total_units = (uint32_t)rows_total * segs;
        constexpr int kUnits = 1, kMinCtas = 3;
        static std::atomic<int> occ{0};
        const int per_sm = ctas_per_sm(swiglu_quant_hot_kernel<kUnits, kMinCtas, kActSigmoidMul>, 0, occ);
        const size_t ctas = ((size_t)total_units + kUnits * 8 - 1) / (kUnits * 8);
        launch_hot(swiglu_quant_hot_kernel<kUnits, kMinCtas, kActSigmoidMul>, clamp_grid(ctas, (size_t)dev.sms * per_sm), 0,
                   s, (const uint16_t*)gate, (const uint16_t*)x, packed, scales, live_units, total_units, cols,
                   global_scale, blk_mn, chunk, make_fast_div(segs), make_fast_div((uint32_t)blk_mn));
        return check_launch(what);
    }
    if (dtype == CLEF_F32 && use_hot() && hot_scale_ok(global_scale) && cols % 512 == 0 && total_blocks / 32 < 0x7fffffffull && aligned(x, 32) &&
        aligned(gate, 32)) {
        launch_unit_quant_f32<2>(s, dev, (const float*)gate, (const float*)x, packed, scales, rows, rows_total, cols, global_scale,
                                 blk_mn, chunk);
        return check_launch(what);
    }
    if (dtype == CLEF_BF16) {
        launch_quantise_generic<Bf16, kActSigmoidMul>(s, dev, gate, x, packed, scales, rows, rows_total, cols, global_scale,
                                                      blk_mn, chunk);
    } else {
        launch_quantise_generic<F32, kActSigmoidMul>(s, dev, gate, x, packed, scales, rows, rows_total, cols, global_scale,
                                                     blk_mn, chunk);
    }
    return check_launch(what);
}

int clef_sigmoid_mul_quantise_nvfp4(clef_stream_t stream, const void* x, const void* gate, uint8_t* packed,
                                    uint8_t* scales, int rows, int cols, float global_scale, int blk_mn, int chunk,
                                    int dtype) {
    return clef_sigmoid_mul_quantise_nvfp4_impl(stream, x, gate, packed, scales, rows, cols, global_scale, blk_mn, chunk, dtype, CLEF_SF_DEFAULT);
}

int clef_sigmoid_mul_quantise_nvfp4_ex(clef_stream_t stream, const void* x, const void* gate, uint8_t* packed,
                                    uint8_t* scales, int rows, int cols, float global_scale, int blk_mn, int chunk,
                                    int dtype, int sf_layout) {
    return clef_sigmoid_mul_quantise_nvfp4_impl(stream, x, gate, packed, scales, rows, cols, global_scale, blk_mn, chunk, dtype, sf_layout);
}

int clef_copy_bytes(clef_stream_t stream, void* dst, size_t dst_offset, const void* src, size_t src_offset, size_t bytes) {
    const char* what = "clef_copy_bytes";
    if (!dst || !src) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (bytes == 0) return CLEF_OK;
    uint8_t* d = static_cast<uint8_t*>(dst) + dst_offset;
    const uint8_t* s8 = static_cast<const uint8_t*>(src) + src_offset;
    if (d < s8 + bytes && s8 < d + bytes) return fail(CLEF_ERR_INVALID, "%s: the ranges overlap", what);
    DeviceInfo dev;
    if (int r = device_info(dev)) return r;
    static std::atomic<int> occ{0};
    const int per_sm = ctas_per_sm(copy_bytes_kernel, 0, occ);
    const size_t threads = (reinterpret_cast<uintptr_t>(d) ^ reinterpret_cast<uintptr_t>(s8)) & 31 ? bytes : bytes / 32 + 64;
    launch_hot(copy_bytes_kernel, clamp_grid((threads + kCtaThreads - 1) / kCtaThreads, (size_t)dev.sms * per_sm), 0,
               as_stream(stream), d, s8, bytes);
    return check_launch(what);
}

int clef_add(clef_stream_t stream, void* out, const void* a, const void* b, size_t total, int dtype) {
    const char* what = "clef_add";
    if (int r = check_dtype(dtype, what)) return r;
    if (!out || !a || !b) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (!aligned(out, 16) || !aligned(a, 16) || !aligned(b, 16)) {
        return fail(CLEF_ERR_INVALID, "%s: pointers must be 16-byte aligned", what);
    }
    if (total == 0) return CLEF_OK;
    DeviceInfo dev;
    if (int r = device_info(dev)) return r;
    cudaStream_t s = as_stream(stream);
    if (dtype == CLEF_BF16 && use_hot() && total >= 16 && total / 16 < 0xffffffffull && aligned(out, 32) && aligned(a, 32) &&
        aligned(b, 32)) {
        static std::atomic<int> occ{0};
        const int per_sm = ctas_per_sm(add_hot_kernel, 0, occ);
        const size_t blocks = total / 16;
        launch_hot(add_hot_kernel, clamp_grid((blocks + kCtaThreads - 1) / kCtaThreads, (size_t)dev.sms * per_sm), 0, s,
                   (uint16_t*)out, (const uint16_t*)a, (const uint16_t*)b, (uint32_t)blocks);
        if (int r = check_launch(what)) return r;
        const size_t done = blocks * 16;
        if (done == total) return CLEF_OK;
        a = (const uint16_t*)a + done;
        b = (const uint16_t*)b + done;
        out = (uint16_t*)out + done;
        total -= done;
    }
    const size_t quads = (total + 3) / 4;
    if (dtype == CLEF_BF16) {
        static std::atomic<int> occ{0};
        const int per_sm = ctas_per_sm(add_generic_kernel<Bf16>, 0, occ);
        add_generic_kernel<Bf16><<<clamp_grid((quads + kCtaThreads - 1) / kCtaThreads, (size_t)dev.sms * per_sm), kCtaThreads,
                                   0, s>>>((uint16_t*)out, (const uint16_t*)a, (const uint16_t*)b, total);
    } else {
        static std::atomic<int> occ{0};
        const int per_sm = ctas_per_sm(add_generic_kernel<F32>, 0, occ);
        add_generic_kernel<F32><<<clamp_grid((quads + kCtaThreads - 1) / kCtaThreads, (size_t)dev.sms * per_sm), kCtaThreads,
                                  0, s>>>((float*)out, (const float*)a, (const float*)b, total);
    }
    return check_launch(what);
}

}  // extern "C"
