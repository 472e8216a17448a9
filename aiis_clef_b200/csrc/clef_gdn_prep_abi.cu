// C-ABI of the elementwise kernels in front of the Gated-DeltaNet scan (causal convolution + silu with the
// per-token maps, history save, gate transform, splitting copies). Declarations and the reference interfaces:
// include/clef_fused.h. Asynchronous on the caller's stream, no allocation, no synchronisation, grids that depend
// on the shape arguments only.

#include "../../include/clef_fused.h"

#include <atomic>

#include "abi_support.cuh"
#include "kernels_gdn_prep.cuh"

using namespace clef;
using namespace clef::abi;

namespace {

template <typename T>
void launch_conv(cudaStream_t s, const DeviceInfo& dev, void* out, const void* x, const float* w, int rows, int channels,
                 int k, const int32_t* seq_start, const void* history, const int32_t* slot_map) {
    if (k == 4 && channels % 8 == 0 && use_hot()) {   // 4 channels per thread, three CTAs per SM (measured)
        static std::atomic<int> occ{0};
        // 8,192 channels (16 + 16 heads of q and k and 32 of v, 128 wide) is the engine's mixed row: its stride is compiled in
        auto kernel = channels == 8192 ? causal_conv_silu_c4_kernel<4, 8, 3, 8192, T> : causal_conv_silu_c4_kernel<4, 8, 3, 0, T>;
        const int per_sm = ctas_per_sm(kernel, 0, occ);
        const size_t items = (size_t)((rows + 7) / 8) * (channels / 4);
        launch_hot(kernel, clamp_grid((items + kCtaThreads - 1) / kCtaThreads, (size_t)dev.sms * per_sm), 0, s,
                   (Storage<T>*)out, (const Storage<T>*)x, w, rows, channels, (const int*)seq_start,
                   (const Storage<T>*)history, (const int*)slot_map, make_fast_div((uint32_t)(channels / 4)));
        return;
    }
    static std::atomic<int> occ{0};
    auto kernel = causal_conv_silu_generic_kernel<T>;
    const int per_sm = ctas_per_sm(kernel, 0, occ);
    const size_t items = (size_t)rows * channels;
    kernel<<<clamp_grid((items + kCtaThreads - 1) / kCtaThreads, (size_t)dev.sms * per_sm), kCtaThreads, 0, s>>>(
        (Storage<T>*)out, (const Storage<T>*)x, w, rows, channels, k, seq_start, (const Storage<T>*)history, slot_map);
}

template <typename T>
void launch_split(cudaStream_t s, const DeviceInfo& dev, const void* in, void* o0, void* o1, void* o2, size_t rows,
                  const SplitPlan& plan) {
    static std::atomic<int> occ{0};
    auto kernel = split_rows_kernel<T>;
    const int per_sm = ctas_per_sm(kernel, 0, occ);
    const size_t items = rows * (size_t)(plan.in_width / (16 / T::kBytes));
    kernel<<<clamp_grid((items + kCtaThreads - 1) / kCtaThreads, (size_t)dev.sms * per_sm), kCtaThreads, 0, s>>>(
        (const Storage<T>*)in, (Storage<T>*)o0, (Storage<T>*)o1, (Storage<T>*)o2, rows, plan);
}

int split_impl(const char* what, clef_stream_t stream, const void* in, void* o0, void* o1, void* o2, size_t rows,
               const SplitPlan& plan, int dtype) {
    const int per = dtype == CLEF_BF16 ? 8 : 4;
    for (int i = 0; i < plan.n_out; ++i) {
        if (plan.width[i] <= 0 || plan.width[i] % per != 0) {
            return fail(CLEF_ERR_INVALID, "%s: every part must be a positive multiple of %d values wide (16 bytes)", what, per);
        }
    }
    if (!aligned(in, 16) || !aligned(o0, 16) || !aligned(o1, 16) || (o2 && !aligned(o2, 16))) {
        return fail(CLEF_ERR_INVALID, "%s: pointers must be 16-byte aligned", what);
    }
    if (rows == 0) return CLEF_OK;
    if (rows * (size_t)plan.in_width >= ((size_t)1 << 40)) return fail(CLEF_ERR_TOO_LARGE, "%s: too many values", what);
    DeviceInfo dev;
    if (int r = device_info(dev)) return r;
    if (dtype == CLEF_BF16) {
        launch_split<Bf16>(as_stream(stream), dev, in, o0, o1, o2, rows, plan);
    } else {
        launch_split<F32>(as_stream(stream), dev, in, o0, o1, o2, rows, plan);
    }
    return check_launch(what);
}

}  // namespace

extern "C" {

int clef_causal_conv_silu(clef_stream_t stream, void* out, const void* x, const float* w, int rows, int channels, int k,
                          const int32_t* seq_start, const void* history, const int32_t* slot_map, int dtype) {
    const char* what = "clef_causal_conv_silu";
    if (int r = check_dtype(dtype, what)) return r;
    if (!out || !x || !w) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (rows < 0 || channels <= 0 || k <= 0) return fail(CLEF_ERR_INVALID, "%s: rows %d channels %d k %d", what, rows, channels, k);
    if (out == x) return fail(CLEF_ERR_INVALID, "%s: out must not alias x (a row is read by the k - 1 rows after it)", what);
    if (!aligned(out, 16) || !aligned(x, 16) || !aligned(w, 16) || (history && !aligned(history, 16))) {
        return fail(CLEF_ERR_INVALID, "%s: pointers must be 16-byte aligned", what);
    }
    if ((size_t)rows * channels >= ((size_t)1 << 34)) return fail(CLEF_ERR_TOO_LARGE, "%s: %d x %d values", what, rows, channels);
    if (rows == 0) return CLEF_OK;
    DeviceInfo dev;
    if (int r = device_info(dev)) return r;
    if (dtype == CLEF_BF16) {
        launch_conv<Bf16>(as_stream(stream), dev, out, x, w, rows, channels, k, seq_start, history, slot_map);
    } else {
        launch_conv<F32>(as_stream(stream), dev, out, x, w, rows, channels, k, seq_start, history, slot_map);
    }
    return check_launch(what);
}

int clef_conv_hist_save(clef_stream_t stream, void* hist, const void* src, const int32_t* saves, int n_saves, int rows,
                        int k, int channels, int dtype) {
    const char* what = "clef_conv_hist_save";
    if (int r = check_dtype(dtype, what)) return r;
    if (n_saves < 0 || rows < 0 || k < 1 || channels <= 0) {
        return fail(CLEF_ERR_INVALID, "%s: n_saves %d rows %d k %d channels %d", what, n_saves, rows, k, channels);
    }
    if (n_saves == 0) return CLEF_OK;
    if (!hist || !src || !saves) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    const int per = dtype == CLEF_BF16 ? 8 : 4;
    if (!aligned(hist, 16) || !aligned(src, 16) || channels % per != 0) {
        return fail(CLEF_ERR_INVALID, "%s: pointers 16-byte aligned and channels a multiple of %d", what, per);
    }
    DeviceInfo dev;
    if (int r = device_info(dev)) return r;
    if (dtype == CLEF_BF16) {
        conv_hist_save_kernel<Bf16><<<n_saves, kCtaThreads, 0, as_stream(stream)>>>((const uint16_t*)src, (uint16_t*)hist, saves,
                                                                                  n_saves, rows, k, channels);
    } else {
        conv_hist_save_kernel<F32><<<n_saves, kCtaThreads, 0, as_stream(stream)>>>((const float*)src, (float*)hist, saves, n_saves,
                                                                                 rows, k, channels);
    }
    return check_launch(what);
}

int clef_gdn_gates(clef_stream_t stream, const void* a, const void* b, const float* a_log, const float* dt_bias,
                   float* decay, float* beta, int tokens, int heads, int dtype) {
    const char* what = "clef_gdn_gates";
    if (int r = check_dtype(dtype, what)) return r;
    if (!a || !b || !a_log || !dt_bias || !decay || !beta) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (tokens < 0 || heads <= 0 || (long long)tokens * heads > 0x7fffffffLL) {
        return fail(CLEF_ERR_INVALID, "%s: tokens %d heads %d", what, tokens, heads);
    }
    if (tokens == 0) return CLEF_OK;
    DeviceInfo dev;
    if (int r = device_info(dev)) return r;
    const int total = tokens * heads;
    const unsigned grid = clamp_grid(((size_t)total + kCtaThreads - 1) / kCtaThreads, (size_t)dev.sms * 8);
    if (dtype == CLEF_BF16) {
        gdn_gates_kernel<Bf16><<<grid, kCtaThreads, 0, as_stream(stream)>>>((const uint16_t*)a, (const uint16_t*)b, a_log, dt_bias,
                                                                         decay, beta, total, heads);
    } else {
        gdn_gates_kernel<F32><<<grid, kCtaThreads, 0, as_stream(stream)>>>((const float*)a, (const float*)b, a_log, dt_bias, decay,
                                                                        beta, total, heads);
    }
    return check_launch(what);
}

int clef_gdn_prep(clef_stream_t stream, const void* mixed, float* v_out, void* q_hi, void* q_lo, void* k_hi, void* k_lo,
                  float* kn, int seq_len, int heads, int kh, int kd, int conv_dim, float q_scale, int dtype) {
    const char* what = "clef_gdn_prep";
    if (int r = check_dtype(dtype, what)) return r;
    if (!mixed || !v_out || !q_hi || !q_lo || !k_hi || !k_lo || !kn) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (seq_len < 0 || heads <= 0 || kh <= 0 || heads % kh != 0) {
        return fail(CLEF_ERR_INVALID, "%s: seq_len %d heads %d kh %d (heads must be a multiple of kh)", what, seq_len, heads, kh);
    }
    if (kd != kGdnKd) return fail(CLEF_ERR_INVALID, "%s: kd %d (the scan's operand layout is built for 128)", what, kd);
    if ((long long)conv_dim < 2LL * kh * kd + (long long)heads * kd || conv_dim % 8 != 0) {
        return fail(CLEF_ERR_INVALID, "%s: conv_dim %d must hold q, k (kh x kd each) and v (heads x kd) and be a multiple of 8",
                    what, conv_dim);
    }
    if (!aligned(mixed, 16) || !aligned(v_out, 16) || !aligned(q_hi, 16) || !aligned(q_lo, 16) || !aligned(k_hi, 16) ||
        !aligned(k_lo, 16) || !aligned(kn, 16)) {
        return fail(CLEF_ERR_INVALID, "%s: pointers must be 16-byte aligned", what);
    }
    if (seq_len == 0) return CLEF_OK;
    DeviceInfo dev;
    if (int r = device_info(dev)) return r;
    const int nchunks = (seq_len + kGdnChunk - 1) / kGdnChunk;
    const size_t warps = (size_t)nchunks * kGdnChunk * kh;
    if (warps >= 0x7fffffffull || (size_t)seq_len * heads * (kGdnKd / 8) >= 0x7fffffffull) {
        return fail(CLEF_ERR_TOO_LARGE, "%s: seq_len %d x heads %d exceeds the 32-bit item range", what, seq_len, heads);
    }
    const unsigned grid = clamp_grid((warps + kCtaThreads / 32 - 1) / (kCtaThreads / 32), (size_t)dev.sms * 8);
    const FastDiv kh_div = make_fast_div((uint32_t)kh), vvec_div = make_fast_div((uint32_t)heads * (kGdnKd / 8));
    if (dtype == CLEF_BF16) {
        gdn_prep_kernel<Bf16><<<grid, kCtaThreads, 0, as_stream(stream)>>>(
            (const uint16_t*)mixed, v_out, (uint8_t*)q_hi, (uint8_t*)q_lo, (uint8_t*)k_hi, (uint8_t*)k_lo, kn, seq_len, heads, kh,
            nchunks, conv_dim, q_scale, kh_div, vvec_div);
    } else {
        gdn_prep_kernel<F32><<<grid, kCtaThreads, 0, as_stream(stream)>>>(
            (const float*)mixed, v_out, (uint8_t*)q_hi, (uint8_t*)q_lo, (uint8_t*)k_hi, (uint8_t*)k_lo, kn, seq_len, heads, kh,
            nchunks, conv_dim, q_scale, kh_div, vvec_div);
    }
    return check_launch(what);
}

int clef_gdn_conv_prep(clef_stream_t stream, const void* x, const float* w, float* v_out, void* q_hi, void* q_lo, void* k_hi,
                       void* k_lo, float* kn, int rows, int channels, int k, const int32_t* seq_start, const void* history,
                       const int32_t* slot_map, int heads, int kh, int kd, float q_scale, int dtype) {
    const char* what = "clef_gdn_conv_prep";
    if (int r = check_dtype(dtype, what)) return r;
    if (!x || !w || !v_out || !q_hi || !q_lo || !k_hi || !k_lo || !kn) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (rows < 0 || channels <= 0 || k <= 0 || heads <= 0 || kh <= 0 || heads % kh != 0) {
        return fail(CLEF_ERR_INVALID, "%s: rows %d channels %d k %d heads %d kh %d", what, rows, channels, k, heads, kh);
    }
    if (kd != kGdnKd) return fail(CLEF_ERR_INVALID, "%s: kd %d (the scan's operand layout is built for 128)", what, kd);
    if ((long long)channels != 2LL * kh * kd + (long long)heads * kd) {
        return fail(CLEF_ERR_INVALID, "%s: channels %d must be q, k (kh x kd each) and v (heads x kd)", what, channels);
    }
    if (!aligned(x, 16) || !aligned(w, 16) || !aligned(v_out, 16) || !aligned(q_hi, 16) || !aligned(q_lo, 16) ||
        !aligned(k_hi, 16) || !aligned(k_lo, 16) || !aligned(kn, 16) || (history && !aligned(history, 16))) {
        return fail(CLEF_ERR_INVALID, "%s: pointers must be 16-byte aligned", what);
    }
    // One launch for 4 taps and 1, 2 or 4 value heads per key head (the repeat count is compiled in); other shapes, and
    // the shape-general kernel choice, decline: the caller then runs clef_causal_conv_silu + clef_gdn_prep.
    if (k != 4 || !use_hot() || (heads != kh && heads != 2 * kh && heads != 4 * kh)) return CLEF_DECLINED;
    if (rows == 0) return CLEF_OK;
    if ((size_t)rows * channels >= ((size_t)1 << 34)) return fail(CLEF_ERR_TOO_LARGE, "%s: %d x %d values", what, rows, channels);
    DeviceInfo dev;
    if (int r = device_info(dev)) return r;
    const int nchunks = (rows + kGdnChunk - 1) / kGdnChunk;
    const size_t items = (size_t)nchunks * (kGdnChunk / 8) * (channels / kGdnKd);
    const FastDiv groups_div = make_fast_div((uint32_t)(channels / kGdnKd));
    auto launch = [&](auto kernel, std::atomic<int>& occ, auto* xp, auto* hp) {
        const int per_sm = ctas_per_sm(kernel, 0, occ);
        launch_hot(kernel, clamp_grid((items + kCtaThreads / 32 - 1) / (kCtaThreads / 32), (size_t)dev.sms * per_sm), 0,
                   as_stream(stream), xp, w, v_out, (uint8_t*)q_hi, (uint8_t*)q_lo, (uint8_t*)k_hi, (uint8_t*)k_lo, kn, rows,
                   channels, (const int*)seq_start, hp, (const int*)slot_map, heads, kh, nchunks, q_scale, groups_div);
    };
    static std::atomic<int> occ[6];
    const int ratio = heads / kh;
#define CLEF_GDN_FUSED(RATIO, SLOT)                                                                                          \
    if (dtype == CLEF_BF16) launch(gdn_conv_prep_kernel<Bf16, 4, 8, 3, RATIO>, occ[SLOT], (const uint16_t*)x, (const uint16_t*)history); \
    else launch(gdn_conv_prep_kernel<F32, 4, 8, 3, RATIO>, occ[SLOT + 1], (const float*)x, (const float*)history);
    if (ratio == 1) {
        CLEF_GDN_FUSED(1, 0)
    } else if (ratio == 2) {
        CLEF_GDN_FUSED(2, 2)
    } else {
        CLEF_GDN_FUSED(4, 4)
    }
#undef CLEF_GDN_FUSED
    return check_launch(what);
}

int clef_split_q_gate(clef_stream_t stream, const void* qg, void* q, void* gate, int tokens, int heads, int head_dim,
                      int dtype) {
    const char* what = "clef_split_q_gate";
    if (int r = check_dtype(dtype, what)) return r;
    if (!qg || !q || !gate) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (tokens < 0 || heads <= 0 || head_dim <= 0) return fail(CLEF_ERR_INVALID, "%s: tokens %d heads %d head_dim %d", what, tokens, heads, head_dim);
    SplitPlan plan{2 * head_dim, 2, {0, head_dim, 0}, {head_dim, head_dim, 0}};
    return split_impl(what, stream, qg, q, gate, nullptr, (size_t)tokens * heads, plan, dtype);
}

int clef_split_qkv(clef_stream_t stream, const void* mixed, void* q, void* k, void* v, int tokens, int kh, int kd, int vh,
                   int vd, int dtype) {
    const char* what = "clef_split_qkv";
    if (int r = check_dtype(dtype, what)) return r;
    if (!mixed || !q || !k || !v) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (tokens < 0 || kh <= 0 || kd <= 0 || vh <= 0 || vd <= 0) {
        return fail(CLEF_ERR_INVALID, "%s: tokens %d kh %d kd %d vh %d vd %d", what, tokens, kh, kd, vh, vd);
    }
    const int qk = kh * kd, vw = vh * vd;
    SplitPlan plan{2 * qk + vw, 3, {0, qk, 2 * qk}, {qk, qk, vw}};
    return split_impl(what, stream, mixed, q, k, v, (size_t)tokens, plan, dtype);
}

int clef_repeat_interleave(clef_stream_t stream, const void* src, void* out, int tokens, int kh, int ratio, int dim,
                           int dtype) {
    const char* what = "clef_repeat_interleave";
    if (int r = check_dtype(dtype, what)) return r;
    if (!src || !out) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    const int per = dtype == CLEF_BF16 ? 8 : 4;
    if (tokens < 0 || kh <= 0 || ratio <= 0 || dim <= 0 || dim % per != 0) {
        return fail(CLEF_ERR_INVALID, "%s: tokens %d kh %d ratio %d dim %d (dim a multiple of %d)", what, tokens, kh, ratio, dim, per);
    }
    if (!aligned(src, 16) || !aligned(out, 16)) return fail(CLEF_ERR_INVALID, "%s: pointers must be 16-byte aligned", what);
    if (tokens == 0) return CLEF_OK;
    DeviceInfo dev;
    if (int r = device_info(dev)) return r;
    const size_t head_rows_out = (size_t)tokens * kh * ratio;
    const size_t items = head_rows_out * (size_t)(dim / per);
    if (dtype == CLEF_BF16) {
        static std::atomic<int> occ{0};
        const int per_sm = ctas_per_sm(repeat_interleave_kernel<Bf16>, 0, occ);
        repeat_interleave_kernel<Bf16><<<clamp_grid((items + kCtaThreads - 1) / kCtaThreads, (size_t)dev.sms * per_sm), kCtaThreads, 0,
                                         as_stream(stream)>>>((const uint16_t*)src, (uint16_t*)out, head_rows_out, ratio, dim);
    } else {
        static std::atomic<int> occ{0};
        const int per_sm = ctas_per_sm(repeat_interleave_kernel<F32>, 0, occ);
        repeat_interleave_kernel<F32><<<clamp_grid((items + kCtaThreads - 1) / kCtaThreads, (size_t)dev.sms * per_sm), kCtaThreads, 0,
                                        as_stream(stream)>>>((const float*)src, (float*)out, head_rows_out, ratio, dim);
    }
    return check_launch(what);
}

}  // extern "C"
