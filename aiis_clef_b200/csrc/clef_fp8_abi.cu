// C-ABI of the FP8 (E4M3) activation quantisers. Declarations and the reference interfaces:
// include/clef_fused.h. Same contract as the other entry points: asynchronous on the caller's stream,
// no allocation, no synchronisation, grids that depend on the shape arguments only.

#include "../../include/clef_fused.h"

#include <atomic>

#include "abi_support.cuh"
#include "kernels_fp8.cuh"

using namespace clef;
using namespace clef::abi;

namespace {

constexpr int kFp8MaxCols = 16384;   // 8 vectors of 8 values per thread of a 256-thread CTA

template <typename T, int MODE, int KMAX>
void launch_fp8_rows_k(cudaStream_t s, const DeviceInfo& dev, const void* a, const void* b, const float* weight,
                       uint8_t* out, uint16_t* scales, uint16_t* bf_out, int rows, int cols, float eps) {
    static std::atomic<int> occ{0};
    auto kernel = fp8_rows_kernel<T, MODE, KMAX>;
    const int per_sm = ctas_per_sm(kernel, 0, occ);
    kernel<<<clamp_grid((size_t)rows, (size_t)dev.sms * per_sm), kCtaThreads, 0, s>>>(
        (const Storage<T>*)a, (const Storage<T>*)b, weight, out, scales, bf_out, rows, cols, eps);
}

template <typename T, int MODE>
void launch_fp8_rows(cudaStream_t s, const DeviceInfo& dev, const void* a, const void* b, const float* weight,
                     uint8_t* out, uint16_t* scales, uint16_t* bf_out, int rows, int cols, float eps) {
    const int k = (cols + 2047) / 2048;
    if (k <= 1) launch_fp8_rows_k<T, MODE, 1>(s, dev, a, b, weight, out, scales, bf_out, rows, cols, eps);
    else if (k <= 2) launch_fp8_rows_k<T, MODE, 2>(s, dev, a, b, weight, out, scales, bf_out, rows, cols, eps);
    else if (k <= 3) launch_fp8_rows_k<T, MODE, 3>(s, dev, a, b, weight, out, scales, bf_out, rows, cols, eps);
    else if (k <= 4) launch_fp8_rows_k<T, MODE, 4>(s, dev, a, b, weight, out, scales, bf_out, rows, cols, eps);
    else if (k <= 6) launch_fp8_rows_k<T, MODE, 6>(s, dev, a, b, weight, out, scales, bf_out, rows, cols, eps);
    else launch_fp8_rows_k<T, MODE, 8>(s, dev, a, b, weight, out, scales, bf_out, rows, cols, eps);
}

int fp8_rows_impl(const char* what, int mode, clef_stream_t stream, const void* a, const void* b, const float* weight,
                  uint8_t* out, uint16_t* scales, uint16_t* bf_out, int rows, int cols, float eps, int dtype) {
    if (int r = check_dtype(dtype, what)) return r;
    if (!a || !out || !scales || (mode == kFp8SwiGLU && !b) || (mode == kFp8RmsNorm && !weight)) {
        return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    }
    if (rows < 0 || cols <= 0 || cols % 8 != 0) {
        return fail(CLEF_ERR_INVALID, "%s: rows %d, cols %d (cols must be a positive multiple of 8)", what, rows, cols);
    }
    if (cols > kFp8MaxCols) return fail(CLEF_ERR_TOO_LARGE, "%s: cols %d above %d", what, cols, kFp8MaxCols);
    if (!aligned(a, 16) || (b && !aligned(b, 16)) || !aligned(out, 8) || !aligned(scales, 2) ||
        (weight && !aligned(weight, 16)) || (bf_out && !aligned(bf_out, 16))) {
        return fail(CLEF_ERR_INVALID, "%s: activations, weight and the bf16 output must be 16-byte aligned, codes 8-byte", what);
    }
    if (rows == 0) return CLEF_OK;
    DeviceInfo dev;
    if (int r = device_info(dev)) return r;
    cudaStream_t s = as_stream(stream);
    if (use_hot() && mode == kFp8RmsNorm && (cols == 2048 || cols == 4096) && aligned(a, 32) &&
        aligned(out, 16) && (!bf_out || aligned(bf_out, 32))) {
        const size_t groups = ((size_t)rows + 7) / 8;
        const size_t smem = (size_t)cols * sizeof(float);
#define CLEF_FP8_HOT(NB, MODE, T)                                                                                   \
    {                                                                                                               \
        static std::atomic<int> occ{0};                                                                             \
        const int per_sm = ctas_per_sm(fp8_rows_hot_kernel<NB, MODE, T>, smem, occ);                                \
        launch_hot(fp8_rows_hot_kernel<NB, MODE, T>, clamp_grid(groups, (size_t)dev.sms * per_sm), smem, s,         \
                   (const Storage<T>*)a, weight, out, scales, bf_out, rows, eps);                                   \
    }
        if (dtype == CLEF_BF16) {
            if (cols == 2048) CLEF_FP8_HOT(4, kFp8RmsNorm, Bf16) else CLEF_FP8_HOT(8, kFp8RmsNorm, Bf16)
        } else {
            if (cols == 2048) CLEF_FP8_HOT(4, kFp8RmsNorm, F32) else CLEF_FP8_HOT(8, kFp8RmsNorm, F32)
        }
#undef CLEF_FP8_HOT
        return check_launch(what);
    }
    if (use_hot() && mode != kFp8RmsNorm && aligned(a, 32) && (!b || aligned(b, 32)) && aligned(out, 16)) {
        // cols = 512 * WPR * BPL with BPL 3 or 4 blocks per lane and WPR 1, 2, 4 or 8 warps per row
        const int bpl = (cols % 1536 == 0) ? 3 : ((cols % 2048 == 0) ? 4 : 0);
        const int wpr = bpl ? cols / (512 * bpl) : 0;
        if (wpr == 1 || wpr == 2 || wpr == 4 || wpr == 8) {
#define CLEF_FP8_TEAM_T(MODE, BPL, WPR, T)                                                                          \
    {                                                                                                               \
        static std::atomic<int> occ{0};                                                                             \
        const int per_sm = ctas_per_sm(fp8_team_hot_kernel<MODE, BPL, WPR, T>, 0, occ);                             \
        const size_t ctas = ((size_t)rows + (8 / WPR) - 1) / (8 / WPR);                                             \
        launch_hot(fp8_team_hot_kernel<MODE, BPL, WPR, T>, clamp_grid(ctas, (size_t)dev.sms * per_sm), 0, s,        \
                   (const Storage<T>*)a, (const Storage<T>*)b, out, scales, rows);                                  \
    }
#define CLEF_FP8_TEAM(MODE, BPL, WPR)                                                \
    {                                                                                \
        if (dtype == CLEF_BF16) CLEF_FP8_TEAM_T(MODE, BPL, WPR, Bf16)                \
        else CLEF_FP8_TEAM_T(MODE, BPL, WPR, F32)                                    \
    }
#define CLEF_FP8_TEAM_W(MODE, BPL)                                      \
    if (wpr == 1) CLEF_FP8_TEAM(MODE, BPL, 1)                           \
    else if (wpr == 2) CLEF_FP8_TEAM(MODE, BPL, 2)                      \
    else if (wpr == 4) CLEF_FP8_TEAM(MODE, BPL, 4)                      \
    else CLEF_FP8_TEAM(MODE, BPL, 8)
            if (mode == kFp8Plain) {
                if (bpl == 3) { CLEF_FP8_TEAM_W(kFp8Plain, 3) } else { CLEF_FP8_TEAM_W(kFp8Plain, 4) }
            } else {
                if (bpl == 3) { CLEF_FP8_TEAM_W(kFp8SwiGLU, 3) } else { CLEF_FP8_TEAM_W(kFp8SwiGLU, 4) }
            }
#undef CLEF_FP8_TEAM_W
#undef CLEF_FP8_TEAM
#undef CLEF_FP8_TEAM_T
            return check_launch(what);
        }
    }
#define CLEF_FP8_DISPATCH(MODE)                                                                                 \
    if (dtype == CLEF_BF16) launch_fp8_rows<Bf16, MODE>(s, dev, a, b, weight, out, scales, bf_out, rows, cols, eps); \
    else launch_fp8_rows<F32, MODE>(s, dev, a, b, weight, out, scales, bf_out, rows, cols, eps);
    if (mode == kFp8Plain) {
        CLEF_FP8_DISPATCH(kFp8Plain)
    } else if (mode == kFp8SwiGLU) {
        CLEF_FP8_DISPATCH(kFp8SwiGLU)
    } else {
        CLEF_FP8_DISPATCH(kFp8RmsNorm)
    }
#undef CLEF_FP8_DISPATCH
    return check_launch(what);
}

template <typename T, int HMAX>
void launch_fp8_gated(cudaStream_t s, const DeviceInfo& dev, const void* x, const void* gate, const float* weight,
                      uint8_t* out, uint16_t* scales, int tokens, int cols, float eps, int vh, int rows_live) {
    static std::atomic<int> occ{0};
    auto kernel = fp8_gated_kernel<T, HMAX>;
    const int per_sm = ctas_per_sm(kernel, 0, occ);
    kernel<<<clamp_grid((size_t)tokens, (size_t)dev.sms * per_sm), kCtaThreads, 0, s>>>(
        (const Storage<T>*)x, (const Storage<T>*)gate, weight, out, scales, tokens, cols, eps, vh, rows_live);
}

}  // namespace

extern "C" {

int clef_quantise_fp8(clef_stream_t stream, const void* x, uint8_t* out, uint16_t* scales, int rows, int cols,
                      int dtype) {
    return fp8_rows_impl("clef_quantise_fp8", kFp8Plain, stream, x, nullptr, nullptr, out, scales, nullptr, rows, cols,
                         0.0f, dtype);
}

int clef_swiglu_quantise_fp8(clef_stream_t stream, const void* gate, const void* up, uint8_t* out, uint16_t* scales,
                             int rows, int cols, int dtype) {
    return fp8_rows_impl("clef_swiglu_quantise_fp8", kFp8SwiGLU, stream, gate, up, nullptr, out, scales, nullptr, rows,
                         cols, 0.0f, dtype);
}

int clef_rms_norm_fp8_bf16(clef_stream_t stream, const void* x, const float* weight, uint8_t* q_out,
                           uint16_t* q_scales, uint16_t* bf_out, int rows, int cols, float eps, int dtype) {
    return fp8_rows_impl("clef_rms_norm_fp8_bf16", kFp8RmsNorm, stream, x, nullptr, weight, q_out, q_scales, bf_out, rows,
                         cols, eps, dtype);
}

int clef_rms_norm_gated_quantise_fp8(clef_stream_t stream, const void* x, const void* gate, const float* weight,
                                     uint8_t* out, uint16_t* scales, int rows, int cols, float eps, int vh,
                                     int rows_live, int dtype) {
    const char* what = "clef_rms_norm_gated_quantise_fp8";
    if (int r = check_dtype(dtype, what)) return r;
    if (!x || !gate || !weight || !out || !scales) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (rows < 0 || cols <= 0 || cols % 4 != 0 || vh <= 0 || rows % vh != 0 || rows_live < 0 || rows_live > rows) {
        return fail(CLEF_ERR_INVALID, "%s: rows %d (a multiple of vh %d), rows_live %d, cols %d (a multiple of 4)", what,
                    rows, vh, rows_live, cols);
    }
    if (cols > 256) return fail(CLEF_ERR_TOO_LARGE, "%s: head width %d above 256", what, cols);
    if (vh > 64) return fail(CLEF_ERR_TOO_LARGE, "%s: %d head rows per token above 64", what, vh);
    if (!aligned(x, 16) || !aligned(gate, 16) || !aligned(weight, 16) || !aligned(out, 4) || !aligned(scales, 2)) {
        return fail(CLEF_ERR_INVALID, "%s: x, gate and weight must be 16-byte aligned, codes 4-byte", what);
    }
    const int tokens = rows / vh;
    if (tokens == 0) return CLEF_OK;
    DeviceInfo dev;
    if (int r = device_info(dev)) return r;
    cudaStream_t s = as_stream(stream);
    if (use_hot() && cols == 128 && rows_live == rows && (vh == 8 || vh == 16 || vh == 32 || vh == 64) &&
        aligned(x, 32) && aligned(gate, 32) && aligned(out, 16)) {
#define CLEF_FP8_GATED_HOT_T(STEPS, WPT, T)                                                                       \
    {                                                                                                             \
        static std::atomic<int> occ{0};                                                                           \
        const int per_sm = ctas_per_sm(fp8_gated_hot_kernel<STEPS, WPT, T>, 0, occ);                              \
        const size_t ctas = ((size_t)tokens + (8 / WPT) - 1) / (8 / WPT);                                         \
        launch_hot(fp8_gated_hot_kernel<STEPS, WPT, T>, clamp_grid(ctas, (size_t)dev.sms * per_sm), 0, s,         \
                   (const Storage<T>*)x, (const Storage<T>*)gate, weight, out, scales, tokens, eps);              \
    }
#define CLEF_FP8_GATED_HOT(STEPS, WPT)                                            \
    {                                                                             \
        if (dtype == CLEF_BF16) CLEF_FP8_GATED_HOT_T(STEPS, WPT, Bf16)            \
        else CLEF_FP8_GATED_HOT_T(STEPS, WPT, F32)                                \
    }
        // one step per warp, vh / 8 warps per token: measured ahead of two steps per warp (which spills at 128 registers)
        if (vh == 8) CLEF_FP8_GATED_HOT(1, 1)
        else if (vh == 16) CLEF_FP8_GATED_HOT(1, 2)
        else if (vh == 32) CLEF_FP8_GATED_HOT(1, 4)
        else CLEF_FP8_GATED_HOT(1, 8)
#undef CLEF_FP8_GATED_HOT
#undef CLEF_FP8_GATED_HOT_T
        return check_launch(what);
    }
    const int hmax = (vh + 7) / 8;
#define CLEF_FP8_GATED(T)                                                                                          \
    if (hmax <= 1) launch_fp8_gated<T, 1>(s, dev, x, gate, weight, out, scales, tokens, cols, eps, vh, rows_live);     \
    else if (hmax <= 2) launch_fp8_gated<T, 2>(s, dev, x, gate, weight, out, scales, tokens, cols, eps, vh, rows_live); \
    else if (hmax <= 4) launch_fp8_gated<T, 4>(s, dev, x, gate, weight, out, scales, tokens, cols, eps, vh, rows_live); \
    else launch_fp8_gated<T, 8>(s, dev, x, gate, weight, out, scales, tokens, cols, eps, vh, rows_live);
    if (dtype == CLEF_BF16) {
        CLEF_FP8_GATED(Bf16)
    } else {
        CLEF_FP8_GATED(F32)
    }
#undef CLEF_FP8_GATED
    return check_launch(what);
}

}  // extern "C"
