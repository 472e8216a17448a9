// C-ABI of the fused elementwise kernels: argument checks, kernel selection, grid sizing, launch.
// Declarations and the reference interface each entry point replaces: include/clef_fused.h.
//
// Nothing here allocates, synchronises or copies; every launch is asynchronous on the caller's
// stream and its grid depends only on the shape arguments, so the calls can be captured in a CUDA
// graph and replayed while only buffer CONTENTS change (the reference's geometry-keyed replay).

#include "../../include/clef_fused.h"

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "abi_support.cuh"
#include "internal.hpp"
#include "kernels_generic.cuh"
#include "kernels_hot.cuh"
#include "unit_quant_f32_launch.cuh"

namespace {
thread_local char g_error[512] = "";
}

namespace clef {
int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}
}  // namespace clef

namespace {
std::atomic<int> g_kernel_choice{0};
std::atomic<int> g_scale_layout{0};
}

namespace clef {
int kernel_choice() { return g_kernel_choice.load(std::memory_order_relaxed); }
int scale_layout() { return g_scale_layout.load(std::memory_order_relaxed); }
}  // namespace clef


using namespace clef;
using namespace clef::abi;

extern "C" {

const char* clef_last_error(void) { return g_error; }

int clef_version(void) { return 100; }

void clef_set_kernel_choice(int choice) {
    g_kernel_choice.store(choice == 1 ? 1 : 0, std::memory_order_relaxed);
}

int clef_set_scale_layout(int layout) {
    if (layout != CLEF_SF_ACTIVATION && layout != CLEF_SF_INTERLEAVED) {
        return fail(CLEF_ERR_INVALID, "clef_set_scale_layout: layout %d", layout);
    }
    g_scale_layout.store(layout, std::memory_order_relaxed);
    return CLEF_OK;
}

int clef_sf_atom_for_tile_m(int tile_m, int* blk_mn, int* chunk) {
    if (tile_m <= 0) {
        return fail(CLEF_ERR_INVALID, "clef_sf_atom_for_tile_m: tile_m %d", tile_m);
    }
    int atom = 0;
    if (tile_m < 128) {
        atom = 128;
    } else {
        const int candidates[4] = {128, 96, 64, 32};
        for (int c : candidates) {
            if (tile_m % c == 0) {
                atom = c;
                break;
            }
        }
    }
    if (atom == 0) {
        return fail(CLEF_ERR_INVALID, "clef_sf_atom_for_tile_m: tile_m %d is not a multiple of 32", tile_m);
    }
    if (blk_mn) *blk_mn = atom;
    if (chunk) *chunk = atom * 4;
    return CLEF_OK;
}

int clef_nvfp4_sizes(int rows, int cols, int blk_mn, int* rows_padded, size_t* packed_bytes, size_t* scale_bytes) {
    if (rows < 0 || cols <= 0 || cols % 16 != 0 || blk_mn <= 0) {
        return fail(CLEF_ERR_INVALID, "clef_nvfp4_sizes: rows %d cols %d blk_mn %d", rows, cols, blk_mn);
    }
    const long long padded = ((long long)rows + blk_mn - 1) / blk_mn * blk_mn;
    if (padded > 0x7fffffffLL) {
        return fail(CLEF_ERR_TOO_LARGE, "clef_nvfp4_sizes: %lld padded rows", padded);
    }
    if (rows_padded) *rows_padded = (int)padded;
    if (packed_bytes) *packed_bytes = (size_t)padded * (size_t)(cols / 2);
    if (scale_bytes) *scale_bytes = (size_t)padded * (size_t)(cols / 16);
    return CLEF_OK;
}

int clef_embed_gather(clef_stream_t stream, const void* table, const int32_t* ids, void* out, int tokens, int hidden,
                      int dtype) {
    if (int r = check_dtype(dtype, "clef_embed_gather")) return r;
    if (!table || !ids || !out) return fail(CLEF_ERR_INVALID, "clef_embed_gather: null pointer");
    if (tokens < 0 || hidden <= 0) return fail(CLEF_ERR_INVALID, "clef_embed_gather: tokens %d hidden %d", tokens, hidden);
    const size_t row_bytes = (size_t)hidden * (dtype == CLEF_BF16 ? 2 : 4);
    if (row_bytes % 16 != 0 || !aligned(table, 16) || !aligned(out, 16)) {
        return fail(CLEF_ERR_INVALID, "clef_embed_gather: rows of %zu bytes / pointers must be 16-byte aligned", row_bytes);
    }
    if (tokens == 0) return CLEF_OK;
    DeviceInfo dev;
    if (int r = device_info(dev)) return r;
    const bool hot_ok = use_hot() && aligned(table, 32) && aligned(out, 32);
    if (hot_ok && (row_bytes == 4096 || row_bytes == 8192 || row_bytes == 2048 || row_bytes == 1024)) {
        const size_t groups = ((size_t)tokens + 7) / 8;
#define CLEF_EMBED_HOT(CH)                                                                                       \
    {                                                                                                            \
        static std::atomic<int> occ{0};                                                                          \
        const int per_sm = ctas_per_sm(embed_gather_hot_kernel<CH>, 0, occ);                                     \
        launch_hot(embed_gather_hot_kernel<CH>, clamp_grid(groups, (size_t)dev.sms * per_sm), 0, as_stream(stream), \
                   (const uint8_t*)table, (const int*)ids, (uint8_t*)out, tokens);                                \
    }
        switch (row_bytes / 1024) {
            case 1: CLEF_EMBED_HOT(1) break;
            case 2: CLEF_EMBED_HOT(2) break;
            case 4: CLEF_EMBED_HOT(4) break;
            default: CLEF_EMBED_HOT(8) break;
        }
#undef CLEF_EMBED_HOT
        return check_launch("clef_embed_gather");
    }
    static std::atomic<int> occ{0};
    const int per_sm = ctas_per_sm(embed_gather_generic_kernel, 0, occ);
    const size_t vecs = (size_t)tokens * (row_bytes / 16);
    embed_gather_generic_kernel<<<clamp_grid((vecs + kCtaThreads - 1) / kCtaThreads, (size_t)dev.sms * per_sm),
                                  kCtaThreads, 0, as_stream(stream)>>>((const uint8_t*)table, ids, (uint8_t*)out,
                                                                       tokens, row_bytes);
    return check_launch("clef_embed_gather");
}

// ---- rms_norm family -----------------------------------------------------------------------------

}  // extern "C"

template <typename T, bool QUANT>
static int launch_rms_norm_generic(cudaStream_t stream, const DeviceInfo& dev, const void* x, const float* weight,
                                   void* out, uint8_t* packed, uint8_t* scales, int rows, int rows_total, int cols,
                                   float eps, float global_scale, int blk_mn, int chunk) {
    static std::atomic<int> occ{0};
    auto kernel = rms_norm_generic_kernel<T, QUANT>;
    const int per_sm = ctas_per_sm(kernel, 0, occ);
    const int rpb = kCtaThreads / ref_threads_per_row(cols);
    const size_t groups = ((size_t)rows_total + rpb - 1) / rpb;
    kernel<<<clamp_grid(groups, (size_t)dev.sms * per_sm), kCtaThreads, 0, stream>>>(
        (const Storage<T>*)x, weight, (Storage<T>*)out, packed, scales, rows, rows_total, cols, eps, global_scale,
        blk_mn, chunk);
    return CLEF_OK;
}

extern "C" {

int clef_rms_norm(clef_stream_t stream, const void* x, const float* weight, void* out, int rows, int cols, float eps,
                  int dtype) {
    if (int r = check_dtype(dtype, "clef_rms_norm")) return r;
    if (!x || !out) return fail(CLEF_ERR_INVALID, "clef_rms_norm: null pointer");
    if (rows < 0 || cols <= 0 || cols % 4 != 0) {
        return fail(CLEF_ERR_INVALID, "clef_rms_norm: rows %d, cols %d (cols must be a positive multiple of 4)", rows, cols);
    }
    if (!aligned(x, 16) || !aligned(out, 16) || (weight && !aligned(weight, 16))) {
        return fail(CLEF_ERR_INVALID, "clef_rms_norm: pointers must be 16-byte aligned");
    }
    if (rows == 0) return CLEF_OK;
    DeviceInfo dev;
    if (int r = device_info(dev)) return r;
    if (dtype == CLEF_BF16 && use_hot() && (cols == 2048 || cols == 4096) && aligned(x, 32) && aligned(out, 32)) {
        const size_t groups = ((size_t)rows + 7) / 8;
        const size_t smem = (size_t)cols * sizeof(float);
        if (cols == 2048) {
            static std::atomic<int> occ{0};
            const int per_sm = ctas_per_sm(rms_norm_hot_kernel<4>, smem, occ);
            launch_hot(rms_norm_hot_kernel<4>, clamp_grid(groups, (size_t)dev.sms * per_sm), smem, as_stream(stream),
                       (const uint16_t*)x, weight, (uint16_t*)out, rows, eps);
        } else {
            static std::atomic<int> occ{0};
            const int per_sm = ctas_per_sm(rms_norm_hot_kernel<8>, smem, occ);
            launch_hot(rms_norm_hot_kernel<8>, clamp_grid(groups, (size_t)dev.sms * per_sm), smem, as_stream(stream),
                       (const uint16_t*)x, weight, (uint16_t*)out, rows, eps);
        }
        return check_launch("clef_rms_norm");
    }
    if (dtype == CLEF_F32 && use_hot() && (cols == 2048 || cols == 4096) && aligned(x, 32) && aligned(out, 32)) {
        const size_t groups = ((size_t)rows + 7) / 8;
        const size_t smem = (size_t)cols * sizeof(float);
        if (cols == 2048) {
            static std::atomic<int> occ{0};
            const int per_sm = ctas_per_sm(rms_norm_f32_hot_kernel<4>, smem, occ);
            launch_hot(rms_norm_f32_hot_kernel<4>, clamp_grid(groups, (size_t)dev.sms * per_sm), smem, as_stream(stream),
                       (const float*)x, weight, (float*)out, rows, eps);
        } else {
            static std::atomic<int> occ{0};
            const int per_sm = ctas_per_sm(rms_norm_f32_hot_kernel<8>, smem, occ);
            launch_hot(rms_norm_f32_hot_kernel<8>, clamp_grid(groups, (size_t)dev.sms * per_sm), smem, as_stream(stream),
                       (const float*)x, weight, (float*)out, rows, eps);
        }
        return check_launch("clef_rms_norm");
    }
    if (dtype == CLEF_BF16) {
        launch_rms_norm_generic<Bf16, false>(as_stream(stream), dev, x, weight, out, nullptr, nullptr, rows, rows, cols,
                                             eps, 0.0f, 1, 4);
    } else {
        launch_rms_norm_generic<F32, false>(as_stream(stream), dev, x, weight, out, nullptr, nullptr, rows, rows, cols,
                                            eps, 0.0f, 1, 4);
    }
    return check_launch("clef_rms_norm");
}

}  // extern "C"

// RMSNorm + NVFP4 of x, or (addend != NULL) of the stored sum x + addend, which is also written to sum_out.
static int rms_norm_quantise_impl(const char* what, clef_stream_t stream, const void* x, const void* addend,
                                  void* sum_out, const float* weight, uint8_t* packed, uint8_t* scales, int rows,
                                  int cols, float eps, float global_scale, int blk_mn, int chunk, int dtype,
                                  int sf_layout) {
    if (int r = check_dtype(dtype, what)) return r;
    if (!x || !weight || !packed || !scales) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (addend && !sum_out) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (int r = check_scale_layout(what, rows, cols, blk_mn, &chunk, sf_layout)) return r;   // folds the tile order into chunk
    if (!aligned(x, 16) || !aligned(weight, 16) || !aligned(packed, 8) || (addend && (!aligned(addend, 16) || !aligned(sum_out, 16)))) {
        return fail(CLEF_ERR_INVALID, "%s: activations and weight must be 16-byte aligned, packed 8-byte aligned", what);
    }
    int rows_total = 0;
    if (int r = clef_nvfp4_sizes(rows, cols, blk_mn, &rows_total, nullptr, nullptr)) return r;
    if (rows_total == 0) return CLEF_OK;
    DeviceInfo dev;
    if (int r = device_info(dev)) return r;
    cudaStream_t s = as_stream(stream);
    if (dtype == CLEF_BF16 && use_hot() && hot_scale_ok(global_scale) && (cols == 2048 || cols == 4096) && aligned(x, 32) &&
        (!addend || (aligned(addend, 32) && aligned(sum_out, 32)))) {
        const size_t groups = ((size_t)rows_total + 7) / 8;
        const size_t smem = (size_t)cols * sizeof(float);
        const FastDiv atom_div = make_fast_div((uint32_t)blk_mn);
#define CLEF_RMSQ_HOT(NB, ADD)                                                                                     \
    {                                                                                                              \
        static std::atomic<int> occ{0};                                                                            \
        const int per_sm = ctas_per_sm(rms_norm_quant_hot_kernel<NB, ADD>, smem, occ);                             \
        launch_hot(rms_norm_quant_hot_kernel<NB, ADD>, clamp_grid(groups, (size_t)dev.sms * per_sm), smem, s,      \
                   (const uint16_t*)x, (const uint16_t*)addend, (uint16_t*)sum_out, weight, packed, scales, rows,  \
                   rows_total, eps, global_scale, blk_mn, chunk, atom_div, (const int*)nullptr);                   \
    }
        if (cols == 2048) {
            if (addend) CLEF_RMSQ_HOT(4, true) else CLEF_RMSQ_HOT(4, false)
        } else {
            if (addend) CLEF_RMSQ_HOT(8, true) else CLEF_RMSQ_HOT(8, false)
        }
#undef CLEF_RMSQ_HOT
        return check_launch(what);
    }
    if (dtype == CLEF_F32 && use_hot() && hot_scale_ok(global_scale) && (cols == 2048 || cols == 4096) && aligned(x, 32) &&
        (!addend || (aligned(addend, 32) && aligned(sum_out, 32)))) {
        // f32 activations (the reference engine's residual stream): the tuned kernel's f32 form
        const size_t groups = ((size_t)rows_total + 7) / 8;
        const size_t smem = (size_t)cols * sizeof(float);
        const FastDiv atom_div = make_fast_div((uint32_t)blk_mn);
        auto launch = [&](auto kernel, std::atomic<int>& occ) {
            const int per_sm = ctas_per_sm(kernel, smem, occ);
            launch_hot(kernel, clamp_grid(groups, (size_t)dev.sms * per_sm), smem, s, (const float*)x, (const float*)addend,
                       (float*)sum_out, weight, packed, scales, rows, rows_total, eps, global_scale, blk_mn, chunk, atom_div,
                       (const int*)nullptr);
        };
        static std::atomic<int> occ[4];
        if (cols == 2048) {
            if (addend) launch(rms_norm_quant_f32_hot_kernel<4, true>, occ[0]);
            else launch(rms_norm_quant_f32_hot_kernel<4>, occ[1]);
        } else {
            if (addend) launch(rms_norm_quant_f32_hot_kernel<8, true>, occ[2]);
            else launch(rms_norm_quant_f32_hot_kernel<8>, occ[3]);
        }
        return check_launch(what);
    }
    if (addend) {   // shape-general path: the add, then the norm + quantiser on the stored sum
        if (int r = clef_add(stream, sum_out, x, addend, (size_t)rows * cols, dtype)) return r;
        x = sum_out;
    }
    if (dtype == CLEF_BF16) {
        launch_rms_norm_generic<Bf16, true>(s, dev, x, weight, nullptr, packed, scales, rows, rows_total, cols, eps,
                                            global_scale, blk_mn, chunk);
    } else {
        launch_rms_norm_generic<F32, true>(s, dev, x, weight, nullptr, packed, scales, rows, rows_total, cols, eps,
                                           global_scale, blk_mn, chunk);
    }
    return check_launch(what);
}

extern "C" {

int clef_rms_norm_quantise_nvfp4(clef_stream_t stream, const void* x, const float* weight, uint8_t* packed,
                                 uint8_t* scales, int rows, int cols, float eps, float global_scale, int blk_mn,
                                 int chunk, int dtype) {
    return rms_norm_quantise_impl("clef_rms_norm_quantise_nvfp4", stream, x, nullptr, nullptr, weight, packed, scales,
                                  rows, cols, eps, global_scale, blk_mn, chunk, dtype, CLEF_SF_DEFAULT);
}

int clef_rms_norm_quantise_nvfp4_ex(clef_stream_t stream, const void* x, const float* weight, uint8_t* packed,
                                    uint8_t* scales, int rows, int cols, float eps, float global_scale, int blk_mn,
                                    int chunk, int dtype, int sf_layout) {
    return rms_norm_quantise_impl("clef_rms_norm_quantise_nvfp4_ex", stream, x, nullptr, nullptr, weight, packed, scales,
                                  rows, cols, eps, global_scale, blk_mn, chunk, dtype, sf_layout);
}

int clef_add_rms_norm_quantise_nvfp4(clef_stream_t stream, void* sum_out, const void* a, const void* b,
                                     const float* weight, uint8_t* packed, uint8_t* scales, int rows, int cols,
                                     float eps, float global_scale, int blk_mn, int chunk, int dtype) {
    if (!b || !sum_out) return fail(CLEF_ERR_INVALID, "clef_add_rms_norm_quantise_nvfp4: null pointer");
    return rms_norm_quantise_impl("clef_add_rms_norm_quantise_nvfp4", stream, a, b, sum_out, weight, packed, scales,
                                  rows, cols, eps, global_scale, blk_mn, chunk, dtype, CLEF_SF_DEFAULT);
}

int clef_add_rms_norm_quantise_nvfp4_ex(clef_stream_t stream, void* sum_out, const void* a, const void* b,
                                        const float* weight, uint8_t* packed, uint8_t* scales, int rows, int cols,
                                        float eps, float global_scale, int blk_mn, int chunk, int dtype, int sf_layout) {
    if (!b || !sum_out) return fail(CLEF_ERR_INVALID, "clef_add_rms_norm_quantise_nvfp4_ex: null pointer");
    return rms_norm_quantise_impl("clef_add_rms_norm_quantise_nvfp4_ex", stream, a, b, sum_out, weight, packed, scales,
                                  rows, cols, eps, global_scale, blk_mn, chunk, dtype, sf_layout);
}

// Embedding gather + RMSNorm + NVFP4 in one pass over the gathered row (hidden 2048 or 4096); other shapes run the
// two entry points it stands for.
static int embed_rms_norm_quantise_impl(const char* what, clef_stream_t stream, const void* table, const int32_t* ids,
                                        void* h_out, const float* weight, uint8_t* packed, uint8_t* scales, int tokens,
                                        int hidden, float eps, float global_scale, int blk_mn, int chunk, int dtype,
                                        int sf_layout) {
    if (int r = check_dtype(dtype, what)) return r;
    if (!table || !ids || !h_out || !weight || !packed || !scales) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (tokens < 0 || hidden <= 0) return fail(CLEF_ERR_INVALID, "%s: tokens %d hidden %d", what, tokens, hidden);
    int folded = chunk;
    if (int r = check_scale_layout(what, tokens, hidden, blk_mn, &folded, sf_layout)) return r;
    int rows_total = 0;
    if (int r = clef_nvfp4_sizes(tokens, hidden, blk_mn, &rows_total, nullptr, nullptr)) return r;
    if (rows_total == 0) return CLEF_OK;
    DeviceInfo dev;
    if (int r = device_info(dev)) return r;
    if (dtype == CLEF_BF16 && use_hot() && hot_scale_ok(global_scale) && (hidden == 2048 || hidden == 4096) && aligned(table, 32) &&
        aligned(h_out, 32) && aligned(weight, 16) && aligned(packed, 8)) {
        const size_t groups = ((size_t)rows_total + 7) / 8;
        const size_t smem = (size_t)hidden * sizeof(float);
        const FastDiv atom_div = make_fast_div((uint32_t)blk_mn);
        auto launch = [&](auto kernel, std::atomic<int>& occ) {
            const int per_sm = ctas_per_sm(kernel, smem, occ);
            launch_hot(kernel, clamp_grid(groups, (size_t)dev.sms * per_sm), smem, as_stream(stream), (const uint16_t*)table,
                       (const uint16_t*)nullptr, (uint16_t*)h_out, weight, packed, scales, tokens, rows_total, eps, global_scale,
                       blk_mn, folded, atom_div, (const int*)ids);
        };
        static std::atomic<int> occ[2];
        if (hidden == 2048) launch(rms_norm_quant_hot_kernel<4, false, true>, occ[0]);
        else launch(rms_norm_quant_hot_kernel<8, false, true>, occ[1]);
        return check_launch(what);
    }
    if (dtype == CLEF_F32 && use_hot() && hot_scale_ok(global_scale) && (hidden == 2048 || hidden == 4096) && aligned(table, 32) &&
        aligned(h_out, 32) && aligned(weight, 16) && aligned(packed, 8)) {
        const size_t groups = ((size_t)rows_total + 7) / 8;
        const size_t smem = (size_t)hidden * sizeof(float);
        const FastDiv atom_div = make_fast_div((uint32_t)blk_mn);
        auto launch = [&](auto kernel, std::atomic<int>& occ) {
            const int per_sm = ctas_per_sm(kernel, smem, occ);
            launch_hot(kernel, clamp_grid(groups, (size_t)dev.sms * per_sm), smem, as_stream(stream), (const float*)table,
                       (const float*)nullptr, (float*)h_out, weight, packed, scales, tokens, rows_total, eps, global_scale, blk_mn,
                       folded, atom_div, (const int*)ids);
        };
        static std::atomic<int> occ[2];
        if (hidden == 2048) launch(rms_norm_quant_f32_hot_kernel<4, false, true>, occ[0]);
        else launch(rms_norm_quant_f32_hot_kernel<8, false, true>, occ[1]);
        return check_launch(what);
    }
    if (int r = clef_embed_gather(stream, table, ids, h_out, tokens, hidden, dtype)) return r;
    return rms_norm_quantise_impl(what, stream, h_out, nullptr, nullptr, weight, packed, scales, tokens, hidden, eps, global_scale,
                                  blk_mn, chunk, dtype, sf_layout);
}

int clef_embed_rms_norm_quantise_nvfp4(clef_stream_t stream, const void* table, const int32_t* ids, void* h_out,
                                       const float* weight, uint8_t* packed, uint8_t* scales, int tokens, int hidden,
                                       float eps, float global_scale, int blk_mn, int chunk, int dtype) {
    return embed_rms_norm_quantise_impl("clef_embed_rms_norm_quantise_nvfp4", stream, table, ids, h_out, weight, packed, scales,
                                        tokens, hidden, eps, global_scale, blk_mn, chunk, dtype, CLEF_SF_DEFAULT);
}

int clef_embed_rms_norm_quantise_nvfp4_ex(clef_stream_t stream, const void* table, const int32_t* ids, void* h_out,
                                          const float* weight, uint8_t* packed, uint8_t* scales, int tokens, int hidden,
                                          float eps, float global_scale, int blk_mn, int chunk, int dtype, int sf_layout) {
    return embed_rms_norm_quantise_impl("clef_embed_rms_norm_quantise_nvfp4_ex", stream, table, ids, h_out, weight, packed,
                                        scales, tokens, hidden, eps, global_scale, blk_mn, chunk, dtype, sf_layout);
}

// ---- gated rms_norm family -------------------------------------------------------------------------

}  // extern "C"

template <typename T, bool QUANT>
static void launch_gated_generic(cudaStream_t stream, const DeviceInfo& dev, const void* x, const void* gate,
                                 const float* weight, void* out, uint8_t* packed, uint8_t* scales, int rows_live,
                                 int rows_total, int cols, float eps, float global_scale, int blk_mn, int chunk,
                                 int vh) {
    static std::atomic<int> occ{0};
    auto kernel = rms_norm_gated_generic_kernel<T, QUANT>;
    const int per_sm = ctas_per_sm(kernel, 0, occ);
    const int rpb = kCtaThreads / ref_threads_per_row(cols);
    const size_t groups = ((size_t)rows_total + rpb - 1) / rpb;
    kernel<<<clamp_grid(groups, (size_t)dev.sms * per_sm), kCtaThreads, 0, stream>>>(
        (const Storage<T>*)x, (const Storage<T>*)gate, weight, (Storage<T>*)out, packed, scales, rows_live,
        rows_total, cols, eps, global_scale, blk_mn, chunk, vh);
}

extern "C" {

int clef_rms_norm_gated(clef_stream_t stream, const void* x, const void* gate, const float* weight, void* out,
                        int rows, int cols, float eps, int dtype) {
    const char* what = "clef_rms_norm_gated";
    if (int r = check_dtype(dtype, what)) return r;
    if (!x || !out) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (rows < 0 || cols <= 0 || cols % 4 != 0) {
        return fail(CLEF_ERR_INVALID, "%s: rows %d, cols %d (cols must be a positive multiple of 4)", what, rows, cols);
    }
    if (!aligned(x, 16) || !aligned(out, 16) || (gate && !aligned(gate, 16)) || (weight && !aligned(weight, 16))) {
        return fail(CLEF_ERR_INVALID, "%s: pointers must be 16-byte aligned", what);
    }
    if (rows == 0) return CLEF_OK;
    DeviceInfo dev;
    if (int r = device_info(dev)) return r;
    if (dtype == CLEF_BF16 && use_hot() && cols == 128 && gate && weight && aligned(x, 32) && aligned(gate, 32) &&
        aligned(out, 32)) {
        static std::atomic<int> occ{0};
        const int per_sm = ctas_per_sm(gated_norm_hot_kernel, 0, occ);
        const size_t groups = ((size_t)rows + 63) / 64;
        launch_hot(gated_norm_hot_kernel, clamp_grid(groups, (size_t)dev.sms * per_sm), 0, as_stream(stream),
                   (const uint16_t*)x, (const uint16_t*)gate, weight, (uint16_t*)out, rows, eps);
        return check_launch(what);
    }
    if (dtype == CLEF_F32 && use_hot() && cols == 128 && gate && weight && aligned(x, 32) && aligned(gate, 32) &&
        aligned(out, 32)) {
        static std::atomic<int> occ{0};
        const int per_sm = ctas_per_sm(gated_norm_f32_hot_kernel, 0, occ);
        const size_t groups = ((size_t)rows + 63) / 64;
        launch_hot(gated_norm_f32_hot_kernel, clamp_grid(groups, (size_t)dev.sms * per_sm), 0, as_stream(stream),
                   (const float*)x, (const float*)gate, weight, (float*)out, rows, eps);
        return check_launch(what);
    }
    if (dtype == CLEF_BF16) {
        launch_gated_generic<Bf16, false>(as_stream(stream), dev, x, gate, weight, out, nullptr, nullptr, rows, rows,
                                          cols, eps, 0.0f, 1, 4, 1);
    } else {
        launch_gated_generic<F32, false>(as_stream(stream), dev, x, gate, weight, out, nullptr, nullptr, rows, rows,
                                         cols, eps, 0.0f, 1, 4, 1);
    }
    return check_launch(what);
}

static int clef_rms_norm_gated_quantise_nvfp4_impl(clef_stream_t stream, const void* x, const void* gate, const float* weight,
                                       uint8_t* packed, uint8_t* scales, int rows, int cols, float eps,
                                       float global_scale, int blk_mn, int chunk, int vh, int rows_live, int dtype, int sf_layout) {
    const char* what = "clef_rms_norm_gated_quantise_nvfp4";
    if (int r = check_dtype(dtype, what)) return r;
    if (!x || !gate || !weight || !packed || !scales) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (vh <= 0 || cols <= 0 || cols % 16 != 0) {
        return fail(CLEF_ERR_INVALID, "%s: vh %d, cols %d (cols must be a multiple of 16)", what, vh, cols);
    }
    if ((long long)vh * cols > 0x7fffffffLL) return fail(CLEF_ERR_TOO_LARGE, "%s: vh*cols overflows", what);
    if (rows < 0 || rows % vh != 0 || rows_live < 0 || rows_live > rows) {
        return fail(CLEF_ERR_INVALID, "%s: rows %d must be a multiple of vh %d and rows_live %d <= rows", what, rows, vh,
                    rows_live);
    }
    if (int r = check_scale_layout(what, rows / vh, vh * cols, blk_mn, &chunk, sf_layout)) return r;   // folds the tile order into chunk
    if ((rows / vh) % blk_mn != 0) {
        return fail(CLEF_ERR_INVALID, "%s: rows/vh = %d tokens is not a multiple of blk_mn %d (rows counts padding)", what,
                    rows / vh, blk_mn);
    }
    if (!aligned(x, 16) || !aligned(gate, 16) || !aligned(weight, 16) || !aligned(packed, 8)) {
        return fail(CLEF_ERR_INVALID, "%s: x, gate and weight must be 16-byte aligned, packed 8-byte aligned", what);
    }
    if (rows == 0) return CLEF_OK;
    DeviceInfo dev;
    if (int r = device_info(dev)) return r;
    cudaStream_t s = as_stream(stream);
    if (dtype == CLEF_BF16 && use_hot() && hot_scale_ok(global_scale) && cols == 128 && aligned(x, 32) && aligned(gate, 32)) {
        static std::atomic<int> occ{0};
        const int per_sm = ctas_per_sm(gated_norm_quant_hot_kernel, 0, occ);
        const size_t groups = ((size_t)rows + 63) / 64;   // 64 head rows per CTA step
        launch_hot(gated_norm_quant_hot_kernel, clamp_grid(groups, (size_t)dev.sms * per_sm), 0, s, (const uint16_t*)x,
                   (const uint16_t*)gate, weight, packed, scales, rows_live, rows, eps, global_scale, blk_mn, chunk, vh,
                   make_fast_div((uint32_t)vh), make_fast_div((uint32_t)blk_mn));
        return check_launch(what);
    }
    if (dtype == CLEF_F32 && use_hot() && hot_scale_ok(global_scale) && cols == 128 && aligned(x, 32) && aligned(gate, 32)) {
        static std::atomic<int> occ{0};
        const int per_sm = ctas_per_sm(gated_norm_quant_f32_hot_kernel, 0, occ);
        const size_t groups = ((size_t)rows + 63) / 64;   // 64 head rows per CTA step
        launch_hot(gated_norm_quant_f32_hot_kernel, clamp_grid(groups, (size_t)dev.sms * per_sm), 0, s, (const float*)x,
                   (const float*)gate, weight, packed, scales, rows_live, rows, eps, global_scale, blk_mn, chunk, vh,
                   make_fast_div((uint32_t)vh), make_fast_div((uint32_t)blk_mn));
        return check_launch(what);
    }
    if (dtype == CLEF_BF16) {
        launch_gated_generic<Bf16, true>(s, dev, x, gate, weight, nullptr, packed, scales, rows_live, rows, cols, eps,
                                         global_scale, blk_mn, chunk, vh);
    } else {
        launch_gated_generic<F32, true>(s, dev, x, gate, weight, nullptr, packed, scales, rows_live, rows, cols, eps,
                                        global_scale, blk_mn, chunk, vh);
    }
    return check_launch(what);
}

int clef_rms_norm_gated_quantise_nvfp4(clef_stream_t stream, const void* x, const void* gate, const float* weight,
                                       uint8_t* packed, uint8_t* scales, int rows, int cols, float eps,
                                       float global_scale, int blk_mn, int chunk, int vh, int rows_live, int dtype) {
    return clef_rms_norm_gated_quantise_nvfp4_impl(stream, x, gate, weight, packed, scales, rows, cols, eps, global_scale, blk_mn, chunk, vh, rows_live, dtype, CLEF_SF_DEFAULT);
}

int clef_rms_norm_gated_quantise_nvfp4_ex(clef_stream_t stream, const void* x, const void* gate, const float* weight,
                                       uint8_t* packed, uint8_t* scales, int rows, int cols, float eps,
                                       float global_scale, int blk_mn, int chunk, int vh, int rows_live, int dtype, int sf_layout) {
    return clef_rms_norm_gated_quantise_nvfp4_impl(stream, x, gate, weight, packed, scales, rows, cols, eps, global_scale, blk_mn, chunk, vh, rows_live, dtype, sf_layout);
}

// ---- swiglu / quantise -------------------------------------------------------------------------------

int clef_swiglu(clef_stream_t stream, const void* gate, const void* up, void* out, size_t total, int dtype) {
    const char* what = "clef_swiglu";
    if (int r = check_dtype(dtype, what)) return r;
    if (!gate || !up || !out) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (!aligned(gate, 16) || !aligned(up, 16) || !aligned(out, 16)) {
        return fail(CLEF_ERR_INVALID, "%s: pointers must be 16-byte aligned", what);
    }
    if (total == 0) return CLEF_OK;
    DeviceInfo dev;
    if (int r = device_info(dev)) return r;
    if (dtype == CLEF_BF16 && use_hot() && total >= 16 && total / 16 < 0xffffffffull && aligned(gate, 32) &&
        aligned(up, 32) && aligned(out, 32)) {
        static std::atomic<int> occ{0};
        const int per_sm = ctas_per_sm(swiglu_hot_kernel<kActSwiGLU>, 0, occ);
        const size_t blocks = total / 16;
        launch_hot(swiglu_hot_kernel<kActSwiGLU>, clamp_grid((blocks + kCtaThreads - 1) / kCtaThreads, (size_t)dev.sms * per_sm), 0,
                   as_stream(stream), (const uint16_t*)gate, (const uint16_t*)up, (uint16_t*)out, (uint32_t)blocks);
        if (int r = check_launch(what)) return r;
        const size_t done = blocks * 16;
        if (done == total) return CLEF_OK;
        gate = (const uint16_t*)gate + done;   // the last total % 16 values go through the shape-general kernel
        up = (const uint16_t*)up + done;
        out = (uint16_t*)out + done;
        total -= done;
    }
    const size_t quads = (total + 3) / 4;
    if (dtype == CLEF_BF16) {
        static std::atomic<int> occ{0};
        const int per_sm = ctas_per_sm(swiglu_generic_kernel<Bf16>, 0, occ);
        swiglu_generic_kernel<Bf16><<<clamp_grid((quads + kCtaThreads - 1) / kCtaThreads, (size_t)dev.sms * per_sm),
                                      kCtaThreads, 0, as_stream(stream)>>>((const uint16_t*)gate, (const uint16_t*)up,
                                                                           (uint16_t*)out, total);
    } else {
        static std::atomic<int> occ{0};
        const int per_sm = ctas_per_sm(swiglu_generic_kernel<F32>, 0, occ);
        swiglu_generic_kernel<F32><<<clamp_grid((quads + kCtaThreads - 1) / kCtaThreads, (size_t)dev.sms * per_sm),
                                     kCtaThreads, 0, as_stream(stream)>>>((const float*)gate, (const float*)up,
                                                                          (float*)out, total);
    }
    return check_launch(what);
}

static int clef_quantise_nvfp4_impl(clef_stream_t stream, const void* x, uint8_t* packed, uint8_t* scales, int rows, int cols,
                        float global_scale, int blk_mn, int chunk, int dtype, int sf_layout) {
    const char* what = "clef_quantise_nvfp4";
    if (int r = check_dtype(dtype, what)) return r;
    if (!x || !packed || !scales) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (int r = check_scale_layout(what, rows, cols, blk_mn, &chunk, sf_layout)) return r;   // folds the tile order into chunk
    if (!aligned(x, 16) || !aligned(packed, 8)) {
        return fail(CLEF_ERR_INVALID, "%s: x must be 16-byte aligned, packed 8-byte aligned", what);
    }
    int rows_total = 0;
    if (int r = clef_nvfp4_sizes(rows, cols, blk_mn, &rows_total, nullptr, nullptr)) return r;
    if (rows_total == 0) return CLEF_OK;
    DeviceInfo dev;
    if (int r = device_info(dev)) return r;
    if (dtype == CLEF_BF16 && use_hot() && hot_scale_ok(global_scale) && cols % 512 == 0 && (size_t)rows_total * (cols / 512) < 0x7fffffffull &&
        aligned(x, 32)) {
        constexpr int kUnits = 1;   // one unit in flight per warp (plus its prefetched successor): 9.2 us against 9.6 with two at 8,192 x 2048
        static std::atomic<int> occ{0};
        const int per_sm = ctas_per_sm(quantise_hot_kernel<kUnits>, 0, occ);
        const uint32_t segs = (uint32_t)(cols / 512);
        const uint32_t live_units = (uint32_t)rows * segs, total_units = (uint32_t)rows_total * segs;
        const size_t ctas = ((size_t)total_units + kUnits * 8 - 1) / (kUnits * 8);
        launch_hot(quantise_hot_kernel<kUnits>, clamp_grid(ctas, (size_t)dev.sms * per_sm), 0, as_stream(stream),
                   (const uint16_t*)x, packed, scales, live_units, total_units, cols, global_scale, blk_mn, chunk,
                   make_fast_div(segs), make_fast_div((uint32_t)blk_mn));
        return check_launch(what);
    }
    if (dtype == CLEF_F32 && use_hot() && hot_scale_ok(global_scale) && cols % 512 == 0 && (size_t)rows_total * (cols / 512) < 0x7fffffffull &&
        aligned(x, 32)) {
        launch_unit_quant_f32<0>(as_stream(stream), dev, (const float*)x, nullptr, packed, scales, rows, rows_total, cols,
                                 global_scale, blk_mn, chunk);
        return check_launch(what);
    }
    if (dtype == CLEF_BF16) {
        launch_quantise_generic<Bf16, kActNone>(as_stream(stream), dev, x, nullptr, packed, scales, rows, rows_total, cols,
                                             global_scale, blk_mn, chunk);
    } else {
        launch_quantise_generic<F32, kActNone>(as_stream(stream), dev, x, nullptr, packed, scales, rows, rows_total, cols,
                                            global_scale, blk_mn, chunk);
    }
    return check_launch(what);
}

int clef_quantise_nvfp4(clef_stream_t stream, const void* x, uint8_t* packed, uint8_t* scales, int rows, int cols,
                        float global_scale, int blk_mn, int chunk, int dtype) {
    return clef_quantise_nvfp4_impl(stream, x, packed, scales, rows, cols, global_scale, blk_mn, chunk, dtype, CLEF_SF_DEFAULT);
}

int clef_quantise_nvfp4_ex(clef_stream_t stream, const void* x, uint8_t* packed, uint8_t* scales, int rows, int cols,
                        float global_scale, int blk_mn, int chunk, int dtype, int sf_layout) {
    return clef_quantise_nvfp4_impl(stream, x, packed, scales, rows, cols, global_scale, blk_mn, chunk, dtype, sf_layout);
}

static int clef_swiglu_quantise_nvfp4_impl(clef_stream_t stream, const void* gate, const void* up, uint8_t* packed,
                               uint8_t* scales, int rows, int cols, float global_scale, int blk_mn, int chunk,
                               int dtype, int sf_layout) {
    const char* what = "clef_swiglu_quantise_nvfp4";
    if (int r = check_dtype(dtype, what)) return r;
    if (!gate || !up || !packed || !scales) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (int r = check_scale_layout(what, rows, cols, blk_mn, &chunk, sf_layout)) return r;   // folds the tile order into chunk
    if (!aligned(gate, 16) || !aligned(up, 16) || !aligned(packed, 8)) {
        return fail(CLEF_ERR_INVALID, "%s: gate and up must be 16-byte aligned, packed 8-byte aligned", what);
    }
    int rows_total = 0;
    if (int r = clef_nvfp4_sizes(rows, cols, blk_mn, &rows_total, nullptr, nullptr)) return r;
    if (rows_total == 0) return CLEF_OK;
    DeviceInfo dev;
    if (int r = device_info(dev)) return r;
    cudaStream_t s = as_stream(stream);
    const size_t total_blocks = (size_t)rows_total * (cols / 16);
    if (dtype == CLEF_BF16 && use_hot() && hot_scale_ok(global_scale) && cols % 512 == 0 && total_blocks / 32 < 0x7fffffffull && aligned(gate, 32) &&
        aligned(up, 32)) {
        const uint32_t segs = (uint32_t)(cols / 512);
        const uint32_t live_units = (uint32_t)rows * segs, total_units = (uint32_t)rows_total * segs;
        // One unit in flight per warp (plus its prefetched successor) at three CTAs per SM measured best on B200
        // among 1-3 units x 2-5 CTAs (38.9 us against 40.7 to 45.3 us at 8,192 x 6144).
        constexpr int kUnits = 1, kMinCtas = 3;
        static std::atomic<int> occ{0};
        const int per_sm = ctas_per_sm(swiglu_quant_hot_kernel<kUnits, kMinCtas, kActSwiGLU>, 0, occ);
        const size_t ctas = ((size_t)total_units + kUnits * 8 - 1) / (kUnits * 8);
        launch_hot(swiglu_quant_hot_kernel<kUnits, kMinCtas, kActSwiGLU>, clamp_grid(ctas, (size_t)dev.sms * per_sm), 0, s,
                   (const uint16_t*)gate, (const uint16_t*)up, packed, scales, live_units, total_units, cols,
                   global_scale, blk_mn, chunk, make_fast_div(segs), make_fast_div((uint32_t)blk_mn));
        return check_launch(what);
    }
    if (dtype == CLEF_F32 && use_hot() && hot_scale_ok(global_scale) && cols % 512 == 0 && total_blocks / 32 < 0x7fffffffull && aligned(gate, 32) &&
        aligned(up, 32)) {
        launch_unit_quant_f32<1>(s, dev, (const float*)gate, (const float*)up, packed, scales, rows, rows_total, cols,
                                 global_scale, blk_mn, chunk);
        return check_launch(what);
    }
    if (dtype == CLEF_BF16) {
        launch_quantise_generic<Bf16, kActSwiGLU>(s, dev, gate, up, packed, scales, rows, rows_total, cols, global_scale,
                                            blk_mn, chunk);
    } else {
        launch_quantise_generic<F32, kActSwiGLU>(s, dev, gate, up, packed, scales, rows, rows_total, cols, global_scale,
                                           blk_mn, chunk);
    }
    return check_launch(what);
}

int clef_swiglu_quantise_nvfp4(clef_stream_t stream, const void* gate, const void* up, uint8_t* packed,
                               uint8_t* scales, int rows, int cols, float global_scale, int blk_mn, int chunk,
                               int dtype) {
    return clef_swiglu_quantise_nvfp4_impl(stream, gate, up, packed, scales, rows, cols, global_scale, blk_mn, chunk, dtype, CLEF_SF_DEFAULT);
}

int clef_swiglu_quantise_nvfp4_ex(clef_stream_t stream, const void* gate, const void* up, uint8_t* packed,
                               uint8_t* scales, int rows, int cols, float global_scale, int blk_mn, int chunk,
                               int dtype, int sf_layout) {
    return clef_swiglu_quantise_nvfp4_impl(stream, gate, up, packed, scales, rows, cols, global_scale, blk_mn, chunk, dtype, sf_layout);
}

// ---- rope ----------------------------------------------------------------------------------------------

static int check_rope_shape(const char* what, int rows, int heads, int head_dim, int rotary_dim) {
    if (rows < 0 || heads <= 0 || head_dim <= 0 || rotary_dim < 0) {
        return fail(CLEF_ERR_INVALID, "%s: rows %d heads %d head_dim %d rotary_dim %d", what, rows, heads, head_dim,
                    rotary_dim);
    }
    if (head_dim % 4 != 0 || rotary_dim % 8 != 0 || rotary_dim > head_dim) {
        return fail(CLEF_ERR_INVALID,
                    "%s: head_dim %d must be a multiple of 4 and rotary_dim %d a multiple of 8 not above it", what,
                    head_dim, rotary_dim);
    }
    return CLEF_OK;
}

int clef_rope(clef_stream_t stream, void* out, const void* x, const float* cos_table, const float* sin_table,
              int rows, int heads, int head_dim, int rotary_dim, const int32_t* seq_start, const int32_t* pos_base,
              const int32_t* pos_map, int dtype) {
    const char* what = "clef_rope";
    if (int r = check_dtype(dtype, what)) return r;
    if (!out || !x || !cos_table || !sin_table) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (int r = check_rope_shape(what, rows, heads, head_dim, rotary_dim)) return r;
    if (out == x) return fail(CLEF_ERR_INVALID, "%s: out must not alias x", what);
    if (!aligned(x, 16) || !aligned(out, 16) || !aligned(cos_table, 16) || !aligned(sin_table, 16)) {
        return fail(CLEF_ERR_INVALID, "%s: pointers must be 16-byte aligned", what);
    }
    if (rows == 0) return CLEF_OK;
    DeviceInfo dev;
    if (int r = device_info(dev)) return r;
    cudaStream_t s = as_stream(stream);
    const size_t hot_items = (size_t)rows * heads * (head_dim / 32);
    if (dtype == CLEF_BF16 && use_hot() && head_dim % 32 == 0 && rotary_dim % 32 == 0 && hot_items < 0x7fffffffull &&
        aligned(x, 32) && aligned(out, 32)) {
        static std::atomic<int> occ{0};
        const int per_sm = ctas_per_sm(rope_hot_kernel<false, false>, 0, occ);
        const size_t ctas = (hot_items + kCtaThreads - 1) / kCtaThreads, cap = (size_t)dev.sms * per_sm;
        auto kernel = rope_launch_is_short(ctas, cap) ? rope_hot_kernel<false, true> : rope_hot_kernel<false, false>;
        launch_hot(kernel, balanced_grid(ctas, cap), 0, s, (uint16_t*)out, (const uint16_t*)x, cos_table, sin_table,
                   (uint32_t)hot_items, heads, head_dim, rotary_dim, (const int*)seq_start, (const int*)pos_base,
                   (const int*)pos_map, make_fast_div((uint32_t)(head_dim / 32)), make_fast_div((uint32_t)heads), KvCacheDest{});
        return check_launch(what);
    }
    const size_t f32_items = (size_t)rows * heads * (head_dim / 16);
    if (dtype == CLEF_F32 && use_hot() && head_dim % 16 == 0 && rotary_dim % 16 == 0 && f32_items < 0x7fffffffull &&
        aligned(x, 32) && aligned(out, 32)) {
        RopeSegmentsF32 segs{};
        segs.x[0] = (const float*)x;
        segs.out[0] = (float*)out;
        segs.end_item[0] = (uint32_t)f32_items;
        segs.heads_div[0] = make_fast_div((uint32_t)heads);
        static std::atomic<int> occ{0};
        const int per_sm = ctas_per_sm(rope_f32_hot_kernel<1>, 0, occ);
        launch_hot(rope_f32_hot_kernel<1>, clamp_grid((f32_items + kCtaThreads - 1) / kCtaThreads, (size_t)dev.sms * per_sm), 0, s,
                   segs, cos_table, sin_table, head_dim, rotary_dim, (const int*)seq_start, (const int*)pos_base,
                   (const int*)pos_map, make_fast_div((uint32_t)(head_dim / 16)));
        return check_launch(what);
    }
    const size_t items = (size_t)rows * heads * ((rotary_dim / 8) + (head_dim - rotary_dim) / 4);
    if (dtype == CLEF_BF16) {
        static std::atomic<int> occ{0};
        const int per_sm = ctas_per_sm(rope_generic_kernel<Bf16>, 0, occ);
        rope_generic_kernel<Bf16><<<clamp_grid((items + kCtaThreads - 1) / kCtaThreads, (size_t)dev.sms * per_sm),
                                    kCtaThreads, 0, s>>>((uint16_t*)out, (const uint16_t*)x, cos_table, sin_table, rows,
                                                         heads, head_dim, rotary_dim, seq_start, pos_base, pos_map);
    } else {
        static std::atomic<int> occ{0};
        const int per_sm = ctas_per_sm(rope_generic_kernel<F32>, 0, occ);
        rope_generic_kernel<F32><<<clamp_grid((items + kCtaThreads - 1) / kCtaThreads, (size_t)dev.sms * per_sm),
                                   kCtaThreads, 0, s>>>((float*)out, (const float*)x, cos_table, sin_table, rows, heads,
                                                        head_dim, rotary_dim, seq_start, pos_base, pos_map);
    }
    return check_launch(what);
}

int clef_qk_norm_rope(clef_stream_t stream, const void* x, const float* weight, const float* cos_table,
                      const float* sin_table, void* out, void* gate_out, int rows, int heads, int head_dim,
                      int rotary_dim, float eps, const int32_t* seq_start, const int32_t* pos_base,
                      const int32_t* pos_map, int dtype) {
    const char* what = "clef_qk_norm_rope";
    if (int r = check_dtype(dtype, what)) return r;
    if (!x || !weight || !cos_table || !sin_table || !out) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (int r = check_rope_shape(what, rows, heads, head_dim, rotary_dim)) return r;
    if (head_dim > 1024) return fail(CLEF_ERR_TOO_LARGE, "%s: head_dim %d above 1024", what, head_dim);
    if (!aligned(x, 16) || !aligned(out, 16) || !aligned(weight, 16) || (gate_out && !aligned(gate_out, 16))) {
        return fail(CLEF_ERR_INVALID, "%s: pointers must be 16-byte aligned", what);
    }
    if (rows == 0) return CLEF_OK;
    DeviceInfo dev;
    if (int r = device_info(dev)) return r;
    if (dtype == CLEF_BF16 && use_hot() && (head_dim == 128 || head_dim == 256) && rotary_dim == 64 && rows < 0x3fffffff &&
        aligned(x, 32) && aligned(out, 32) && (!gate_out || aligned(gate_out, 32))) {
        // head_dim 256 with a gate: the gate halves are copy items after the normed rows (from a multiple of 8)
        const size_t hot_items = (head_dim == 256 && gate_out) ? (((size_t)rows + 7) & ~(size_t)7) + rows : (size_t)rows;
        const size_t hot_groups = (hot_items + 63) / 64;
        const FastDiv heads_div = make_fast_div((uint32_t)heads);
        auto launch = [&](auto kernel, std::atomic<int>& occ) {
            const int per_sm = ctas_per_sm(kernel, 0, occ);
            launch_hot(kernel, balanced_grid(hot_groups, (size_t)dev.sms * per_sm), 0, as_stream(stream), (const uint16_t*)x,
                       weight, cos_table, sin_table, (uint16_t*)out, (uint16_t*)gate_out, (uint32_t)rows, eps,
                       (const int*)seq_start, (const int*)pos_base, (const int*)pos_map, heads_div, KvCacheDest{});
        };
        static std::atomic<int> occ[4];
        if (head_dim == 128) {
            if (gate_out) launch(qk_norm_rope_hot_kernel<true, false>, occ[0]);
            else launch(qk_norm_rope_hot_kernel<false, false>, occ[1]);
        } else {
            if (gate_out) launch(qk_norm_rope_hd256_hot_kernel<true, false>, occ[2]);
            else launch(qk_norm_rope_hd256_hot_kernel<false, false>, occ[3]);
        }
        return check_launch(what);
    }
    if (dtype == CLEF_F32 && use_hot() && (head_dim == 128 || head_dim == 256) && rotary_dim == 64 && rows < 0x3fffffff) {
        // f32 activations: one warp per head row, two rows in flight per warp
        const size_t hot_groups = ((size_t)rows + 15) / 16;
        const FastDiv heads_div = make_fast_div((uint32_t)heads);
        auto launch = [&](auto kernel, std::atomic<int>& occ) {
            const int per_sm = ctas_per_sm(kernel, 0, occ);
            launch_hot(kernel, clamp_grid(hot_groups, (size_t)dev.sms * per_sm), 0, as_stream(stream), (const float*)x, weight,
                       cos_table, sin_table, (float*)out, (float*)gate_out, (uint32_t)rows, eps, (const int*)seq_start,
                       (const int*)pos_base, (const int*)pos_map, heads_div);
        };
        static std::atomic<int> occ[4];
        if (head_dim == 128) {
            if (gate_out) launch(qk_norm_rope_f32_hot_kernel<128, true>, occ[0]);
            else launch(qk_norm_rope_f32_hot_kernel<128, false>, occ[1]);
        } else {
            if (gate_out) launch(qk_norm_rope_f32_hot_kernel<256, true>, occ[2]);
            else launch(qk_norm_rope_f32_hot_kernel<256, false>, occ[3]);
        }
        return check_launch(what);
    }
    const size_t smem = (size_t)8 * head_dim * sizeof(float);
    const size_t groups = ((size_t)rows + 7) / 8;
    if (dtype == CLEF_BF16) {
        static std::atomic<int> occ{0};
        const int per_sm = ctas_per_sm(qk_norm_rope_generic_kernel<Bf16, Bf16, false>, smem, occ);
        qk_norm_rope_generic_kernel<Bf16, Bf16, false><<<clamp_grid(groups, (size_t)dev.sms * per_sm), kCtaThreads, smem,
                                            as_stream(stream)>>>((const uint16_t*)x, weight, cos_table, sin_table,
                                                                 (uint16_t*)out, (uint16_t*)gate_out, rows, heads,
                                                                 head_dim, rotary_dim, eps, seq_start, pos_base, pos_map,
                                                                 nullptr, nullptr);
    } else {
        static std::atomic<int> occ{0};
        const int per_sm = ctas_per_sm(qk_norm_rope_generic_kernel<F32, F32, false>, smem, occ);
        qk_norm_rope_generic_kernel<F32, F32, false><<<clamp_grid(groups, (size_t)dev.sms * per_sm), kCtaThreads, smem,
                                           as_stream(stream)>>>((const float*)x, weight, cos_table, sin_table,
                                                                (float*)out, (float*)gate_out, rows, heads, head_dim,
                                                                rotary_dim, eps, seq_start, pos_base, pos_map, nullptr,
                                                                nullptr);
    }
    return check_launch(what);
}

int clef_rope_tables(clef_stream_t stream, const int32_t* positions, float* cos_out, float* sin_out, int rows,
                     int rotary_dim, float theta) {
    const char* what = "clef_rope_tables";
    if (!positions || !cos_out || !sin_out) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (rows < 0 || rotary_dim <= 0 || rotary_dim % 2 != 0) {
        return fail(CLEF_ERR_INVALID, "%s: rows %d rotary_dim %d", what, rows, rotary_dim);
    }
    if (rows == 0) return CLEF_OK;
    DeviceInfo dev;
    if (int r = device_info(dev)) return r;
    static std::atomic<int> occ{0};
    const int per_sm = ctas_per_sm(rope_tables_kernel, 0, occ);
    const size_t total = (size_t)rows * rotary_dim;
    rope_tables_kernel<<<clamp_grid((total + kCtaThreads - 1) / kCtaThreads, (size_t)dev.sms * per_sm), kCtaThreads, 0,
                         as_stream(stream)>>>(positions, cos_out, sin_out, rows, rotary_dim, theta);
    return check_launch(what);
}

}  // extern "C"
