// Helpers shared by the translation units that hold C-ABI entry points: device facts, occupancy
// cache, the programmatic-dependent-launch wrapper, argument checks. Header-only (inline), not installed.
#pragma once

#include <atomic>
#include <cstdint>
#include <cstdlib>

#include <cuda_runtime.h>

#include "../../include/clef_fused.h"
#include "internal.hpp"
#include "kernels_generic.cuh"

namespace clef {
namespace abi {

struct DeviceInfo {
    int sms = 0;
    int cc_major = 0;
};

// Per-device facts, looked up once per device (no allocation; attribute queries only).
inline int device_info(DeviceInfo& out) {
    static std::atomic<int> cached_sms[64];
    static std::atomic<int> cached_cc[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        return fail(CLEF_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    }
    if (dev < 0 || dev >= 64) {
        return fail(CLEF_ERR_CUDA, "device ordinal %d out of range", dev);
    }
    int sms = cached_sms[dev].load(std::memory_order_relaxed);
    int cc = cached_cc[dev].load(std::memory_order_relaxed);
    if (sms == 0) {
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (e == cudaSuccess) {
            e = cudaDeviceGetAttribute(&cc, cudaDevAttrComputeCapabilityMajor, dev);
        }
        if (e != cudaSuccess) {
            return fail(CLEF_ERR_CUDA, "cudaDeviceGetAttribute: %s", cudaGetErrorString(e));
        }
        cached_sms[dev].store(sms, std::memory_order_relaxed);
        cached_cc[dev].store(cc, std::memory_order_relaxed);
    }
    if (cc != 10) {
        return fail(CLEF_ERR_CUDA, "this library holds sm_100a code only; device %d is compute capability %d.x", dev,
                    cc);
    }
    out.sms = sms;
    out.cc_major = cc;
    return CLEF_OK;
}

// Resident CTAs per SM of a kernel (cached per kernel instantiation by the caller's static).
template <typename K>
int ctas_per_sm(K kernel, size_t dyn_smem, std::atomic<int>& cache) {
    int n = cache.load(std::memory_order_relaxed);
    if (n > 0) {
        return n;
    }
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, clef::kCtaThreads, dyn_smem) != cudaSuccess || n < 1) {
        (void)cudaGetLastError();
        n = 1;
    }
    cache.store(n, std::memory_order_relaxed);
    return n;
}

// Launch of a tuned kernel. With programmatic dependent launch (default; CLEF_PDL=0 turns it off) the
// kernel may begin its argument-only prologue while the stream's previous kernel drains; the kernels
// wait for that kernel before touching any activation or output (common.cuh, pdl_wait_prior_grids).
inline bool pdl_enabled() {
    static const int on = [] {
        const char* v = getenv("CLEF_PDL");
        return (v && v[0] == '0') ? 0 : 1;
    }();
    return on != 0;
}

template <typename... KArgs, typename... Args>
void launch_hot(void (*kernel)(KArgs...), unsigned grid, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(clef::kCtaThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    (void)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);   // errors surface in check_launch
}

// Whether a grid-stride launch of `ctas_wanted` CTA-sized pieces on `cap` resident CTAs is short enough (at most
// six rounds per thread) for the RoPE kernels' hoisted-load form; see rope_hot_kernel.
inline bool rope_launch_is_short(size_t ctas_wanted, size_t cap) { return ctas_wanted <= 6 * cap; }

inline unsigned clamp_grid(size_t wanted, size_t cap) {
    size_t g = wanted < cap ? wanted : cap;
    return (unsigned)(g < 1 ? 1 : g);
}

// A grid for `wanted` CTA-sized pieces on `cap` resident CTAs in which every CTA runs the same number of rounds:
// ceil(wanted / rounds) CTAs with rounds = ceil(wanted / cap), instead of `cap` CTAs whose last round is part empty.
// For kernels with many resident CTAs per SM (an SM then holds one CTA fewer at most).
inline unsigned balanced_grid(size_t wanted, size_t cap) {
    if (wanted <= cap || cap == 0) return clamp_grid(wanted, cap);
    const size_t rounds = (wanted + cap - 1) / cap;
    return (unsigned)((wanted + rounds - 1) / rounds);
}

inline int check_launch(const char* what) {
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        return fail(CLEF_ERR_CUDA, "%s: launch failed: %s", what, cudaGetErrorString(e));
    }
    return CLEF_OK;
}

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

inline int check_dtype(int dtype, const char* what) {
    if (dtype != CLEF_BF16 && dtype != CLEF_F32) {
        return fail(CLEF_ERR_INVALID, "%s: dtype %d is neither CLEF_BF16 nor CLEF_F32", what, dtype);
    }
    return CLEF_OK;
}

// Checks the shape and the scale-tile arguments of an NVFP4 entry point and folds the tile order into `chunk` the way
// the kernels take it (negated for the interleaved order; nvfp4_codec.cuh, SfLayout). `sf_layout` is the call's own
// choice or CLEF_SF_DEFAULT for the process default (clef_set_scale_layout).
inline int check_scale_layout(const char* what, int rows, int cols, int blk_mn, int* chunk, int sf_layout) {
    if (rows < 0 || cols <= 0) {
        return fail(CLEF_ERR_INVALID, "%s: rows %d / cols %d", what, rows, cols);
    }
    if (cols % 64 != 0) {
        return fail(CLEF_ERR_INVALID,
                    "%s: cols %d is not a multiple of 64 (four 16-value blocks fill one scale group)", what, cols);
    }
    if (blk_mn <= 0 || *chunk != blk_mn * 4) {
        return fail(CLEF_ERR_INVALID, "%s: scale atom blk_mn %d / chunk %d (chunk must be blk_mn * 4)", what, blk_mn,
                    *chunk);
    }
    if (sf_layout == CLEF_SF_DEFAULT) sf_layout = scale_layout();
    if (sf_layout != CLEF_SF_ACTIVATION && sf_layout != CLEF_SF_INTERLEAVED) {
        return fail(CLEF_ERR_INVALID, "%s: scale-tile order %d", what, sf_layout);
    }
    if (sf_layout == CLEF_SF_INTERLEAVED) {
        if (blk_mn % 32 != 0) {   // the order interleaves 32-row groups: row r sits at (r % 32) * (blk_mn / 32) + r / 32
            return fail(CLEF_ERR_INVALID, "%s: the interleaved scale-tile order needs blk_mn %% 32 == 0 (blk_mn %d)", what,
                        blk_mn);
        }
        *chunk = -*chunk;
    }
    return CLEF_OK;
}

inline bool use_hot() { return kernel_choice() != 1; }

// The tuned quantising kernels cover the global scales real checkpoints carry; see kHotGlobalScaleMin.
inline bool hot_scale_ok(float global_scale) {
    return global_scale >= kHotGlobalScaleMin && global_scale <= kHotGlobalScaleMax;
}

inline cudaStream_t as_stream(clef_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

template <typename T>
using Storage = typename T::storage;


// ACT: kActNone (a only), kActSwiGLU (a = gate, b = up), kActSigmoidMul (a = gate, b = the gated values).
template <typename T, int ACT>
inline void launch_quantise_generic(cudaStream_t stream, const DeviceInfo& dev, const void* a, const void* b,
                                    uint8_t* packed, uint8_t* scales, int rows, int rows_total, int cols,
                                    float global_scale, int blk_mn, int chunk) {
    static std::atomic<int> occ{0};
    auto kernel = quantise_generic_kernel<T, ACT>;
    const int per_sm = ctas_per_sm(kernel, 0, occ);
    const size_t blocks = (size_t)rows_total * (cols / 16);
    kernel<<<clamp_grid((blocks + kCtaThreads - 1) / kCtaThreads, (size_t)dev.sms * per_sm), kCtaThreads, 0, stream>>>(
        (const Storage<T>*)a, (const Storage<T>*)b, packed, scales, rows, rows_total, cols, global_scale, blk_mn, chunk);
}

}  // namespace abi
}  // namespace clef
