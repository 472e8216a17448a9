// Host-side companions of the fused kernels (declared in include/clef_host.h): the device handle,
// the host-slice launchers that stream row tiles through two CUDA streams, the per-token maps of a
// pass, the rung ladder and the multi-GPU row split. The kernels themselves are reached only through
// the C-ABI of clef_fused.h; there is no CPU implementation of any of them in this library.

#include "../../include/clef_host.h"

#include <algorithm>
#include <cstring>
#include <mutex>
#include <vector>

#include <cuda_runtime.h>

#include "internal.hpp"

using clef::fail;

namespace {

constexpr int kStreams = 2;

#define CLEF_CUDA(call)                                                                               \
    do {                                                                                              \
        const cudaError_t e__ = (call);                                                               \
        if (e__ != cudaSuccess) {                                                                     \
            return fail(CLEF_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e__));                     \
        }                                                                                             \
    } while (0)

inline size_t round_up(size_t v, size_t n) { return (v + n - 1) / n * n; }
inline size_t elem_bytes(int dtype) { return dtype == CLEF_BF16 ? 2 : 4; }

}  // namespace

// One staging slot per stream: a device arena that holds one row tile's inputs and outputs.
struct clef_device {
    int ordinal = 0;
    cudaStream_t streams[kStreams] = {nullptr, nullptr};
    cudaEvent_t slot_free[kStreams] = {nullptr, nullptr};
    cudaEvent_t fence[kStreams] = {nullptr, nullptr};   // orders the two streams at the start and the end of a call
    void* arena[kStreams] = {nullptr, nullptr};
    size_t arena_bytes[kStreams] = {0, 0};
    void* consts = nullptr;       // small operands (weights, tables): two halves, used by alternate calls
    size_t consts_bytes = 0;
    int consts_gen = 0;           // the half the current call uses
    cudaEvent_t gen_done[2][kStreams] = {{nullptr, nullptr}, {nullptr, nullptr}};   // last work that read a half
    bool pipelined = false;       // host-slice calls return once their work is enqueued (clef_device_set_pipelined)
    std::mutex lock;              // one host-slice call at a time per handle
};

namespace {

// Set the handle's device current for the duration of a call.
struct DeviceScope {
    int previous = -1;
    bool ok = false;
    explicit DeviceScope(const clef_device* dev) {
        if (cudaGetDevice(&previous) == cudaSuccess && cudaSetDevice(dev->ordinal) == cudaSuccess) {
            ok = true;
        }
    }
    ~DeviceScope() {
        if (previous >= 0) {
            cudaSetDevice(previous);
        }
    }
};

// Declares the scope and refuses the call when the handle's device cannot be made current (the launches and
// copies would otherwise go to whatever device the caller had selected, on this handle's streams).
#define CLEF_DEVICE_SCOPE(dev, what)                                                                   \
    DeviceScope scope(dev);                                                                            \
    if (!scope.ok) return fail(CLEF_ERR_CUDA, "%s: cannot select device %d", what, (dev)->ordinal)

int ensure_arena(clef_device* dev, int slot, size_t bytes) {
    if (dev->arena_bytes[slot] >= bytes) {
        return CLEF_OK;
    }
    // Growth happens on the first call of a shape only; steady-state calls allocate nothing.
    CLEF_CUDA(cudaStreamSynchronize(dev->streams[slot]));
    if (dev->arena[slot]) {
        CLEF_CUDA(cudaFree(dev->arena[slot]));
        dev->arena[slot] = nullptr;
        dev->arena_bytes[slot] = 0;
    }
    const size_t want = round_up(bytes + bytes / 8, 1 << 20);
    CLEF_CUDA(cudaMalloc(&dev->arena[slot], want));
    dev->arena_bytes[slot] = want;
    return CLEF_OK;
}

int ensure_consts(clef_device* dev, size_t bytes) {
    if (dev->consts_bytes >= bytes) {
        return CLEF_OK;
    }
    for (int s = 0; s < kStreams; ++s) {
        CLEF_CUDA(cudaStreamSynchronize(dev->streams[s]));
    }
    if (dev->consts) {
        CLEF_CUDA(cudaFree(dev->consts));
        dev->consts = nullptr;
        dev->consts_bytes = 0;
    }
    const size_t want = round_up(bytes, 1 << 16);
    CLEF_CUDA(cudaMalloc(&dev->consts, want));
    dev->consts_bytes = want;
    return CLEF_OK;
}

// A per-row stream of a tiled call: `row_bytes` bytes per row at `host`, staged at `offset` of the slot.
struct RowStream {
    const void* host_in = nullptr;   // input: copied host -> device before the launch
    void* host_out = nullptr;        // output: copied device -> host after the launch
    size_t row_bytes = 0;
    size_t offset = 0;               // byte offset inside the slot's arena (256-byte aligned)
};

// Drives `launch(stream, slot_base, first_row, n_rows, n_rows_padded)` over row tiles of `tile_rows`
// (a multiple of `atom`), alternating between the two streams. Inputs are copied for the live rows of
// the tile, outputs for its padded rows (`pad_outputs`) or its live rows.
template <typename Launch>
int run_tiled(clef_device* dev, int rows, int atom, int tile_rows, std::vector<RowStream>& streams_in,
              std::vector<RowStream>& streams_out, bool pad_outputs, Launch launch) {
    size_t slot_bytes = 0;
    for (auto* list : {&streams_in, &streams_out}) {
        for (RowStream& r : *list) {
            r.offset = slot_bytes;
            slot_bytes += round_up(r.row_bytes * (size_t)tile_rows, 256);
        }
    }
    for (int s = 0; s < kStreams; ++s) {
        if (int rc = ensure_arena(dev, s, slot_bytes)) return rc;
    }
    // Device pointers a caller passes (clef_device_alloc / clef_device_upload) are ordered on stream 0 only:
    // stream 1 starts this call behind everything stream 0 holds so far.
    CLEF_CUDA(cudaEventRecord(dev->fence[0], dev->streams[0]));
    CLEF_CUDA(cudaStreamWaitEvent(dev->streams[1], dev->fence[0], 0));
    const int rows_padded = (int)round_up((size_t)rows, (size_t)atom);
    int tile = 0;
    for (int r0 = 0; r0 < rows_padded; r0 += tile_rows, ++tile) {
        const int s = tile % kStreams;
        cudaStream_t st = dev->streams[s];
        char* base = static_cast<char*>(dev->arena[s]);
        const int n_padded = std::min(tile_rows, rows_padded - r0);
        const int n_live = std::max(0, std::min(n_padded, rows - r0));
        // The slot's previous tile must have left the arena (its downloads are ordered on `st`, so
        // stream order already guarantees it; the event documents the dependency).
        CLEF_CUDA(cudaStreamWaitEvent(st, dev->slot_free[s], 0));
        for (const RowStream& in : streams_in) {
            if (n_live > 0) {
                CLEF_CUDA(cudaMemcpyAsync(base + in.offset,
                                          static_cast<const char*>(in.host_in) + (size_t)r0 * in.row_bytes,
                                          (size_t)n_live * in.row_bytes, cudaMemcpyHostToDevice, st));
            }
        }
        if (int rc = launch(st, base, r0, n_live, n_padded)) return rc;
        for (const RowStream& out : streams_out) {
            const int n = pad_outputs ? n_padded : n_live;
            if (n > 0) {
                CLEF_CUDA(cudaMemcpyAsync(static_cast<char*>(out.host_out) + (size_t)r0 * out.row_bytes,
                                          base + out.offset, (size_t)n * out.row_bytes, cudaMemcpyDeviceToHost, st));
            }
        }
        CLEF_CUDA(cudaEventRecord(dev->slot_free[s], st));
    }
    for (int s = 0; s < kStreams; ++s) {
        // the half of the constants arena this call read may be rewritten once this point is reached
        CLEF_CUDA(cudaEventRecord(dev->gen_done[dev->consts_gen][s], dev->streams[s]));
    }
    // ... and what the caller enqueues on stream 0 next (an upload over an operand, clef_device_free) comes
    // behind the tiles that ran on stream 1.
    CLEF_CUDA(cudaEventRecord(dev->fence[1], dev->streams[1]));
    CLEF_CUDA(cudaStreamWaitEvent(dev->streams[0], dev->fence[1], 0));
    if (!dev->pipelined) {
        for (int s = 0; s < kStreams; ++s) {
            CLEF_CUDA(cudaStreamSynchronize(dev->streams[s]));
        }
    }
    return CLEF_OK;
}

// Rows per tile: large enough to keep the copy engines busy, small enough to pipeline a pass.
int pick_tile_rows(int rows, int atom, size_t bytes_per_row) {
    const size_t target = (size_t)24 << 20;   // about 24 MiB of traffic per tile
    size_t t = std::max<size_t>(1, target / std::max<size_t>(1, bytes_per_row));
    t = std::max<size_t>(atom, t / atom * atom);
    const size_t padded = round_up((size_t)rows, (size_t)atom);
    return (int)std::min(t, padded);
}

int check_handle(const clef_device* dev, const char* what) {
    if (!dev) return fail(CLEF_ERR_INVALID, "%s: null device handle", what);
    return CLEF_OK;
}

// Upload small constant operands to the front of the consts arena on both streams' timeline.
int upload_consts(clef_device* dev, std::initializer_list<std::pair<const void*, size_t>> items,
                  std::vector<void*>& device_ptrs) {
    size_t total = 0;
    for (const auto& it : items) total += round_up(it.second, 256);
    const size_t half = round_up(total, 1 << 16);
    if (int rc = ensure_consts(dev, 2 * half)) return rc;
    // Alternate calls use alternate halves, so that (in pipelined mode) this call's constants can be uploaded while
    // the previous call's kernels still read theirs; the half is free once the call before that has passed the
    // events recorded at its end.
    dev->consts_gen ^= 1;
    for (int s = 0; s < kStreams; ++s) {
        CLEF_CUDA(cudaStreamWaitEvent(dev->streams[0], dev->gen_done[dev->consts_gen][s], 0));
    }
    size_t off = (size_t)dev->consts_gen * (dev->consts_bytes / 2);
    for (const auto& it : items) {
        void* dst = static_cast<char*>(dev->consts) + off;
        device_ptrs.push_back(it.first ? dst : nullptr);
        if (it.first && it.second) {
            CLEF_CUDA(cudaMemcpyAsync(dst, it.first, it.second, cudaMemcpyHostToDevice, dev->streams[0]));
        }
        off += round_up(it.second, 256);
    }
    // Both streams read the constants: order stream 1 after the copies issued on stream 0.
    cudaEvent_t ready = dev->slot_free[0];
    CLEF_CUDA(cudaEventRecord(ready, dev->streams[0]));
    CLEF_CUDA(cudaStreamWaitEvent(dev->streams[1], ready, 0));
    return CLEF_OK;
}

}  // namespace

extern "C" {

// ---- device handle -----------------------------------------------------------------------------------
int clef_device_open(int ordinal, clef_device** out) {
    if (!out) return fail(CLEF_ERR_INVALID, "clef_device_open: null out pointer");
    int count = 0;
    CLEF_CUDA(cudaGetDeviceCount(&count));
    if (ordinal < 0 || ordinal >= count) {
        return fail(CLEF_ERR_INVALID, "clef_device_open: device %d of %d", ordinal, count);
    }
    int major = 0;
    CLEF_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, ordinal));
    if (major != 10) {
        return fail(CLEF_ERR_CUDA, "clef_device_open: device %d is compute capability %d.x; this library holds sm_100a code only",
                    ordinal, major);
    }
    clef_device* dev = new clef_device();
    dev->ordinal = ordinal;
    const int rc = [&]() -> int {
        CLEF_DEVICE_SCOPE(dev, "clef_device_open");
        // The reference runs its one stream at the highest priority (src/cuda/mod.rs:610-628).
        int least = 0, greatest = 0;
        CLEF_CUDA(cudaDeviceGetStreamPriorityRange(&least, &greatest));
        for (int s = 0; s < kStreams; ++s) {
            CLEF_CUDA(cudaStreamCreateWithPriority(&dev->streams[s], cudaStreamNonBlocking, greatest));
            CLEF_CUDA(cudaEventCreateWithFlags(&dev->slot_free[s], cudaEventDisableTiming));
            CLEF_CUDA(cudaEventCreateWithFlags(&dev->fence[s], cudaEventDisableTiming));
            CLEF_CUDA(cudaEventCreateWithFlags(&dev->gen_done[0][s], cudaEventDisableTiming));
            CLEF_CUDA(cudaEventCreateWithFlags(&dev->gen_done[1][s], cudaEventDisableTiming));
        }
        return CLEF_OK;
    }();
    if (rc != CLEF_OK) {
        clef_device_close(dev);   // destroys whatever was created before the failing step (the message stays)
        return rc;
    }
    *out = dev;
    return CLEF_OK;
}

int clef_device_close(clef_device* dev) {
    if (!dev) return CLEF_OK;
    {
        DeviceScope scope(dev);
        for (int s = 0; s < kStreams; ++s) {
            if (dev->streams[s]) {
                cudaStreamSynchronize(dev->streams[s]);
                cudaStreamDestroy(dev->streams[s]);
            }
            if (dev->slot_free[s]) cudaEventDestroy(dev->slot_free[s]);
            if (dev->fence[s]) cudaEventDestroy(dev->fence[s]);
            if (dev->gen_done[0][s]) cudaEventDestroy(dev->gen_done[0][s]);
            if (dev->gen_done[1][s]) cudaEventDestroy(dev->gen_done[1][s]);
            if (dev->arena[s]) cudaFree(dev->arena[s]);
        }
        if (dev->consts) cudaFree(dev->consts);
    }
    delete dev;
    return CLEF_OK;
}

int clef_device_ordinal(const clef_device* dev) { return dev ? dev->ordinal : -1; }

clef_stream_t clef_device_stream(clef_device* dev) { return dev ? (clef_stream_t)dev->streams[0] : nullptr; }

int clef_device_synchronize(clef_device* dev) {
    if (int rc = check_handle(dev, "clef_device_synchronize")) return rc;
    CLEF_DEVICE_SCOPE(dev, "clef_device_synchronize");
    for (int s = 0; s < kStreams; ++s) {
        CLEF_CUDA(cudaStreamSynchronize(dev->streams[s]));
    }
    return CLEF_OK;
}

int clef_device_set_pipelined(clef_device* dev, int on) {
    if (int rc = check_handle(dev, "clef_device_set_pipelined")) return rc;
    std::lock_guard<std::mutex> guard(dev->lock);
    dev->pipelined = on != 0;
    if (!dev->pipelined) {
        CLEF_DEVICE_SCOPE(dev, "clef_device_set_pipelined");
        for (int s = 0; s < kStreams; ++s) {
            CLEF_CUDA(cudaStreamSynchronize(dev->streams[s]));
        }
    }
    return CLEF_OK;
}

int clef_device_alloc(clef_device* dev, size_t bytes, void** out) {
    if (int rc = check_handle(dev, "clef_device_alloc")) return rc;
    if (!out) return fail(CLEF_ERR_INVALID, "clef_device_alloc: null out pointer");
    CLEF_DEVICE_SCOPE(dev, "clef_device_alloc");
    CLEF_CUDA(cudaMallocAsync(out, bytes ? bytes : 1, dev->streams[0]));
    return CLEF_OK;
}

int clef_device_free(clef_device* dev, void* ptr) {
    if (int rc = check_handle(dev, "clef_device_free")) return rc;
    if (!ptr) return CLEF_OK;
    CLEF_DEVICE_SCOPE(dev, "clef_device_free");
    CLEF_CUDA(cudaFreeAsync(ptr, dev->streams[0]));
    return CLEF_OK;
}

int clef_device_upload(clef_device* dev, void* dst_device, const void* src_host, size_t bytes) {
    if (int rc = check_handle(dev, "clef_device_upload")) return rc;
    if ((!dst_device || !src_host) && bytes) return fail(CLEF_ERR_INVALID, "clef_device_upload: null pointer");
    CLEF_DEVICE_SCOPE(dev, "clef_device_upload");
    CLEF_CUDA(cudaMemcpyAsync(dst_device, src_host, bytes, cudaMemcpyHostToDevice, dev->streams[0]));
    return CLEF_OK;
}

int clef_device_download(clef_device* dev, void* dst_host, const void* src_device, size_t bytes) {
    if (int rc = check_handle(dev, "clef_device_download")) return rc;
    if ((!dst_host || !src_device) && bytes) return fail(CLEF_ERR_INVALID, "clef_device_download: null pointer");
    CLEF_DEVICE_SCOPE(dev, "clef_device_download");
    CLEF_CUDA(cudaMemcpyAsync(dst_host, src_device, bytes, cudaMemcpyDeviceToHost, dev->streams[0]));
    CLEF_CUDA(cudaStreamSynchronize(dev->streams[0]));
    return CLEF_OK;
}

int clef_host_alloc_pinned(size_t bytes, void** out) {
    if (!out) return fail(CLEF_ERR_INVALID, "clef_host_alloc_pinned: null out pointer");
    CLEF_CUDA(cudaHostAlloc(out, bytes ? bytes : 1, cudaHostAllocDefault));
    return CLEF_OK;
}

int clef_host_free_pinned(void* ptr) {
    if (ptr) CLEF_CUDA(cudaFreeHost(ptr));
    return CLEF_OK;
}

// ---- host-slice launchers --------------------------------------------------------------------------------
int clef_host_embed_gather(clef_device* dev, const void* table_device, const int32_t* ids, void* out, int tokens,
                           int hidden, int dtype) {
    const char* what = "clef_host_embed_gather";
    if (int rc = check_handle(dev, what)) return rc;
    if (!table_device || !ids || !out) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (tokens < 0 || hidden <= 0 || (dtype != CLEF_BF16 && dtype != CLEF_F32)) {
        return fail(CLEF_ERR_INVALID, "%s: tokens %d hidden %d dtype %d", what, tokens, hidden, dtype);
    }
    if (tokens == 0) return CLEF_OK;
    std::lock_guard<std::mutex> guard(dev->lock);
    CLEF_DEVICE_SCOPE(dev, "clef_host_embed_gather");
    const size_t row = (size_t)hidden * elem_bytes(dtype);
    std::vector<RowStream> in{{ids, nullptr, sizeof(int32_t), 0}};
    std::vector<RowStream> outs{{nullptr, out, row, 0}};
    const int tile = pick_tile_rows(tokens, 128, row);
    return run_tiled(dev, tokens, 1, tile, in, outs, false,
                     [&](cudaStream_t st, char* base, int, int n_live, int) -> int {
                         return clef_embed_gather(st, table_device, (const int32_t*)(base + in[0].offset),
                                                  base + outs[0].offset, n_live, hidden, dtype);
                     });
}

static int host_quant_common(clef_device* dev, const char* what, int rows, int cols, int tile_m, int dtype,
                             int* blk_mn, int* chunk) {
    if (int rc = check_handle(dev, what)) return rc;
    if (dtype != CLEF_BF16 && dtype != CLEF_F32) return fail(CLEF_ERR_INVALID, "%s: dtype %d", what, dtype);
    if (rows < 0 || cols <= 0 || cols % 64 != 0) {
        return fail(CLEF_ERR_INVALID, "%s: rows %d, cols %d (cols must be a multiple of 64)", what, rows, cols);
    }
    return clef_sf_atom_for_tile_m(tile_m, blk_mn, chunk);
}

int clef_host_quantise_nvfp4(clef_device* dev, const void* x, uint8_t* packed, uint8_t* scales, int rows, int cols,
                             float global_scale, int tile_m, int dtype) {
    const char* what = "clef_host_quantise_nvfp4";
    int blk_mn = 0, chunk = 0;
    if (int rc = host_quant_common(dev, what, rows, cols, tile_m, dtype, &blk_mn, &chunk)) return rc;
    if (!x || !packed || !scales) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (rows == 0) return CLEF_OK;
    std::lock_guard<std::mutex> guard(dev->lock);
    CLEF_DEVICE_SCOPE(dev, "clef_host_quantise_nvfp4");
    const size_t row_in = (size_t)cols * elem_bytes(dtype);
    std::vector<RowStream> in{{x, nullptr, row_in, 0}};
    std::vector<RowStream> outs{{nullptr, packed, (size_t)cols / 2, 0}, {nullptr, scales, (size_t)cols / 16, 0}};
    const int tile = pick_tile_rows(rows, blk_mn, row_in + cols / 2 + cols / 16);
    return run_tiled(dev, rows, blk_mn, tile, in, outs, true,
                     [&](cudaStream_t st, char* base, int, int n_live, int) -> int {
                         return clef_quantise_nvfp4(st, base + in[0].offset, (uint8_t*)(base + outs[0].offset),
                                                    (uint8_t*)(base + outs[1].offset), n_live, cols, global_scale,
                                                    blk_mn, chunk, dtype);
                     });
}

// Device::quantise_fp8 (src/cuda/mod.rs:1065-1092): FP8 codes [rows, cols] and one u16 scale word per row.
int clef_host_quantise_fp8(clef_device* dev, const void* x, uint8_t* out, uint16_t* scales, int rows, int cols,
                           int dtype) {
    const char* what = "clef_host_quantise_fp8";
    if (int rc = check_handle(dev, what)) return rc;
    if (dtype != CLEF_BF16 && dtype != CLEF_F32) return fail(CLEF_ERR_INVALID, "%s: dtype %d", what, dtype);
    if (rows < 0 || cols <= 0 || cols % 8 != 0) {
        return fail(CLEF_ERR_INVALID, "%s: rows %d, cols %d (cols must be a multiple of 8)", what, rows, cols);
    }
    if (!x || !out || !scales) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (rows == 0) return CLEF_OK;
    std::lock_guard<std::mutex> guard(dev->lock);
    CLEF_DEVICE_SCOPE(dev, "clef_host_quantise_fp8");
    const size_t row_in = (size_t)cols * elem_bytes(dtype);
    std::vector<RowStream> in{{x, nullptr, row_in, 0}};
    std::vector<RowStream> outs{{nullptr, out, (size_t)cols, 0}, {nullptr, scales, sizeof(uint16_t), 0}};
    const int tile = pick_tile_rows(rows, 128, row_in + cols + 2);
    return run_tiled(dev, rows, 1, tile, in, outs, false,
                     [&](cudaStream_t st, char* base, int, int n_live, int) -> int {
                         return clef_quantise_fp8(st, base + in[0].offset, (uint8_t*)(base + outs[0].offset),
                                                  (uint16_t*)(base + outs[1].offset), n_live, cols, dtype);
                     });
}

int clef_host_rms_norm_quantise_nvfp4(clef_device* dev, const void* x, const float* weight, uint8_t* packed,
                                      uint8_t* scales, int rows, int cols, float eps, float global_scale, int tile_m,
                                      int dtype) {
    const char* what = "clef_host_rms_norm_quantise_nvfp4";
    int blk_mn = 0, chunk = 0;
    if (int rc = host_quant_common(dev, what, rows, cols, tile_m, dtype, &blk_mn, &chunk)) return rc;
    if (!x || !weight || !packed || !scales) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (rows == 0) return CLEF_OK;
    std::lock_guard<std::mutex> guard(dev->lock);
    CLEF_DEVICE_SCOPE(dev, "clef_host_rms_norm_quantise_nvfp4");
    std::vector<void*> consts;
    if (int rc = upload_consts(dev, {{weight, (size_t)cols * sizeof(float)}}, consts)) return rc;
    const size_t row_in = (size_t)cols * elem_bytes(dtype);
    std::vector<RowStream> in{{x, nullptr, row_in, 0}};
    std::vector<RowStream> outs{{nullptr, packed, (size_t)cols / 2, 0}, {nullptr, scales, (size_t)cols / 16, 0}};
    const int tile = pick_tile_rows(rows, blk_mn, row_in + cols / 2 + cols / 16);
    return run_tiled(dev, rows, blk_mn, tile, in, outs, true,
                     [&](cudaStream_t st, char* base, int, int n_live, int n_padded) -> int {
                         if (n_live == 0) {   // a tile of padding only: zero codes, zero scales
                             if (cudaMemsetAsync(base + outs[0].offset, 0, (size_t)n_padded * (cols / 2), st) != cudaSuccess ||
                                 cudaMemsetAsync(base + outs[1].offset, 0, (size_t)n_padded * (cols / 16), st) != cudaSuccess) {
                                 return fail(CLEF_ERR_CUDA, "%s: cudaMemsetAsync failed", what);
                             }
                             return CLEF_OK;
                         }
                         return clef_rms_norm_quantise_nvfp4(st, base + in[0].offset, (const float*)consts[0],
                                                             (uint8_t*)(base + outs[0].offset),
                                                             (uint8_t*)(base + outs[1].offset), n_live, cols, eps,
                                                             global_scale, blk_mn, chunk, dtype);
                     });
}

int clef_host_swiglu_quantise_nvfp4(clef_device* dev, const void* gate, const void* up, uint8_t* packed,
                                    uint8_t* scales, int rows, int cols, float global_scale, int tile_m, int dtype) {
    const char* what = "clef_host_swiglu_quantise_nvfp4";
    int blk_mn = 0, chunk = 0;
    if (int rc = host_quant_common(dev, what, rows, cols, tile_m, dtype, &blk_mn, &chunk)) return rc;
    if (!gate || !up || !packed || !scales) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (rows == 0) return CLEF_OK;
    std::lock_guard<std::mutex> guard(dev->lock);
    CLEF_DEVICE_SCOPE(dev, "clef_host_swiglu_quantise_nvfp4");
    const size_t row_in = (size_t)cols * elem_bytes(dtype);
    std::vector<RowStream> in{{gate, nullptr, row_in, 0}, {up, nullptr, row_in, 0}};
    std::vector<RowStream> outs{{nullptr, packed, (size_t)cols / 2, 0}, {nullptr, scales, (size_t)cols / 16, 0}};
    const int tile = pick_tile_rows(rows, blk_mn, 2 * row_in + cols / 2 + cols / 16);
    return run_tiled(dev, rows, blk_mn, tile, in, outs, true,
                     [&](cudaStream_t st, char* base, int, int n_live, int) -> int {
                         return clef_swiglu_quantise_nvfp4(st, base + in[0].offset, base + in[1].offset,
                                                           (uint8_t*)(base + outs[0].offset),
                                                           (uint8_t*)(base + outs[1].offset), n_live, cols,
                                                           global_scale, blk_mn, chunk, dtype);
                     });
}

int clef_host_rms_norm_gated_quantise_nvfp4(clef_device* dev, const void* x, const void* gate, const float* weight,
                                            uint8_t* packed, uint8_t* scales, int rows, int cols, int vh, float eps,
                                            float global_scale, int tile_m, int dtype) {
    const char* what = "clef_host_rms_norm_gated_quantise_nvfp4";
    if (vh <= 0 || cols <= 0 || rows < 0 || rows % (vh > 0 ? vh : 1) != 0) {
        return fail(CLEF_ERR_INVALID, "%s: rows %d must be a multiple of vh %d", what, rows, vh);
    }
    int blk_mn = 0, chunk = 0;
    const int tokens = rows / vh;
    if (int rc = host_quant_common(dev, what, tokens, vh * cols, tile_m, dtype, &blk_mn, &chunk)) return rc;
    if (!x || !gate || !weight || !packed || !scales) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (rows == 0) return CLEF_OK;
    std::lock_guard<std::mutex> guard(dev->lock);
    CLEF_DEVICE_SCOPE(dev, "clef_host_rms_norm_gated_quantise_nvfp4");
    std::vector<void*> consts;
    if (int rc = upload_consts(dev, {{weight, (size_t)cols * sizeof(float)}}, consts)) return rc;
    // Tiles are cut in TOKENS; a token row carries vh head rows.
    const size_t tok_in = (size_t)vh * cols * elem_bytes(dtype);
    const size_t flat = (size_t)vh * cols;
    std::vector<RowStream> in{{x, nullptr, tok_in, 0}, {gate, nullptr, tok_in, 0}};
    std::vector<RowStream> outs{{nullptr, packed, flat / 2, 0}, {nullptr, scales, flat / 16, 0}};
    const int tile = pick_tile_rows(tokens, blk_mn, 2 * tok_in + flat / 2 + flat / 16);
    return run_tiled(dev, tokens, blk_mn, tile, in, outs, true,
                     [&](cudaStream_t st, char* base, int, int n_live, int n_padded) -> int {
                         return clef_rms_norm_gated_quantise_nvfp4(
                             st, base + in[0].offset, base + in[1].offset, (const float*)consts[0],
                             (uint8_t*)(base + outs[0].offset), (uint8_t*)(base + outs[1].offset), n_padded * vh, cols,
                             eps, global_scale, blk_mn, chunk, vh, n_live * vh, dtype);
                     });
}

// ---- the reference's plain host-slice wrappers (src/cuda/mod.rs:853-973) ---------------------------------

int clef_host_rms_norm(clef_device* dev, const void* x, const float* weight, void* out, int rows, int cols, float eps,
                       int dtype) {
    const char* what = "clef_host_rms_norm";
    if (int rc = check_handle(dev, what)) return rc;
    if (dtype != CLEF_BF16 && dtype != CLEF_F32) return fail(CLEF_ERR_INVALID, "%s: dtype %d", what, dtype);
    if (rows < 0 || cols <= 0 || cols % 4 != 0) return fail(CLEF_ERR_INVALID, "%s: rows %d, cols %d (cols must be a multiple of 4)", what, rows, cols);
    if (!x || !out) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (rows == 0) return CLEF_OK;
    std::lock_guard<std::mutex> guard(dev->lock);
    CLEF_DEVICE_SCOPE(dev, "clef_host_rms_norm");
    std::vector<void*> consts;
    if (int rc = upload_consts(dev, {{weight, (size_t)cols * sizeof(float)}}, consts)) return rc;
    const size_t row = (size_t)cols * elem_bytes(dtype);
    std::vector<RowStream> in{{x, nullptr, row, 0}};
    std::vector<RowStream> outs{{nullptr, out, row, 0}};
    const int tile = pick_tile_rows(rows, 128, 2 * row);
    return run_tiled(dev, rows, 1, tile, in, outs, false, [&](cudaStream_t st, char* base, int, int n_live, int) -> int {
        return clef_rms_norm(st, base + in[0].offset, (const float*)consts[0], base + outs[0].offset, n_live, cols, eps, dtype);
    });
}

int clef_host_rms_norm_gated(clef_device* dev, const void* x, const void* gate, const float* weight, void* out, int rows,
                             int cols, float eps, int dtype) {
    const char* what = "clef_host_rms_norm_gated";
    if (int rc = check_handle(dev, what)) return rc;
    if (dtype != CLEF_BF16 && dtype != CLEF_F32) return fail(CLEF_ERR_INVALID, "%s: dtype %d", what, dtype);
    if (rows < 0 || cols <= 0 || cols % 4 != 0) return fail(CLEF_ERR_INVALID, "%s: rows %d, cols %d (cols must be a multiple of 4)", what, rows, cols);
    if (!x || !out) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (rows == 0) return CLEF_OK;
    std::lock_guard<std::mutex> guard(dev->lock);
    CLEF_DEVICE_SCOPE(dev, "clef_host_rms_norm_gated");
    std::vector<void*> consts;
    if (int rc = upload_consts(dev, {{weight, (size_t)cols * sizeof(float)}}, consts)) return rc;
    const size_t row = (size_t)cols * elem_bytes(dtype);
    std::vector<RowStream> in{{x, nullptr, row, 0}};
    if (gate) in.push_back({gate, nullptr, row, 0});
    std::vector<RowStream> outs{{nullptr, out, row, 0}};
    const int tile = pick_tile_rows(rows, 128, (gate ? 3 : 2) * row);
    return run_tiled(dev, rows, 1, tile, in, outs, false, [&](cudaStream_t st, char* base, int, int n_live, int) -> int {
        return clef_rms_norm_gated(st, base + in[0].offset, gate ? base + in[1].offset : nullptr, (const float*)consts[0],
                                   base + outs[0].offset, n_live, cols, eps, dtype);
    });
}

int clef_host_swiglu(clef_device* dev, const void* gate, const void* up, void* out, size_t total, int dtype) {
    const char* what = "clef_host_swiglu";
    if (int rc = check_handle(dev, what)) return rc;
    if (dtype != CLEF_BF16 && dtype != CLEF_F32) return fail(CLEF_ERR_INVALID, "%s: dtype %d", what, dtype);
    if (total % 4 != 0) return fail(CLEF_ERR_INVALID, "%s: total %zu must be a multiple of 4", what, total);
    if (!gate || !up || !out) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (total == 0) return CLEF_OK;
    // the flat arrays are cut into "rows" of the largest power of two up to 4,096 values that divides their length
    size_t width = 4;
    while (width < 4096 && total % (2 * width) == 0) width *= 2;
    if (total / width > 0x7fffffffull) return fail(CLEF_ERR_TOO_LARGE, "%s: %zu values", what, total);
    const int rows = (int)(total / width);
    std::lock_guard<std::mutex> guard(dev->lock);
    CLEF_DEVICE_SCOPE(dev, "clef_host_swiglu");
    const size_t row = width * elem_bytes(dtype);
    std::vector<RowStream> in{{gate, nullptr, row, 0}, {up, nullptr, row, 0}};
    std::vector<RowStream> outs{{nullptr, out, row, 0}};
    const int tile = pick_tile_rows(rows, 128, 3 * row);
    return run_tiled(dev, rows, 1, tile, in, outs, false, [&](cudaStream_t st, char* base, int, int n_live, int) -> int {
        return clef_swiglu(st, base + in[0].offset, base + in[1].offset, base + outs[0].offset, (size_t)n_live * width, dtype);
    });
}

int clef_host_causal_conv_silu(clef_device* dev, const void* x, const float* w, void* out, int rows, int channels, int k,
                               int dtype) {
    const char* what = "clef_host_causal_conv_silu";
    if (int rc = check_handle(dev, what)) return rc;
    if (dtype != CLEF_BF16 && dtype != CLEF_F32) return fail(CLEF_ERR_INVALID, "%s: dtype %d", what, dtype);
    if (rows < 0 || channels <= 0 || k <= 0) return fail(CLEF_ERR_INVALID, "%s: rows %d channels %d k %d", what, rows, channels, k);
    if (!x || !w || !out) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (rows == 0) return CLEF_OK;
    std::lock_guard<std::mutex> guard(dev->lock);
    CLEF_DEVICE_SCOPE(dev, "clef_host_causal_conv_silu");
    std::vector<void*> consts;
    if (int rc = upload_consts(dev, {{w, (size_t)channels * k * sizeof(float)}}, consts)) return rc;
    // a row's taps reach k - 1 rows back, so the sequence goes through as ONE tile (a single sequence without history,
    // as Device::causal_conv_silu runs it)
    const size_t row = (size_t)channels * elem_bytes(dtype);
    std::vector<RowStream> in{{x, nullptr, row, 0}};
    std::vector<RowStream> outs{{nullptr, out, row, 0}};
    return run_tiled(dev, rows, 1, rows, in, outs, false, [&](cudaStream_t st, char* base, int, int n_live, int) -> int {
        return clef_causal_conv_silu(st, base + outs[0].offset, base + in[0].offset, (const float*)consts[0], n_live, channels, k,
                                     nullptr, nullptr, nullptr, dtype);
    });
}

int clef_host_rope_tables(clef_device* dev, const int32_t* positions, float* cos_out, float* sin_out, int count,
                          int rotary_dim, float theta) {
    const char* what = "clef_host_rope_tables";
    if (int rc = check_handle(dev, what)) return rc;
    if (count < 0 || rotary_dim <= 0 || rotary_dim % 2 != 0) return fail(CLEF_ERR_INVALID, "%s: count %d rotary_dim %d", what, count, rotary_dim);
    if (!positions || !cos_out || !sin_out) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (count == 0) return CLEF_OK;
    std::lock_guard<std::mutex> guard(dev->lock);
    CLEF_DEVICE_SCOPE(dev, "clef_host_rope_tables");
    const size_t row = (size_t)rotary_dim * sizeof(float);
    std::vector<RowStream> in{{positions, nullptr, sizeof(int32_t), 0}};
    std::vector<RowStream> outs{{nullptr, cos_out, row, 0}, {nullptr, sin_out, row, 0}};
    const int tile = pick_tile_rows(count, 128, 2 * row + 4);
    return run_tiled(dev, count, 1, tile, in, outs, false, [&](cudaStream_t st, char* base, int, int n_live, int) -> int {
        return clef_rope_tables(st, (const int32_t*)(base + in[0].offset), (float*)(base + outs[0].offset),
                                (float*)(base + outs[1].offset), n_live, rotary_dim, theta);
    });
}

int clef_host_rope(clef_device* dev, void* out, const void* x, const float* cos_table, const float* sin_table,
                   int table_rows, int rows, int heads, int head_dim, int rotary_dim, const int32_t* pos_map,
                   int dtype) {
    const char* what = "clef_host_rope";
    if (int rc = check_handle(dev, what)) return rc;
    if (!out || !x || !cos_table || !sin_table) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    if (dtype != CLEF_BF16 && dtype != CLEF_F32) return fail(CLEF_ERR_INVALID, "%s: dtype %d", what, dtype);
    if (rows < 0 || heads <= 0 || head_dim <= 0 || rotary_dim <= 0 || table_rows <= 0) {
        return fail(CLEF_ERR_INVALID, "%s: rows %d heads %d head_dim %d rotary_dim %d table_rows %d", what, rows, heads,
                    head_dim, rotary_dim, table_rows);
    }
    if (rows == 0) return CLEF_OK;
    // Positions are checked on the host: the kernel indexes the tables with them unchecked.
    std::vector<int32_t> iota;
    if (!pos_map) {
        iota.resize(rows);
        for (int i = 0; i < rows; ++i) iota[i] = i;
        pos_map = iota.data();
    }
    for (int i = 0; i < rows; ++i) {
        if (pos_map[i] < 0 || pos_map[i] >= table_rows) {
            return fail(CLEF_ERR_INVALID, "%s: position %d of row %d is outside the %d-row tables", what, pos_map[i], i,
                        table_rows);
        }
    }
    std::lock_guard<std::mutex> guard(dev->lock);
    CLEF_DEVICE_SCOPE(dev, "clef_host_rope");
    const size_t table_bytes = (size_t)table_rows * rotary_dim * sizeof(float);
    std::vector<void*> consts;
    if (int rc = upload_consts(dev, {{cos_table, table_bytes}, {sin_table, table_bytes}}, consts)) return rc;
    const size_t row = (size_t)heads * head_dim * elem_bytes(dtype);
    std::vector<RowStream> in{{x, nullptr, row, 0}, {pos_map, nullptr, sizeof(int32_t), 0}};
    std::vector<RowStream> outs{{nullptr, out, row, 0}};
    const int tile = pick_tile_rows(rows, 128, 2 * row);
    const int rc = run_tiled(dev, rows, 1, tile, in, outs, false,
                             [&](cudaStream_t st, char* base, int, int n_live, int) -> int {
                                 return clef_rope(st, base + outs[0].offset, base + in[0].offset, (const float*)consts[0],
                                                  (const float*)consts[1], n_live, heads, head_dim, rotary_dim, nullptr,
                                                  nullptr, (const int32_t*)(base + in[1].offset), dtype);
                             });
    if (rc == CLEF_OK && dev->pipelined && !iota.empty()) {
        // the position map of this call lives in a local buffer: its uploads must finish before it goes away
        for (int s = 0; s < kStreams; ++s) {
            CLEF_CUDA(cudaStreamSynchronize(dev->streams[s]));
        }
    }
    return rc;
}

// ---- per-token maps -----------------------------------------------------------------------------------------
namespace {
// Rungs::body_at (src/gpu.rs:711-733): the head rungs up to `top`, their multiples by 2..slots up to `top`, and
// `top` itself when no rung reaches it; `top` is max(max_chunk, granule), NOT rounded to the granule.
std::vector<size_t> body_rungs(size_t slots, size_t max_chunk, size_t* top_out) {
    static const size_t head[8] = {64, 128, 256, 512, 1024, 2048, 4096, 8192};   // src/gpu.rs:689
    const size_t top = std::max<size_t>(max_chunk, CLEF_CHUNK_GRANULE);
    std::vector<size_t> rungs;
    for (size_t r : head) {
        if (r <= top) rungs.push_back(r);
    }
    for (size_t k = 2; k <= slots; ++k) {
        for (size_t r : head) {
            if (k * r <= top) rungs.push_back(k * r);
        }
    }
    if (rungs.empty() || *std::max_element(rungs.begin(), rungs.end()) < top) rungs.push_back(top);
    std::sort(rungs.begin(), rungs.end());
    rungs.erase(std::unique(rungs.begin(), rungs.end()), rungs.end());
    if (top_out) *top_out = top;
    return rungs;
}
}  // namespace

int clef_pass_geometries(size_t slots, size_t max_chunk, size_t* out, size_t cap) {
    // src/gpu.rs:779-795 (pass_geometries) on Rungs::body_at(max_chunk).
    if (slots == 0) slots = 1;
    size_t top = 0;
    const std::vector<size_t> rungs = body_rungs(slots, max_chunk, &top);
    std::vector<size_t> geoms = rungs;
    // The reference also caps totals at the engine's admission limit (max_batch_tokens), which in the
    // shipped configuration is not below slots * top; that product is the cap used here.
    const size_t max_graph = slots * top;
    for (size_t k = 2; k <= slots; ++k) {
        for (size_t r : rungs) {
            const size_t total = k * r;
            if (total > top && total <= k * top && total <= max_graph) geoms.push_back(total);
        }
    }
    std::sort(geoms.begin(), geoms.end());
    geoms.erase(std::unique(geoms.begin(), geoms.end()), geoms.end());
    if (out) {
        for (size_t i = 0; i < geoms.size() && i < cap; ++i) out[i] = geoms[i];
    }
    return (int)geoms.size();
}

int clef_rungs_decompose(size_t tokens, size_t slots, size_t max_chunk, size_t* bases, size_t* rows, size_t cap) {
    // Rungs::decompose, src/gpu.rs:762-775, on Rungs::body_at(max_chunk).
    if (slots == 0) slots = 1;
    const std::vector<size_t> rungs = body_rungs(slots, max_chunk, nullptr);
    const size_t smallest = rungs.front();
    size_t n = 0, base = 0;
    while (base < tokens) {
        const size_t rem = tokens - base;
        size_t pick = 0;
        for (size_t r : rungs) {
            if (r <= rem) pick = std::max(pick, r);
        }
        if (pick == 0) pick = smallest;
        if (n < cap) {
            if (bases) bases[n] = base;
            if (rows) rows[n] = pick;
        }
        ++n;
        base += pick;
    }
    return (int)n;
}

int clef_pass_maps_build(const clef_chunk_spec* chunks, size_t n_chunks, size_t capacity, int check_geometry,
                         size_t slots, size_t max_chunk, clef_pass_maps* m) {
    const char* what = "clef_pass_maps_build";
    if (!m || (!chunks && n_chunks)) return fail(CLEF_ERR_INVALID, "%s: null pointer", what);
    const size_t granule = CLEF_CHUNK_GRANULE;
    size_t total = 0;
    for (size_t i = 0; i < n_chunks; ++i) {
        if (chunks[i].rows == 0 || chunks[i].rows % granule != 0) {
            return fail(CLEF_ERR_INVALID, "%s: a chunk of %zu rows is not a positive granule multiple", what,
                        chunks[i].rows);
        }
        if (!chunks[i].ids || chunks[i].ids_len == 0) {
            return fail(CLEF_ERR_INVALID, "%s: a request has at least one token", what);
        }
        if (chunks[i].pos >= chunks[i].ids_len) {
            return fail(CLEF_ERR_INVALID, "%s: chunk %zu starts at %zu, past its %zu-token request", what, i,
                        chunks[i].pos, chunks[i].ids_len);
        }
        for (size_t j = i + 1; j < n_chunks; ++j) {
            if (chunks[i].slot == chunks[j].slot) {
                return fail(CLEF_ERR_INVALID, "%s: two chunks of one pass share slot %zu -- their keys would alias", what,
                            chunks[i].slot);
            }
        }
        total += chunks[i].rows;
    }
    if (check_geometry && n_chunks) {
        std::vector<size_t> geoms(4096);
        const int n = clef_pass_geometries(slots, max_chunk, geoms.data(), geoms.size());
        if (n < 0 || !std::binary_search(geoms.begin(), geoms.begin() + std::min<size_t>(n, geoms.size()), total)) {
            return fail(CLEF_ERR_INVALID, "%s: a pass of %zu rows is not a graphed geometry -- it would run eager", what,
                        total);
        }
    }
    if (total > 0x7fffffffu || capacity > 0x7fffffffu) return fail(CLEF_ERR_TOO_LARGE, "%s: pass too large", what);
    m->total = total;
    m->cache_len = n_chunks ? 0x7fffffff : 0;
    const int32_t cap = (int32_t)capacity;
    size_t off = 0, granule_index = 0;
    for (size_t i = 0; i < n_chunks; ++i) {
        const clef_chunk_spec& x = chunks[i];
        const size_t pad = x.rows;
        const size_t real = std::min(pad, x.ids_len - x.pos);
        if (m->rows_real) m->rows_real[i] = real;
        if (m->offs) m->offs[i] = off;
        const int32_t base = (int32_t)x.slot * cap;
        for (size_t t = 0; t < pad; ++t) {
            const size_t row = off + t;
            if (m->ids) m->ids[row] = t < real ? x.ids[x.pos + t] : x.ids[x.ids_len - 1];
            if (m->seq_start) m->seq_start[row] = (int32_t)off;
            if (m->seq_end) m->seq_end[row] = (int32_t)(off + real);
            if (m->cpos) m->cpos[row] = base + (int32_t)x.pos + (int32_t)t;
            if (m->cbase) m->cbase[row] = base;
            if (m->slot_map) m->slot_map[row] = (int32_t)x.slot;
            if (m->rope_pos) m->rope_pos[row] = (int32_t)x.pos + (int32_t)t;
        }
        m->cache_len = std::min(m->cache_len, base + (int32_t)x.pos);
        if (m->hist_save) {
            m->hist_save[2 * i] = (uint32_t)(off + real - 1);
            m->hist_save[2 * i + 1] = (uint32_t)x.slot;
        }
        for (size_t k = 0; k < pad / granule; ++k, ++granule_index) {
            if (m->chunk_start) m->chunk_start[granule_index] = (k == 0 && i > 0) ? 1 : 0;
            if (m->state_slot) m->state_slot[granule_index] = (int32_t)x.slot;
        }
        off += pad;
    }
    return CLEF_OK;
}

int clef_shard_rows(int rows, int blk_mn, int n_shards, int shard, int* first_row, int* n_rows) {
    if (rows < 0 || blk_mn <= 0 || n_shards <= 0 || shard < 0 || shard >= n_shards) {
        return fail(CLEF_ERR_INVALID, "clef_shard_rows: rows %d blk_mn %d shard %d of %d", rows, blk_mn, shard, n_shards);
    }
    const long long atoms = ((long long)rows + blk_mn - 1) / blk_mn;
    const long long per = (atoms + n_shards - 1) / n_shards;
    const long long first = std::min<long long>((long long)shard * per * blk_mn, rows);
    const long long last = std::min<long long>(((long long)shard + 1) * per * blk_mn, rows);
    if (first_row) *first_row = (int)first;
    if (n_rows) *n_rows = (int)(last - first);
    return CLEF_OK;
}

}  // extern "C"
