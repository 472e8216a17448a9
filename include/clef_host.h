/* clef_host.h -- host-side companions of the fused kernels, C ABI.
 *
 * Three pieces the reference keeps in Rust next to its launch layer, restated in C++ behind plain C
 * entry points so the reference (or any other host language) can bind them:
 *
 *  1. A device handle with stream-ordered buffers: `Device::open`, `alloc`, `upload`, `download`,
 *     `sync` of aiis-clef src/cuda/mod.rs:604-660, 3971-4051, 4255-4275, 4947.
 *  2. Host-slice launchers: the reference's convenience wrappers that take host slices, upload,
 *     launch and download (`Device::rms_norm`, `swiglu`, `rope_apply`, `quantise_nvfp4`:
 *     src/cuda/mod.rs:853-1075). Here they stream row tiles through two CUDA streams so the upload of
 *     one tile overlaps the kernel and the download of the previous one. These are what the
 *     end-to-end figure of the benchmark times. Host pointers may be pageable, but only pinned memory
 *     (clef_host_alloc_pinned, or any cudaHostAlloc / cudaHostRegister memory) copies asynchronously.
 *  3. The per-token maps of a pass: `pass_maps` of src/gpu.rs:948-1013 (ids, seq_start, seq_end, cpos,
 *     cbase, slot_map, rope_pos per row; chunk_start, state_slot per 64-row granule), the rung ladder of
 *     src/gpu.rs:689-775, and the row-range split used to spread one pass over several GPUs.
 *
 * Status codes are those of clef_fused.h; clef_last_error() reports the message.
 */
#ifndef CLEF_HOST_H
#define CLEF_HOST_H

#include <stddef.h>
#include <stdint.h>

#include "clef_fused.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct clef_device clef_device;

/* ---- device handle (src/cuda/mod.rs:604-660) ---------------------------------------------------- */
/* Opens device `ordinal` (the reference always opens 0), creates its streams. */
int clef_device_open(int ordinal, clef_device** out);
int clef_device_close(clef_device* dev);
int clef_device_ordinal(const clef_device* dev);
/* The stream every *_dev call of this handle should be given (a cudaStream_t). */
clef_stream_t clef_device_stream(clef_device* dev);
int clef_device_synchronize(clef_device* dev);
/* Pipelined mode (off by default): a host-slice call (clef_host_*) returns as soon as its copies and launches are
 * enqueued, so consecutive calls overlap (the uploads of the next call run under the downloads of the previous
 * one); outputs are complete in host memory after clef_device_synchronize. The caller keeps every host buffer of a
 * call, inputs and weights included, alive and unchanged until then. Switching it off synchronises. */
int clef_device_set_pipelined(clef_device* dev, int on);
/* Stream-ordered device memory (src/cuda/mod.rs:3971-4051); not for use inside a stream capture. alloc, upload
 * and free are enqueued on the handle's stream (clef_device_stream) and return at once; download waits for its
 * copy. A host-slice call that is given such a pointer (clef_host_embed_gather's table) starts behind them on
 * both of the handle's streams, and a free or an upload issued after the call comes behind all of its tiles. */
int clef_device_alloc(clef_device* dev, size_t bytes, void** out);
int clef_device_free(clef_device* dev, void* ptr);
int clef_device_upload(clef_device* dev, void* dst_device, const void* src_host, size_t bytes);
int clef_device_download(clef_device* dev, void* dst_host, const void* src_device, size_t bytes);
/* Pinned host memory for the host-slice launchers. */
int clef_host_alloc_pinned(size_t bytes, void** out);
int clef_host_free_pinned(void* ptr);

/* ---- host-slice launchers (src/cuda/mod.rs:853-1075) ------------------------------------------------
 * Every pointer is a HOST pointer. Each call returns after its outputs are complete in host memory.
 * Output sizes are those of clef_nvfp4_sizes (rows padded to the scale atom of `tile_m`). */
int clef_host_embed_gather(clef_device* dev, const void* table_device, const int32_t* ids, void* out, int tokens,
                           int hidden, int dtype);   /* the table stays on the device (it is a model weight) */
int clef_host_quantise_nvfp4(clef_device* dev, const void* x, uint8_t* packed, uint8_t* scales, int rows, int cols,
                             float global_scale, int tile_m, int dtype);
int clef_host_quantise_fp8(clef_device* dev, const void* x, uint8_t* out, uint16_t* scales, int rows, int cols,
                           int dtype);             /* Device::quantise_fp8, src/cuda/mod.rs:1065-1092 */
int clef_host_rms_norm_quantise_nvfp4(clef_device* dev, const void* x, const float* weight, uint8_t* packed,
                                      uint8_t* scales, int rows, int cols, float eps, float global_scale, int tile_m,
                                      int dtype);
int clef_host_swiglu_quantise_nvfp4(clef_device* dev, const void* gate, const void* up, uint8_t* packed,
                                    uint8_t* scales, int rows, int cols, float global_scale, int tile_m, int dtype);
/* rows = live head rows (tokens * vh), as in Device::rms_norm_gated_quantise_nvfp4_dev. */
int clef_host_rms_norm_gated_quantise_nvfp4(clef_device* dev, const void* x, const void* gate, const float* weight,
                                            uint8_t* packed, uint8_t* scales, int rows, int cols, int vh, float eps,
                                            float global_scale, int tile_m, int dtype);
/* Device::rms_norm (src/cuda/mod.rs:853-879): out = x * inv_rms * (1 + weight); weight may be NULL (no weight). */
int clef_host_rms_norm(clef_device* dev, const void* x, const float* weight, void* out, int rows, int cols, float eps,
                       int dtype);
/* Device::rms_norm_gated (src/cuda/mod.rs:881-909): out = x * inv_rms * weight * silu(gate); gate and weight may be
 * NULL as in the kernel. */
int clef_host_rms_norm_gated(clef_device* dev, const void* x, const void* gate, const float* weight, void* out, int rows,
                             int cols, float eps, int dtype);
/* Device::swiglu (src/cuda/mod.rs:911-933): out = silu(gate) * up over flat arrays of `total` values (a multiple of 4). */
int clef_host_swiglu(clef_device* dev, const void* gate, const void* up, void* out, size_t total, int dtype);
/* Device::causal_conv_silu (src/cuda/mod.rs:935-945): one sequence of `rows` tokens without history, w [channels, k]. */
int clef_host_causal_conv_silu(clef_device* dev, const void* x, const float* w, void* out, int rows, int channels, int k,
                               int dtype);
/* Device::rope_tables (src/cuda/mod.rs:947-973): cos_out, sin_out [count, rotary_dim] for the given positions. */
int clef_host_rope_tables(clef_device* dev, const int32_t* positions, float* cos_out, float* sin_out, int count,
                          int rotary_dim, float theta);
/* pos_map may be NULL (position = row index), as in Device::rope_apply. cos/sin: [table_rows, rotary_dim]. */
int clef_host_rope(clef_device* dev, void* out, const void* x, const float* cos_table, const float* sin_table,
                   int table_rows, int rows, int heads, int head_dim, int rotary_dim, const int32_t* pos_map,
                   int dtype);

/* ---- per-token maps (src/gpu.rs:905-1013) ------------------------------------------------------------- */
typedef struct clef_chunk_spec {
    const uint32_t* ids; /* the request's token ids */
    size_t ids_len;
    size_t pos;          /* first position of this chunk inside the request */
    size_t slot;         /* KV / state slot of the request */
    size_t rows;         /* padded rows of the chunk: a positive multiple of the 64-row granule */
} clef_chunk_spec;

/* Caller-allocated outputs; `total` = sum of chunk rows, `granules` = total / 64. */
typedef struct clef_pass_maps {
    uint32_t* ids;       /* [total] pad rows repeat the request's last id */
    int32_t* seq_start;  /* [total] first row of the row's chunk */
    int32_t* seq_end;    /* [total] one past the last REAL row of the row's chunk */
    int32_t* cpos;       /* [total] slot * capacity + pos + t : the KV row a token writes */
    int32_t* cbase;      /* [total] slot * capacity */
    int32_t* slot_map;   /* [total] */
    int32_t* rope_pos;   /* [total] pos + t : the position RoPE rotates by */
    int32_t* chunk_start;/* [granules] 1 on the first granule of every chunk but the first */
    int32_t* state_slot; /* [granules] */
    uint32_t* hist_save; /* [n_chunks * 2] (last real row, slot) */
    size_t* rows_real;   /* [n_chunks] */
    size_t* offs;        /* [n_chunks] */
    int32_t cache_len;   /* out: smallest slot * capacity + pos of the pass (0 for an empty pass) */
    size_t total;        /* out */
} clef_pass_maps;

#define CLEF_CHUNK_GRANULE 64

/* Fills `maps` for one pass. Refuses (CLEF_ERR_INVALID) a chunk whose rows are not a positive
 * multiple of 64, a request with no tokens, and two chunks sharing a slot -- the conditions the
 * reference asserts on. `check_geometry` != 0 also refuses a total that is not on the pass ladder
 * for `slots` KV slots and `max_chunk` rows (src/gpu.rs:779-795). */
int clef_pass_maps_build(const clef_chunk_spec* chunks, size_t n_chunks, size_t capacity, int check_geometry,
                         size_t slots, size_t max_chunk, clef_pass_maps* maps);

/* The pass geometries (src/gpu.rs:779-795) for `slots` and `max_chunk`; writes up to `cap` ascending
 * row counts to `out` and returns how many there are (negative on error). */
int clef_pass_geometries(size_t slots, size_t max_chunk, size_t* out, size_t cap);

/* Rungs::decompose (src/gpu.rs:762-775) on the body ladder: cuts `tokens` into (base, rows) chunks,
 * largest rung first; returns the number of chunks written (at most `cap`). */
int clef_rungs_decompose(size_t tokens, size_t slots, size_t max_chunk, size_t* bases, size_t* rows, size_t cap);

/* Row-range split of one pass over `n_shards` GPUs: contiguous ranges aligned to the scale atom
 * (blk_mn rows) so every shard's NVFP4 outputs are a contiguous slice of the single-GPU outputs.
 * Shard g gets atoms [g * ceil(A / n), (g + 1) * ceil(A / n)), A = ceil(rows / blk_mn). */
int clef_shard_rows(int rows, int blk_mn, int n_shards, int shard, int* first_row, int* n_rows);

#ifdef __cplusplus
}
#endif

#endif /* CLEF_HOST_H */
