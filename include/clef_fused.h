/* clef_fused.h -- C ABI of the B200 (sm_100a) fused per-layer elementwise kernels.
 *
 * Drop-in boundary: each entry point replaces one launcher of aiis-clef's CUDA launch layer
 * (`impl Device` in src/cuda/mod.rs) together with the kernel it launches (kernels/elementwise.cu,
 * kernels/quantise.cu, the conversion / add kernels of attention_mma.cu and head.cu, and the prep kernels
 * of gdn_chunk.cu). The argument
 * order after `stream` is the reference KERNEL's positional parameter list, so a binding only has to pass
 * what it already passes to `launch_builder().arg(..)`.
 *
 * Groups, in the order of this file: layout helpers; the fused path (embedding gather, RMSNorm, gated
 * RMSNorm, SwiGLU, RoPE, each with its NVFP4 quantiser); the steps either side of it in a layer
 * (KV-cache write, sigmoid_mul, residual add, alone and fused); the FP8 (E4M3) quantisers; the
 * elementwise kernels in front of the Gated-DeltaNet scan (kernels/elementwise.cu, and the two prep
 * kernels of kernels/gdn_chunk.cu); process-wide settings. A few entry points
 * fuse several reference launches into one and say so ("one launch", "one pass"); their results equal
 * the reference's chain of kernels byte for byte.
 *
 * Contract of every launch function:
 *   - asynchronous on `stream` (a CUstream / cudaStream_t); no allocation, no synchronisation, no
 *     host<->device copy, so it may be called while the stream is being captured into a CUDA graph;
 *     grid sizes depend only on the shape arguments, never on buffer contents;
 *   - the caller owns every buffer; inputs are never written; outputs are fully written, including
 *     the padding rows of NVFP4 outputs (zero codes, zero scales), so no memset is needed first;
 *   - optional per-token maps are passed as NULL when absent (the reference passes a raw 0);
 *   - returns CLEF_OK, CLEF_DECLINED (shape not served by this entry point: the reference's
 *     `Ok(None)`, caller runs its unfused chain) or a negative error; nothing is launched unless
 *     the return value is CLEF_OK; clef_last_error() gives a message for the calling thread.
 *
 * Activations are bf16 (CLEF_BF16) or f32 (CLEF_F32, the reference engine's residual-stream type);
 * norm weights and RoPE tables are f32 in both cases, ids and maps are int32.
 *
 * NVFP4 output of a [rows x cols] matrix (kernels/quantise.cu:22-52, kernels/nvfp4_quant.h):
 *   packed: rows_padded * cols/2 bytes, E2M1 codes, low nibble = even column;
 *   scales: rows_padded * cols/16 bytes, E4M3, at
 *           ((row / blk_mn) * (cols/64) + block/4) * chunk + (row % blk_mn) * 4 + block % 4;
 *   rows_padded = rows rounded up to blk_mn; (blk_mn, chunk) come from clef_sf_atom_for_tile_m.
 *   global_scale is the checkpoint's per-projection input_global_scale, passed by value.
 */
#ifndef CLEF_FUSED_H
#define CLEF_FUSED_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* clef_stream_t; /* CUstream / cudaStream_t; NULL is the legacy default stream */

enum clef_dtype { CLEF_BF16 = 0, CLEF_F32 = 1 };

enum clef_status {
    CLEF_OK = 0,
    CLEF_DECLINED = 1,          /* shape outside this entry point: fall back to the unfused chain */
    CLEF_ERR_INVALID = -1,      /* null pointer, bad size, bad alignment, bad dtype */
    CLEF_ERR_CUDA = -2,         /* a CUDA runtime call failed (launch error, no sm_100 device...) */
    CLEF_ERR_TOO_LARGE = -3     /* a size beyond a stated maximum */
};

/* Message describing the last non-OK status returned on this thread ("" if none). */
const char* clef_last_error(void);

/* Library version as major*10000 + minor*100 + patch. */
int clef_version(void);

/* src/swizzle.rs:16-30 (blk_mn_for_tile_m, sf_chunk_stride_for_tile_m): the row atom and the tile
 * stride of the scale layout for a GEMM M-tile. tile_m < 128 -> (128, 512); 128 -> (128, 512);
 * 192 -> (96, 384). */
int clef_sf_atom_for_tile_m(int tile_m, int* blk_mn, int* chunk);

/* Output sizes of an NVFP4 quantisation (src/cuda/mod.rs:2183-2187): rows_padded, packed bytes,
 * scale bytes. Any out pointer may be NULL. */
int clef_nvfp4_sizes(int rows, int cols, int blk_mn, int* rows_padded, size_t* packed_bytes, size_t* scale_bytes);

/* embed_gather_kernel (kernels/elementwise.cu:396-407), Device::embed_gather_dev
 * (src/cuda/mod.rs:2908-2928): out[t, :] = table[ids[t], :]. ids must be valid row numbers. */
int clef_embed_gather(clef_stream_t stream, const void* table, const int32_t* ids, void* out, int tokens, int hidden,
                      int dtype);

/* rms_norm_kernel (kernels/elementwise.cu:4-68), Device::rms_norm_dev (src/cuda/mod.rs:2718-2739):
 * out = x * rsqrt(mean(x^2) + eps) * (1 + weight); weight may be NULL (no scaling). cols % 4 == 0. */
int clef_rms_norm(clef_stream_t stream, const void* x, const float* weight, void* out, int rows, int cols, float eps,
                  int dtype);

/* rms_norm_gated_kernel (kernels/elementwise.cu:144-223), Device::rms_norm_gated_dev
 * (src/cuda/mod.rs:2741-2763): out = x * rsqrt(mean(x^2) + eps) * weight * silu(gate); plain weight
 * (no +1); weight and gate may each be NULL (weight skipped; gate = 0). cols % 4 == 0. */
int clef_rms_norm_gated(clef_stream_t stream, const void* x, const void* gate, const float* weight, void* out,
                        int rows, int cols, float eps, int dtype);

/* swiglu_kernel (kernels/elementwise.cu:225-241), Device::swiglu_dev (src/cuda/mod.rs:2765-2782):
 * out[i] = silu(gate[i]) * up[i], i < total. */
int clef_swiglu(clef_stream_t stream, const void* gate, const void* up, void* out, size_t total, int dtype);

/* rope_kernel (kernels/elementwise.cu:276-315), Device::rope_apply_dev (src/cuda/mod.rs:3045-3074):
 * x, out [rows, heads, head_dim]; the first rotary_dim dims of each head are rotated in pairs
 * (j, j + rotary_dim/2) by cos/sin[pos * rotary_dim + j]; the rest are copied.
 * pos = pos_map ? pos_map[row] : (seq_start ? row - seq_start[row] : row) + (pos_base ? *pos_base : 0).
 * The engine passes its per-token `rope_pos` / `cpos` map as pos_map. out must not alias x. */
int clef_rope(clef_stream_t stream, void* out, const void* x, const float* cos_table, const float* sin_table,
              int rows, int heads, int head_dim, int rotary_dim, const int32_t* seq_start, const int32_t* pos_base,
              const int32_t* pos_map, int dtype);

/* qk_norm_rope_kernel (kernels/elementwise.cu:70-142), Device::qk_norm_rope_dev
 * (src/cuda/mod.rs:3008-3043): per-head RMSNorm with (1 + weight), then RoPE as above.
 * rows counts head rows (tokens * heads). With gate_out != NULL the input rows are [q | gate]
 * (2 * head_dim wide) and the gate half is copied to gate_out. The reference serves head_dim 256
 * only; this entry point serves any head_dim % 4 == 0 with the arithmetic of the unfused chain
 * (rms_norm_kernel per head row, then rope_kernel). */
int clef_qk_norm_rope(clef_stream_t stream, const void* x, const float* weight, const float* cos_table,
                      const float* sin_table, void* out, void* gate_out, int rows, int heads, int head_dim,
                      int rotary_dim, float eps, const int32_t* seq_start, const int32_t* pos_base,
                      const int32_t* pos_map, int dtype);

/* rope_tables_kernel (kernels/elementwise.cu:446-462), Device::rope_tables_dev
 * (src/cuda/mod.rs:2983-3005): cos/sin [rows, rotary_dim] f32 of positions[row] / theta^(2i/rotary_dim). */
int clef_rope_tables(clef_stream_t stream, const int32_t* positions, float* cos_out, float* sin_out, int rows,
                     int rotary_dim, float theta);

/* quantise_nvfp4_kernel (kernels/quantise.cu:6-53), Device::quantise_nvfp4_dev
 * (src/cuda/mod.rs:2169-2207). cols % 64 == 0. */
int clef_quantise_nvfp4(clef_stream_t stream, const void* x, uint8_t* packed, uint8_t* scales, int rows, int cols,
                        float global_scale, int blk_mn, int chunk, int dtype);

/* rms_norm_quantise_nvfp4_kernel (kernels/quantise.cu:193-271), Device::rms_norm_quantise_nvfp4_dev
 * (src/cuda/mod.rs:2133-2167): clef_rms_norm followed by clef_quantise_nvfp4 without the f32 round
 * trip, byte-identical to that chain. The reference declines cols != 4096; this serves cols % 64 == 0. */
int clef_rms_norm_quantise_nvfp4(clef_stream_t stream, const void* x, const float* weight, uint8_t* packed,
                                 uint8_t* scales, int rows, int cols, float eps, float global_scale, int blk_mn,
                                 int chunk, int dtype);

/* rms_norm_gated_quantise_nvfp4_kernel (kernels/quantise.cu:57-121),
 * Device::rms_norm_gated_quantise_nvfp4_dev (src/cuda/mod.rs:2269-2302). As in the reference kernel,
 * `rows` counts head rows INCLUDING padding (tokens_padded * vh, tokens_padded a multiple of
 * blk_mn), `rows_live` the head rows that hold data; `cols` is the head width; a token's vh head
 * rows form one quantised row of width vh * cols. packed: rows * cols/2 bytes; scales:
 * (rows / vh) * (vh * cols / 16) bytes. (vh * cols) % 64 == 0, cols % 16 == 0. */
int clef_rms_norm_gated_quantise_nvfp4(clef_stream_t stream, const void* x, const void* gate, const float* weight,
                                       uint8_t* packed, uint8_t* scales, int rows, int cols, float eps,
                                       float global_scale, int blk_mn, int chunk, int vh, int rows_live, int dtype);

/* swiglu_quantise_nvfp4_kernel (kernels/quantise.cu:523-591), Device::swiglu_quantise_nvfp4_dev
 * (src/cuda/mod.rs:2359-2400): clef_swiglu followed by clef_quantise_nvfp4, byte-identical to that
 * chain. gate and up are two dense [rows, cols] matrices. cols % 64 == 0. */
int clef_swiglu_quantise_nvfp4(clef_stream_t stream, const void* gate, const void* up, uint8_t* packed,
                               uint8_t* scales, int rows, int cols, float global_scale, int blk_mn, int chunk,
                               int dtype);

/* ------------------------------------------------------------------------------------------------
 * The steps either side of the fused quantisers in a layer.
 * ------------------------------------------------------------------------------------------------ */

/* to_bf16_kernel (kernels/attention_mma.cu:118-146), launched by Device::attention_dev for q and, without
 * a position map, for k and v (src/cuda/mod.rs:3201-3227): out[off + i] = bf16(x[i]), i < n,
 * off = *off_tokens_dev * off_stride (0 when the pointer is NULL). Round to nearest even. With
 * CLEF_BF16 input this is a copy to the offset. out is always bf16. */
int clef_to_bf16(clef_stream_t stream, void* out, const void* x, size_t n, const int32_t* off_tokens_dev,
                 int off_stride, int dtype);

/* to_bf16_scatter_kernel (kernels/attention_mma.cu:148-171; KvCache::pos_map, src/cuda/mod.rs:5344-5354,
 * the engine's `cpos`, src/gpu.rs:1157): token t = i / stride is written at row pos_map[t] of the cache:
 * out[pos_map[t] * stride + c] = bf16(x[t * stride + c]). stride % 8 == 0, n % stride == 0. */
int clef_to_bf16_scatter(clef_stream_t stream, void* out, const void* x, size_t n, const int32_t* pos_map,
                         int stride, int dtype);

/* The key/value side of Device::attention_dev's prologue in one launch: rope_kernel on k
 * (as clef_rope, same position arguments) followed by the bf16 cache write of k and v
 * (src/cuda/mod.rs:3201-3227). k, v: [tokens, kv_heads, head_dim]; cache_k, cache_v: bf16 caches with
 * rows of kv_heads * head_dim values. Token t lands at cache row cache_map[t] (to_bf16_scatter_kernel),
 * or, with cache_map NULL, at t + *cache_len (to_bf16_kernel; cache_len NULL means 0). Bytes equal
 * clef_rope into an f32 buffer followed by clef_to_bf16(_scatter). No counterpart as ONE kernel in the
 * reference. */
int clef_rope_kv_write(clef_stream_t stream, void* cache_k, void* cache_v, const void* k, const void* v,
                       const float* cos_table, const float* sin_table, int tokens, int kv_heads, int head_dim,
                       int rotary_dim, const int32_t* seq_start, const int32_t* pos_base, const int32_t* pos_map,
                       const int32_t* cache_map, const int32_t* cache_len, int dtype);

/* The two rope_kernel launches of a layer (q, then k, same positions: src/gpu.rs:1722-1725) as one launch.
 * q [rows, q_heads, head_dim] -> q_out, k [rows, kv_heads, head_dim] -> k_out; position arguments as clef_rope. */
int clef_rope_qk(clef_stream_t stream, void* q_out, const void* q, int q_heads, void* k_out, const void* k, int kv_heads,
                 const float* cos_table, const float* sin_table, int rows, int head_dim, int rotary_dim,
                 const int32_t* seq_start, const int32_t* pos_base, const int32_t* pos_map, int dtype);

/* clef_rope on q plus clef_rope_kv_write on k and v in one launch: the whole RoPE + KV-cache prologue of an attention
 * layer (two rope_kernel launches and the k / v conversion launches of the reference). q_out has the activation dtype,
 * the caches are bf16. */
int clef_rope_qkv_write(clef_stream_t stream, void* q_out, const void* q, int q_heads, void* cache_k, void* cache_v,
                        const void* k, const void* v, int kv_heads, const float* cos_table, const float* sin_table,
                        int tokens, int head_dim, int rotary_dim, const int32_t* seq_start, const int32_t* pos_base,
                        const int32_t* pos_map, const int32_t* cache_map, const int32_t* cache_len, int dtype);

/* As clef_rope_kv_write with the per-head RMSNorm of qk_norm_rope_kernel in front of the rotation
 * (the k call of src/gpu.rs:1711-1713): k_raw -> norm with (1 + weight) -> RoPE -> bf16 -> cache. */
int clef_qk_norm_rope_kv_write(clef_stream_t stream, void* cache_k, void* cache_v, const void* k_raw, const void* v,
                               const float* weight, const float* cos_table, const float* sin_table, int tokens,
                               int kv_heads, int head_dim, int rotary_dim, float eps, const int32_t* seq_start,
                               const int32_t* pos_base, const int32_t* pos_map, const int32_t* cache_map,
                               const int32_t* cache_len, int dtype);

/* sigmoid_mul_kernel (kernels/elementwise.cu:344-359), Device::sigmoid_mul_dev (src/cuda/mod.rs:2838-2856):
 * out[i] = x[i] * sigmoid(gate[i]) in the reference's two forms (x * 1 / (1 + __expf(-g)) for whole
 * quads, x * (1 / (1 + __expf(-g))) for the total % 4 tail). */
int clef_sigmoid_mul(clef_stream_t stream, void* out, const void* x, const void* gate, size_t total, int dtype);

/* sigmoid_mul_kernel followed by quantise_nvfp4_kernel without the round trip: the gated attention output
 * as the NVFP4 operand of o_proj (src/gpu.rs:1750-1753 with run_projection_dev's quantiser). x and gate
 * are dense [rows, cols]; bytes equal clef_sigmoid_mul (f32) followed by clef_quantise_nvfp4.
 * cols % 64 == 0. No counterpart as ONE kernel in the reference. */
int clef_sigmoid_mul_quantise_nvfp4(clef_stream_t stream, const void* x, const void* gate, uint8_t* packed,
                                    uint8_t* scales, int rows, int cols, float global_scale, int blk_mn, int chunk,
                                    int dtype);

/* copy_kernel, copy_u8_kernel, copy_range_u8_kernel (kernels/elementwise.cu:317-342), Device::copy_into,
 * Device::copy_bytes, Device::copy_bytes_at (src/cuda/mod.rs:4642-4720): `bytes` bytes from src + src_offset to
 * dst + dst_offset, device to device, inside the pass's graph. Any alignment; the ranges must not overlap
 * (copy_into of `values` f32 values is bytes = 4 * values). */
int clef_copy_bytes(clef_stream_t stream, void* dst, size_t dst_offset, const void* src, size_t src_offset, size_t bytes);

/* add_kernel (kernels/head.cu:117-129), Device::add_dev (src/cuda/mod.rs:1686-1704): out = a + b.
 * out may be a or b. */
int clef_add(clef_stream_t stream, void* out, const void* a, const void* b, size_t total, int dtype);

/* The residual add and the next layer's norm + quantiser in one pass over the row: sum = a + b is
 * written to sum_out (which may be a) in the activation dtype, and rms_norm_quantise_nvfp4 of that stored
 * sum to packed/scales. Bytes equal clef_add followed by clef_rms_norm_quantise_nvfp4 on sum_out.
 * No counterpart as ONE kernel in the reference. */
int clef_add_rms_norm_quantise_nvfp4(clef_stream_t stream, void* sum_out, const void* a, const void* b,
                                     const float* weight, uint8_t* packed, uint8_t* scales, int rows, int cols,
                                     float eps, float global_scale, int blk_mn, int chunk, int dtype);

/* The first layer's token-embedding gather and its norm + quantiser in one pass over the gathered row
 * (embed_dev followed by fused_norm_quantise_nvfp4, src/gpu.rs:1792-1798 and :461-474): row t of the table row
 * ids[t] is copied to h_out[t] (the residual stream) and rms_norm_quantise_nvfp4 of it goes to packed/scales.
 * Bytes equal clef_embed_gather followed by clef_rms_norm_quantise_nvfp4 on h_out. One kernel for bf16 and
 * hidden 2048 or 4096 (9H/2 + 9H/16 + 4 bytes per row instead of 13H/2 + 9H/16 + 4); other shapes run the two
 * entry points. No counterpart as ONE kernel in the reference. */
int clef_embed_rms_norm_quantise_nvfp4(clef_stream_t stream, const void* table, const int32_t* ids, void* h_out,
                                       const float* weight, uint8_t* packed, uint8_t* scales, int tokens, int hidden,
                                       float eps, float global_scale, int blk_mn, int chunk, int dtype);

/* ------------------------------------------------------------------------------------------------
 * FP8 (E4M3) activation quantisers, for the FP8 projections of a mixed NVFP4 + FP8 checkpoint.
 * Per quantised row: scale = amax / 448, stored as the upper 16 bits of that f32 (one uint16 per row);
 * code = e4m3(|v| / scale) with the sign bit, one byte per value, dense [rows, cols]. cols % 8 == 0,
 * cols <= 16384.
 * ------------------------------------------------------------------------------------------------ */

/* quantise_fp8_kernel (kernels/quantise.cu:454-514), Device::quantise_fp8_dev (src/cuda/mod.rs:2246-2266).
 * Every row is quantised from its own values; the reference kernel reads row blockIdx.x for all rows of
 * a block, which is the same thing only when a row has a CTA to itself (cols > 1792). */
int clef_quantise_fp8(clef_stream_t stream, const void* x, uint8_t* out, uint16_t* scales, int rows, int cols,
                      int dtype);

/* swiglu_quantise_fp8_kernel (kernels/quantise.cu:390-452), Device::swiglu_quantise_fp8_dev
 * (src/cuda/mod.rs:2402-2427): clef_swiglu followed by clef_quantise_fp8. The reference declines
 * cols > 12288. */
int clef_swiglu_quantise_fp8(clef_stream_t stream, const void* gate, const void* up, uint8_t* out, uint16_t* scales,
                             int rows, int cols, int dtype);

/* rms_norm_fp8_bf16_kernel (kernels/quantise.cu:273-381), Device::rms_norm_fp8_bf16_dev
 * (src/cuda/mod.rs:2330-2358): one pass gives the FP8 codes and row scales of the normalised row AND its
 * bf16 copy (bf_out, [rows, cols]; may be NULL). Equals clef_rms_norm -> clef_quantise_fp8 / clef_to_bf16.
 * The reference declines cols != 4096. */
int clef_rms_norm_fp8_bf16(clef_stream_t stream, const void* x, const float* weight, uint8_t* q_out,
                           uint16_t* q_scales, uint16_t* bf_out, int rows, int cols, float eps, int dtype);

/* rms_norm_gated_quantise_fp8_kernel (kernels/quantise.cu:123-191), Device::rms_norm_gated_quantise_fp8_dev
 * (src/cuda/mod.rs:2304-2328): `rows` head rows of width `cols` (vh per token, rows % vh == 0), one scale
 * per TOKEN (rows / vh of them); head rows >= rows_live hold no data and are not written. The reference
 * serves cols == 128 and vh <= 32; here cols <= 256, vh <= 64. */
int clef_rms_norm_gated_quantise_fp8(clef_stream_t stream, const void* x, const void* gate, const float* weight,
                                     uint8_t* out, uint16_t* scales, int rows, int cols, float eps, int vh,
                                     int rows_live, int dtype);

/* ------------------------------------------------------------------------------------------------
 * Elementwise kernels in front of the Gated-DeltaNet scan.
 * ------------------------------------------------------------------------------------------------ */

/* causal_conv_silu_kernel (kernels/elementwise.cu:243-274), Device::causal_conv_silu_dev
 * (src/cuda/mod.rs:2784-2812): depthwise causal convolution over the token axis with k taps, then silu.
 * x, out [rows, channels]; w [channels, k] f32. seq_start[t] (optional) is the first row of token t's sequence:
 * taps before it come from history [slots, k - 1, channels] of slot slot_map[t] (slot 0 without a map) when
 * history is given, and are skipped otherwise. out must not alias x. */
int clef_causal_conv_silu(clef_stream_t stream, void* out, const void* x, const float* w, int rows, int channels, int k,
                          const int32_t* seq_start, const void* history, const int32_t* slot_map, int dtype);

/* conv_hist_save_kernel (kernels/elementwise.cu:463-485), Device::conv_hist_save_dev (src/cuda/mod.rs:2814-2836):
 * for each pair saves[2 i] = row, saves[2 i + 1] = slot (the pass maps' hist_save), rows row - (k - 2) .. row of src
 * become the history of the slot. Pairs with a row outside [k - 2, rows) are ignored, as in the reference. */
int clef_conv_hist_save(clef_stream_t stream, void* hist, const void* src, const int32_t* saves, int n_saves, int rows,
                        int k, int channels, int dtype);

/* gdn_prep_kernel (kernels/gdn_chunk.cu:1176-1239), Device::gdn_prep_dev (src/cuda/mod.rs:3606-3647): the convolved
 * row [q (kh x kd) | k (kh x kd) | v (heads x kd)] of each of seq_len tokens (row stride conv_dim) becomes the chunked
 * scan's operands: q and k heads L2-normalised (q times q_scale), each value split into a bf16 pair hi + lo and stored
 * in the scan's swizzled layout, heads * ceil(seq_len / 64) * 2 * 64 * 128 bytes per buffer, k heads repeated
 * heads / kh times; kn = normalised k as f32 [seq_len, heads, kd]; v_out = v as f32 [seq_len, heads * kd]. kd must be
 * 128. Rows of the last chunk past seq_len are written as zeros (the reference allocates the buffers zeroed). */
int clef_gdn_prep(clef_stream_t stream, const void* mixed, float* v_out, void* q_hi, void* q_lo, void* k_hi, void* k_lo,
                  float* kn, int seq_len, int heads, int kh, int kd, int conv_dim, float q_scale, int dtype);

/* gdn_conv_prep_kernel (kernels/gdn_chunk.cu:1008-1172), Device::gdn_conv_prep_dev (src/cuda/mod.rs:3649-3707):
 * clef_causal_conv_silu followed by clef_gdn_prep in one launch, the convolved rows staying in f32 in between (as
 * in the reference). x [rows, channels] with channels = 2 kh kd + heads kd, w [channels, k] f32; the maps as for
 * clef_causal_conv_silu; outputs as for clef_gdn_prep. Returns CLEF_DECLINED (run the two calls) for a tap count
 * other than 4, for heads / kh other than 1, 2 or 4, and under clef_set_kernel_choice(1). */
int clef_gdn_conv_prep(clef_stream_t stream, const void* x, const float* w, float* v_out, void* q_hi, void* q_lo, void* k_hi,
                       void* k_lo, float* kn, int rows, int channels, int k, const int32_t* seq_start, const void* history,
                       const int32_t* slot_map, int heads, int kh, int kd, float q_scale, int dtype);

/* gdn_gates_kernel (kernels/elementwise.cu:361-377), Device::gdn_gates_dev (src/cuda/mod.rs:2858-2882):
 * beta = sigmoid(b), decay = -exp(a_log[h]) * softplus(a + dt_bias[h]) for a, b [tokens, heads]; outputs are f32. */
int clef_gdn_gates(clef_stream_t stream, const void* a, const void* b, const float* a_log, const float* dt_bias,
                   float* decay, float* beta, int tokens, int heads, int dtype);

/* split_q_gate_kernel (kernels/elementwise.cu:378-395), Device::split_q_gate_dev (src/cuda/mod.rs:2884-2906):
 * qg [tokens, heads, 2 * head_dim] -> q and gate [tokens, heads, head_dim]. */
int clef_split_q_gate(clef_stream_t stream, const void* qg, void* q, void* gate, int tokens, int heads, int head_dim,
                      int dtype);

/* split_qkv_kernel (kernels/elementwise.cu:409-427), Device::split_qkv_dev (src/cuda/mod.rs:2930-2958):
 * mixed [tokens, 2 kh kd + vh vd] -> q, k [tokens, kh kd] and v [tokens, vh vd]. */
int clef_split_qkv(clef_stream_t stream, const void* mixed, void* q, void* k, void* v, int tokens, int kh, int kd, int vh,
                   int vd, int dtype);

/* repeat_interleave_kernel (kernels/elementwise.cu:429-445), Device::repeat_interleave_dev
 * (src/cuda/mod.rs:2959-2982): out[t, h * ratio + r, :] = src[t, h, :] for r < ratio. */
int clef_repeat_interleave(clef_stream_t stream, const void* src, void* out, int tokens, int kh, int ratio, int dim,
                           int dtype);

/* Order of the rows inside a [blk_mn rows x 4 blocks] scale tile:
 *   CLEF_SF_ACTIVATION   row r at byte 4 r: the reference's activation-side ("conflict-free") order,
 *                        kernels/quantise.cu:34-41, src/swizzle.rs:64-65. Default.
 *   CLEF_SF_INTERLEAVED  row r at byte 4 ((r % 32) * (blk_mn / 32) + r / 32): the 32 x 4 x 4 order of
 *                        src/swizzle.rs:66-68 that block-scaled tensor-core GEMMs (tcgen05) read directly.
 *                        Needs blk_mn % 32 == 0 (refused otherwise).
 * The order is a property of the GEMM that consumes the operands. clef_set_scale_layout sets the PROCESS-WIDE
 * default that the NVFP4 entry points above use; it is read when a call is made, so it is baked into a CUDA graph
 * at capture time, and it is shared by every thread. A caller with two consumers (a mixed checkpoint, two
 * threads) passes the order per call instead: every NVFP4 entry point has an `_ex` form with one more argument,
 * `sf_layout` = CLEF_SF_ACTIVATION, CLEF_SF_INTERLEAVED or CLEF_SF_DEFAULT (the process default), as the
 * reference passes `conflict_free` per call (src/swizzle.rs:64-69). */
#define CLEF_SF_DEFAULT (-1)
#define CLEF_SF_ACTIVATION 0
#define CLEF_SF_INTERLEAVED 1
int clef_set_scale_layout(int layout);
int clef_quantise_nvfp4_ex(clef_stream_t stream, const void* x, uint8_t* packed, uint8_t* scales, int rows, int cols,
                           float global_scale, int blk_mn, int chunk, int dtype, int sf_layout);
int clef_rms_norm_quantise_nvfp4_ex(clef_stream_t stream, const void* x, const float* weight, uint8_t* packed,
                                    uint8_t* scales, int rows, int cols, float eps, float global_scale, int blk_mn,
                                    int chunk, int dtype, int sf_layout);
int clef_rms_norm_gated_quantise_nvfp4_ex(clef_stream_t stream, const void* x, const void* gate, const float* weight,
                                          uint8_t* packed, uint8_t* scales, int rows, int cols, float eps,
                                          float global_scale, int blk_mn, int chunk, int vh, int rows_live, int dtype,
                                          int sf_layout);
int clef_swiglu_quantise_nvfp4_ex(clef_stream_t stream, const void* gate, const void* up, uint8_t* packed,
                                  uint8_t* scales, int rows, int cols, float global_scale, int blk_mn, int chunk,
                                  int dtype, int sf_layout);
int clef_sigmoid_mul_quantise_nvfp4_ex(clef_stream_t stream, const void* x, const void* gate, uint8_t* packed,
                                       uint8_t* scales, int rows, int cols, float global_scale, int blk_mn, int chunk,
                                       int dtype, int sf_layout);
int clef_add_rms_norm_quantise_nvfp4_ex(clef_stream_t stream, void* sum_out, const void* a, const void* b,
                                        const float* weight, uint8_t* packed, uint8_t* scales, int rows, int cols,
                                        float eps, float global_scale, int blk_mn, int chunk, int dtype, int sf_layout);
int clef_embed_rms_norm_quantise_nvfp4_ex(clef_stream_t stream, const void* table, const int32_t* ids, void* h_out,
                                          const float* weight, uint8_t* packed, uint8_t* scales, int tokens, int hidden,
                                          float eps, float global_scale, int blk_mn, int chunk, int dtype, int sf_layout);

/* Kernel selection: 0 = automatic (tuned kernel when the shape has one; default), 1 = always the shape-general
 * kernel (tests, measurements). Process-wide; not part of the reference interface. */
void clef_set_kernel_choice(int choice);

#ifdef __cplusplus
}
#endif

#endif /* CLEF_FUSED_H */
