// Tuned sm_100a kernels for bf16 activations at the shapes the fused layer runs at.
//
// Common shape of every kernel here: persistent CTAs (grid = SM count x resident CTAs), each lane
// moves 32 contiguous bytes per access (256-bit ld/st, a warp covers 1 KiB), so one lane owns
// one whole 16-value NVFP4 block; row reductions are warp shuffles arranged to reproduce the
// reference's summation tree; nothing is staged through global scratch memory.
#pragma once

#include "common.cuh"
#include "nvfp4_codec.cuh"

namespace clef {

// Unpack a 32-byte chunk of 16 bf16 values to f32.
__device__ __forceinline__ void unpack16(const U8x32& d, float* v) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        v[2 * i] = bf16_lo(d.w[i]);
        v[2 * i + 1] = bf16_hi(d.w[i]);
    }
}

// ---------------------------------------------------------------------------------------------
// RMSNorm + NVFP4 quantiser, cols = NB * 512 (NB = 4: 2048, NB = 8: 4096), one warp per row.
//
// Reference association (kernels/quantise.cu:207-237 with 256 threads, equal to
// kernels/elementwise.cu:22-52 for cols >= 1793): reference thread `sub` adds quads sub, sub+256, ..;
// warps of 32 consecutive `sub` join by the 16,8,4,2,1 tree; the 8 warp sums join by the 4,2,1 tree.
// Here lane L holds chunks c = L + 32 j (j < NB), i.e. quads 4c + k (k < 4), so
//   sub            = k + 4 L + 128 (j & 1)        reference lane = k + 4 (L & 7)
//   reference warp = (L >> 3) + 4 (j & 1)
// and the same tree is: in-lane over j (stride 2, ascending), shuffles over L bits 2,1,0, in-lane
// over k (k^2 then k^1), in-lane over j & 1, shuffles over L bit 4 then L bit 3.
// ---------------------------------------------------------------------------------------------
template <int NB>
__device__ __forceinline__ float row_sum_squares_256(const U8x32* d) {
    float p[2][4];
#pragma unroll
    for (int j0 = 0; j0 < 2; ++j0) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float acc = 0.0f;
#pragma unroll
            for (int j = j0; j < NB; j += 2) {
                const uint32_t a = d[j].w[2 * k], b = d[j].w[2 * k + 1];
                acc = __fadd_rn(acc, quad_sq(make_float4(bf16_lo(a), bf16_hi(a), bf16_lo(b), bf16_hi(b))));
            }
            p[j0][k] = acc;
        }
    }
#pragma unroll
    for (int off = 4; off > 0; off >>= 1) {
#pragma unroll
        for (int j0 = 0; j0 < 2; ++j0) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                p[j0][k] = __fadd_rn(p[j0][k], __shfl_xor_sync(kFullMask, p[j0][k], off));
            }
        }
    }
    float w[2];
#pragma unroll
    for (int j0 = 0; j0 < 2; ++j0) {
        w[j0] = __fadd_rn(__fadd_rn(p[j0][0], p[j0][2]), __fadd_rn(p[j0][1], p[j0][3]));
    }
    float t = __fadd_rn(w[0], w[1]);
    t = __fadd_rn(t, __shfl_xor_sync(kFullMask, t, 16));
    t = __fadd_rn(t, __shfl_xor_sync(kFullMask, t, 8));
    return t;
}

template <int NB>
__global__ void __launch_bounds__(kCtaThreads)
rms_norm_quant_hot_kernel(const uint16_t* __restrict__ x, const float* __restrict__ weight,
                          uint8_t* __restrict__ packed, uint8_t* __restrict__ scales, int rows, int rows_total,
                          float eps, float global_scale, int blk_mn, int chunk) {
    constexpr int COLS = NB * 512;
    constexpr int BLOCKS = COLS / 16;
    __shared__ float s_inv[kInvScaleTableSize];
    extern __shared__ float4 s_w[];   // (1 + w), transposed so lane L reads s_w[(4 j + q) * 32 + L]
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;

    int row = blockIdx.x * 8 + warp;
    U8x32 d[NB];
    const bool first_live = row < rows;
    if (first_live) {
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            d[j] = ldg_stream_v8(x + (size_t)row * COLS + (size_t)(lane + 32 * j) * 16);
        }
    }
    fill_inv_scale_table(s_inv, global_scale);
    for (int idx = threadIdx.x; idx < COLS / 4; idx += kCtaThreads) {
        const int l = idx & 31, q = (idx >> 5) & 3, j = idx >> 7;
        const float4 w = *reinterpret_cast<const float4*>(weight + (l + 32 * j) * 16 + 4 * q);
        s_w[idx] = make_float4(1.0f + w.x, 1.0f + w.y, 1.0f + w.z, 1.0f + w.w);
    }
    __syncthreads();

    bool loaded = first_live;
    for (; row < rows_total; row += gridDim.x * 8) {
        uint8_t* prow = packed + (size_t)row * (COLS / 2);
        if (row >= rows) {
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                const int b = lane + 32 * j;
                store_block(prow, scales, (size_t)b * 8, scale_offset(row, b, BLOCKS, blk_mn, chunk), 0u, 0u, 0u);
            }
            continue;
        }
        if (!loaded) {
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                d[j] = ldg_stream_v8(x + (size_t)row * COLS + (size_t)(lane + 32 * j) * 16);
            }
        }
        loaded = false;
        const float inv = inv_rms(row_sum_squares_256<NB>(d), COLS, eps);
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            float v[16];
            unpack16(d[j], v);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 w = s_w[(4 * j + q) * 32 + lane];
                v[4 * q + 0] = v[4 * q + 0] * inv * w.x;
                v[4 * q + 1] = v[4 * q + 1] * inv * w.y;
                v[4 * q + 2] = v[4 * q + 2] * inv * w.z;
                v[4 * q + 3] = v[4 * q + 3] * inv * w.w;
            }
            uint32_t stored, lo, hi;
            quantise16(v, global_scale, s_inv, stored, lo, hi);
            const int b = lane + 32 * j;
            store_block(prow, scales, (size_t)b * 8, scale_offset(row, b, BLOCKS, blk_mn, chunk), stored, lo, hi);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// SwiGLU + NVFP4 quantiser (kernels/quantise.cu:523-591): silu(gate) * up, one lane per block,
// UNROLL blocks in flight per lane. Rows in [rows, rows_total) are zero-filled.
// ---------------------------------------------------------------------------------------------
template <int UNROLL>
__global__ void __launch_bounds__(kCtaThreads)
swiglu_quant_hot_kernel(const uint16_t* __restrict__ gate, const uint16_t* __restrict__ up,
                        uint8_t* __restrict__ packed, uint8_t* __restrict__ scales, int rows, int rows_total,
                        int cols, float global_scale, int blk_mn, int chunk) {
    __shared__ float s_inv[kInvScaleTableSize];
    const int blocks = cols >> 4;
    const size_t live_blocks = (size_t)rows * blocks;
    const size_t total_blocks = (size_t)rows_total * blocks;
    const size_t stride = (size_t)gridDim.x * kCtaThreads;
    size_t idx0 = (size_t)blockIdx.x * kCtaThreads + threadIdx.x;

    U8x32 g[UNROLL], u[UNROLL];
#pragma unroll
    for (int k = 0; k < UNROLL; ++k) {
        const size_t idx = idx0 + k * stride;
        if (idx < live_blocks) {
            g[k] = ldg_stream_v8(gate + idx * 16);
            u[k] = ldg_stream_v8(up + idx * 16);
        }
    }
    fill_inv_scale_table(s_inv, global_scale);
    __syncthreads();

    bool loaded = true;
    for (; idx0 < total_blocks; idx0 += UNROLL * stride) {
        if (!loaded) {
#pragma unroll
            for (int k = 0; k < UNROLL; ++k) {
                const size_t idx = idx0 + k * stride;
                if (idx < live_blocks) {
                    g[k] = ldg_stream_v8(gate + idx * 16);
                    u[k] = ldg_stream_v8(up + idx * 16);
                }
            }
        }
        loaded = false;
#pragma unroll
        for (int k = 0; k < UNROLL; ++k) {
            const size_t idx = idx0 + k * stride;
            if (idx >= total_blocks) {
                break;
            }
            const int row = (int)(idx / blocks);
            const int blk = (int)(idx - (size_t)row * blocks);
            uint32_t stored = 0, lo = 0, hi = 0;
            if (idx < live_blocks) {
                float v[16], w[16];
                unpack16(g[k], v);
                unpack16(u[k], w);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    v[i] = silu_ieee_div(v[i]) * w[i];
                }
                quantise16(v, global_scale, s_inv, stored, lo, hi);
            }
            store_block(packed, scales, idx * 8, scale_offset(row, blk, blocks, blk_mn, chunk), stored, lo, hi);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Gated RMSNorm + NVFP4 quantiser for 128-wide heads (kernels/quantise.cu:57-121).
// Eight lanes own one head row (8 chunks of 16), a warp handles 4 head rows per step.
// Reference association: lane l of a warp holds quad l; tree 16,8,4,2,1 over l. Here lane m (of 8)
// holds quads 4m + k, so the tree is: shuffles over m bits 2,1,0, then in-lane k^2, k^1.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kCtaThreads)
gated_norm_quant_hot_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ gate,
                            const float* __restrict__ weight, uint8_t* __restrict__ packed,
                            uint8_t* __restrict__ scales, int rows_live, int rows_total, float eps,
                            float global_scale, int blk_mn, int chunk, int vh) {
    constexpr int COLS = 128;
    __shared__ float s_inv[kInvScaleTableSize];
    const int lane = threadIdx.x & 31;
    const int m = lane & 7;
    const int blocks = vh * (COLS / 16);

    // Head row handled by this lane group in step s: (global group index) + s * (groups in grid).
    const size_t groups_in_grid = (size_t)gridDim.x * (kCtaThreads / 8);
    size_t hrow = (size_t)blockIdx.x * (kCtaThreads / 8) + (threadIdx.x >> 3);

    U8x32 dx, dg;
    if (hrow < (size_t)rows_live) {
        dx = ldg_stream_v8(x + hrow * COLS + m * 16);
        dg = ldg_stream_v8(gate + hrow * COLS + m * 16);
    }
    float w[16];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const float4 t = *reinterpret_cast<const float4*>(weight + m * 16 + 4 * q);
        w[4 * q] = t.x;
        w[4 * q + 1] = t.y;
        w[4 * q + 2] = t.z;
        w[4 * q + 3] = t.w;
    }
    fill_inv_scale_table(s_inv, global_scale);
    __syncthreads();

    bool loaded = true;
    // Every lane of a warp runs the same number of steps (the shuffles need the full warp).
    const size_t warp_first = hrow - (size_t)((lane >> 3));
    for (size_t base = warp_first; base < (size_t)rows_total; base += groups_in_grid, hrow += groups_in_grid) {
        const bool in_range = hrow < (size_t)rows_total;
        const bool live = hrow < (size_t)rows_live;
        if (!loaded && live) {
            dx = ldg_stream_v8(x + hrow * COLS + m * 16);
            dg = ldg_stream_v8(gate + hrow * COLS + m * 16);
        }
        loaded = false;
        float v[16];
        float p[4] = {0.f, 0.f, 0.f, 0.f};
        if (live) {
            unpack16(dx, v);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                p[k] = __fadd_rn(0.0f, quad_sq(make_float4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3])));
            }
        }
#pragma unroll
        for (int off = 4; off > 0; off >>= 1) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                p[k] = __fadd_rn(p[k], __shfl_xor_sync(kFullMask, p[k], off));
            }
        }
        if (!in_range) {
            continue;
        }
        const int token = (int)(hrow / vh);
        const int head = (int)(hrow - (size_t)token * vh);
        uint32_t stored = 0, lo = 0, hi = 0;
        if (live) {
            const float total = __fadd_rn(__fadd_rn(p[0], p[2]), __fadd_rn(p[1], p[3]));
            const float inv = inv_rms(total, COLS, eps);
            float g[16];
            unpack16(dg, g);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                v[i] = v[i] * inv * w[i] * silu_fast_div(g[i]);
            }
            quantise16(v, global_scale, s_inv, stored, lo, hi);
        }
        store_block(packed, scales, hrow * (COLS / 2) + (size_t)m * 8,
                    scale_offset(token, head * (COLS / 16) + m, blocks, blk_mn, chunk), stored, lo, hi);
    }
}

// ---------------------------------------------------------------------------------------------
// Partial RoPE (kernels/elementwise.cu:276-315) for head_dim % 32 == 0, rotary_dim % 32 == 0.
// A head row is head_dim/16 chunks of 32 bytes. Work items per head row: rotary_dim/32 "rotating"
// items (chunk i of the lower half together with its partner chunk i + rotary_dim/32) followed by
// (head_dim - rotary_dim)/32 "copy" items (two pass-through chunks each); one lane per item, so
// every lane moves 64 bytes in and 64 bytes out.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kCtaThreads)
rope_hot_kernel(uint16_t* __restrict__ out, const uint16_t* __restrict__ x, const float* __restrict__ cos_t,
                const float* __restrict__ sin_t, int rows, int heads, int head_dim, int rotary_dim,
                const int* __restrict__ seq_start, const int* __restrict__ pos_base,
                const int* __restrict__ pos_map) {
    const int rot_items = rotary_dim >> 5;
    const int items = head_dim >> 5;
    const size_t total = (size_t)rows * heads * items;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const size_t head_row = idx / items;
        const int item = (int)(idx - head_row * items);
        const uint16_t* xr = x + head_row * head_dim;
        uint16_t* orow = out + head_row * head_dim;
        if (item < rot_items) {
            const int row = (int)(head_row / heads);
            const int pos = rope_position(row, seq_start, pos_base, pos_map);
            const int half = rotary_dim >> 1;
            const U8x32 dlo = ldg_stream_v8(xr + item * 16);
            const U8x32 dhi = ldg_stream_v8(xr + half + item * 16);
            const float* cp = cos_t + (size_t)pos * rotary_dim + item * 16;
            const float* sp = sin_t + (size_t)pos * rotary_dim + item * 16;
            float lo[16], hi[16];
            unpack16(dlo, lo);
            unpack16(dhi, hi);
            U8x32 olo, ohi;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 c = __ldg(reinterpret_cast<const float4*>(cp) + q);
                const float4 s = __ldg(reinterpret_cast<const float4*>(sp) + q);
                float a0, b0, a1, b1, a2, b2, a3, b3;
                rope_pair(lo[4 * q], hi[4 * q], c.x, s.x, a0, b0);
                rope_pair(lo[4 * q + 1], hi[4 * q + 1], c.y, s.y, a1, b1);
                rope_pair(lo[4 * q + 2], hi[4 * q + 2], c.z, s.z, a2, b2);
                rope_pair(lo[4 * q + 3], hi[4 * q + 3], c.w, s.w, a3, b3);
                olo.w[2 * q] = pack_bf16x2(a0, a1);
                olo.w[2 * q + 1] = pack_bf16x2(a2, a3);
                ohi.w[2 * q] = pack_bf16x2(b0, b1);
                ohi.w[2 * q + 1] = pack_bf16x2(b2, b3);
            }
            stg_v8(orow + item * 16, olo);
            stg_v8(orow + half + item * 16, ohi);
        } else {
            const int c0 = rotary_dim + (item - rot_items) * 32;
            const U8x32 a = ldg_stream_v8(xr + c0);
            const U8x32 b = ldg_stream_v8(xr + c0 + 16);
            stg_v8(orow + c0, a);
            stg_v8(orow + c0 + 16, b);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Embedding gather (kernels/elementwise.cu:396-407) for rows of a multiple of 1 KiB: one warp per
// token row, every lane moves CH chunks of 32 bytes.
// ---------------------------------------------------------------------------------------------
template <int CH>
__global__ void __launch_bounds__(kCtaThreads)
embed_gather_hot_kernel(const uint8_t* __restrict__ table, const int* __restrict__ ids, uint8_t* __restrict__ out,
                        int tokens) {
    constexpr size_t ROW_BYTES = (size_t)CH * 1024;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    for (int t = blockIdx.x * 8 + warp; t < tokens; t += gridDim.x * 8) {
        const uint8_t* src = table + (size_t)__ldg(ids + t) * ROW_BYTES;
        uint8_t* dst = out + (size_t)t * ROW_BYTES;
        U8x32 d[CH];
#pragma unroll
        for (int j = 0; j < CH; ++j) {
            d[j] = ldg_stream_v8(src + (size_t)(lane + 32 * j) * 32);
        }
#pragma unroll
        for (int j = 0; j < CH; ++j) {
            stg_v8(dst + (size_t)(lane + 32 * j) * 32, d[j]);
        }
    }
}

}  // namespace clef
