// Shape-general kernels for every entry point, for bf16 and f32 activations.
//
// These keep the reference kernels' work decomposition (which thread sums which quad, which
// tree joins the partial sums), so their f32 results equal the reference's by construction for
// every shape the entry points accept. The tuned kernels in kernels_hot.cuh cover the shapes
// the benchmark names and are checked against these and against the CPU oracle.
#pragma once

#include "common.cuh"
#include "nvfp4_codec.cuh"

namespace clef {

constexpr int kCtaThreads = 256;

// Row sum of squares in the association of kernels/elementwise.cu:22-52: thread `sub` of a team of
// `tpr` threads adds quads sub, sub+tpr, ...; each warp joins with the 16..1 tree; the team's
// warps join with the 4,2,1 tree (missing warps contribute exact zeros). `s_part` has one float
// per warp of the CTA. All threads of the CTA must call this (it synchronises the CTA).
template <typename T>
__device__ __forceinline__ float team_sum_squares(const typename T::storage* xrow, bool active, int cols, int tpr,
                                                  float* s_part) {
    const int sub = threadIdx.x % tpr;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int wpr = tpr >> 5;
    const int c4 = cols >> 2;
    float acc = 0.0f;
    if (active) {
        for (int i = sub; i < c4; i += tpr) {
            acc = __fadd_rn(acc, quad_sq(load_quad<T>(xrow, i)));
        }
    }
    acc = warp_tree_sum(acc);
    if (wpr == 1) {
        return acc;
    }
    if (lane == 0) {
        s_part[warp] = acc;
    }
    __syncthreads();
    const int first = (warp / wpr) * wpr;
    // (a CTA whose 8 warps do not divide into teams leaves a partial last team: it reads in range and its sum is unused)
    float t = (lane < wpr && first + lane < kCtaThreads / 32) ? s_part[first + lane] : 0.0f;
#pragma unroll
    for (int off = 4; off > 0; off >>= 1) {
        t = __fadd_rn(t, __shfl_xor_sync(kFullMask, t, off));
    }
    t = __shfl_sync(kFullMask, t, 0);   // lanes >= 8 summed zeros among themselves
    __syncthreads();                    // s_part is reused by the next row group
    return t;
}

// Store one quantised block: 8 packed bytes and its scale byte.
__device__ __forceinline__ void store_block(uint8_t* packed, uint8_t* scales, size_t packed_offset, size_t scale_off,
                                            uint32_t stored, uint32_t lo, uint32_t hi) {
    *reinterpret_cast<uint2*>(packed + packed_offset) = make_uint2(lo, hi);
    scales[scale_off] = (uint8_t)stored;
}

// ---------------------------------------------------------------------------------------------
// rms_norm (kernels/elementwise.cu:4-68) and rms_norm_quantise_nvfp4 (kernels/quantise.cu:193-271).
// QUANT == false: out[row] = x*inv*(1+w) (or x*inv without weight), rows < `rows`.
// QUANT == true : rows in [0, rows_padded) are written; live rows are quantised, pad rows zeroed.
// ---------------------------------------------------------------------------------------------
template <typename T, bool QUANT>
__global__ void __launch_bounds__(kCtaThreads)
rms_norm_generic_kernel(const typename T::storage* __restrict__ x, const float* __restrict__ weight,
                        typename T::storage* __restrict__ out, uint8_t* __restrict__ packed,
                        uint8_t* __restrict__ scales, int rows, int rows_total, int cols, float eps,
                        float global_scale, int blk_mn, int chunk) {
    __shared__ float s_part[kCtaThreads / 32];
    __shared__ float s_inv[kInvScaleTableSize];
    const int tpr = ref_threads_per_row(cols);
    const int rpb = kCtaThreads / tpr;
    const int team = threadIdx.x / tpr;
    const int sub = threadIdx.x % tpr;
    if (QUANT) {
        fill_inv_scale_table(s_inv, global_scale);
        __syncthreads();
    }
    const int groups = (rows_total + rpb - 1) / rpb;
    for (int group = blockIdx.x; group < groups; group += gridDim.x) {
        // Threads beyond the last whole team (tpr = 160, 192 or 224 does not divide 256) take no row. The reference
        // kernels let them run as a partial team on the NEXT block's first row, racing with that block; the intended
        // arithmetic, one team of tpr threads per row, is what is computed here.
        const bool in_team = team < rpb;
        const int row = group * rpb + team;
        const bool live = in_team && row < rows;
        const typename T::storage* xrow = x + (size_t)row * cols;
        const float total = team_sum_squares<T>(xrow, live, cols, tpr, s_part);
        if (!in_team) {
            continue;
        }
        if (!QUANT) {
            if (live) {
                const float inv = inv_rms(total, cols, eps);
                typename T::storage* orow = out + (size_t)row * cols;
                const int c4 = cols >> 2;
                for (int i = sub; i < c4; i += tpr) {
                    const float4 v = load_quad<T>(xrow, i);
                    float4 o;
                    if (weight) {
                        const float4 w = *reinterpret_cast<const float4*>(weight + 4 * i);
                        o = make_float4(v.x * inv * (1.0f + w.x), v.y * inv * (1.0f + w.y), v.z * inv * (1.0f + w.z),
                                        v.w * inv * (1.0f + w.w));
                    } else {
                        o = make_float4(v.x * inv, v.y * inv, v.z * inv, v.w * inv);
                    }
                    store_quad<T>(orow, i, o);
                }
            }
        } else if (row < rows_total) {
            const int blocks = cols >> 4;
            if (live) {
                const float inv = inv_rms(total, cols, eps);
                for (int b = sub; b < blocks; b += tpr) {
                    float v[16];
                    load_block16<T>(xrow + b * 16, v);
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float w = weight ? weight[b * 16 + i] : 0.0f;
                        v[i] = weight ? v[i] * inv * (1.0f + w) : v[i] * inv;
                    }
                    uint32_t stored, lo, hi;
                    quantise16(v, global_scale, s_inv, stored, lo, hi);
                    store_block(packed, scales, (size_t)row * (cols >> 1) + (size_t)b * 8,
                                scale_offset(row, b, blocks, blk_mn, chunk), stored, lo, hi);
                }
            } else {
                for (int b = sub; b < blocks; b += tpr) {
                    store_block(packed, scales, (size_t)row * (cols >> 1) + (size_t)b * 8,
                                scale_offset(row, b, blocks, blk_mn, chunk), 0u, 0u, 0u);
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// rms_norm_gated (kernels/elementwise.cu:144-223) and rms_norm_gated_quantise_nvfp4
// (kernels/quantise.cu:57-121): out = x*inv*w*silu(gate), plain weight, approximate divide.
// QUANT: a token's `vh` head rows of width `cols` form one quantised row of width vh*cols;
// head rows in [rows_live, rows_total) are padding (zero codes, zero scales).
// ---------------------------------------------------------------------------------------------
template <typename T, bool QUANT>
__global__ void __launch_bounds__(kCtaThreads)
rms_norm_gated_generic_kernel(const typename T::storage* __restrict__ x, const typename T::storage* __restrict__ gate,
                              const float* __restrict__ weight, typename T::storage* __restrict__ out,
                              uint8_t* __restrict__ packed, uint8_t* __restrict__ scales, int rows_live,
                              int rows_total, int cols, float eps, float global_scale, int blk_mn, int chunk, int vh) {
    __shared__ float s_part[kCtaThreads / 32];
    __shared__ float s_inv[kInvScaleTableSize];
    const int tpr = ref_threads_per_row(cols);
    const int rpb = kCtaThreads / tpr;
    const int team = threadIdx.x / tpr;
    const int sub = threadIdx.x % tpr;
    if (QUANT) {
        fill_inv_scale_table(s_inv, global_scale);
        __syncthreads();
    }
    const int groups = (rows_total + rpb - 1) / rpb;
    for (int group = blockIdx.x; group < groups; group += gridDim.x) {
        const bool in_team = team < rpb;   // see rms_norm_generic_kernel
        const int row = group * rpb + team;
        const bool live = in_team && row < rows_live;
        const typename T::storage* xrow = x + (size_t)row * cols;
        const typename T::storage* grow = gate ? gate + (size_t)row * cols : nullptr;
        const float total = team_sum_squares<T>(xrow, live, cols, tpr, s_part);
        if (!in_team) {
            continue;
        }
        if (!QUANT) {
            if (live) {
                const float inv = inv_rms(total, cols, eps);
                typename T::storage* orow = out + (size_t)row * cols;
                const int c4 = cols >> 2;
                for (int i = sub; i < c4; i += tpr) {
                    const float4 v = load_quad<T>(xrow, i);
                    const float4 g = grow ? load_quad<T>(grow, i) : make_float4(0.f, 0.f, 0.f, 0.f);
                    float4 o;
                    if (weight) {
                        const float4 w = *reinterpret_cast<const float4*>(weight + 4 * i);
                        o = make_float4(v.x * inv * w.x * silu_fast_div(g.x), v.y * inv * w.y * silu_fast_div(g.y),
                                        v.z * inv * w.z * silu_fast_div(g.z), v.w * inv * w.w * silu_fast_div(g.w));
                    } else {
                        o = make_float4(v.x * inv * silu_fast_div(g.x), v.y * inv * silu_fast_div(g.y),
                                        v.z * inv * silu_fast_div(g.z), v.w * inv * silu_fast_div(g.w));
                    }
                    store_quad<T>(orow, i, o);
                }
            }
        } else if (row < rows_total) {
            const int head_blocks = cols >> 4;
            const int blocks = vh * head_blocks;
            const int token = row / vh;
            const int head = row - token * vh;
            const float inv = live ? inv_rms(total, cols, eps) : 0.0f;
            for (int b = sub; b < head_blocks; b += tpr) {
                uint32_t stored = 0, lo = 0, hi = 0;
                if (live) {
                    float v[16], g[16];
                    load_block16<T>(xrow + b * 16, v);
                    load_block16<T>(grow + b * 16, g);
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        v[i] = v[i] * inv * weight[b * 16 + i] * silu_fast_div(g[i]);
                    }
                    quantise16(v, global_scale, s_inv, stored, lo, hi);
                }
                store_block(packed, scales, (size_t)row * (cols >> 1) + (size_t)b * 8,
                            scale_offset(token, head * head_blocks + b, blocks, blk_mn, chunk), stored, lo, hi);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// swiglu (kernels/elementwise.cu:225-241): out = (g / (1 + __expf(-g))) * u over a flat array.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kCtaThreads)
swiglu_generic_kernel(const typename T::storage* __restrict__ gate, const typename T::storage* __restrict__ up,
                      typename T::storage* __restrict__ out, size_t total) {
    const size_t quads = total >> 2;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < quads; i += stride) {
        const float4 g = load_quad<T>(gate, i);
        const float4 u = load_quad<T>(up, i);
        store_quad<T>(out, i,
                      make_float4(silu_ieee_div(g.x) * u.x, silu_ieee_div(g.y) * u.y, silu_ieee_div(g.z) * u.z,
                                  silu_ieee_div(g.w) * u.w));
    }
    if (blockIdx.x == 0 && threadIdx.x < (total & 3)) {
        const size_t k = (quads << 2) + threadIdx.x;
        float g, u;
        if (T::kBytes == 2) {
            g = __uint_as_float((uint32_t)reinterpret_cast<const uint16_t*>(gate)[k] << 16);
            u = __uint_as_float((uint32_t)reinterpret_cast<const uint16_t*>(up)[k] << 16);
            reinterpret_cast<uint16_t*>(out)[k] = (uint16_t)(pack_bf16x2(silu_ieee_div(g) * u, 0.0f) & 0xffffu);
        } else {
            g = reinterpret_cast<const float*>(gate)[k];
            u = reinterpret_cast<const float*>(up)[k];
            reinterpret_cast<float*>(out)[k] = silu_ieee_div(g) * u;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// quantise_nvfp4 (kernels/quantise.cu:6-53), swiglu_quantise_nvfp4 (kernels/quantise.cu:523-591) and
// sigmoid_mul (kernels/elementwise.cu:344-359) followed by quantise_nvfp4:
// one thread per 16-value block, rows in [0, rows_total) written, pad rows zeroed.
// ---------------------------------------------------------------------------------------------
template <typename T, int ACT>
__global__ void __launch_bounds__(kCtaThreads)
quantise_generic_kernel(const typename T::storage* __restrict__ a, const typename T::storage* __restrict__ b,
                        uint8_t* __restrict__ packed, uint8_t* __restrict__ scales, int rows, int rows_total, int cols,
                        float global_scale, int blk_mn, int chunk) {
    __shared__ float s_inv[kInvScaleTableSize];
    fill_inv_scale_table(s_inv, global_scale);
    __syncthreads();
    const int blocks = cols >> 4;
    const size_t total_blocks = (size_t)rows_total * blocks;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total_blocks; idx += stride) {
        const int row = (int)(idx / blocks);
        const int blk = (int)(idx - (size_t)row * blocks);
        uint32_t stored = 0, lo = 0, hi = 0;
        if (row < rows) {
            float v[16];
            load_block16<T>(a + (size_t)row * cols + blk * 16, v);
            if (ACT != kActNone) {   // a = gate, b = up (SwiGLU) or the gated values (sigmoid_mul)
                float u[16];
                load_block16<T>(b + (size_t)row * cols + blk * 16, u);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    v[i] = gated_literal<(ACT == kActNone ? kActSwiGLU : ACT)>(v[i], u[i]);
                }
            }
            quantise16(v, global_scale, s_inv, stored, lo, hi);
        }
        store_block(packed, scales, (size_t)row * (cols >> 1) + (size_t)blk * 8,
                    scale_offset(row, blk, blocks, blk_mn, chunk), stored, lo, hi);
    }
}

// ---------------------------------------------------------------------------------------------
// Position of a token row for RoPE (kernels/elementwise.cu:300-303).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ int rope_position(int row, const int* seq_start, const int* pos_base, const int* pos_map) {
    return pos_map ? pos_map[row] : (seq_start ? row - seq_start[row] : row) + (pos_base ? pos_base[0] : 0);
}

// rope (kernels/elementwise.cu:276-315): one thread per (row, head, 4 consecutive dims of the lower
// half of the rotary span plus their partners), or per 4 pass-through dims.
template <typename T>
__global__ void __launch_bounds__(kCtaThreads)
rope_generic_kernel(typename T::storage* __restrict__ out, const typename T::storage* __restrict__ x,
                    const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rows, int heads,
                    int head_dim, int rotary_dim, const int* __restrict__ seq_start,
                    const int* __restrict__ pos_base, const int* __restrict__ pos_map) {
    // Work items per head: half/4 rotating quads (each also owns the partner quad half dims up)
    // followed by (head_dim - rotary_dim)/4 pass-through quads.
    const int half = rotary_dim >> 1;
    const int rot_items = half >> 2;
    const int pass_items = (head_dim - rotary_dim) >> 2;
    const int items = rot_items + pass_items;
    const size_t total = (size_t)rows * heads * items;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const size_t head_row = idx / items;
        const int item = (int)(idx - head_row * items);
        const int row = (int)(head_row / heads);
        const typename T::storage* xr = x + head_row * head_dim;
        typename T::storage* orow = out + head_row * head_dim;
        if (item < rot_items) {
            const int pos = rope_position(row, seq_start, pos_base, pos_map);
            const float4 c = *reinterpret_cast<const float4*>(cos_t + (size_t)pos * rotary_dim + 4 * item);
            const float4 s = *reinterpret_cast<const float4*>(sin_t + (size_t)pos * rotary_dim + 4 * item);
            const float4 lo = load_quad<T>(xr, item);
            const float4 hi = load_quad<T>(xr + half, item);
            float4 olo, ohi;
            rope_pair(lo.x, hi.x, c.x, s.x, olo.x, ohi.x);
            rope_pair(lo.y, hi.y, c.y, s.y, olo.y, ohi.y);
            rope_pair(lo.z, hi.z, c.z, s.z, olo.z, ohi.z);
            rope_pair(lo.w, hi.w, c.w, s.w, olo.w, ohi.w);
            store_quad<T>(orow, item, olo);
            store_quad<T>(orow + half, item, ohi);
        } else {
            const int q = (rotary_dim >> 2) + (item - rot_items);
            store_quad<T>(orow, q, load_quad<T>(xr, q));
        }
    }
}

// qk_norm_rope (kernels/elementwise.cu:70-142), any head_dim: one warp per head row; the row is
// normalised with the (1 + w) weight, staged in shared memory, rotated, and written; with
// gate_out the input row is [q | gate] and the gate half is copied out.
// TO is the storage type of `out` (T itself, or Bf16 when the rows go to a KV cache); with KV the head rows of
// token t are written at cache row cache_map[t], or t + *cache_len without a map (kernels/attention_mma.cu:118-171).
template <typename T, typename TO, bool KV>
__global__ void __launch_bounds__(kCtaThreads)
qk_norm_rope_generic_kernel(const typename T::storage* __restrict__ x, const float* __restrict__ weight,
                            const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                            typename TO::storage* __restrict__ out, typename T::storage* __restrict__ gate_out,
                            int rows, int heads, int head_dim, int rotary_dim, float eps,
                            const int* __restrict__ seq_start, const int* __restrict__ pos_base,
                            const int* __restrict__ pos_map, const int* __restrict__ cache_map,
                            const int* __restrict__ cache_len) {
    extern __shared__ float s_rows[];   // 8 warps x head_dim floats
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    float* r = s_rows + (size_t)warp * head_dim;
    const int c4 = head_dim >> 2;
    const int stride = gate_out ? 2 * head_dim : head_dim;
    const int tpr = ref_threads_per_row(head_dim);   // the chain's rms_norm team; a warp emulates it below
    const int half = rotary_dim >> 1;
    for (int row = blockIdx.x * 8 + warp; row < rows; row += gridDim.x * 8) {
        const typename T::storage* xr = x + (size_t)row * stride;
        const int t = row / heads;
        // Partial sums of the tpr "reference threads", 32 at a time, then the reference trees.
        float warp_sums[8];
        const int wpr = tpr >> 5;
#pragma unroll 1
        for (int w = 0; w < wpr; ++w) {
            float acc = 0.0f;
            for (int i = w * 32 + lane; i < c4; i += tpr) {
                acc = __fadd_rn(acc, quad_sq(load_quad<T>(xr, i)));
            }
            warp_sums[w] = warp_tree_sum(acc);
        }
        float total = warp_sums[0];
        if (wpr > 1) {
            float tsum[8];
#pragma unroll
            for (int w = 0; w < 8; ++w) tsum[w] = (w < wpr) ? warp_sums[w] : 0.0f;
#pragma unroll
            for (int off = 4; off > 0; off >>= 1) {
#pragma unroll
                for (int l = 0; l < 4; ++l) {
                    if (l < off) tsum[l] = __fadd_rn(tsum[l], tsum[l + off]);
                }
            }
            total = tsum[0];
        }
        const float inv = inv_rms(total, head_dim, eps);
        for (int i = lane; i < c4; i += 32) {
            const float4 v = load_quad<T>(xr, i);
            const float4 w = *reinterpret_cast<const float4*>(weight + 4 * i);
            *reinterpret_cast<float4*>(r + 4 * i) =
                make_float4(v.x * inv * (1.0f + w.x), v.y * inv * (1.0f + w.y), v.z * inv * (1.0f + w.z),
                            v.w * inv * (1.0f + w.w));
        }
        __syncwarp();
        const int pos = rope_position(t, seq_start, pos_base, pos_map);
        for (int p = lane; p < half; p += 32) {
            const float c = cos_t[(size_t)pos * rotary_dim + p];
            const float s = sin_t[(size_t)pos * rotary_dim + p];
            float olo, ohi;
            rope_pair(r[p], r[p + half], c, s, olo, ohi);
            r[p] = olo;
            r[p + half] = ohi;
        }
        __syncwarp();
        size_t out_row = (size_t)row;
        if (KV) {
            const size_t cache_row = cache_map ? (size_t)cache_map[t] : (size_t)t + (size_t)(cache_len ? cache_len[0] : 0);
            out_row = cache_row * (size_t)heads + (size_t)(row - t * heads);
        }
        typename TO::storage* orow = out + out_row * head_dim;
        for (int i = lane; i < c4; i += 32) {
            store_quad<TO>(orow, i, *reinterpret_cast<const float4*>(r + 4 * i));
        }
        if (gate_out) {
            typename T::storage* grow = gate_out + (size_t)row * head_dim;
            for (int i = lane; i < c4; i += 32) {
                if (T::kBytes == 2) {
                    *reinterpret_cast<uint2*>(grow + 4 * i) = *reinterpret_cast<const uint2*>(xr + head_dim + 4 * i);
                } else {
                    *reinterpret_cast<float4*>(grow + 4 * i) = *reinterpret_cast<const float4*>(xr + head_dim + 4 * i);
                }
            }
        }
        __syncwarp();
    }
}

// embed_gather (kernels/elementwise.cu:396-407): out[t, :] = table[ids[t], :], 16 bytes per thread.
static __global__ void __launch_bounds__(kCtaThreads)
embed_gather_generic_kernel(const uint8_t* __restrict__ table, const int* __restrict__ ids, uint8_t* __restrict__ out,
                            int tokens, size_t row_bytes) {
    const size_t vecs_per_row = row_bytes >> 4;
    const size_t total = (size_t)tokens * vecs_per_row;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const size_t t = idx / vecs_per_row;
        const size_t v = idx - t * vecs_per_row;
        const uint4 val = ldg_stream_v4(table + (size_t)ids[t] * row_bytes + (v << 4));
        stg_v4(out + t * row_bytes + (v << 4), val);
    }
}

// rope_tables (kernels/elementwise.cu:446-462): cos/sin of pos / theta^(2i/rot), both halves alike.
static __global__ void __launch_bounds__(kCtaThreads)
rope_tables_kernel(const int* __restrict__ positions, float* __restrict__ cos_out, float* __restrict__ sin_out,
                   int rows, int rotary_dim, float theta) {
    const int half = rotary_dim / 2;
    const size_t total = (size_t)rows * rotary_dim;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int row = (int)(idx / rotary_dim);
        const int j = (int)(idx - (size_t)row * rotary_dim);
        const int i = j % half;
        const float inv_freq = 1.0f / powf(theta, 2.0f * (float)i / (float)rotary_dim);
        const float f = (float)positions[row] * inv_freq;
        cos_out[idx] = cosf(f);
        sin_out[idx] = sinf(f);
    }
}

}  // namespace clef
