// Shape-general kernels for the steps either side of the fused quantisers in a layer: the bf16
// KV-cache write (alone, and fused behind the key-side RoPE), attention-output gating
// (sigmoid_mul), the residual add. T = Bf16 or F32 is the storage type of the activations; the KV
// cache is always bf16. The tuned bf16 counterparts live in kernels_hot.cuh.
#pragma once

#include "kernels_generic.cuh"
#include "kernels_hot.cuh"

namespace clef {

// 8 consecutive values -> 16 bytes of bf16 (round to nearest even, NaN -> 0x7FFF as __float2bfloat16).
template <typename T>
__device__ __forceinline__ uint4 load8_as_bf16(const typename T::storage* p);
template <>
__device__ __forceinline__ uint4 load8_as_bf16<Bf16>(const uint16_t* p) {
    return ldg_stream_v4(p);
}
template <>
__device__ __forceinline__ uint4 load8_as_bf16<F32>(const float* p) {
    const uint4 a = ldg_stream_v4(p), b = ldg_stream_v4(p + 4);
    return make_uint4(pack_bf16x2(__uint_as_float(a.x), __uint_as_float(a.y)),
                      pack_bf16x2(__uint_as_float(a.z), __uint_as_float(a.w)),
                      pack_bf16x2(__uint_as_float(b.x), __uint_as_float(b.y)),
                      pack_bf16x2(__uint_as_float(b.z), __uint_as_float(b.w)));
}

template <typename T>
__device__ __forceinline__ uint16_t load1_as_bf16(const typename T::storage* p);
template <>
__device__ __forceinline__ uint16_t load1_as_bf16<Bf16>(const uint16_t* p) {
    return *p;
}
template <>
__device__ __forceinline__ uint16_t load1_as_bf16<F32>(const float* p) {
    return (uint16_t)(pack_bf16x2(*p, 0.0f) & 0xffffu);
}

// ---------------------------------------------------------------------------------------------
// to_bf16_kernel / to_bf16_scatter_kernel (kernels/attention_mma.cu:118-171): out[dst(t) * stride + c] =
// bf16(x[t * stride + c]) for token t, dst(t) = kv_cache_row(t). `vecs` = n / 8 vectors of 8 values;
// without a map the n % 8 tail values are converted one by one (as the reference does); the scatter
// form has no tail (stride % 8 == 0 and n % stride == 0 are required by the launcher).
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kCtaThreads)
to_bf16_rows_kernel(const typename T::storage* __restrict__ x, uint16_t* __restrict__ out, uint32_t vecs, uint32_t tail,
                    const int* __restrict__ pos_map, const int* __restrict__ off_tokens, int stride,
                    FastDiv vecs_per_token) {
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    const uint32_t step = gridDim.x * blockDim.x;
    const size_t base = pos_map ? 0 : (size_t)(off_tokens ? off_tokens[0] : 0) * (size_t)stride;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += step) {
        size_t dst = base + (size_t)i * 8;
        if (pos_map) {
            const uint32_t token = fast_div(i, vecs_per_token);
            dst = (size_t)pos_map[token] * (size_t)stride + (size_t)(i - token * vecs_per_token.d) * 8;
        }
        stg_v4(out + dst, load8_as_bf16<T>(x + (size_t)i * 8));
    }
    if (blockIdx.x == 0 && threadIdx.x < tail) {
        const size_t k = (size_t)vecs * 8 + threadIdx.x;
        out[base + k] = load1_as_bf16<T>(x + k);
    }
}

// ---------------------------------------------------------------------------------------------
// Key-side RoPE (kernels/elementwise.cu:276-315) with the bf16 cache write of
// kernels/attention_mma.cu:118-171 as its store, and the value rows converted and written in the
// same launch: work items are the rope items of the key rows (see rope_generic_kernel) followed by
// the quads of the value rows. The rotated f32 values are rounded to bf16 once, which is what the
// reference's rope_kernel + to_bf16(_scatter)_kernel pair produces.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kCtaThreads)
rope_kv_write_generic_kernel(uint16_t* __restrict__ cache_k, uint16_t* __restrict__ cache_v,
                             const typename T::storage* __restrict__ k, const typename T::storage* __restrict__ v,
                             const float* __restrict__ cos_t, const float* __restrict__ sin_t, int tokens, int heads,
                             int head_dim, int rotary_dim, const int* __restrict__ seq_start,
                             const int* __restrict__ pos_base, const int* __restrict__ pos_map,
                             const int* __restrict__ cache_map, const int* __restrict__ cache_len) {
    const int half = rotary_dim >> 1;
    const int rot_items = half >> 2;
    const int items = rot_items + ((head_dim - rotary_dim) >> 2);
    const int row_quads = head_dim >> 2;
    const size_t key_items = (size_t)tokens * heads * items;
    const size_t total = key_items + (size_t)tokens * heads * row_quads;
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += step) {
        const bool is_value = idx >= key_items;
        const size_t local = is_value ? idx - key_items : idx;
        const int per_row = is_value ? row_quads : items;
        const size_t head_row = local / per_row;
        const int item = (int)(local - head_row * per_row);
        const int token = (int)(head_row / heads);
        const int head = (int)(head_row - (size_t)token * heads);
        const size_t dst = (kv_cache_row(token, cache_map, cache_len) * (size_t)heads + head) * (size_t)head_dim;
        if (is_value) {
            store_quad<Bf16>(cache_v + dst, item, load_quad<T>(v + head_row * head_dim, item));
            continue;
        }
        const typename T::storage* xr = k + head_row * head_dim;
        uint16_t* orow = cache_k + dst;
        if (item < rot_items) {
            const int pos = rope_position(token, seq_start, pos_base, pos_map);
            const float4 c = *reinterpret_cast<const float4*>(cos_t + (size_t)pos * rotary_dim + 4 * item);
            const float4 s = *reinterpret_cast<const float4*>(sin_t + (size_t)pos * rotary_dim + 4 * item);
            const float4 lo = load_quad<T>(xr, item);
            const float4 hi = load_quad<T>(xr + half, item);
            float4 olo, ohi;
            rope_pair(lo.x, hi.x, c.x, s.x, olo.x, ohi.x);
            rope_pair(lo.y, hi.y, c.y, s.y, olo.y, ohi.y);
            rope_pair(lo.z, hi.z, c.z, s.z, olo.z, ohi.z);
            rope_pair(lo.w, hi.w, c.w, s.w, olo.w, ohi.w);
            store_quad<Bf16>(orow, item, olo);
            store_quad<Bf16>(orow + half, item, ohi);
        } else {
            const int q = (rotary_dim >> 2) + (item - rot_items);
            store_quad<Bf16>(orow, q, load_quad<T>(xr, q));
        }
    }
}

// ---------------------------------------------------------------------------------------------
// sigmoid_mul (kernels/elementwise.cu:344-359): out = x * 1.0f / (1.0f + __expf(-gate)) for whole
// quads, x * (1.0f / (1.0f + __expf(-gate))) for the total % 4 tail values (the reference's two forms).
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kCtaThreads)
sigmoid_mul_generic_kernel(typename T::storage* __restrict__ out, const typename T::storage* __restrict__ x,
                           const typename T::storage* __restrict__ gate, size_t total) {
    const size_t quads = total >> 2;
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < quads; i += step) {
        const float4 v = load_quad<T>(x, i);
        const float4 g = load_quad<T>(gate, i);
        store_quad<T>(out, i,
                      make_float4(gated_literal<kActSigmoidMul>(g.x, v.x), gated_literal<kActSigmoidMul>(g.y, v.y),
                                  gated_literal<kActSigmoidMul>(g.z, v.z), gated_literal<kActSigmoidMul>(g.w, v.w)));
    }
    if (blockIdx.x == 0 && threadIdx.x < (total & 3)) {
        const size_t k = (quads << 2) + threadIdx.x;
        if (T::kBytes == 2) {
            const float v = __uint_as_float((uint32_t)reinterpret_cast<const uint16_t*>(x)[k] << 16);
            const float g = __uint_as_float((uint32_t)reinterpret_cast<const uint16_t*>(gate)[k] << 16);
            const float r = v * __fdiv_rn(1.0f, __fadd_rn(1.0f, __expf(-g)));
            reinterpret_cast<uint16_t*>(out)[k] = (uint16_t)(pack_bf16x2(r, 0.0f) & 0xffffu);
        } else {
            const float v = reinterpret_cast<const float*>(x)[k];
            const float g = reinterpret_cast<const float*>(gate)[k];
            reinterpret_cast<float*>(out)[k] = v * __fdiv_rn(1.0f, __fadd_rn(1.0f, __expf(-g)));
        }
    }
}

// ---------------------------------------------------------------------------------------------
// add (kernels/head.cu:117-129): out = a + b over a flat array; out may be a or b.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kCtaThreads)
add_generic_kernel(typename T::storage* out, const typename T::storage* a, const typename T::storage* b, size_t total) {
    const size_t quads = total >> 2;
    const size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < quads; i += step) {
        const float4 x = load_quad<T>(a, i);
        const float4 y = load_quad<T>(b, i);
        store_quad<T>(out, i, make_float4(__fadd_rn(x.x, y.x), __fadd_rn(x.y, y.y), __fadd_rn(x.z, y.z), __fadd_rn(x.w, y.w)));
    }
    if (blockIdx.x == 0 && threadIdx.x < (total & 3)) {
        const size_t k = (quads << 2) + threadIdx.x;
        if (T::kBytes == 2) {
            const float x = __uint_as_float((uint32_t)reinterpret_cast<const uint16_t*>(a)[k] << 16);
            const float y = __uint_as_float((uint32_t)reinterpret_cast<const uint16_t*>(b)[k] << 16);
            reinterpret_cast<uint16_t*>(out)[k] = (uint16_t)(pack_bf16x2(__fadd_rn(x, y), 0.0f) & 0xffffu);
        } else {
            reinterpret_cast<float*>(out)[k] =
                __fadd_rn(reinterpret_cast<const float*>(a)[k], reinterpret_cast<const float*>(b)[k]);
        }
    }
}

// add for bf16, 16 values per lane per step (32-byte accesses); `blocks` = total / 16, the tail is the caller's.
static __global__ void __launch_bounds__(kCtaThreads)
add_hot_kernel(uint16_t* out, const uint16_t* a, const uint16_t* b, uint32_t blocks) {
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    const uint32_t step = gridDim.x * kCtaThreads;
    for (uint32_t i = blockIdx.x * kCtaThreads + threadIdx.x; i < blocks; i += step) {
        f32x2 x[8], y[8];
        unpack16_quadpairs(ldg_stream_v8(a + (size_t)i * 16), x);
        unpack16_quadpairs(ldg_stream_v8(b + (size_t)i * 16), y);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            x[k] = f2_add(x[k], y[k]);
        }
        stg_v8(out + (size_t)i * 16, pack16_bf16(x));
    }
}

// copy_kernel, copy_u8_kernel, copy_range_u8_kernel (kernels/elementwise.cu:317-342): device-to-device copies inside a
// captured pass. One kernel for the three: 32 bytes per thread where both addresses allow, single bytes for a ragged
// head and tail or for addresses that are not congruent modulo 32.
static __global__ void __launch_bounds__(kCtaThreads)
copy_bytes_kernel(uint8_t* __restrict__ dst, const uint8_t* __restrict__ src, size_t bytes) {
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    const size_t tid = (size_t)blockIdx.x * kCtaThreads + threadIdx.x, step = (size_t)gridDim.x * kCtaThreads;
    const uintptr_t da = reinterpret_cast<uintptr_t>(dst), sa = reinterpret_cast<uintptr_t>(src);
    if (((da ^ sa) & 31) != 0) {   // not congruent: bytes
        for (size_t i = tid; i < bytes; i += step) dst[i] = src[i];
        return;
    }
    size_t head = (32 - (da & 31)) & 31;
    if (head > bytes) head = bytes;
    const size_t chunks = (bytes - head) / 32, tail = head + chunks * 32;
    if (tid < head) dst[tid] = src[tid];
    for (size_t c = tid; c < chunks; c += step) stg_v8(dst + head + c * 32, ldg_stream_v8(src + head + c * 32));
    if (tail + tid < bytes) dst[tail + tid] = src[tail + tid];   // fewer than 32 bytes
}

}  // namespace clef
