// Shared device helpers: vector memory access, bf16 <-> f32, and the reductions whose
// floating-point association must equal the reference kernels' (see sumsq notes below).
#pragma once

#include <cstdint>
#include <cuda_runtime.h>
#include <cuda_bf16.h>

namespace clef {

constexpr int kWarp = 32;
constexpr unsigned kFullMask = 0xffffffffu;

// Activation element types of the C-ABI `dtype` argument.
struct Bf16 {
    using storage = uint16_t;
    static constexpr int kBytes = 2;
};
struct F32 {
    using storage = float;
    static constexpr int kBytes = 4;
};

// ---------------------------------------------------------------------------------------------
// bf16 <-> f32 on bit patterns. Widening is exact. Narrowing is round-to-nearest-even
// (cvt.rn.bf16x2.f32), which is also what the reference's integer formula in
// kernels/quantise.cu:375-378 computes for finite values.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float bf16_lo(uint32_t pair) { return __uint_as_float(pair << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t pair) { return __uint_as_float(pair & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// ---------------------------------------------------------------------------------------------
// Global memory access. Streaming data is read once and written once, so loads bypass L1
// allocation and stores are marked evict-first-ish (.cs) where the caller says so.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 ldg_stream_v4(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}
__device__ __forceinline__ uint2 ldg_stream_v2(const void* p) {
    uint2 r;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p));
    return r;
}
// 256-bit load (sm_100): one lane fetches 32 contiguous bytes, a warp 1 KiB.
struct U8x32 {
    uint32_t w[8];
};
__device__ __forceinline__ U8x32 ldg_stream_v8(const void* p) {
    U8x32 r;
    asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r.w[0]), "=r"(r.w[1]), "=r"(r.w[2]), "=r"(r.w[3]), "=r"(r.w[4]), "=r"(r.w[5]), "=r"(r.w[6]),
                   "=r"(r.w[7])
                 : "l"(p));
    return r;
}
__device__ __forceinline__ void stg_v8(void* p, const U8x32& v) {
    asm volatile("st.global.v8.u32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v.w[0]), "r"(v.w[1]), "r"(v.w[2]),
                 "r"(v.w[3]), "r"(v.w[4]), "r"(v.w[5]), "r"(v.w[6]), "r"(v.w[7])
                 : "memory");
}
__device__ __forceinline__ void stg_v4(void* p, uint4 v) {
    asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void stg_v2(void* p, uint2 v) {
    asm volatile("st.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}

// Programmatic dependent launch (sm_90+). A kernel launched with the programmatic-serialisation
// attribute may start while the previous kernel of the stream is still draining: it signals at once
// that its own successor may be scheduled, does the work that depends on no earlier kernel (tables
// built from launch arguments and from constant weights), and only then waits for every earlier grid
// to have completed and flushed its writes. All reads of activations and all global writes come after
// pdl_wait_prior_grids(). Without the launch attribute both instructions do nothing.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait_prior_grids() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// L2 prefetch hint for the 128-byte line holding p. The row-structured kernels issue it for their FIRST round of
// activations before pdl_wait_prior_grids(): the hint moves the line from DRAM towards L2 and returns nothing
// to the SM, so it cannot observe a value (L2 is the point of coherence; a line the previous kernel is still
// writing is updated in place). Its only effect is that the first round's DRAM latency runs under the previous
// kernel's tail instead of after it. p must lie inside the tensor the kernel is going to read.
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// Load 4 consecutive activations (one "quad" = the reference's float4) as f32.
template <typename T>
__device__ __forceinline__ float4 load_quad(const typename T::storage* base, size_t quad_index);
template <>
__device__ __forceinline__ float4 load_quad<Bf16>(const uint16_t* base, size_t quad_index) {
    const uint2 r = *reinterpret_cast<const uint2*>(base + quad_index * 4);
    return make_float4(bf16_lo(r.x), bf16_hi(r.x), bf16_lo(r.y), bf16_hi(r.y));
}
template <>
__device__ __forceinline__ float4 load_quad<F32>(const float* base, size_t quad_index) {
    return *reinterpret_cast<const float4*>(base + quad_index * 4);
}
template <typename T>
__device__ __forceinline__ void store_quad(typename T::storage* base, size_t quad_index, float4 v);
template <>
__device__ __forceinline__ void store_quad<Bf16>(uint16_t* base, size_t quad_index, float4 v) {
    *reinterpret_cast<uint2*>(base + quad_index * 4) = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
}
template <>
__device__ __forceinline__ void store_quad<F32>(float* base, size_t quad_index, float4 v) {
    *reinterpret_cast<float4*>(base + quad_index * 4) = v;
}

// Load one 16-value block as f32.
// One activation value widened to f32 / narrowed from f32 (round to nearest even).
template <typename T>
__device__ __forceinline__ float load_scalar(const typename T::storage* p);
template <>
__device__ __forceinline__ float load_scalar<Bf16>(const uint16_t* p) {
    return __uint_as_float((uint32_t)(*p) << 16);
}
template <>
__device__ __forceinline__ float load_scalar<F32>(const float* p) {
    return *p;
}
template <typename T>
__device__ __forceinline__ void store_scalar(typename T::storage* p, float v);
template <>
__device__ __forceinline__ void store_scalar<Bf16>(uint16_t* p, float v) {
    *p = (uint16_t)(pack_bf16x2(v, 0.0f) & 0xffffu);
}
template <>
__device__ __forceinline__ void store_scalar<F32>(float* p, float v) {
    *p = v;
}

template <typename T>
__device__ __forceinline__ void load_block16(const typename T::storage* p, float* v);
template <>
__device__ __forceinline__ void load_block16<Bf16>(const uint16_t* p, float* v) {
    const uint4 a = *reinterpret_cast<const uint4*>(p);
    const uint4 b = *reinterpret_cast<const uint4*>(p + 8);
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        v[2 * i] = bf16_lo(w[i]);
        v[2 * i + 1] = bf16_hi(w[i]);
    }
}
template <>
__device__ __forceinline__ void load_block16<F32>(const float* p, float* v) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 q = *reinterpret_cast<const float4*>(p + 4 * i);
        v[4 * i] = q.x;
        v[4 * i + 1] = q.y;
        v[4 * i + 2] = q.z;
        v[4 * i + 3] = q.w;
    }
}

// ---------------------------------------------------------------------------------------------
// Sum of squares of one quad, (x*x + y*y) + (z*z + w*w), with the contraction the reference
// build applies to that expression (kernels/elementwise.cu:29, kernels/quantise.cu:75,214):
// CLEF_SUMSQ_FMA 1: each pair is fma(a, a, b*b); 2: fma(b, b, a*a); 0: no FMA.
// Written with explicit rounding intrinsics so the compiler cannot re-associate or re-fuse.
// ---------------------------------------------------------------------------------------------
#ifndef CLEF_SUMSQ_FMA
#define CLEF_SUMSQ_FMA 1
#endif
__device__ __forceinline__ float pair_sq(float a, float b) {
#if CLEF_SUMSQ_FMA == 1
    return __fmaf_rn(a, a, __fmul_rn(b, b));
#elif CLEF_SUMSQ_FMA == 2
    return __fmaf_rn(b, b, __fmul_rn(a, a));
#else
    return __fadd_rn(__fmul_rn(a, a), __fmul_rn(b, b));
#endif
}
__device__ __forceinline__ float quad_sq(float4 v) { return __fadd_rn(pair_sq(v.x, v.y), pair_sq(v.z, v.w)); }

// RoPE pair, lo*c - hi*s and hi*c + lo*s (kernels/elementwise.cu:308-309), same idea; the two
// expressions are contracted independently by the reference build:
//   CLEF_ROPE_FMA_LO 1: fma(lo, c, -(hi*s))   2: fma(-hi, s, lo*c)   0: no FMA
//   CLEF_ROPE_FMA_HI 1: fma(hi, c, lo*s)      2: fma(lo, s, hi*c)    0: no FMA
#ifndef CLEF_ROPE_FMA_LO
#define CLEF_ROPE_FMA_LO 1
#endif
#ifndef CLEF_ROPE_FMA_HI
#define CLEF_ROPE_FMA_HI 2
#endif
__device__ __forceinline__ void rope_pair(float lo, float hi, float c, float s, float& out_lo, float& out_hi) {
#if CLEF_ROPE_FMA_LO == 1
    out_lo = __fmaf_rn(lo, c, -__fmul_rn(hi, s));
#elif CLEF_ROPE_FMA_LO == 2
    out_lo = __fmaf_rn(-hi, s, __fmul_rn(lo, c));
#else
    out_lo = __fsub_rn(__fmul_rn(lo, c), __fmul_rn(hi, s));
#endif
#if CLEF_ROPE_FMA_HI == 1
    out_hi = __fmaf_rn(hi, c, __fmul_rn(lo, s));
#elif CLEF_ROPE_FMA_HI == 2
    out_hi = __fmaf_rn(lo, s, __fmul_rn(hi, c));
#else
    out_hi = __fadd_rn(__fmul_rn(hi, c), __fmul_rn(lo, s));
#endif
}

// Warp tree the reference uses everywhere: shfl_down by 16, 8, 4, 2, 1; lane 0 holds
// ((..)+(..)) in that association. A xor butterfly computes the same tree in every lane
// (f32 addition is commutative), which saves the broadcast.
__device__ __forceinline__ float warp_tree_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        v = __fadd_rn(v, __shfl_xor_sync(kFullMask, v, off));
    }
    return v;
}

// 1 / sqrt(total / cols + eps) with IEEE division and square root, as the reference writes it.
__device__ __forceinline__ float inv_rms(float total, int cols, float eps) {
    return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, (float)cols), eps)));
}

// Threads the reference assigns to one row of the plain / gated norm (kernels/elementwise.cu:8).
__host__ __device__ __forceinline__ int ref_threads_per_row(int cols) {
    const int t = ((cols + 255) / 256) * 32;
    return t < 32 ? 32 : (t > 256 ? 256 : t);
}

// silu pieces, spelled exactly like the reference so the same hardware approximations are used:
//   swiglu:      (g / (1 + __expf(-g))) * u          IEEE divide, approximate exp
//   gated norm:  __fdividef(g, 1 + __expf(-g))       approximate divide, approximate exp
__device__ __forceinline__ float silu_ieee_div(float g) { return __fdiv_rn(g, __fadd_rn(1.0f, __expf(-g))); }
__device__ __forceinline__ float silu_fast_div(float g) { return __fdividef(g, __fadd_rn(1.0f, __expf(-g))); }

// The two gated products that share one kernel structure. First input g, second input x:
//   kActSwiGLU      (g / (1 + __expf(-g))) * x          kernels/elementwise.cu:225-241, g = gate, x = up
//   kActSigmoidMul  x * 1.0f / (1.0f + __expf(-g))      kernels/elementwise.cu:344-353, g = gate, x = attention output
enum GatedAct { kActNone = -1, kActSwiGLU = 0, kActSigmoidMul = 1 };

template <int ACT>
__device__ __forceinline__ float gated_literal(float g, float x) {
    return ACT == kActSwiGLU ? silu_ieee_div(g) * x : __fdiv_rn(x * 1.0f, __fadd_rn(1.0f, __expf(-g)));
}


}  // namespace clef
