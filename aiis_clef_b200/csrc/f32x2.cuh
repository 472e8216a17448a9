// Packed-pair fp32 arithmetic (sm_100 `*.f32x2`): one instruction issues two IEEE fp32 operations.
// Each half is rounded exactly like the scalar round-to-nearest form, so results are bit-identical
// to scalar code; what is saved is issue slots, which is what bounds the quantising kernels.
// Built on the compiler's float2 builtins so the register allocator pairs the halves itself.
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

namespace clef {

using f32x2 = float2;   // {x = first value, y = second value}

__device__ __forceinline__ f32x2 f2_pack(float lo, float hi) { return make_float2(lo, hi); }
__device__ __forceinline__ void f2_unpack(f32x2 v, float& lo, float& hi) {
    lo = v.x;
    hi = v.y;
}
__device__ __forceinline__ f32x2 f2_splat(float v) { return make_float2(v, v); }
__device__ __forceinline__ f32x2 f2_mul(f32x2 a, f32x2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ f32x2 f2_add(f32x2 a, f32x2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ f32x2 f2_fma(f32x2 a, f32x2 b, f32x2 c) { return __ffma2_rn(a, b, c); }

// A 32-bit word holding two bf16 values -> the pair {element 0, element 1} widened exactly.
__device__ __forceinline__ f32x2 f2_from_bf16x2(uint32_t word) {
    return make_float2(__uint_as_float(word << 16), __uint_as_float(word & 0xffff0000u));
}

// NaN-propagating 3-input maximum (sm_100): max(acc, |a|, |b|), NaN if any input is NaN.
__device__ __forceinline__ float max3_abs_nan(float acc, float a, float b) {
    float r;
    asm("max.NaN.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(acc), "f"(fabsf(a)), "f"(fabsf(b)));
    return r;
}

// NaN-propagating 2-input maximum.
__device__ __forceinline__ float fmaxf_nan(float a, float b) {
    float r;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}

// 3-input minimum of magnitudes: min(acc, |a|, |b|); a NaN input is ignored.
__device__ __forceinline__ float min3_abs(float acc, float a, float b) {
    float r;
    asm("min.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(acc), "f"(fabsf(a)), "f"(fabsf(b)));
    return r;
}

}  // namespace clef
