// The short silu forms' building blocks, shared by the tuned kernels (kernels_hot.cuh) and the GEMM-epilogue
// quantiser (nvfp4_epilogue.cuh). See kernels_hot.cuh for the derivations and the exhaustive device-side checks.
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

namespace clef {

constexpr float kSiluFastMaxAbs = 44.0f;
constexpr float kNegLog2e = -1.4426950408889634f;

__device__ __forceinline__ float ex2_approx(float t) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(t));
    return r;
}
__device__ __forceinline__ float rcp_approx(float d) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(d));
    return r;
}

// silu(g) = g / (1 + __expf(-g)) with the IEEE quotient for ANY f32 g with |g| <= 44: e = ex2.approx(g * -log2 e),
// d = 1 + e, one Newton step on rcp.approx(d), q0 = g * r, one exact-remainder correction. Equals div.rn for every
// f32 g of the range (all patterns are compared on the device by the tests); the sign of g is copied onto the
// result (d > 0, so the exact quotient has the sign of g, and the short form loses the sign of a zero).
__device__ __forceinline__ float silu_ieee_refined_f32(float g) {
    const float d = __fadd_rn(1.0f, ex2_approx(__fmul_rn(g, kNegLog2e)));
    float r = rcp_approx(d);
    r = __fmaf_rn(__fmaf_rn(-d, r, 1.0f), r, r);
    const float q0 = __fmul_rn(g, r);
    const float q = __fmaf_rn(__fmaf_rn(-d, q0, g), r, q0);
    return __uint_as_float((__float_as_uint(q) & 0x7fffffffu) | (__float_as_uint(g) & 0x80000000u));
}

}  // namespace clef
