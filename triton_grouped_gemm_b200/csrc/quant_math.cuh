// Arithmetic shared by the quantiser kernels and by GEMM epilogues that quantise their output:
// the exact operation order that reproduces the reference's torch casts bit for bit.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>

namespace b200 {

// two fp32 -> two e4m3 bytes (round to nearest even, finite values saturate at +-448,
// NaN -> 0x7f); low byte = first value
__device__ __forceinline__ uint32_t cvt_e4m3x2(float a, float b) {
  return static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3));
}

// The reference writes `448.0 / amax` with a Python scalar on the left; torch evaluates that
// as reciprocal(amax) * 448 (two roundings), which differs from a single IEEE division in
// the last bit often enough to flip e4m3 bytes.  Reproduce the two roundings.
__device__ __forceinline__ float inv_scale_448(float amax) { return __fmul_rn(__frcp_rn(amax), 448.0f); }

__device__ __forceinline__ float silu_mul_round_bf16(float g, float u) {
  // silu has no reference bit pattern to reproduce (the torch oracle rounds the activation to
  // bf16, which absorbs a 2^-21 relative error in all but ~1e-4 of the elements), so the
  // exponential and the quotient use the special-function unit: ex2.approx and rcp.approx
  // instead of ~25 instructions of IEEE expf and division per element, which kept this kernel
  // at half of the memory roofline.  g << 0: exp(-g) = inf, g / inf = -0.
  const float act = __fmul_rn(__fdividef(g, 1.0f + __expf(-g)), u);
  return __bfloat162float(__float2bfloat16_rn(act));
}

}  // namespace b200
