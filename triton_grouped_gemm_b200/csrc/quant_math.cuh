// Arithmetic shared by the quantiser kernels and by GEMM epilogues that quantise their output:
// the exact operation order that reproduces the reference's torch casts bit for bit.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>

namespace b200 {

__device__ __forceinline__ float to_f32(uint16_t raw, int is_fp16) {
  if (is_fp16) return __half2float(__ushort_as_half(raw));
  return __uint_as_float(static_cast<uint32_t>(raw) << 16);
}

__device__ __forceinline__ float abs_max8(const uint4& v, int is_fp16) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m = fmaxf(m, fabsf(to_f32(static_cast<uint16_t>(w[i] & 0xFFFFu), is_fp16)));
    m = fmaxf(m, fabsf(to_f32(static_cast<uint16_t>(w[i] >> 16), is_fp16)));
  }
  return m;
}

// two fp32 -> two e4m3 bytes (round to nearest even, finite values saturate at +-448,
// NaN -> 0x7f); low byte = first value
__device__ __forceinline__ uint32_t cvt_e4m3x2(float a, float b) {
  return static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3));
}

// The reference writes `448.0 / amax` with a Python scalar on the left; torch evaluates that
// as reciprocal(amax) * 448 (two roundings), which differs from a single IEEE division in
// the last bit often enough to flip e4m3 bytes.  Reproduce the two roundings.
__device__ __forceinline__ float inv_scale_448(float amax) { return __fmul_rn(__frcp_rn(amax), 448.0f); }

// eight 16-bit values times `inv` -> eight e4m3 bytes: the per-chunk arithmetic of the 1x128
// activation quantiser (fp32 product rounded to nearest, then the saturating conversion)
__device__ __forceinline__ uint2 quant8_e4m3(const uint4& v, float inv, int is_fp16) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  uint32_t out[2];
#pragma unroll
  for (int p = 0; p < 2; ++p) {
    const float f0 = __fmul_rn(to_f32(static_cast<uint16_t>(w[2 * p] & 0xFFFFu), is_fp16), inv);
    const float f1 = __fmul_rn(to_f32(static_cast<uint16_t>(w[2 * p] >> 16), is_fp16), inv);
    const float f2 = __fmul_rn(to_f32(static_cast<uint16_t>(w[2 * p + 1] & 0xFFFFu), is_fp16), inv);
    const float f3 = __fmul_rn(to_f32(static_cast<uint16_t>(w[2 * p + 1] >> 16), is_fp16), inv);
    out[p] = cvt_e4m3x2(f0, f1) | (cvt_e4m3x2(f2, f3) << 16);
  }
  return make_uint2(out[0], out[1]);
}

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
