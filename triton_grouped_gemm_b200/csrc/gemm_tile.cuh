// Tile constants and the TMEM -> global epilogue shared by the 16-bit grouped GEMM kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace b200 {

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;  // 64 16-bit elements = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kNumThreads = 192;
constexpr int kSwizzle128 = 2;

__device__ __forceinline__ uint32_t pack2_16bit(float lo, float hi, int is_fp16) {
  if (is_fp16) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// One thread = one accumulator row (TMEM lane).  Reads kBlockN fp32 columns in chunks of 32,
// optionally scales them ((acc * row_scale) * col_scale[col], the order the reference's FP8
// kernels use), rounds once to the 16-bit output type and writes 16-byte vectors; columns
// >= n and rows with !row_ok are skipped.  The tcgen05.ld itself is executed by every lane
// (warp-aligned).  col_scale points at the scale of column 0 of the output row's group.
template <int kBlockN, bool kScaled>
__device__ __forceinline__ void store_acc_row_16bit(uint32_t t_addr, uint16_t* c_row, bool row_ok, int col_base,
                                                    int n, int is_fp16, float row_scale = 1.0f,
                                                    const float* __restrict__ col_scale = nullptr) {
#pragma unroll 1
  for (int c = 0; c < kBlockN / 32; ++c) {
    uint32_t r[32];
    tmem_ld_32x32b_x32(t_addr + c * 32, r);
    tmem_ld_wait();
    const int col0 = col_base + c * 32;
    if (row_ok && col0 < n) {
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        if (col0 + v * 8 < n) {
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[v * 8 + e]);
          if constexpr (kScaled) {
            const float4 s0 = __ldg(reinterpret_cast<const float4*>(col_scale + col0 + v * 8));
            const float4 s1 = __ldg(reinterpret_cast<const float4*>(col_scale + col0 + v * 8 + 4));
            const float cs[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = __fmul_rn(__fmul_rn(f[e], row_scale), cs[e]);
          }
          uint32_t p[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) p[e] = pack2_16bit(f[2 * e], f[2 * e + 1], is_fp16);
          *reinterpret_cast<uint4*>(c_row + col0 + v * 8) = make_uint4(p[0], p[1], p[2], p[3]);
        }
      }
    }
  }
}

// Same footprint, all zeros (a K-grouped output whose group is empty).
template <int kBlockN>
__device__ __forceinline__ void store_zero_row_16bit(uint16_t* c_row, bool row_ok, int col_base, int n) {
  if (!row_ok) return;
#pragma unroll 1
  for (int col = col_base; col < col_base + kBlockN && col < n; col += 8)
    *reinterpret_cast<uint4*>(c_row + col) = make_uint4(0, 0, 0, 0);
}

}  // namespace b200
