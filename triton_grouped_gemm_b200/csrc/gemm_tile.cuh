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

// Warp-collective variant for warps whose 32 rows are all valid: 64-column chunks are rounded,
// staged in shared memory in the 128-byte-swizzle layout (conflict-free 16-byte stores) and
// written with one TMA store per chunk; two 4 KB staging buffers per warp alternate so the
// next chunk is converted while the previous one drains.  The tensor map clips columns >= n
// and rows past the end of the tensor.  `stage` is this warp's 8 KB (1024-byte aligned),
// `sel` its current buffer; z >= 0 selects a 3-D map (x = column, y = row, z).
constexpr int kEpiStageBytesPerWarp = 2 * 32 * 128;

template <int kBlockN, bool kScaled>
__device__ __forceinline__ void store_acc_warp_tma(uint32_t t_addr, const CUtensorMap* tm_c, uint8_t* stage, int& sel,
                                                   int row_warp0, int z, int col_base, int n, int is_fp16, int lane,
                                                   float row_scale = 1.0f,
                                                   const float* __restrict__ col_scale = nullptr) {
#pragma unroll 1
  for (int c = 0; c < kBlockN / 64; ++c) {
    const int col0 = col_base + c * 64;
    if (col0 >= n) break;
    uint32_t r[64];
    {
      uint32_t(&lo)[32] = *reinterpret_cast<uint32_t(*)[32]>(&r[0]);
      uint32_t(&hi)[32] = *reinterpret_cast<uint32_t(*)[32]>(&r[32]);
      tmem_ld_32x32b_x32(t_addr + c * 64, lo);
      tmem_ld_32x32b_x32(t_addr + c * 64 + 32, hi);
    }
    tmem_ld_wait();
    if (lane == 0) tma_store_wait_read<1>();  // the buffer written two chunks ago has been read
    __syncwarp();
    uint8_t* buf = stage + sel * (32 * 128);
#pragma unroll
    for (int v = 0; v < 8; ++v) {
      float f[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[v * 8 + e]);
      if constexpr (kScaled) {
        if (col0 + v * 8 < n) {
          const float4 s0 = __ldg(reinterpret_cast<const float4*>(col_scale + col0 + v * 8));
          const float4 s1 = __ldg(reinterpret_cast<const float4*>(col_scale + col0 + v * 8 + 4));
          const float cs[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = __fmul_rn(__fmul_rn(f[e], row_scale), cs[e]);
        }
      }
      uint32_t p[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) p[e] = pack2_16bit(f[2 * e], f[2 * e + 1], is_fp16);
      *reinterpret_cast<uint4*>(buf + lane * 128 + ((v ^ (lane & 7)) << 4)) = make_uint4(p[0], p[1], p[2], p[3]);
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      if (z >= 0) tma_store_3d(tm_c, smem_u32(buf), col0, row_warp0, z);
      else tma_store_2d(tm_c, smem_u32(buf), col0, row_warp0);
      tma_store_commit();
    }
    sel ^= 1;
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

// CTA-pair (cta_group::2) variant of the M-grouped kernels, 256 x 256 tiles (gemm_pair.cu).
// `want_ctas` <= 0: as many CTAs as are co-resident.  tm_b must describe 128-row (K-major) or
// 64 x 64 (MN-major) boxes; tm_a 128-row boxes; tm_c 32 x 64 boxes.
template <bool kBMnMajor, bool kFp8>
int launch_m_grouped_pair(const CUtensorMap& tm_a, const CUtensorMap& tm_b, const CUtensorMap& tm_c, void* c,
                          const void* sizes, int sizes_is_i64, int num_groups, int masked_stride, long long m_rows,
                          int n, int k, int in_fmt, int out_fp16, const float* a_scale, const float* b_scale,
                          int want_ctas, cudaStream_t stream);
// Scratch of the balanced K-grouped scheduler (int32 words): [0] tile counter, [1..63] unused,
// then starts[G], tokens[G], order[G] (written by the plan kernel in gemm_bf16_k.cu).
constexpr int kPlanHeaderWords = 64;

// CTA-pair variant of the balanced K-grouped kernels, 256 x 256 tiles (gemm_k_pair.cu).  The plan
// kernel must already be queued on `stream`.  16-bit: tm_a / tm_b 64 x 64 boxes over
// [K_TOTAL, M_DIM] / [K_TOTAL, N_DIM]; fp8: 128-byte x 128-row boxes over [M, K_TOTAL] / [N, K_TOTAL].
template <bool kFp8>
int launch_k_grouped_pair(const CUtensorMap& tm_a, const CUtensorMap& tm_b, const CUtensorMap& tm_c, void* c,
                          int num_groups, int m_dim, int n_dim, int in_fmt, int out_fp16, const float* a_scale,
                          const float* b_scale, int* scratch, int want_ctas, cudaStream_t stream);
// Validates a K-grouped workspace and queues the plan kernel on it: scratch[kPlanHeaderWords + ...] =
// starts[G] (first token of each group), tokens[G], order[G] (groups by falling token count).
// *out = nullptr when workspace is null (gemm_bf16_k.cu).
int k_grouped_plan_into(void* workspace, long long workspace_bytes, const void* sizes, int sizes_is_i64,
                        int num_groups, const char* who, int** out, cudaStream_t stream);
// -1 = use the pair kernel when the problem is large enough, 0 = never, 1 = whenever possible
extern int g_cta_pair_mode;
int pair_kernel_grid();

}  // namespace b200
