// Block-scaled FP8 (e4m3) M-grouped and masked M-grouped GEMM for sm_100a:
//   C[m, n] = sum_kb ( sum_{k in kb} a8[m,k] * b8[g,n,k] ) * as[m, kb] * bs[g, n/128, kb]   -> bf16
// with one fp32 scale per 1x128 block of A (along K) and per 128x128 block of B.
//
// The fp32 scales cannot be given to the tensor core (its block scaling is UE8M0 per 32
// elements), so every 128-wide k-block is multiplied into a FRESH TMEM buffer and promoted
// in software: promotion warps read the partial sums with tcgen05.ld, multiply by the
// combined scale and accumulate in fp32 registers.  Two TMEM buffers alternate per k-block,
// so the tensor core works on k-block i+1 while k-block i is being promoted.
//
// Warp roles (one persistent CTA per SM):
//   warp 0              TMA producer (same ring as the 16-bit kernels; a k-block is 128 bytes
//                       per row, so the stage layout is identical)
//   warp 1              MMA issuer: 4 x tcgen05.mma kind::f8f6f4 (128 x BLOCK_N x 32) per k-block
//   warps 2, 3          idle (they complete warpgroup 0, which gives its registers away)
//   warps 4..4+BLOCK_N/32-1   promotion + epilogue: warp (quarter = warp%4, half = (warp-4)/4)
//                       owns TMEM lanes [32*quarter, +32) and columns [128*half, +128), i.e.
//                       exactly one 128-wide scale block of B per thread; these warpgroups
//                       raise their register budget (setmaxnreg) to hold 128 fp32 accumulators
#include <cuda_bf16.h>

#include "../../include/b200gemm.h"
#include "common.cuh"
#include "gemm_tile.cuh"

namespace b200 {

template <int kBlockN>
struct Fp8BlockCfg {
  static constexpr int kStages = kBlockN == 256 ? 4 : 6;
  static constexpr int kPromoWarps = kBlockN / 32;  // 4 lane quarters x (kBlockN/128) column halves
  static constexpr int kThreads = 128 + 32 * kPromoWarps;
  // 384 threads start at 168 registers each; warpgroup 0 drops to 72 and the two promotion
  // warpgroups rise to 216 (128*72 + 256*216 <= 64K).  256 threads (BLOCK_N = 128) already
  // get 255 each and need no re-balancing.
  static constexpr bool kRebalance = kBlockN == 256;
  static constexpr int kABytes = kBlockM * 128;
  static constexpr int kBBytes = kBlockN * 128;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kEpiOffset = kStages * kStageBytes;  // one 4 KB store-staging buffer per promotion warp
  static constexpr int kBarOffset = kEpiOffset + kPromoWarps * 32 * 128;
  static constexpr int kNumBars = 2 * kStages + 4;
  static constexpr int kDynamicBytes = kBarOffset + kNumBars * 8 + 16 + 1024;
};

template <int kBlockN>
__global__ void __launch_bounds__(Fp8BlockCfg<kBlockN>::kThreads, 1)
fp8_block_m_grouped_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                           const __grid_constant__ CUtensorMap tm_c, __nv_bfloat16* __restrict__ c_ptr, const float* __restrict__ a_scale,
                           const float* __restrict__ b_scale, const void* __restrict__ sizes, int sizes_i64,
                           int num_groups, int masked_stride, int n, int k, unsigned* status) {
  using L = Fp8BlockCfg<kBlockN>;
  constexpr int kStages = L::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + L::kBarOffset;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tmem_full_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto tmem_empty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem + L::kBarOffset + L::kNumBars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kBarOffset + L::kNumBars * 8 + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_tiles = (n + kBlockN - 1) / kBlockN;
  const int num_kb = (k + 127) / 128;
  const int n_blocks = (n + 127) / 128;  // scale blocks of B along n
  constexpr uint32_t kTmemCols = 2 * kBlockN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tmem_full_bar(a), 1);
      mbar_init(tmem_empty_bar(a), L::kPromoWarps);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tmap(&tm_a);
    prefetch_tmap(&tm_b);
    prefetch_tmap(&tm_c);
  }
  if (warp == 1) {
    tmem_alloc<1>(smem_u32(const_cast<uint32_t*>(tmem_holder)), kTmemCols);
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp < 4) {
  if constexpr (L::kRebalance) warpgroup_reg_dec<72>();
  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    GroupWalker w;
    w.init(sizes, sizes_i64, num_groups, masked_stride, kBlockM);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok; tile += gridDim.x) {
      const int mt = tile / n_tiles;
      const int nt = tile - mt * n_tiles;
      if (!w.seek(mt)) break;
      const int row0 = static_cast<int>(w.tile_row0(mt));
      const int g = w.g;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag, status, kDevTimeoutProducer)) {
          ok = false;
          break;
        }
        if (lane == 0) {
          const uint32_t a_dst = smem_base + stage * L::kStageBytes;
          mbar_arrive_expect_tx(full_bar(stage), L::kStageBytes);
          tma_load_2d(a_dst, &tm_a, full_bar(stage), kb * 128, row0);
          tma_load_3d(a_dst + L::kABytes, &tm_b, full_bar(stage), kb * 128, nt * kBlockN, g);
        }
        __syncwarp();
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    GroupWalker w;
    w.init(sizes, sizes_i64, num_groups, masked_stride, kBlockM);
    const uint32_t idesc = make_instr_desc(0u, 0u, 0u, 0u, kBlockM, kBlockN);  // e4m3 x e4m3 -> f32
    int stage = 0;
    uint32_t phase = 0;
    uint32_t it = 0;  // k-blocks issued so far: TMEM buffer = it & 1
    bool ok = true;
    for (int tile = blockIdx.x; ok; tile += gridDim.x) {
      const int mt = tile / n_tiles;
      if (!w.seek(mt)) break;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const uint32_t buf = it & 1u;
        const uint32_t buf_phase = (it >> 1) & 1u;
        if (!wait_bounded(tmem_empty_bar(buf), buf_phase ^ 1u, abort_flag, status, kDevTimeoutMma) ||
            !wait_bounded(full_bar(stage), phase, abort_flag, status, kDevTimeoutMma)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        if (lane == 0) {
          const uint32_t a_addr = smem_base + stage * L::kStageBytes;
          const uint32_t b_addr = a_addr + L::kABytes;
          const uint32_t d_tmem = tmem_base + buf * kBlockN;
#pragma unroll
          for (int k32 = 0; k32 < 4; ++k32) {
            const uint64_t a_desc = make_smem_desc(a_addr + k32 * 32, 16, 1024, kSwizzle128);
            const uint64_t b_desc = make_smem_desc(b_addr + k32 * 32, 16, 1024, kSwizzle128);
            umma<1, true>(d_tmem, a_desc, b_desc, idesc, k32 != 0 ? 1u : 0u);
          }
          umma_commit_1cta(empty_bar(stage));
          umma_commit_1cta(tmem_full_bar(buf));
        }
        __syncwarp();
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  }
  } else {
    // ------------------------------------------------------------ promotion + epilogue
    if constexpr (L::kRebalance) warpgroup_reg_inc<216>();
    GroupWalker w;
    w.init(sizes, sizes_i64, num_groups, masked_stride, kBlockM);
    const int quarter = warp & 3;
    const int half = (warp - 4) >> 2;
    uint32_t it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok; tile += gridDim.x) {
      const int mt = tile / n_tiles;
      const int nt = tile - mt * n_tiles;
      if (!w.seek(mt)) break;
      const long long row = w.tile_row0(mt) + quarter * 32 + lane;
      const bool row_ok = row < w.group_row_end();
      const int col_base = nt * kBlockN + half * 128;
      // scales of this thread: its row of A, and the one 128-wide block of B it covers
      const float* as_row = a_scale + (row_ok ? row : 0) * static_cast<long long>(num_kb);
      int nb = col_base >> 7;
      if (nb >= n_blocks) nb = n_blocks - 1;  // columns past n: results are discarded
      const float* bs_blk = b_scale + (static_cast<long long>(w.g) * n_blocks + nb) * num_kb;
      float acc[128];
#pragma unroll
      for (int j = 0; j < 128; ++j) acc[j] = 0.f;
      // Software pipeline over 32-column chunks: two tcgen05.ld are kept in flight (t0, t1)
      // while the previous two chunks are multiplied in, so the TMEM read latency overlaps
      // the FMAs; the first two chunks of k-block kb+1 are requested before the last FMAs of kb.
      uint32_t t0[32], t1[32];
      const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + half * 128;
      float s_next = __ldg(as_row) * __ldg(bs_blk);
      if (!wait_bounded(tmem_full_bar(it & 1u), (it >> 1) & 1u, abort_flag, status, kDevTimeoutPromote)) break;
      tc_fence_after_sync();
      tmem_ld_32x32b_x32(t_lane + (it & 1u) * kBlockN, t0);
      tmem_ld_32x32b_x32(t_lane + (it & 1u) * kBlockN + 32, t1);
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const float s = s_next;
        const bool more = kb + 1 < num_kb;
        if (more) s_next = __ldg(as_row + kb + 1) * __ldg(bs_blk + kb + 1);
        const uint32_t buf = it & 1u;
        const uint32_t t_addr = t_lane + buf * kBlockN;
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = fmaf(s, __uint_as_float(t0[j]), acc[j]);
        tmem_ld_32x32b_x32(t_addr + 64, t0);
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[32 + j] = fmaf(s, __uint_as_float(t1[j]), acc[32 + j]);
        tmem_ld_32x32b_x32(t_addr + 96, t1);
        tmem_ld_wait();
        // every column of this buffer is in registers now: hand it back to the MMA warp
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(tmem_empty_bar(buf));
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[64 + j] = fmaf(s, __uint_as_float(t0[j]), acc[64 + j]);
        if (more) {
          const uint32_t nit = it + 1;
          if (!wait_bounded(tmem_full_bar(nit & 1u), (nit >> 1) & 1u, abort_flag, status, kDevTimeoutPromote)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          tmem_ld_32x32b_x32(t_lane + (nit & 1u) * kBlockN, t0);
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[96 + j] = fmaf(s, __uint_as_float(t1[j]), acc[96 + j]);
        if (more) tmem_ld_32x32b_x32(t_lane + ((it + 1) & 1u) * kBlockN + 32, t1);
      }
      if (!ok) break;
      const long long row_w0 = w.tile_row0(mt) + quarter * 32;
      if (row_w0 + 32 <= w.group_row_end()) {
        // all 32 rows of this warp are valid: round, stage in the 128-byte-swizzle layout and
        // let TMA write 64-column chunks (the tensor map clips columns >= n)
        uint8_t* buf = smem + L::kEpiOffset + (warp - 4) * (32 * 128);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int col0 = col_base + c * 64;
          if (col0 < n) {
            if (lane == 0) tma_store_wait_read<0>();
            __syncwarp();
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              uint32_t p[4];
#pragma unroll
              for (int e = 0; e < 4; ++e)
                p[e] = pack2_16bit(acc[c * 64 + v * 8 + 2 * e], acc[c * 64 + v * 8 + 2 * e + 1], 0);
              *reinterpret_cast<uint4*>(buf + lane * 128 + ((v ^ (lane & 7)) << 4)) = make_uint4(p[0], p[1], p[2], p[3]);
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tm_c, smem_u32(buf), col0, static_cast<int>(row_w0));
              tma_store_commit();
            }
          }
        }
      } else if (row_ok) {
        __nv_bfloat16* c_row = c_ptr + row * static_cast<long long>(n);
#pragma unroll
        for (int v = 0; v < 16; ++v) {
          const int col = col_base + v * 8;
          if (col < n) {
            uint32_t p[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) p[e] = pack2_16bit(acc[v * 8 + 2 * e], acc[v * 8 + 2 * e + 1], 0);
            *reinterpret_cast<uint4*>(c_row + col) = make_uint4(p[0], p[1], p[2], p[3]);
          }
        }
      }
    }
    if (lane == 0) tma_store_wait_all<0>();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(4000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_base, kTmemCols);
  }
}

template <int kBlockN>
static int launch_fp8_block(const CUtensorMap& tm_a, const CUtensorMap& tm_b, const CUtensorMap& tm_c, void* c, const float* a_scale,
                            const float* b_scale, const void* sizes, int sizes_is_i64, int num_groups,
                            int masked_stride, int n, int k, int grid, cudaStream_t stream) {
  using L = Fp8BlockCfg<kBlockN>;
  auto kern = fp8_block_m_grouped_kernel<kBlockN>;
  B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes));
  kern<<<grid, L::kThreads, L::kDynamicBytes, stream>>>(tm_a, tm_b, tm_c, static_cast<__nv_bfloat16*>(c), a_scale, b_scale,
                                                        sizes, sizes_is_i64, num_groups, masked_stride, n, k,
                                                        device_status_ptr());
  B200_CUDA(cudaGetLastError());
  return 0;
}

static int fp8_block_common(const void* a, const float* a_scale, const void* b, const float* b_scale, void* c,
                            const void* sizes, int sizes_is_i64, int num_groups, int64_t m_rows, int masked_stride,
                            int n, int k, int num_sms, void* stream_v, const char* who) {
  B200_REQUIRE(num_groups >= 0 && m_rows >= 0 && n >= 0 && k >= 0, "%s: negative dimension", who);
  if (num_groups == 0 || m_rows == 0 || n == 0) return 0;
  B200_REQUIRE(k > 0, "%s: k must be positive", who);
  B200_REQUIRE(a && b && c && sizes && a_scale && b_scale, "%s: null pointer", who);
  B200_REQUIRE(k % 16 == 0, "%s: TMA required 16-byte alignment: k bytes (k=%d)", who, k);
  B200_REQUIRE(n % 8 == 0, "%s: n must be a multiple of 8 (n=%d)", who, n);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(a) & 15) == 0 && (reinterpret_cast<uintptr_t>(b) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(c) & 15) == 0,
               "%s: a, b and c must be 16-byte aligned", who);
  B200_REQUIRE(m_rows < (1ll << 31), "%s: m_rows must fit in int32", who);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const int sms = sm_count();
  B200_REQUIRE(sms > 0, "%s: no CUDA device", who);
  const int grid = (num_sms > 0 && num_sms < sms) ? num_sms : sms;
  const long long m_tiles_est = (m_rows + kBlockM - 1) / kBlockM;
  const int block_n = (n <= 128 || m_tiles_est * ((n + 255) / 256) < grid) ? 128 : 256;
  CUtensorMap tm_a, tm_b;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(k), static_cast<uint64_t>(m_rows)};
    const uint64_t strides[1] = {static_cast<uint64_t>(k)};
    const uint32_t box[2] = {128, kBlockM};
    int rc = encode_tmap(&tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, "A");
    if (rc) return rc;
  }
  {
    const uint64_t dims[3] = {static_cast<uint64_t>(k), static_cast<uint64_t>(n), static_cast<uint64_t>(num_groups)};
    const uint64_t strides[2] = {static_cast<uint64_t>(k), static_cast<uint64_t>(k) * n};
    const uint32_t box[3] = {128, static_cast<uint32_t>(block_n), 1};
    int rc = encode_tmap(&tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, b, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                         "B[G,N,K]");
    if (rc) return rc;
  }
  CUtensorMap tm_c;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(n), static_cast<uint64_t>(m_rows)};
    const uint64_t strides[1] = {static_cast<uint64_t>(n) * 2};
    const uint32_t box[2] = {64, 32};
    int rc = encode_tmap(&tm_c, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, c, dims, strides, box,
                         CU_TENSOR_MAP_SWIZZLE_128B, "C");
    if (rc) return rc;
  }
  if (block_n == 256)
    return launch_fp8_block<256>(tm_a, tm_b, tm_c, c, a_scale, b_scale, sizes, sizes_is_i64, num_groups, masked_stride, n, k,
                                 grid, stream);
  return launch_fp8_block<128>(tm_a, tm_b, tm_c, c, a_scale, b_scale, sizes, sizes_is_i64, num_groups, masked_stride, n, k,
                               grid, stream);
}

}  // namespace b200

extern "C" {

int b200gemm_fp8_m_grouped_block(const void* a, const float* a_scale, const void* b, const float* b_scale, void* c,
                                 const void* sizes, int sizes_is_i64, int num_groups, int64_t m_rows, int n, int k,
                                 int rows_padded, int num_sms, void* stream) {
  return b200::fp8_block_common(a, a_scale, b, b_scale, c, sizes, sizes_is_i64, num_groups, m_rows,
                                rows_padded ? -1 : 0, n, k, num_sms, stream, "b200gemm_fp8_m_grouped_block");
}

int b200gemm_fp8_m_grouped_masked_block(const void* a, const float* a_scale, const void* b, const float* b_scale,
                                        void* out, const void* masked_m, int sizes_is_i64, int num_groups,
                                        int expected_m, int n, int k, int num_sms, void* stream) {
  if (expected_m <= 0)
    return b200::set_error(b200::kErrInvalidArgument, "b200gemm_fp8_m_grouped_masked_block: expected_m must be positive");
  return b200::fp8_block_common(a, a_scale, b, b_scale, out, masked_m, sizes_is_i64, num_groups,
                                static_cast<int64_t>(num_groups) * expected_m, expected_m, n, k, num_sms, stream,
                                "b200gemm_fp8_m_grouped_masked_block");
}

}  // extern "C"
