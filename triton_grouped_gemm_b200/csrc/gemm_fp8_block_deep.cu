// Block-scaled FP8 (e4m3) M-grouped GEMM, "deep" CTA-pair form: 256 x 128 tiles, FOUR TMEM buffers.
//
// Same product as gemm_fp8_block.cu (1x128 activation scales x 128x128 weight scales, promoted in
// software per 128-wide k-block).  That kernel's 256 x 256 pair tile leaves room for only two
// 256-column TMEM buffers, and its pace is set by the length of the hand-over loop
//   MMA -> commit -> promotion warps wake, read TMEM (with half of their FMAs between the two
//   loads, for want of registers) -> arrive -> MMA warp wakes
// that two buffers cannot hide.  Here the tile is 128 columns wide: four 128-column buffers are in
// flight, a promotion thread owns 64 columns (64 accumulators + two 64-register staging sets fit
// the 224-register budget), so a buffer is released as soon as its single TMEM load has landed -
// no arithmetic inside the loop - and the next buffer's load is issued before this one's FMAs.
// The price is shared-memory traffic per output column (the A tile is re-read for every 128
// columns instead of every 256), which the measurements have to justify.
//
//   warp 0   TMA producer   warp 1   MMA issuer (leader CTA)   warps 2, 3  idle
//   warps 4..11  promotion + epilogue: warp (quarter = warp % 4, half = (warp - 4) / 4) owns TMEM
//                lanes [32 quarter, +32) and columns [64 half, +64) of the current buffer
// CTA r of the pair holds rows [128 r, +128) of A and of the accumulators and supplies rows
// [64 r, +64) of the B tile; plain cta_group::2 TMA loads, no multicast.
#include <cuda_bf16.h>

#include "../../include/b200gemm.h"
#include "common.cuh"
#include "gemm_tile.cuh"

namespace b200 {

struct Fp8DeepCfg {
  static constexpr int kBlockN = 128;
  static constexpr int kBufs = 4;
  static constexpr int kStages = 7;
  static constexpr int kBRows = 64;
  static constexpr int kPromoWarps = 8;
  static constexpr int kThreads = 128 + 32 * kPromoWarps;
  static constexpr int kABytes = kBlockM * 128;
  static constexpr int kBBytes = kBRows * 128;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kEpiOffset = kStages * kStageBytes;
  static constexpr int kBarOffset = kEpiOffset + 8 * 32 * 128;
  static constexpr int kNumBars = 2 * kStages + 2 * kBufs;
  static constexpr int kDynamicBytes = kBarOffset + kNumBars * 8 + 16 + 1024;
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Fp8DeepCfg::kThreads, 1)
fp8_block_m_grouped_deep_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                                const __grid_constant__ CUtensorMap tm_c, __nv_bfloat16* __restrict__ c_ptr,
                                const float* __restrict__ a_scale, const float* __restrict__ b_scale,
                                const void* __restrict__ sizes, int sizes_i64, int num_groups, int masked_stride,
                                long long m_rows, int n, int k, const int* __restrict__ b_map, int num_b,
                                unsigned* status) {
  using L = Fp8DeepCfg;
  constexpr int kBlockN = L::kBlockN;
  constexpr int kStages = L::kStages;
  constexpr int kBufs = L::kBufs;
  constexpr int kTileM = 2 * kBlockM;
  auto weight_of = [&](int g) -> int {
    if (!b_map) return g;
    const int v = __ldg(b_map + g);
    return v < 0 ? 0 : (v >= num_b ? num_b - 1 : v);
  };
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + L::kBarOffset;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tmem_full_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto tmem_empty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + kBufs + a); };
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem + L::kBarOffset + L::kNumBars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kBarOffset + L::kNumBars * 8 + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int first_tile = blockIdx.x >> 1;
  const int tile_step = gridDim.x >> 1;
  const int n_tiles = (n + kBlockN - 1) / kBlockN;
  const int num_kb = (k + 127) / 128;
  const int n_blocks = (n + 127) / 128;
  constexpr uint32_t kTmemCols = kBufs * kBlockN;  // 512

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < kBufs; ++a) {
      mbar_init(tmem_full_bar(a), 1);
      mbar_init(tmem_empty_bar(a), L::kPromoWarps * 2);
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
    tmem_alloc<2>(smem_u32(const_cast<uint32_t*>(tmem_holder)), kTmemCols);
    tmem_relinquish<2>();
  }
  tc_fence_before_sync();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp < 4) {
    warpgroup_reg_dec<56>();
    if (warp == 0) {
      // ------------------------------------------------------------ TMA producer
      GroupWalker w;
      w.init(sizes, sizes_i64, num_groups, masked_stride, kTileM, m_rows);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = first_tile; ok; tile += tile_step) {
        const int mt = tile / n_tiles;
        const int nt = tile - mt * n_tiles;
        if (!w.seek(mt)) break;
        const int row0 = static_cast<int>(w.tile_row0(mt)) + static_cast<int>(rank) * kBlockM;
        const int col0 = nt * kBlockN + static_cast<int>(rank) * L::kBRows;
        const int g = weight_of(w.g);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag, status, kDevTimeoutProducer)) {
            ok = false;
            break;
          }
          if (lane == 0) {
            const uint32_t a_dst = smem_base + stage * L::kStageBytes;
            const uint32_t leader_full = mapa_u32(full_bar(stage), 0);
            if (rank == 0) mbar_arrive_expect_tx(full_bar(stage), 2 * L::kStageBytes);
            tma_load_2d_pair(a_dst, &tm_a, leader_full, kb * 128, row0);
            tma_load_3d_pair(a_dst + L::kABytes, &tm_b, leader_full, kb * 128, col0, g);
          }
          __syncwarp();
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    } else if (warp == 1) {
      // ------------------------------------------------------------ MMA issuer (leader CTA)
      GroupWalker w;
      w.init(sizes, sizes_i64, num_groups, masked_stride, kTileM, m_rows);
      const uint32_t idesc = make_instr_desc(0u, 0u, 0u, 0u, kTileM, kBlockN);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t it = 0;  // k-blocks issued so far: TMEM buffer = it % kBufs
      bool ok = rank == 0;
      for (int tile = first_tile; ok; tile += tile_step) {
        const int mt = tile / n_tiles;
        if (!w.seek(mt)) break;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const uint32_t buf = it & (kBufs - 1);
          const uint32_t buf_phase = (it / kBufs) & 1u;
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
              umma<2, true>(d_tmem, a_desc, b_desc, idesc, k32 != 0 ? 1u : 0u);
            }
            umma_commit_2cta(empty_bar(stage), 0x3);
            umma_commit_2cta(tmem_full_bar(buf), 0x3);
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
    warpgroup_reg_inc<224>();
    GroupWalker w;
    w.init(sizes, sizes_i64, num_groups, masked_stride, kTileM, m_rows);
    const int quarter = warp & 3;
    const int half = (warp - 4) >> 2;
    uint32_t it = 0;
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + half * 64;
    uint8_t* stage_buf = smem + L::kEpiOffset + (warp - 4) * (32 * 128);
    bool ok = true;
    for (int tile = first_tile; ok; tile += tile_step) {
      const int mt = tile / n_tiles;
      const int nt = tile - mt * n_tiles;
      if (!w.seek(mt)) break;
      const long long row_w0 = w.tile_row0(mt) + static_cast<long long>(rank) * kBlockM + quarter * 32;
      const long long row = row_w0 + lane;
      const bool row_ok = row < w.group_row_end();
      const int col0 = nt * kBlockN + half * 64;
      const float* as_row = a_scale + (row_ok ? row : 0) * static_cast<long long>(num_kb);
      int nb = nt;  // both halves of a 128-column tile lie in one scale block of B
      if (nb >= n_blocks) nb = n_blocks - 1;
      const float* bs_blk = b_scale + (static_cast<long long>(weight_of(w.g)) * n_blocks + nb) * num_kb;
      unsigned long long acc2[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) acc2[j] = 0ull;
      uint32_t ta[64], tb[64];
      float fa_next = __ldg(as_row), fb_next = __ldg(bs_blk);
      if (!wait_bounded(tmem_full_bar(it & (kBufs - 1)), (it / kBufs) & 1u, abort_flag, status, kDevTimeoutPromote)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      tmem_ld_32x32b_x64(t_lane + (it & (kBufs - 1)) * kBlockN, ta);
      // one k-block: `cur` holds (or is about to hold) this k-block's partial sums; release the buffer
      // as soon as the load has landed, start the next buffer's load into `nxt`, then do the FMAs
      auto step = [&](uint32_t (&cur)[64], uint32_t (&nxt)[64], int kb) -> bool {
        const float s_cur = fa_next * fb_next;
        const unsigned long long s2 = pack_f32x2(__float_as_uint(s_cur), __float_as_uint(s_cur));
        const bool more = kb + 1 < num_kb;
        const uint32_t buf = it & (kBufs - 1);
        tmem_ld_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(tmem_empty_bar(buf), 0);
        if (more) {
          fa_next = __ldg(as_row + kb + 1);
          fb_next = __ldg(bs_blk + kb + 1);
          const uint32_t nit = it + 1;
          if (!wait_bounded(tmem_full_bar(nit & (kBufs - 1)), (nit / kBufs) & 1u, abort_flag, status, kDevTimeoutPromote))
            return false;
          tc_fence_after_sync();
          tmem_ld_32x32b_x64(t_lane + (nit & (kBufs - 1)) * kBlockN, nxt);
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) fma_f32x2(acc2[j], s2, pack_f32x2(cur[2 * j], cur[2 * j + 1]));
        ++it;
        return true;
      };
      for (int kb = 0; kb < num_kb; kb += 2) {
        if (!step(ta, tb, kb)) {
          ok = false;
          break;
        }
        if (kb + 1 < num_kb && !step(tb, ta, kb + 1)) {
          ok = false;
          break;
        }
      }
      if (!ok) break;
      // nothing is in flight here (the last step starts no load), so the next tile starts with ta again
      float acc[64];
#pragma unroll
      for (int j = 0; j < 32; ++j) unpack_f32x2(acc2[j], acc[2 * j], acc[2 * j + 1]);
      if (col0 < n) {
        if (row_w0 + 32 <= w.group_row_end()) {
          if (lane == 0) tma_store_wait_read<0>();
          __syncwarp();
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            uint32_t p[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) p[e] = pack2_16bit(acc[v * 8 + 2 * e], acc[v * 8 + 2 * e + 1], 0);
            *reinterpret_cast<uint4*>(stage_buf + lane * 128 + ((v ^ (lane & 7)) << 4)) = make_uint4(p[0], p[1], p[2], p[3]);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tm_c, smem_u32(stage_buf), col0, static_cast<int>(row_w0));
            tma_store_commit();
          }
        } else if (row_ok) {
          __nv_bfloat16* c_row = c_ptr + row * static_cast<long long>(n);
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            const int col = col0 + v * 8;
            if (col < n) {
              uint32_t p[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) p[e] = pack2_16bit(acc[v * 8 + 2 * e], acc[v * 8 + 2 * e + 1], 0);
              *reinterpret_cast<uint4*>(c_row + col) = make_uint4(p[0], p[1], p[2], p[3]);
            }
          }
        }
      }
    }
    if (lane == 0) tma_store_wait_all<0>();
    if (ok && w.overflow && rank == 0 && warp == 4 && lane == 0 && status) atomicOr(status, kDevBadGroupSize);
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(4000);
    __syncthreads();
  }
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<2>(tmem_base, kTmemCols);
  }
}

// tm_a: 128-byte x 128-row boxes over a [m_rows, k]; tm_b: 128-byte x 64-row boxes over b [num_b, n, k];
// tm_c: 64-column x 32-row boxes over c [m_rows, n] (bf16).  `grid` = CTAs wanted (SM budget).
int launch_fp8_block_deep(const CUtensorMap& tm_a, const CUtensorMap& tm_b, const CUtensorMap& tm_c, void* c,
                          const float* a_scale, const float* b_scale, const void* sizes, int sizes_is_i64,
                          int num_groups, int masked_stride, long long m_rows, int n, int k, const int* b_map, int num_b,
                          int grid, cudaStream_t stream) {
  using L = Fp8DeepCfg;
  auto kern = fp8_block_m_grouped_deep_kernel;
  B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes));
  static int resident[64] = {0};
  int dev = 0;
  B200_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return set_error(kErrUnsupported, "device index %d out of range", dev);
  if (!resident[dev]) {
    cudaLaunchConfig_t q = {};
    q.gridDim = dim3(2, 1, 1);
    q.blockDim = dim3(L::kThreads, 1, 1);
    q.dynamicSmemBytes = L::kDynamicBytes;
    cudaLaunchAttribute qa[1];
    qa[0].id = cudaLaunchAttributeClusterDimension;
    qa[0].val.clusterDim.x = 2;
    qa[0].val.clusterDim.y = 1;
    qa[0].val.clusterDim.z = 1;
    q.attrs = qa;
    q.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kern, &q) != cudaSuccess || clusters <= 0) {
      cudaGetLastError();
      clusters = sm_count() / 2;
    }
    resident[dev] = 2 * clusters;
  }
  grid = (grid < resident[dev] ? grid : resident[dev]) & ~1;
  if (grid < 2) return set_error(kErrUnsupported, "the CTA-pair kernel needs at least 2 SMs");
  kern<<<grid, L::kThreads, L::kDynamicBytes, stream>>>(tm_a, tm_b, tm_c, static_cast<__nv_bfloat16*>(c), a_scale, b_scale,
                                                        sizes, sizes_is_i64, num_groups, masked_stride, m_rows, n, k, b_map,
                                                        num_b, device_status_ptr());
  B200_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace b200
