// CTA-pair (tcgen05 cta_group::2) M-grouped GEMM: a cluster of two CTAs on two SMs works on
// one 256 x 256 output tile.  CTA r of the pair owns rows [128 r, 128 r + 128) of the tile
// (its own A slice and its own 128 TMEM lanes) and supplies columns [128 r, 128 r + 128) of
// B_g; the leader CTA (rank 0) issues one tcgen05.mma.cta_group::2 per K step that reads both
// CTAs' shared memory and writes both CTAs' TMEM.  Per CTA and k-block this loads 16 KB of A
// and 16 KB of B instead of 16 + 32 KB, which takes a third off the shared-memory and L2
// traffic of the single-CTA kernel.  No multicast: each CTA fetches its own slices with
// plain (cta_group::2) TMA loads that signal the leader's mbarrier.
//
// Barriers (same shared-memory offsets in both CTAs):
//   full[s]        leader only, 1 arrival (the leader's producer expects the bytes of both CTAs;
//                  both CTAs' TMA loads complete on it)
//   empty[s]       in each CTA, 1 arrival: tcgen05.commit from the leader, delivered to both
//   tmem_full[a]   in each CTA, 1 arrival: tcgen05.commit from the leader, delivered to both
//   tmem_empty[a]  leader only, 8 arrivals (4 epilogue warps x 2 CTAs, remote arrive)
//
// Tiles are numbered in padded tile space with 256-row tiles; when a group's last tile holds
// <= 128 rows the second CTA of the pair computes rows it never stores.
#include "../../include/b200gemm.h"
#include "common.cuh"
#include "gemm_tile.cuh"

namespace b200 {

constexpr int kPairTileM = 256;
constexpr int kPairTileN = 256;
constexpr int kPairStages = 6;

struct PairSmem {
  static constexpr int kABytes = 128 * 128;
  static constexpr int kBBytes = 128 * 128;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kEpiOffset = kPairStages * kStageBytes;
  static constexpr int kBarOffset = kEpiOffset + 4 * kEpiStageBytesPerWarp;
  static constexpr int kNumBars = 2 * kPairStages + 4;
  static constexpr int kDynamicBytes = kBarOffset + kNumBars * 8 + 16 + 1024;
};

template <bool kBMnMajor, bool kFp8>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kNumThreads, 1)
m_grouped_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                      const __grid_constant__ CUtensorMap tm_c, void* __restrict__ c_ptr,
                      const void* __restrict__ sizes, int sizes_i64, int num_groups, int masked_stride,
                      long long m_rows, int n, int k, int in_fmt, int out_fp16, const float* __restrict__ a_scale,
                      const float* __restrict__ b_scale, unsigned* status) {
  static_assert(!(kFp8 && kBMnMajor), "fp8 operands are K-major only");
  using L = PairSmem;
  constexpr int kStages = kPairStages;
  constexpr int kElemsPerKb = kFp8 ? 128 : 64;
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
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int n_tiles = (n + kPairTileN - 1) / kPairTileN;
  const int num_kb = (k + kElemsPerKb - 1) / kElemsPerKb;
  constexpr uint32_t kTmemCols = 512;  // two 256-column accumulators

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tmem_full_bar(a), 1);
      mbar_init(tmem_empty_bar(a), 8);
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
  cluster_sync_all();  // both CTAs' barriers exist before anyone signals across the pair
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    GroupWalker w;
    w.init(sizes, sizes_i64, num_groups, masked_stride, kPairTileM, m_rows);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = pair_id; ok; tile += num_pairs) {
      const int mt = tile / n_tiles;
      const int nt = tile - mt * n_tiles;
      if (!w.seek(mt)) break;
      const int row0 = static_cast<int>(w.tile_row0(mt)) + static_cast<int>(rank) * 128;
      const int col0 = nt * kPairTileN + static_cast<int>(rank) * 128;
      const int g = w.g;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag, status, kDevTimeoutProducer)) {
          ok = false;
          break;
        }
        if (lane == 0) {
          const uint32_t a_dst = smem_base + stage * L::kStageBytes;
          const uint32_t b_dst = a_dst + L::kABytes;
          const uint32_t leader_full = mapa_u32(full_bar(stage), 0);
          // one arrival per phase, made by the leader for the bytes of BOTH CTAs; the peer's
          // copies may complete on the leader's barrier before this expect-tx is posted, which
          // only drives the pending byte count negative until the arrival lands.  (A second,
          // remote arrive.expect_tx from the peer serialises the pipeline: ~0.7 us per k-block.)
          if (rank == 0) mbar_arrive_expect_tx(full_bar(stage), 2 * L::kStageBytes);
          tma_load_2d_pair(a_dst, &tm_a, leader_full, kb * kElemsPerKb, row0);
          if constexpr (!kBMnMajor) {
            tma_load_3d_pair(b_dst, &tm_b, leader_full, kb * kElemsPerKb, col0, g);
          } else {
#pragma unroll
            for (int j = 0; j < 2; ++j)
              tma_load_3d_pair(b_dst + j * (kBlockK * 128), &tm_b, leader_full, col0 + j * 64, kb * kBlockK, g);
          }
        }
        __syncwarp();
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (rank == 0) {
      GroupWalker w;
      w.init(sizes, sizes_i64, num_groups, masked_stride, kPairTileM, m_rows);
      const uint32_t a_fmt = kFp8 ? static_cast<uint32_t>(in_fmt & 0xF) : static_cast<uint32_t>(in_fmt);
      const uint32_t b_fmt = kFp8 ? static_cast<uint32_t>((in_fmt >> 4) & 0xF) : static_cast<uint32_t>(in_fmt);
      const uint32_t idesc = make_instr_desc(a_fmt, b_fmt, 0u, kBMnMajor ? 1u : 0u, kPairTileM, kPairTileN);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t tile_iter = 0;
      bool ok = true;
      for (int tile = pair_id; ok; tile += num_pairs, ++tile_iter) {
        const int mt = tile / n_tiles;
        if (!w.seek(mt)) break;
        const uint32_t acc = tile_iter & 1u;
        const uint32_t acc_phase = (tile_iter >> 1) & 1u;
        if (!wait_bounded(tmem_empty_bar(acc), acc_phase ^ 1u, abort_flag, status, kDevTimeoutMma)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * kPairTileN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wait_bounded(full_bar(stage), phase, abort_flag, status, kDevTimeoutMma)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          if (lane == 0) {
            const uint32_t a_addr = smem_base + stage * L::kStageBytes;
            const uint32_t b_addr = a_addr + L::kABytes;
#pragma unroll
            for (int k16 = 0; k16 < 4; ++k16) {
              const uint64_t a_desc = make_smem_desc(a_addr + k16 * 32, 16, 1024, kSwizzle128);
              const uint64_t b_desc =
                  kBMnMajor ? make_smem_desc(b_addr + k16 * (kUmmaK * 128), kBlockK * 128, 1024, kSwizzle128)
                            : make_smem_desc(b_addr + k16 * 32, 16, 1024, kSwizzle128);
              umma<2, kFp8>(d_tmem, a_desc, b_desc, idesc, (kb | k16) != 0 ? 1u : 0u);
            }
            umma_commit_2cta(empty_bar(stage), 0x3);
          }
          __syncwarp();
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok && lane == 0) umma_commit_2cta(tmem_full_bar(acc), 0x3);
        __syncwarp();
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    GroupWalker w;
    w.init(sizes, sizes_i64, num_groups, masked_stride, kPairTileM, m_rows);
    const int quarter = warp & 3;
    uint8_t* epi_stage = smem + L::kEpiOffset + quarter * kEpiStageBytesPerWarp;
    int epi_sel = 0;
    uint32_t tile_iter = 0;
    for (int tile = pair_id;; tile += num_pairs, ++tile_iter) {
      const int mt = tile / n_tiles;
      const int nt = tile - mt * n_tiles;
      if (!w.seek(mt)) break;
      const long long row_w0 = w.tile_row0(mt) + static_cast<long long>(rank) * 128 + quarter * 32;
      const long long row = row_w0 + lane;
      const bool row_ok = row < w.group_row_end();
      const uint32_t acc = tile_iter & 1u;
      const uint32_t acc_phase = (tile_iter >> 1) & 1u;
      if (!wait_bounded(tmem_full_bar(acc), acc_phase, abort_flag, status, kDevTimeoutEpilogue)) break;
      tc_fence_after_sync();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kPairTileN;
      uint16_t* c_row = static_cast<uint16_t*>(c_ptr) + row * static_cast<long long>(n);
      float rs = 1.0f;
      const float* cs = nullptr;
      if constexpr (kFp8) {
        rs = row_ok ? __ldg(a_scale + row) : 0.f;
        cs = b_scale + static_cast<long long>(w.g) * n;
      }
      if (row_w0 + 32 <= w.group_row_end())
        store_acc_warp_tma<kPairTileN, kFp8>(t_addr, &tm_c, epi_stage, epi_sel, static_cast<int>(row_w0), -1,
                                             nt * kPairTileN, n, out_fp16, lane, rs, cs);
      else
        store_acc_row_16bit<kPairTileN, kFp8>(t_addr, c_row, row_ok, nt * kPairTileN, n, out_fp16, rs, cs);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tmem_empty_bar(acc), 0);
    }
    if (lane == 0) tma_store_wait_all<0>();
    if (w.overflow && rank == 0 && quarter == 0 && lane == 0 && status) atomicOr(status, kDevBadGroupSize);
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(4000);
  }
  cluster_sync_all();  // neither CTA leaves while the peer may still signal it or write its TMEM
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<2>(tmem_base, kTmemCols);
  }
}

// number of CTAs (an even count) of a persistent launch of `kern` that are co-resident
template <typename Kern>
static int pair_grid_size(Kern kern, int smem_bytes, int want_ctas) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2, 1, 1);
  cfg.blockDim = dim3(kNumThreads, 1, 1);
  cfg.dynamicSmemBytes = smem_bytes;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg) != cudaSuccess || clusters <= 0) {
    cudaGetLastError();
    clusters = want_ctas / 2;
  }
  int ctas = 2 * clusters;
  if (ctas > (want_ctas & ~1)) ctas = want_ctas & ~1;
  return ctas;
}

template <bool kBMnMajor, bool kFp8>
int launch_m_grouped_pair(const CUtensorMap& tm_a, const CUtensorMap& tm_b, const CUtensorMap& tm_c, void* c,
                          const void* sizes, int sizes_is_i64, int num_groups, int masked_stride, long long m_rows,
                          int n, int k, int in_fmt, int out_fp16, const float* a_scale, const float* b_scale,
                          int want_ctas, cudaStream_t stream) {
  auto kern = m_grouped_pair_kernel<kBMnMajor, kFp8>;
  B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PairSmem::kDynamicBytes));
  static int cached_grid[64] = {0};
  int dev = 0;
  B200_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return set_error(kErrUnsupported, "device index %d out of range", dev);
  if (!cached_grid[dev]) cached_grid[dev] = pair_grid_size(kern, PairSmem::kDynamicBytes, sm_count());
  int grid = cached_grid[dev];
  if (want_ctas > 0 && (want_ctas & ~1) < grid) grid = want_ctas & ~1;
  if (grid < 2) return set_error(kErrUnsupported, "the CTA-pair kernel needs at least 2 SMs");
  kern<<<grid, kNumThreads, PairSmem::kDynamicBytes, stream>>>(tm_a, tm_b, tm_c, c, sizes, sizes_is_i64, num_groups,
                                                               masked_stride, m_rows, n, k, in_fmt, out_fp16, a_scale,
                                                               b_scale, device_status_ptr());
  B200_CUDA(cudaGetLastError());
  return 0;
}

// CTAs a persistent launch of the 16-bit pair kernel uses on the current device (0 = error)
int pair_kernel_grid() {
  auto kern = m_grouped_pair_kernel<false, false>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PairSmem::kDynamicBytes) != cudaSuccess)
    return 0;
  return pair_grid_size(kern, PairSmem::kDynamicBytes, sm_count());
}

template int launch_m_grouped_pair<false, false>(const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, void*,
                                                 const void*, int, int, int, long long, int, int, int, int, const float*,
                                                 const float*, int, cudaStream_t);
template int launch_m_grouped_pair<true, false>(const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, void*,
                                                const void*, int, int, int, long long, int, int, int, int, const float*,
                                                const float*, int, cudaStream_t);
template int launch_m_grouped_pair<false, true>(const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, void*,
                                                const void*, int, int, int, long long, int, int, int, int, const float*,
                                                const float*, int, cudaStream_t);

}  // namespace b200
