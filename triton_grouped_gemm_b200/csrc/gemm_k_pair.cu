// CTA-pair (tcgen05 cta_group::2) K-grouped GEMM with the balanced scheduler: a cluster of two
// CTAs on two SMs works on one 256 x 256 tile of C[g] = A_g^T * B_g.  CTA r of the pair loads
// columns [128 r, +128) of the tile's A slice and of its B slice for every k-block (half the
// operand bytes per SM of the single-CTA kernel's 128 x 256 tile) and owns rows [128 r, +128) of
// the accumulator in its own TMEM; the leader (rank 0) issues the MMAs for both.
//
// Unlike the M-grouped pair kernel, a k-block here may need cleaning before it is multiplied
// (the last k-block of a group holds rows of the next group), and each CTA can only clean its
// own shared memory.  So every CTA tracks its own loads on its own full barrier, and the peer
// reports each stage to the leader through a relay warp once it is loaded (and cleaned):
//
//   full[s]        peer: 1 arrival + bytes (its TMA loads of stage s).  Leader: 2 arrivals + bytes:
//                  its own loads, and the peer's relay warp after the peer's full[s] (and
//                  cleaning) - one wait per k-block for the MMA warp, which the tensor core's
//                  shallow queue makes worth having (whatever the issuing warp does between two
//                  k-blocks is idle tensor time)
//   empty[s]       each CTA, 1 arrival: tcgen05.commit from the leader, delivered to both
//   tmem_full[a]   each CTA, 1 arrival: tcgen05.commit from the leader, delivered to both
//   tmem_empty[a]  leader, 8 arrivals: 4 epilogue warps x 2 CTAs
//   sched_full[i]  each CTA, 1 arrival: the leader's producer published tile i - id, group, token
//                  count, first token row - into both CTAs' rings (the peer's copy with a
//                  cluster-scope release); it claims and looks a tile up one tile ahead, in
//                  steps spread over the k-blocks it is loading
//   sched_empty[i] leader, 11 arrivals: every reader of ring slot i in both CTAs
//
// The latency of the relay is hidden by the depth of the operand ring; it is not on the path
// of any role that the tensor core waits for.
//
// Warp roles: 0 = TMA producer (the leader's also claims tiles with atomicAdd), 1 = MMA issuer
// (leader) / relay (peer), 2..5 = epilogue.
#include "../../include/b200gemm.h"
#include "common.cuh"
#include "gemm_tile.cuh"

namespace b200 {

constexpr int kKPairStages = 6;
constexpr int kKPairSchedDepth = 4;

struct KPairSmem {
  static constexpr int kABytes = 128 * 128;  // 16-bit: 2 chunks of [64 tokens][64 m]; fp8: [128 m][128 tokens]
  static constexpr int kBBytes = 128 * 128;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kEpiOffset = kKPairStages * kStageBytes;
  static constexpr int kBarOffset = kEpiOffset + 4 * kEpiStageBytesPerWarp;
  static constexpr int kNumBars = 2 * kKPairStages + 4 + 2 * kKPairSchedDepth;
  static constexpr int kDynamicBytes = kBarOffset + kNumBars * 8 + 16 + kKPairSchedDepth * 16 + 1024;
};

template <bool kFp8>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kNumThreads, 1)
k_grouped_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                      const __grid_constant__ CUtensorMap tm_c, void* __restrict__ c_ptr, int num_groups, int m_dim,
                      int n_dim, int in_fmt, int out_fp16, const float* __restrict__ a_scale,
                      const float* __restrict__ b_scale, int* __restrict__ scratch, unsigned* status) {
  using L = KPairSmem;
  constexpr int kStages = kKPairStages;
  constexpr int kDepth = kKPairSchedDepth;
  constexpr int kTokensPerKb = kFp8 ? 128 : kBlockK;
  constexpr int kTile = 256;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + L::kBarOffset;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tmem_full_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto tmem_empty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  auto sched_full_bar = [&](int i) { return bar_base + 8u * (2 * kStages + 4 + i); };
  auto sched_empty_bar = [&](int i) { return bar_base + 8u * (2 * kStages + 4 + kDepth + i); };
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem + L::kBarOffset + L::kNumBars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kBarOffset + L::kNumBars * 8 + 4);
  volatile int4* sched_info = reinterpret_cast<volatile int4*>(smem + L::kBarOffset + L::kNumBars * 8 + 16);
  const uint32_t sched_info_addr = bar_base + L::kNumBars * 8 + 16;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int m_tiles = (m_dim + kTile - 1) / kTile;
  const int n_tiles = (n_dim + kTile - 1) / kTile;
  const int tiles_per_group = m_tiles * n_tiles;
  const long long num_tiles = static_cast<long long>(tiles_per_group) * num_groups;
  constexpr uint32_t kTmemCols = 512;  // two 256-column accumulators

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), cluster_ctarank() == 0 ? 2 : 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tmem_full_bar(a), 1);
      mbar_init(tmem_empty_bar(a), 8);
    }
    for (int i = 0; i < kDepth; ++i) {
      mbar_init(sched_full_bar(i), 1);
      mbar_init(sched_empty_bar(i), 11);  // leader: MMA + 4 epilogue; peer: producer + relay + 4 epilogue
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

  const int* plan_starts = scratch + kPlanHeaderWords;
  const int* plan_tokens = plan_starts + num_groups;
  const int* plan_order = plan_tokens + num_groups;
  struct TileInfo {
    long long tile;  // -1: no more work (or a wait ran out)
    int g, mt, nt;
    long long tokens, start;
  };
  auto split_tile = [&](long long tile, int& mt, int& nt) {
    const int slot = static_cast<int>(tile / tiles_per_group);
    const int local = static_cast<int>(tile - static_cast<long long>(slot) * tiles_per_group);
    mt = local / n_tiles;
    nt = local - mt * n_tiles;
  };
  // i-th entry of this CTA's ring (every role except the leader's producer)
  auto ring_tile = [&](uint32_t i, unsigned role_bit) -> TileInfo {
    TileInfo ti;
    ti.tile = -1;
    const int slot = i % kDepth;
    if (!wait_bounded_cluster(sched_full_bar(slot), (i / kDepth) & 1u, abort_flag, status, role_bit)) return ti;
    const int t = sched_info[slot].x;
    ti.g = sched_info[slot].y;
    ti.tokens = sched_info[slot].z;
    ti.start = sched_info[slot].w;
    __syncwarp();
    if (lane == 0) mbar_arrive_cluster(sched_empty_bar(slot), 0);
    if (t < num_tiles) {
      ti.tile = t;
      split_tile(t, ti.mt, ti.nt);
    }
    return ti;
  };
  // zero token rows [valid, valid + zero_rows) of the four 64-column chunks of a stage (A: 2,
  // B: 2; a token row keeps its own 128 bytes under the swizzle) so that rows of the next group
  // in the last k-block of a group cannot contribute; 16-bit operands only
  auto clean_tail = [&](int stage, int valid, int zero_rows) {
    const int vec_per_chunk = zero_rows * 8;  // 16-byte vectors
    uint8_t* stage_ptr = smem + stage * L::kStageBytes;
    for (int i = lane; i < 4 * vec_per_chunk; i += 32) {
      const int ch = i / vec_per_chunk;
      const int v = i - ch * vec_per_chunk;
      *reinterpret_cast<uint4*>(stage_ptr + ch * (kBlockK * 128) + valid * 128 + v * 16) = make_uint4(0, 0, 0, 0);
    }
    fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core
    __syncwarp();
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    // Leader: the claim of the next tile (an atomic, ~1 us) and its two dependent plan look-ups
    // are issued one step per k-block while this tile's loads stream, with volatile instructions
    // so that each sits where it is written.
    int nx_t = 0, nx_g = 0, nx_tokens = 0, nx_start = 0, nx_step = 3;
    auto prefetch_step = [&]() {
      if (nx_step == 0) {
        if (lane == 0) asm volatile("atom.global.add.u32 %0, [%1], 1;" : "=r"(nx_t) : "l"(scratch) : "memory");
      } else if (nx_step == 1) {
        nx_t = __shfl_sync(0xFFFFFFFFu, nx_t, 0);
        if (nx_t < num_tiles)
          asm volatile("ld.global.nc.s32 %0, [%1];" : "=r"(nx_g) : "l"(plan_order + nx_t / tiles_per_group));
      } else if (nx_step == 2) {
        if (nx_t < num_tiles) {
          asm volatile("ld.global.nc.s32 %0, [%1];" : "=r"(nx_tokens) : "l"(plan_tokens + nx_g));
          asm volatile("ld.global.nc.s32 %0, [%1];" : "=r"(nx_start) : "l"(plan_starts + nx_g));
        }
      }
      ++nx_step;
    };
    if (rank == 0) nx_step = 0;
    for (uint32_t i = 0; ok; ++i) {
      TileInfo ti;
      if (rank == 0) {
        while (nx_step < 3) prefetch_step();  // first tile, or a tile with fewer than three k-blocks
        // publish the claimed tile (also the end marker) to both CTAs' rings
        const int slot = i % kDepth;
        if (!wait_bounded_cluster(sched_empty_bar(slot), ((i / kDepth) & 1u) ^ 1u, abort_flag, status,
                                  kDevTimeoutProducer))
          break;
        if (lane == 0) {
          sched_info[slot].x = nx_t;
          sched_info[slot].y = nx_g;
          sched_info[slot].z = nx_tokens;
          sched_info[slot].w = nx_start;
          st_shared_cluster_v4(sched_info_addr + 16u * slot, 1, nx_t, nx_g, nx_tokens, nx_start);
          mbar_arrive(sched_full_bar(slot));
          mbar_arrive_cluster_release(sched_full_bar(slot), 1);
        }
        __syncwarp();
        ti.tile = nx_t < num_tiles ? nx_t : -1;
        if (ti.tile >= 0) split_tile(ti.tile, ti.mt, ti.nt);
        ti.g = nx_g;
        ti.tokens = nx_tokens;
        ti.start = nx_start;
        nx_step = 0;
      } else {
        ti = ring_tile(i, kDevTimeoutProducer);
      }
      if (ti.tile < 0) break;
      const int mt = ti.mt, nt = ti.nt;
      const long long start = ti.start;
      const long long tokens = ti.tokens;
      const int num_kb = static_cast<int>((tokens + kTokensPerKb - 1) / kTokensPerKb);
      const int m0 = mt * kTile + static_cast<int>(rank) * 128;
      const int n0 = nt * kTile + static_cast<int>(rank) * 128;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag, status, kDevTimeoutProducer)) {
          ok = false;
          break;
        }
        if (lane == 0) {
          const uint32_t a_dst = smem_base + stage * L::kStageBytes;
          const uint32_t b_dst = a_dst + L::kABytes;
          const int krow = static_cast<int>(start + static_cast<long long>(kb) * kTokensPerKb);
          mbar_arrive_expect_tx(full_bar(stage), L::kStageBytes);
          if constexpr (kFp8) {
            tma_load_2d(a_dst, &tm_a, full_bar(stage), krow, m0);
            tma_load_2d(b_dst, &tm_b, full_bar(stage), krow, n0);
          } else {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              tma_load_2d(a_dst + j * (kBlockK * 128), &tm_a, full_bar(stage), m0 + j * 64, krow);
              tma_load_2d(b_dst + j * (kBlockK * 128), &tm_b, full_bar(stage), n0 + j * 64, krow);
            }
          }
        }
        __syncwarp();
        if (nx_step < 3) prefetch_step();
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1 && rank == 1) {
    // ------------------------------------------------------------ relay (peer CTA)
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (uint32_t i = 0; ok; ++i) {
      const TileInfo ti = ring_tile(i, kDevTimeoutMma);
      if (ti.tile < 0) break;
      const long long tokens = ti.tokens;
      const int num_kb = static_cast<int>((tokens + kTokensPerKb - 1) / kTokensPerKb);
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!wait_bounded(full_bar(stage), phase, abort_flag, status, kDevTimeoutMma)) {
          ok = false;
          break;
        }
        bool cleaned = false;
        if (!kFp8 && kb == num_kb - 1) {
          const int valid = static_cast<int>(tokens - static_cast<long long>(kb) * kBlockK);  // 1..64
          const int zero_rows = (valid + kUmmaK - 1) / kUmmaK * kUmmaK - valid;
          if (zero_rows > 0) {
            clean_tail(stage, valid, zero_rows);
            cleaned = true;
          }
        }
        if (lane == 0) {
          if (cleaned) mbar_arrive_cluster_release(full_bar(stage), 0);
          else mbar_arrive_cluster(full_bar(stage), 0);
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
    const uint32_t a_fmt = kFp8 ? static_cast<uint32_t>(in_fmt & 0xF) : static_cast<uint32_t>(in_fmt);
    const uint32_t b_fmt = kFp8 ? static_cast<uint32_t>((in_fmt >> 4) & 0xF) : static_cast<uint32_t>(in_fmt);
    const uint32_t mn_major = kFp8 ? 0u : 1u;
    const uint32_t idesc = make_instr_desc(a_fmt, b_fmt, mn_major, mn_major, kTile, kTile);
    int stage = 0;
    uint32_t phase = 0;
    uint32_t tile_iter = 0;  // counts non-empty tiles only (same rule in the epilogue)
    bool ok = true;
    for (uint32_t i = 0; ok; ++i) {
      const TileInfo ti = ring_tile(i, kDevTimeoutMma);
      if (ti.tile < 0) break;
      const long long tokens = ti.tokens;
      if (tokens == 0) continue;
      const int num_kb = static_cast<int>((tokens + kTokensPerKb - 1) / kTokensPerKb);
      const uint32_t acc = tile_iter & 1u;
      const uint32_t acc_phase = (tile_iter >> 1) & 1u;
      ++tile_iter;
      if (!wait_bounded_cluster(tmem_empty_bar(acc), acc_phase ^ 1u, abort_flag, status, kDevTimeoutMma)) break;
      tc_fence_after_sync();
      const uint32_t d_tmem = tmem_base + acc * kTile;
      for (int kb = 0; kb < num_kb; ++kb) {
        // both CTAs' operands of this k-block have landed (and the peer's are cleaned)
        if (!wait_bounded_cluster(full_bar(stage), phase, abort_flag, status, kDevTimeoutMma)) {
          ok = false;
          break;
        }
        int k16_steps = kFp8 ? 4 : kBlockK / kUmmaK;
        if (!kFp8 && kb == num_kb - 1) {
          const int valid = static_cast<int>(tokens - static_cast<long long>(kb) * kBlockK);  // 1..64
          k16_steps = (valid + kUmmaK - 1) / kUmmaK;
          const int zero_rows = k16_steps * kUmmaK - valid;
          if (zero_rows > 0) clean_tail(stage, valid, zero_rows);
        }
        tc_fence_after_sync();
        if (lane == 0) {
          const uint32_t a_addr = smem_base + stage * L::kStageBytes;
          const uint32_t b_addr = a_addr + L::kABytes;
          for (int k16 = 0; k16 < k16_steps; ++k16) {
            // MN-major: a K step is 16 token rows of 128 bytes; K-major (fp8): 32 bytes in a row
            const uint32_t step = kFp8 ? 32u : kUmmaK * 128u;
            const uint32_t lbo = kFp8 ? 16u : kBlockK * 128u;
            const uint64_t a_desc = make_smem_desc(a_addr + k16 * step, lbo, 1024, kSwizzle128);
            const uint64_t b_desc = make_smem_desc(b_addr + k16 * step, lbo, 1024, kSwizzle128);
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
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int quarter = warp & 3;
    uint8_t* epi_stage = smem + L::kEpiOffset + quarter * kEpiStageBytesPerWarp;
    int epi_sel = 0;
    uint32_t tile_iter = 0;
    for (uint32_t i = 0;; ++i) {
      const TileInfo ti = ring_tile(i, kDevTimeoutEpilogue);
      if (ti.tile < 0) break;
      const int g = ti.g, mt = ti.mt, nt = ti.nt;
      const long long tokens = ti.tokens;
      const int row_w0 = mt * kTile + static_cast<int>(rank) * 128 + quarter * 32;
      const int row = row_w0 + lane;
      const bool row_ok = row < m_dim;
      uint16_t* c_row = static_cast<uint16_t*>(c_ptr) +
                        (static_cast<long long>(g) * m_dim + row) * static_cast<long long>(n_dim);
      if (tokens == 0) {
        store_zero_row_16bit<kTile>(c_row, row_ok, nt * kTile, n_dim);
        continue;
      }
      const uint32_t acc = tile_iter & 1u;
      const uint32_t acc_phase = (tile_iter >> 1) & 1u;
      ++tile_iter;
      if (!wait_bounded(tmem_full_bar(acc), acc_phase, abort_flag, status, kDevTimeoutEpilogue)) break;
      tc_fence_after_sync();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kTile;
      float rs = 1.0f;
      const float* cs = nullptr;
      if constexpr (kFp8) {
        rs = row_ok ? __ldg(a_scale + static_cast<long long>(g) * m_dim + row) : 0.f;
        cs = b_scale + static_cast<long long>(g) * n_dim;
      }
      if (row_w0 + 32 <= m_dim)
        store_acc_warp_tma<kTile, kFp8>(t_addr, &tm_c, epi_stage, epi_sel, row_w0, g, nt * kTile, n_dim, out_fp16, lane,
                                        rs, cs);
      else
        store_acc_row_16bit<kTile, kFp8>(t_addr, c_row, row_ok, nt * kTile, n_dim, out_fp16, rs, cs);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tmem_empty_bar(acc), 0);
    }
    if (lane == 0) tma_store_wait_all<0>();
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

template <bool kFp8>
int launch_k_grouped_pair(const CUtensorMap& tm_a, const CUtensorMap& tm_b, const CUtensorMap& tm_c, void* c,
                          int num_groups, int m_dim, int n_dim, int in_fmt, int out_fp16, const float* a_scale,
                          const float* b_scale, int* scratch, int want_ctas, cudaStream_t stream) {
  auto kern = k_grouped_pair_kernel<kFp8>;
  B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, KPairSmem::kDynamicBytes));
  static int resident[64] = {0};
  int dev = 0;
  B200_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return set_error(kErrUnsupported, "device index %d out of range", dev);
  if (!resident[dev]) {
    // a cluster of two CTAs per tile; keep only as many CTAs as are co-resident
    cudaLaunchConfig_t q = {};
    q.gridDim = dim3(2, 1, 1);
    q.blockDim = dim3(kNumThreads, 1, 1);
    q.dynamicSmemBytes = KPairSmem::kDynamicBytes;
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
  int grid = resident[dev];
  if (want_ctas > 0 && (want_ctas & ~1) < grid) grid = want_ctas & ~1;
  if (grid < 2) return set_error(kErrUnsupported, "the CTA-pair kernel needs at least 2 SMs");
  kern<<<grid, kNumThreads, KPairSmem::kDynamicBytes, stream>>>(tm_a, tm_b, tm_c, c, num_groups, m_dim, n_dim, in_fmt,
                                                                out_fp16, a_scale, b_scale, scratch,
                                                                device_status_ptr());
  B200_CUDA(cudaGetLastError());
  return 0;
}

template int launch_k_grouped_pair<false>(const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, void*, int, int,
                                          int, int, int, const float*, const float*, int*, int, cudaStream_t);
template int launch_k_grouped_pair<true>(const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, void*, int, int,
                                         int, int, int, const float*, const float*, int*, int, cudaStream_t);

}  // namespace b200
