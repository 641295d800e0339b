// Block-scaled FP8 (e4m3) K-grouped GEMM for sm_100a: the expert weight gradient in FP8.
//
//   out[g, m, n] = sum_{kb in group g} ( sum_{t in kb} x8[m, t] * y8[n, t] ) * xs[m/128, kb] * ys[n/128, kb]   -> bf16
//
// Both operands are outputs of the transposing 128x128 quantiser (b200quant_trans_expand_128x,
// the reference's quant/trans_per_block_quant_expand_128x.py:135-208): x8 [m_dim, m_expand] and
// y8 [n_dim, m_expand] hold the tokens along their inner axis, every expert's tokens padded to a
// multiple of 128, with one fp32 scale per 128x128 block ([dim/128, m_expand/128]).  A k-block of
// 128 tokens therefore never straddles two experts, and the scale of a k-block is ONE scalar per
// 128x128 sub-tile of the output: xs[row block, kb] * ys[column block, kb].  The reference ships
// that quantiser but no kernel that consumes its layout; this one follows the skeleton of its
// per-channel FP8 K-grouped kernel (gemm/FP8/k_grouped_gemm_channel_expert.py:64-140: K-major
// operands, 128-token blocks, tile -> (group, m tile, n tile)).
//
// Structure: the software-promotion pipeline of the block-scaled M-grouped kernel
// (gemm_fp8_block.cu).  Every 128-token k-block is multiplied into a fresh TMEM buffer (two
// alternate), the promotion warps read it with tcgen05.ld, multiply by the k-block's scalar and
// accumulate in fp32 registers; after a group's last k-block the accumulators are rounded once
// and stored with TMA (3-D map over [G, m_dim, n_dim], which clips the m and n tails).
// Experts differ tenfold in tokens and a tile's cost follows its expert's token count; with a
// workspace (the K-grouped kernels' plan: starts, token counts, longest-first order) tiles are
// handed out round-robin in longest-first order, which gives every CTA the same mix.
//   warp 0   TMA producer      warps 1, 2   MMA issuers (pair: leader CTA only; warp 1 owns TMEM buffer 0, warp 2 buffer 1)      warp 3  idle
//   warps 4..11  promotion + epilogue: warp (quarter = warp % 4, half = (warp - 4) / 4) owns TMEM
//                lanes [32 quarter, +32) and columns [128 half, +128) = one scale block of y
// kPair: two CTAs on two SMs share a 256 x 256 tile (tcgen05 cta_group::2), CTA r holding rows
// [128 r, +128) of x and of the accumulator and supplying rows [128 r, +128) of y.
#include <cuda_bf16.h>

#include "../../include/b200gemm.h"
#include "common.cuh"
#include "gemm_tile.cuh"

namespace b200 {

template <bool kPair>
struct Fp8BlockKCfg {
  static constexpr int kBlockN = 256;
  static constexpr int kStages = kPair ? 5 : 3;
  static constexpr int kBRows = kPair ? 128 : kBlockN;
  static constexpr int kPromoWarps = 8;
  static constexpr int kThreads = 128 + 32 * kPromoWarps;
  static constexpr int kABytes = kBlockM * 128;
  static constexpr int kBBytes = kBRows * 128;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kEpiOffset = kStages * kStageBytes;  // one 4 KB store-staging buffer per promotion warp
  static constexpr int kBarOffset = kEpiOffset + 8 * 32 * 128;
  static constexpr int kNumBars = 2 * kStages + 4;  // full / empty ring, tmem_full[2], tmem_empty[2]
  static constexpr int kDynamicBytes = kBarOffset + kNumBars * 8 + 16 + 1024;
};

// Token ranges of the groups in units of 128-token k-blocks: group g covers k-blocks
// [kb0, kb0 + nkb).  Sizes are the padded token counts (multiples of 128); a negative size counts
// as zero and nothing beyond kb_total is ever addressed.
struct KBlockWalker {
  const void* sizes;
  int sizes_i64;
  int num_groups;
  long long kb_total;
  int g;
  long long kb0;
  int nkb;

  __device__ __forceinline__ int load(int i) const {
    long long v = sizes_i64 ? static_cast<const long long*>(sizes)[i]
                            : static_cast<long long>(static_cast<const int*>(sizes)[i]);
    if (v < 0) v = 0;
    long long blocks = (v + 127) >> 7;
    const long long room = kb_total - kb0;
    if (blocks > room) blocks = room > 0 ? room : 0;
    return static_cast<int>(blocks);
  }
  __device__ __forceinline__ void init(const void* sizes_, int sizes_i64_, int num_groups_, long long kb_total_) {
    sizes = sizes_;
    sizes_i64 = sizes_i64_;
    num_groups = num_groups_;
    kb_total = kb_total_;
    g = 0;
    kb0 = 0;
    nkb = num_groups > 0 ? load(0) : 0;
  }
  // move to group `target` (must not decrease between calls)
  __device__ __forceinline__ void seek(int target) {
    while (g < target && g < num_groups) {
      kb0 += nkb;
      ++g;
      nkb = g < num_groups ? load(g) : 0;
    }
  }
  // Slot `slot` of the tile order.  Without a plan the slot IS the group (walk the sizes).  With a
  // plan (starts[G], tokens[G], order[G] written by the plan kernel) slot s is the group with the
  // s-th most tokens: experts differ tenfold in tokens, and handing the tiles out round-robin in
  // that order gives every CTA the same mix of long and short tiles.  Returns the group.
  __device__ __forceinline__ int locate(int slot, const int* __restrict__ plan) {
    if (!plan) {
      seek(slot);
      return slot;
    }
    const int* starts = plan + kPlanHeaderWords;
    const int grp = __ldg(starts + 2 * num_groups + slot);
    long long first = __ldg(starts + grp) >> 7;
    long long blocks = (static_cast<long long>(__ldg(starts + num_groups + grp)) + 127) >> 7;
    if (first > kb_total) first = kb_total;
    if (blocks > kb_total - first) blocks = kb_total - first;
    g = grp;
    kb0 = first;
    nkb = static_cast<int>(blocks);
    return grp;
  }
};

template <bool kPair>
__global__ void __launch_bounds__(Fp8BlockKCfg<kPair>::kThreads, 1)
fp8_block_k_grouped_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_y,
                           const __grid_constant__ CUtensorMap tm_c, const float* __restrict__ x_scale,
                           const float* __restrict__ y_scale, const void* __restrict__ sizes, int sizes_i64,
                           int num_groups, int m_dim, int n_dim, long long kb_total, const int* __restrict__ plan,
                           unsigned* status) {
  using L = Fp8BlockKCfg<kPair>;
  constexpr int kBlockN = L::kBlockN;
  constexpr int kStages = L::kStages;
  constexpr int kCtas = kPair ? 2 : 1;
  constexpr int kTileM = kBlockM * kCtas;
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
  const uint32_t rank = kPair ? cluster_ctarank() : 0u;
  const int first_tile = kPair ? (blockIdx.x >> 1) : blockIdx.x;
  const int tile_step = kPair ? (gridDim.x >> 1) : gridDim.x;
  // Tiles are handed out in rounds of tile_step, alternately forwards and backwards (round r gives
  // this CTA tile r * tile_step + first_tile, or ... + tile_step - 1 - first_tile when r is odd):
  // with the experts in order of falling token count a plain round-robin gives the first CTAs the
  // longer tile of every round, and the excess adds up to the difference between the longest and
  // the shortest tile.  Every role computes the same sequence.
  auto tile_of_round = [&](long long r) -> long long {
    return r * tile_step + ((r & 1) ? (tile_step - 1 - first_tile) : first_tile);
  };
  const int m_tiles = (m_dim + kTileM - 1) / kTileM;
  const int n_tiles = (n_dim + kBlockN - 1) / kBlockN;
  const int tiles_per_group = m_tiles * n_tiles;
  const long long total_tiles = static_cast<long long>(tiles_per_group) * num_groups;
  const int m_blocks = (m_dim + 127) >> 7;
  const int n_blocks = (n_dim + 127) >> 7;
  constexpr uint32_t kTmemCols = 2 * kBlockN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tmem_full_bar(a), 1);
      mbar_init(tmem_empty_bar(a), L::kPromoWarps * kCtas);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tmap(&tm_x);
    prefetch_tmap(&tm_y);
    prefetch_tmap(&tm_c);
  }
  if (warp == 1) {
    tmem_alloc<kCtas>(smem_u32(const_cast<uint32_t*>(tmem_holder)), kTmemCols);
    tmem_relinquish<kCtas>();
  }
  tc_fence_before_sync();
  if constexpr (kPair) cluster_sync_all();
  else __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp < 4) {
    warpgroup_reg_dec<56>();
    if (warp == 0) {
      // ------------------------------------------------------------ TMA producer
      KBlockWalker w;
      w.init(sizes, sizes_i64, num_groups, kb_total);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (long long round = 0, tile = tile_of_round(0); ok && tile < total_tiles; tile = tile_of_round(++round)) {
        const int slot = static_cast<int>(tile / tiles_per_group);
        const int r = static_cast<int>(tile - static_cast<long long>(slot) * tiles_per_group);
        const int mt = r / n_tiles;
        const int nt = r - mt * n_tiles;
        w.locate(slot, plan);
        const int row0 = mt * kTileM + static_cast<int>(rank) * kBlockM;
        const int col0 = nt * kBlockN + static_cast<int>(rank) * L::kBRows;
        for (int kb = 0; kb < w.nkb; ++kb) {
          if (!wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag, status, kDevTimeoutProducer)) {
            ok = false;
            break;
          }
          if (lane == 0) {
            const uint32_t a_dst = smem_base + stage * L::kStageBytes;
            const int tok0 = static_cast<int>((w.kb0 + kb) << 7);
            if constexpr (kPair) {
              const uint32_t leader_full = mapa_u32(full_bar(stage), 0);
              if (rank == 0) mbar_arrive_expect_tx(full_bar(stage), 2 * L::kStageBytes);
              tma_load_2d_pair(a_dst, &tm_x, leader_full, tok0, row0);
              tma_load_2d_pair(a_dst + L::kABytes, &tm_y, leader_full, tok0, col0);
            } else {
              mbar_arrive_expect_tx(full_bar(stage), L::kStageBytes);
              tma_load_2d(a_dst, &tm_x, full_bar(stage), tok0, row0);
              tma_load_2d(a_dst + L::kABytes, &tm_y, full_bar(stage), tok0, col0);
            }
          }
          __syncwarp();
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    } else if (warp == 1 || warp == 2) {
      // ------------------------------------------------------------ MMA issuers (pair: leader only).  Warp 1 issues
      // the k-blocks of TMEM buffer 0, warp 2 those of buffer 1: a warp is blocked in its
      // tcgen05.mma instructions for a good part of a k-block and holds up the promotion warps
      // on its scheduler; two issuers on two schedulers halve that for each of them.
      KBlockWalker w;
      w.init(sizes, sizes_i64, num_groups, kb_total);
      const uint32_t idesc = make_instr_desc(0u, 0u, 0u, 0u, kTileM, kBlockN);  // e4m3 x e4m3 -> f32
      int stage = 0;
      uint32_t phase = 0;
      uint32_t it = 0;  // k-blocks issued so far: TMEM buffer = it & 1
      bool ok = rank == 0;
      for (long long round = 0, tile = tile_of_round(0); ok && tile < total_tiles; tile = tile_of_round(++round)) {
        w.locate(static_cast<int>(tile / tiles_per_group), plan);
        for (int kb = 0; kb < w.nkb; ++kb, ++it) {
          const uint32_t buf = it & 1u;
          const uint32_t buf_phase = (it >> 1) & 1u;
          if (buf != static_cast<uint32_t>(warp - 1)) {  // the other issuer's k-block
            if (++stage == kStages) {
              stage = 0;
              phase ^= 1u;
            }
            continue;
          }
          // operands first, then the drained buffer: the MMAs go out the moment it is handed back
          if (!wait_bounded(full_bar(stage), phase, abort_flag, status, kDevTimeoutMma) ||
              !wait_bounded(tmem_empty_bar(buf), buf_phase ^ 1u, abort_flag, status, kDevTimeoutMma)) {
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
              umma<kCtas, true>(d_tmem, a_desc, b_desc, idesc, k32 != 0 ? 1u : 0u);
            }
            if constexpr (kPair) {
              umma_commit_2cta(empty_bar(stage), 0x3);
              umma_commit_2cta(tmem_full_bar(buf), 0x3);
            } else {
              umma_commit_1cta(empty_bar(stage));
              umma_commit_1cta(tmem_full_bar(buf));
            }
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
    KBlockWalker w;
    w.init(sizes, sizes_i64, num_groups, kb_total);
    const int quarter = warp & 3;
    const int half = (warp - 4) >> 2;
    uint32_t it = 0;
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + half * 128;
    uint8_t* stage_buf = smem + L::kEpiOffset + (warp - 4) * (32 * 128);
    bool ok = true;
    for (long long round = 0, tile = tile_of_round(0); ok && tile < total_tiles; tile = tile_of_round(++round)) {
      const int slot = static_cast<int>(tile / tiles_per_group);
      const int r = static_cast<int>(tile - static_cast<long long>(slot) * tiles_per_group);
      const int mt = r / n_tiles;
      const int nt = r - mt * n_tiles;
      const int g = w.locate(slot, plan);
      const int row_w0 = mt * kTileM + static_cast<int>(rank) * kBlockM + quarter * 32;
      const int col_base = nt * kBlockN + half * 128;
      // the k-block's scalar: xs[row block, kb] * ys[column block, kb], the same for the whole warp
      int rb = (mt * kTileM + static_cast<int>(rank) * kBlockM) >> 7;
      if (rb >= m_blocks) rb = m_blocks - 1;  // rows past m_dim: results are clipped by the store
      int nb = col_base >> 7;
      if (nb >= n_blocks) nb = n_blocks - 1;
      const float* xs_row = x_scale + static_cast<long long>(rb) * kb_total + w.kb0;
      const float* ys_row = y_scale + static_cast<long long>(nb) * kb_total + w.kb0;
      unsigned long long acc2[64];
#pragma unroll
      for (int j = 0; j < 64; ++j) acc2[j] = 0ull;
      const int nkb = w.nkb;
      if (nkb > 0) {
        uint32_t t[64];
        float fa_next = __ldg(xs_row), fb_next = __ldg(ys_row);
        if (!wait_bounded(tmem_full_bar(it & 1u), (it >> 1) & 1u, abort_flag, status, kDevTimeoutPromote)) break;
        tc_fence_after_sync();
        tmem_ld_32x32b_x64(t_lane + (it & 1u) * kBlockN, t);
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const float s_cur = fa_next * fb_next;
          const unsigned long long s2 = pack_f32x2(__float_as_uint(s_cur), __float_as_uint(s_cur));
          const bool more = kb + 1 < nkb;
          const uint32_t buf = it & 1u;
          const uint32_t t_addr = t_lane + buf * kBlockN;
          tmem_ld_wait();
          if (more) {  // next k-block's scale factors: this k-block's FMAs cover their latency
            fa_next = __ldg(xs_row + kb + 1);
            fb_next = __ldg(ys_row + kb + 1);
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) fma_f32x2(acc2[j], s2, pack_f32x2(t[2 * j], t[2 * j + 1]));
          tmem_ld_32x32b_x64(t_addr + 64, t);
          tmem_ld_wait();
          // every column of this buffer is in registers now: hand it back to the MMA warp
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            if constexpr (kPair) mbar_arrive_cluster(tmem_empty_bar(buf), 0);
            else mbar_arrive(tmem_empty_bar(buf));
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) fma_f32x2(acc2[32 + j], s2, pack_f32x2(t[2 * j], t[2 * j + 1]));
          if (more) {
            const uint32_t nit = it + 1;
            if (!wait_bounded(tmem_full_bar(nit & 1u), (nit >> 1) & 1u, abort_flag, status, kDevTimeoutPromote)) {
              ok = false;
              break;
            }
            tc_fence_after_sync();
            tmem_ld_32x32b_x64(t_lane + (nit & 1u) * kBlockN, t);
          }
        }
        if (!ok) break;
      }
      // round once, stage in the 128-byte-swizzle layout, TMA-store 64-column chunks; the 3-D map
      // clips rows >= m_dim and columns >= n_dim (an empty group stores its zero accumulators)
      float acc[128];
#pragma unroll
      for (int j = 0; j < 64; ++j) unpack_f32x2(acc2[j], acc[2 * j], acc[2 * j + 1]);
      if (row_w0 < m_dim) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int col0 = col_base + c * 64;
          if (col0 < n_dim) {
            if (lane == 0) tma_store_wait_read<0>();
            __syncwarp();
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              uint32_t p[4];
#pragma unroll
              for (int e = 0; e < 4; ++e)
                p[e] = pack2_16bit(acc[c * 64 + v * 8 + 2 * e], acc[c * 64 + v * 8 + 2 * e + 1], 0);
              *reinterpret_cast<uint4*>(stage_buf + lane * 128 + ((v ^ (lane & 7)) << 4)) =
                  make_uint4(p[0], p[1], p[2], p[3]);
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_3d(&tm_c, smem_u32(stage_buf), col0, row_w0, g);
              tma_store_commit();
            }
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
  if constexpr (kPair) cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<kCtas>(tmem_base, kTmemCols);
  }
}

template <bool kPair>
static int launch_fp8_block_k(const CUtensorMap& tm_x, const CUtensorMap& tm_y, const CUtensorMap& tm_c,
                              const float* x_scale, const float* y_scale, const void* sizes, int sizes_is_i64,
                              int num_groups, int m_dim, int n_dim, long long kb_total, const int* plan, int grid,
                              cudaStream_t stream) {
  using L = Fp8BlockKCfg<kPair>;
  auto kern = fp8_block_k_grouped_kernel<kPair>;
  B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes));
  if constexpr (kPair) {
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
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(L::kThreads, 1, 1);
    cfg.dynamicSmemBytes = L::kDynamicBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    B200_CUDA(cudaLaunchKernelEx(&cfg, kern, tm_x, tm_y, tm_c, x_scale, y_scale, sizes, sizes_is_i64, num_groups, m_dim,
                                 n_dim, kb_total, plan, device_status_ptr()));
  } else {
    kern<<<grid, L::kThreads, L::kDynamicBytes, stream>>>(tm_x, tm_y, tm_c, x_scale, y_scale, sizes, sizes_is_i64,
                                                          num_groups, m_dim, n_dim, kb_total, plan, device_status_ptr());
  }
  B200_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace b200

extern "C" {

int b200gemm_fp8_k_grouped_block(const void* x8, const float* x_scale, const void* y8, const float* y_scale, void* out,
                                 const void* padded_sizes, int sizes_is_i64, int num_groups, int64_t m_expand,
                                 int m_dim, int n_dim, void* workspace, int64_t workspace_bytes, int num_sms,
                                 void* stream_v) {
  using namespace b200;
  const char* who = "b200gemm_fp8_k_grouped_block";
  B200_REQUIRE(num_groups >= 0 && m_expand >= 0 && m_dim >= 0 && n_dim >= 0, "%s: negative dimension", who);
  if (num_groups == 0 || m_dim == 0 || n_dim == 0) return 0;
  B200_REQUIRE(x8 && y8 && out && padded_sizes && x_scale && y_scale, "%s: null pointer", who);
  B200_REQUIRE(m_expand > 0 && m_expand % 128 == 0, "%s: m_expand (%lld) must be a positive multiple of 128", who,
               (long long)m_expand);
  B200_REQUIRE(m_dim % 128 == 0 && n_dim % 128 == 0,
               "%s: m_dim (%d) and n_dim (%d) must be multiples of 128 (the quantiser's block size)", who, m_dim, n_dim);
  B200_REQUIRE(m_expand < (1ll << 31), "%s: m_expand must fit in int32", who);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(x8) & 15) == 0 && (reinterpret_cast<uintptr_t>(y8) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(out) & 15) == 0,
               "%s: x8, y8 and out must be 16-byte aligned", who);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const int sms = sm_count();
  B200_REQUIRE(sms > 0, "%s: no CUDA device", who);
  const int grid = (num_sms > 0 && num_sms < sms) ? num_sms : sms;
  bool pair = false;
  if (g_cta_pair_mode == 1) pair = grid >= 2;
  else if (g_cta_pair_mode == -1)
    pair = grid >= 2 && m_dim >= 256 && n_dim >= 256 &&
           static_cast<long long>(num_groups) * (m_dim / 256) * ((n_dim + 255) / 256) >= grid / 2;
  CUtensorMap tm_x, tm_y, tm_c;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(m_expand), static_cast<uint64_t>(m_dim)};
    const uint64_t strides[1] = {static_cast<uint64_t>(m_expand)};
    const uint32_t box[2] = {128, kBlockM};
    int rc = encode_tmap(&tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, x8, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                         "x8[m_dim, m_expand]");
    if (rc) return rc;
  }
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(m_expand), static_cast<uint64_t>(n_dim)};
    const uint64_t strides[1] = {static_cast<uint64_t>(m_expand)};
    const uint32_t box[2] = {128, static_cast<uint32_t>(pair ? 128 : 256)};
    int rc = encode_tmap(&tm_y, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, y8, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                         "y8[n_dim, m_expand]");
    if (rc) return rc;
  }
  {
    const uint64_t dims[3] = {static_cast<uint64_t>(n_dim), static_cast<uint64_t>(m_dim),
                              static_cast<uint64_t>(num_groups)};
    const uint64_t strides[2] = {static_cast<uint64_t>(n_dim) * 2, static_cast<uint64_t>(n_dim) * m_dim * 2};
    const uint32_t box[3] = {64, 32, 1};
    int rc = encode_tmap(&tm_c, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, out, dims, strides, box,
                         CU_TENSOR_MAP_SWIZZLE_128B, "out[G, m_dim, n_dim]");
    if (rc) return rc;
  }
  const long long kb_total = m_expand / 128;
  int* plan = nullptr;
  {
    int rc = k_grouped_plan_into(workspace, workspace_bytes, padded_sizes, sizes_is_i64, num_groups, who, &plan, stream);
    if (rc) return rc;
  }
  if (pair)
    return launch_fp8_block_k<true>(tm_x, tm_y, tm_c, x_scale, y_scale, padded_sizes, sizes_is_i64, num_groups, m_dim,
                                    n_dim, kb_total, plan, grid, stream);
  return launch_fp8_block_k<false>(tm_x, tm_y, tm_c, x_scale, y_scale, padded_sizes, sizes_is_i64, num_groups, m_dim,
                                   n_dim, kb_total, plan, grid, stream);
}

}  // extern "C"
