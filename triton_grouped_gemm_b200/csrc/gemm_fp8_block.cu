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
//   warps 1, 2          MMA issuers: 4 x tcgen05.mma kind::f8f6f4 (128 x BLOCK_N x 32) per k-block;
//                       warp 1 issues the k-blocks that go to TMEM buffer 0, warp 2 those of buffer 1.
//                       A warp sits in its blocked tcgen05.mma instructions for ~40 % of a k-block's
//                       time, and the promotion warps that share its scheduler fall that far behind
//                       the others; with two issuers on two schedulers each pair of promotion warps
//                       is held up only every other k-block (+2 %)
//   warp 3              scale producer: for every 16 k-blocks it multiplies a_scale[row, kb] by
//                       b_scale[g, n-block, kb] for this CTA's 128 rows and the tile's two column
//                       halves and leaves the products in shared memory, so that a promotion thread
//                       fetches the scales of two k-blocks with ONE shared-memory load (shared memory
//                       is saturated by the tensor core's operand reads: a load and a shuffle per
//                       k-block cost the promotion warps 8 % of the kernel)
//   warps 4..4+BLOCK_N/32-1   promotion + epilogue: warp (quarter = warp%4, half = (warp-4)/4)
//                       owns TMEM lanes [32*quarter, +32) and columns [128*half, +128), i.e.
//                       exactly one 128-wide scale block of B per thread; these warpgroups
//                       raise their register budget (setmaxnreg) to hold 128 fp32 accumulators
//
// kSwiglu (256-column tiles only): the GEMM is the gate+up projection of a SwiGLU feed-forward
// whose weight rows the caller interleaved in 128-row blocks (tile t = gate block t, then up
// block t), and the epilogue writes act = bf16(silu(bf16(gate)) * bf16(up)) quantised 1x128 -
// e4m3 bytes plus one fp32 scale per row and tile - instead of the bf16 product: the same bytes
// and scales as storing the product and running the SwiGLU quantiser on it, without the round
// trip through HBM.  The warp holding a row's up half passes its values to the warp holding the
// gate half through the two warps' store-staging buffers (mbarrier handshake per tile).
#include <cuda_bf16.h>

#include "../../include/b200gemm.h"
#include "common.cuh"
#include "gemm_tile.cuh"
#include "quant_math.cuh"

namespace b200 {

// kPair: the CTA-pair form (tcgen05 cta_group::2).  Two CTAs on two SMs share a 256 x 256 tile:
// CTA r holds rows [128 r, +128) of A and of the accumulator and supplies columns [128 r, +128)
// of B; the leader (rank 0) issues the MMAs for both, its commits are delivered to both CTAs,
// and both CTAs' promotion warps hand the TMEM buffers back to the leader.  Per CTA a k-block
// is then 16 KB of A plus 16 KB of B, a third less shared-memory and L2 traffic.
template <int kBlockN, bool kPair>
struct Fp8BlockCfg {
  static_assert(!kPair || kBlockN == 256, "the CTA-pair form uses 256-column tiles");
  // 224 KB of shared memory: operand ring + 32 KB store staging + 32 KB scale staging
  static constexpr int kStages = (kPair || kBlockN == 128) ? 5 : 3;
  static constexpr int kBRows = kPair ? 128 : kBlockN;  // rows of B_g this CTA loads per k-block
  static constexpr int kPromoWarps = kBlockN / 32;  // 4 lane quarters x (kBlockN/128) column halves
  static constexpr int kThreads = 128 + 32 * kPromoWarps;
  // 384 threads start at 168 registers each; warpgroup 0 drops to 56 and the two promotion
  // warpgroups rise to 224 (128*56 + 256*224 <= 64K).  256 threads (BLOCK_N = 128) already
  // get 255 each and need no re-balancing.
  static constexpr bool kRebalance = kBlockN == 256;
  // setmaxnreg only moves registers inside the CTA's own allocation (threads x registers at launch);
  // an increase that the decreases do not cover waits for ever
  static constexpr int kRegsLaunch = 168, kRegsMove = 56, kRegsPromo = 224;
  static_assert(!kRebalance || 128 * kRegsMove + (kThreads - 128) * kRegsPromo <= kThreads * kRegsLaunch,
                "register re-balancing must fit the CTA's allocation");
  static constexpr int kABytes = kBlockM * 128;
  static constexpr int kBBytes = kBRows * 128;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kEpiOffset = kStages * kStageBytes;  // one 4 KB store-staging buffer per promotion warp
  // scale products: two buffers x two column halves x 8 k-block pairs x 128 rows x 8 bytes
  // (a buffer covers kScaleChunk = 16 k-blocks; entry [pair][row] = the products of k-blocks 2 pair
  // and 2 pair + 1, so the 32 lanes of a promotion warp read 256 consecutive bytes)
  static constexpr int kScaleChunk = 16;
  static constexpr int kScaleHalfBytes = (kScaleChunk / 2) * kBlockM * 8;  // 8 KB
  static constexpr int kScaleBufBytes = 2 * kScaleHalfBytes;
  static constexpr int kScaleOffset = kEpiOffset + 8 * 32 * 128;
  static constexpr int kBarOffset = kScaleOffset + 2 * kScaleBufBytes;
  // + tmem_full[2], tmem_empty[2], scale_full[2], scale_empty[2], exchange_full[4], exchange_empty[4]
  static constexpr int kNumBars = 2 * kStages + 16;
  static constexpr int kDynamicBytes = kBarOffset + kNumBars * 8 + 16 + 1024;
};

template <int kBlockN, bool kPair, bool kSwiglu>
__global__ void __launch_bounds__(Fp8BlockCfg<kBlockN, kPair>::kThreads, 1)
fp8_block_m_grouped_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                           const __grid_constant__ CUtensorMap tm_c, __nv_bfloat16* __restrict__ c_ptr,
                           const float* __restrict__ a_scale,
                           const float* __restrict__ b_scale, const void* __restrict__ sizes, int sizes_i64,
                           int num_groups, int masked_stride, long long m_rows, int n, int k,
                           const int* __restrict__ b_map, int num_b, float* __restrict__ act_scale_out,
                           unsigned* status) {
  static_assert(!kSwiglu || kBlockN == 256, "the SwiGLU epilogue pairs the two 128-column halves of a 256-column tile");
  using L = Fp8BlockCfg<kBlockN, kPair>;
  // weight matrix of row group g: b[b_map[g]] (clamped into range), or b[g] without a map
  auto weight_of = [&](int g) -> int {
    if (!b_map) return g;
    const int v = __ldg(b_map + g);
    return v < 0 ? 0 : (v >= num_b ? num_b - 1 : v);
  };
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
  auto scale_full_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 4 + a); };
  auto scale_empty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 6 + a); };
  auto xchg_full_bar = [&](int q) { return bar_base + 8u * (2 * kStages + 8 + q); };
  auto xchg_empty_bar = [&](int q) { return bar_base + 8u * (2 * kStages + 12 + q); };
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem + L::kBarOffset + L::kNumBars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kBarOffset + L::kNumBars * 8 + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = kPair ? cluster_ctarank() : 0u;  // 0 = leader of the pair
  const int first_tile = kPair ? (blockIdx.x >> 1) : blockIdx.x;
  const int tile_step = kPair ? (gridDim.x >> 1) : gridDim.x;
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
      mbar_init(tmem_empty_bar(a), L::kPromoWarps * kCtas);
      mbar_init(scale_full_bar(a), 1);  // one arrival of the scale-producer warp
      mbar_init(scale_empty_bar(a), L::kPromoWarps);
    }
    for (int q = 0; q < 4; ++q) {
      mbar_init(xchg_full_bar(q), 1);
      mbar_init(xchg_empty_bar(q), 1);
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
    tmem_alloc<kCtas>(smem_u32(const_cast<uint32_t*>(tmem_holder)), kTmemCols);
    tmem_relinquish<kCtas>();
  }
  tc_fence_before_sync();
  if constexpr (kPair) cluster_sync_all();  // the peer's barriers exist before anyone signals them
  else __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  if (warp < 4) {
  if constexpr (L::kRebalance) warpgroup_reg_dec<L::kRegsMove>();
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
          if constexpr (kPair) {
            // the leader's barrier collects both CTAs' bytes; one arrival per phase (leader)
            const uint32_t leader_full = mapa_u32(full_bar(stage), 0);
            if (rank == 0) mbar_arrive_expect_tx(full_bar(stage), 2 * L::kStageBytes);
            tma_load_2d_pair(a_dst, &tm_a, leader_full, kb * 128, row0);
            tma_load_3d_pair(a_dst + L::kABytes, &tm_b, leader_full, kb * 128, col0, g);
          } else {
            mbar_arrive_expect_tx(full_bar(stage), L::kStageBytes);
            tma_load_2d(a_dst, &tm_a, full_bar(stage), kb * 128, row0);
            tma_load_3d(a_dst + L::kABytes, &tm_b, full_bar(stage), kb * 128, col0, g);
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
    // ------------------------------------------------------------ MMA issuers (pair: leader only); warp 1: TMEM buffer 0, warp 2: buffer 1
    GroupWalker w;
    w.init(sizes, sizes_i64, num_groups, masked_stride, kTileM, m_rows);
    const uint32_t idesc = make_instr_desc(0u, 0u, 0u, 0u, kTileM, kBlockN);  // e4m3 x e4m3 -> f32
    int stage = 0;
    uint32_t phase = 0;
    uint32_t it = 0;  // k-blocks issued so far: TMEM buffer = it & 1
    bool ok = rank == 0;
    for (int tile = first_tile; ok; tile += tile_step) {
      const int mt = tile / n_tiles;
      if (!w.seek(mt)) break;
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const uint32_t buf = it & 1u;
        const uint32_t buf_phase = (it >> 1) & 1u;
        if (buf != static_cast<uint32_t>(warp - 1)) {  // the other issuer's k-block
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
          continue;
        }
        // operands first (they are nearly always there), then the drained buffer: the MMAs go out
        // the moment the promotion warps let go of it
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
  } else {
    // ------------------------------------------------------------ scale producer (warp 3)
    // Lane l serves rows l, l + 32, l + 64 and l + 96 of this CTA's 128.  Per chunk of kScaleChunk k-blocks and column half h the products
    // a_scale[row, kb] * b_scale[weight, n-block of h, kb] go to
    //   products[buffer][h][pair = (kb % 16) / 2][row] = {kb even, kb odd}   (8 bytes)
    // Rows past the end of the tensors read row m_rows - 1 instead (their results are discarded);
    // k-blocks past num_kb get zeros.
    GroupWalker w;
    w.init(sizes, sizes_i64, num_groups, masked_stride, kTileM, m_rows);
    constexpr int kHalves = kBlockN / 128;
    const int row_in_cta = lane;
    uint32_t scale_it = 0;  // chunks produced so far: buffer = scale_it & 1
    bool ok = true;
    for (int tile = first_tile; ok; tile += tile_step) {
      const int mt = tile / n_tiles;
      const int nt = tile - mt * n_tiles;
      if (!w.seek(mt)) break;
      const long long row_c0 = w.tile_row0(mt) + static_cast<long long>(rank) * kBlockM + row_in_cta;
      const int wsel = weight_of(w.g) * n_blocks;
      int bs_off[kHalves];  // first scale of this tile's column half h: b_scale[bs_off[h] + kb]
#pragma unroll
      for (int h = 0; h < kHalves; ++h) {
        int nb = (nt * kBlockN + h * 128) >> 7;
        if (nb >= n_blocks) nb = n_blocks - 1;  // columns past n: results are discarded
        bs_off[h] = (wsel + nb) * num_kb;
      }
      for (int kb0 = 0; kb0 < num_kb; kb0 += L::kScaleChunk) {
        const uint32_t sb = scale_it & 1u;
        if (!wait_bounded(scale_empty_bar(sb), ((scale_it >> 1) & 1u) ^ 1u, abort_flag, status, kDevTimeoutProducer)) {
          ok = false;
          break;
        }
#pragma unroll 1
        for (int j = 0; j < 4; ++j) {
          long long r = row_c0 + 32 * j;
          if (r >= m_rows) r = m_rows - 1;
          const float* ar = a_scale + r * static_cast<long long>(num_kb);
          uint8_t* dst = smem + L::kScaleOffset + sb * L::kScaleBufBytes + (row_in_cta + 32 * j) * 8;
#pragma unroll 2
          for (int pr = 0; pr < L::kScaleChunk / 2; ++pr) {
            const int kb = kb0 + 2 * pr;
            const bool in0 = kb < num_kb, in1 = kb + 1 < num_kb;
            const float a0 = in0 ? __ldg(ar + kb) : 0.f;
            const float a1 = in1 ? __ldg(ar + kb + 1) : 0.f;
#pragma unroll
            for (int h = 0; h < kHalves; ++h) {
              const float b0 = in0 ? __ldg(b_scale + bs_off[h] + kb) : 0.f;
              const float b1 = in1 ? __ldg(b_scale + bs_off[h] + kb + 1) : 0.f;
              *reinterpret_cast<float2*>(dst + h * L::kScaleHalfBytes + pr * (kBlockM * 8)) =
                  make_float2(__fmul_rn(a0, b0), __fmul_rn(a1, b1));
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(scale_full_bar(sb));
        ++scale_it;
      }
    }
  }
  } else {
    // ------------------------------------------------------------ promotion + epilogue
    if constexpr (L::kRebalance) warpgroup_reg_inc<L::kRegsPromo>();
    GroupWalker w;
    w.init(sizes, sizes_i64, num_groups, masked_stride, kTileM, m_rows);
    const int quarter = warp & 3;
    const int half = (warp - 4) >> 2;
    uint32_t it = 0;
    uint32_t scale_it = 0;
    uint32_t xchg_it = 0;  // tiles passed through the gate/up exchange (kSwiglu)
    // this thread's entries of the scale-product buffers: [buffer][half][k-block pair][row] x 8 bytes
    const int srow = quarter * 32 + lane;
    const uint32_t scale_prod = smem_base + L::kScaleOffset + half * L::kScaleHalfBytes + srow * 8;
    // volatile: the load must be issued where it is written (a pair of k-blocks ahead of its
    // use), neither sunk to the use, where its latency would sit on the promotion warps' critical
    // path, nor hoisted above the TMEM load wait
    auto load_scale_pair = [&](uint32_t sb, int kb, float& s0, float& s1) {
      asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];"
                   : "=f"(s0), "=f"(s1)
                   : "r"(scale_prod + sb * L::kScaleBufBytes + ((kb & (L::kScaleChunk - 1)) >> 1) * (kBlockM * 8)));
    };
    bool ok = true;
    for (int tile = first_tile; ok; tile += tile_step) {
      const int mt = tile / n_tiles;
      const int nt = tile - mt * n_tiles;
      if (!w.seek(mt)) break;
      const long long row_w0 = w.tile_row0(mt) + static_cast<long long>(rank) * kBlockM + quarter * 32;
      const long long row = row_w0 + lane;
      const bool row_ok = row < w.group_row_end();
      const int col_base = nt * kBlockN + half * 128;
      // 128 fp32 accumulators as 64 packed pairs (fma.rn.f32x2: two lanes per instruction)
      unsigned long long acc2[64];
#pragma unroll
      for (int j = 0; j < 64; ++j) acc2[j] = 0ull;
      // Per k-block: 64 columns per tcgen05.ld (two loads cover this thread's 128 columns).  The
      // loads are not interleaved with the FMAs of the same registers: a plain load / wait /
      // multiply sequence measured faster than a finer software pipeline; the first load of
      // k-block kb+1 is requested as soon as its buffer is full, before the loop comes around.
      uint32_t t[64];
      const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + half * 128;
      // scale of k-block kb = a_scale[row, kb] * b_scale[g, n-block, kb], multiplied by the scale
      // producers; s_even / s_odd hold the current pair of k-blocks, p_even / p_odd the next pair
      // (requested at the start of the current one)
      uint32_t sb = 0;
      auto begin_chunk = [&]() -> bool {
        sb = scale_it & 1u;
        if (!wait_bounded(scale_full_bar(sb), (scale_it >> 1) & 1u, abort_flag, status, kDevTimeoutPromote))
          return false;
        ++scale_it;
        return true;
      };
      if (!begin_chunk()) break;
      float s_even, s_odd, p_even = 0.f, p_odd = 0.f;
      load_scale_pair(sb, 0, s_even, s_odd);
      if (!wait_bounded(tmem_full_bar(it & 1u), (it >> 1) & 1u, abort_flag, status, kDevTimeoutPromote)) break;
      tc_fence_after_sync();
      tmem_ld_32x32b_x64(t_lane + (it & 1u) * kBlockN, t);
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const bool odd = (kb & 1) != 0;
        const float s_cur = odd ? s_odd : s_even;
        const unsigned long long s2 = pack_f32x2(__float_as_uint(s_cur), __float_as_uint(s_cur));
        const bool more = kb + 1 < num_kb;
        const uint32_t buf = it & 1u;
        const uint32_t t_addr = t_lane + buf * kBlockN;
        tmem_ld_wait();
        // The next pair's products are requested HERE, behind the wait: the same load issued at the
        // top of the loop, while the first TMEM load is in flight, cost 12 % of the kernel
        if (!odd && kb + 2 < num_kb) {
          if (((kb + 2) & (L::kScaleChunk - 1)) == 0) {
            // the next pair opens a new chunk; everything this buffer had to give is in s_even /
            // s_odd already: hand it back to the scale producers
            __syncwarp();
            if (lane == 0) mbar_arrive(scale_empty_bar(sb));
            if (!begin_chunk()) {
              ok = false;
              break;
            }
          }
          load_scale_pair(sb, kb + 2, p_even, p_odd);
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
          if (odd) {
            // end of a pair: the next pair's products arrived long ago
            s_even = p_even;
            s_odd = p_odd;
          }
        }
      }
      if (!ok) break;
      __syncwarp();
      if (lane == 0) mbar_arrive(scale_empty_bar(sb));
      float acc[128];
#pragma unroll
      for (int j = 0; j < 64; ++j) unpack_f32x2(acc2[j], acc[2 * j], acc[2 * j + 1]);
      if (!ok) break;
      if constexpr (kSwiglu) {
        // tile columns [0, 128) hold gate block nt, [128, 256) up block nt of the same 128 outputs
        uint8_t* buf_lo = smem + L::kEpiOffset + quarter * (32 * 128);        // the gate warp's staging buffer
        uint8_t* buf_hi = smem + L::kEpiOffset + (4 + quarter) * (32 * 128);  // the up warp's
        if (half == 1) {
          // up half: round to bf16 (what storing the product would do) and hand over
          if (!wait_bounded(xchg_empty_bar(quarter), (xchg_it & 1u) ^ 1u, abort_flag, status, kDevTimeoutPromote)) break;
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint8_t* buf = c == 0 ? buf_lo : buf_hi;
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              uint32_t p[4];
#pragma unroll
              for (int e = 0; e < 4; ++e)
                p[e] = pack2_16bit(acc[c * 64 + v * 8 + 2 * e], acc[c * 64 + v * 8 + 2 * e + 1], 0);
              *reinterpret_cast<uint4*>(buf + lane * 128 + ((v ^ (lane & 7)) << 4)) = make_uint4(p[0], p[1], p[2], p[3]);
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(xchg_full_bar(quarter));
        } else {
          if (!wait_bounded(xchg_full_bar(quarter), xchg_it & 1u, abort_flag, status, kDevTimeoutPromote)) break;
          float amax = 0.f;
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const uint8_t* buf = c == 0 ? buf_lo : buf_hi;
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              const uint4 u4 = *reinterpret_cast<const uint4*>(buf + lane * 128 + ((v ^ (lane & 7)) << 4));
              const uint32_t uw[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int j = c * 64 + v * 8 + 2 * e;
                const float g0 = __bfloat162float(__float2bfloat16_rn(acc[j]));
                const float g1 = __bfloat162float(__float2bfloat16_rn(acc[j + 1]));
                acc[j] = silu_mul_round_bf16(g0, __uint_as_float(uw[e] << 16));
                acc[j + 1] = silu_mul_round_bf16(g1, __uint_as_float(uw[e] & 0xFFFF0000u));
                amax = fmaxf(amax, fmaxf(fabsf(acc[j]), fabsf(acc[j + 1])));
              }
            }
          }
          __syncwarp();  // every lane has read its row: buf_lo may be reused for the fp8 staging
          amax = fmaxf(amax, 1e-4f);
          const float inv = inv_scale_448(amax);
          const int inter = n >> 1;
          if (row_ok) act_scale_out[row * static_cast<long long>(inter >> 7) + nt] = __fdiv_rn(amax, 448.0f);
          // 16 e4m3 bytes (columns 16 v .. 16 v + 15 of the 128) as one 16-byte vector
          auto quantised16 = [&](int v) -> uint4 {
            uint32_t w4[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int b = 16 * v + 4 * j;
              w4[j] = cvt_e4m3x2(__fmul_rn(acc[b], inv), __fmul_rn(acc[b + 1], inv)) |
                      (cvt_e4m3x2(__fmul_rn(acc[b + 2], inv), __fmul_rn(acc[b + 3], inv)) << 16);
            }
            return make_uint4(w4[0], w4[1], w4[2], w4[3]);
          };
          if (row_w0 + 32 <= w.group_row_end()) {
#pragma unroll
            for (int v = 0; v < 8; ++v)
              *reinterpret_cast<uint4*>(buf_lo + lane * 128 + ((v ^ (lane & 7)) << 4)) = quantised16(v);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tm_c, smem_u32(buf_lo), nt * 128, static_cast<int>(row_w0));
              tma_store_commit();
              tma_store_wait_read<0>();  // the buffer goes back to the up warp below
            }
          } else if (row_ok) {
            uint8_t* out_row = reinterpret_cast<uint8_t*>(c_ptr) + row * static_cast<long long>(inter) + nt * 128;
#pragma unroll
            for (int v = 0; v < 8; ++v) *reinterpret_cast<uint4*>(out_row + v * 16) = quantised16(v);
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(xchg_empty_bar(quarter));
        }
        ++xchg_it;
        continue;
      }
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
    // the sizes added up to more rows than a / c have: the excess was cut off, tell the host
    if (ok && w.overflow && rank == 0 && warp == 4 && lane == 0 && status) atomicOr(status, kDevBadGroupSize);
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(4000);
    __syncthreads();
  }
  if constexpr (kPair) cluster_sync_all();  // the peer may still signal this CTA / write its TMEM
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<kCtas>(tmem_base, kTmemCols);
  }
}

template <int kBlockN, bool kPair, bool kSwiglu = false>
static int launch_fp8_block(const CUtensorMap& tm_a, const CUtensorMap& tm_b, const CUtensorMap& tm_c,
                            void* c, const float* a_scale, const float* b_scale, const void* sizes, int sizes_is_i64,
                            int num_groups, int masked_stride, long long m_rows, int n, int k, const int* b_map, int num_b,
                            int grid, cudaStream_t stream, float* act_scale_out = nullptr) {
  using L = Fp8BlockCfg<kBlockN, kPair>;
  auto kern = fp8_block_m_grouped_kernel<kBlockN, kPair, kSwiglu>;
  B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes));
  if constexpr (kPair) {
    // a cluster of two CTAs per tile; keep only as many CTAs as are co-resident
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
    B200_CUDA(cudaLaunchKernelEx(&cfg, kern, tm_a, tm_b, tm_c, static_cast<__nv_bfloat16*>(c), a_scale, b_scale, sizes,
                                 sizes_is_i64, num_groups, masked_stride, m_rows, n, k, b_map, num_b, act_scale_out,
                                 device_status_ptr()));
  } else {
    kern<<<grid, L::kThreads, L::kDynamicBytes, stream>>>(tm_a, tm_b, tm_c,
                                                          static_cast<__nv_bfloat16*>(c), a_scale,
                                                          b_scale, sizes, sizes_is_i64, num_groups, masked_stride, m_rows,
                                                          n, k, b_map, num_b, act_scale_out, device_status_ptr());
  }
  B200_CUDA(cudaGetLastError());
  return 0;
}

static int fp8_block_common(const void* a, const float* a_scale, const void* b, const float* b_scale, void* c,
                            const void* sizes, int sizes_is_i64, int num_groups, int64_t m_rows, int masked_stride,
                            int n, int k, int num_sms, void* stream_v, const char* who, const int* b_map = nullptr,
                            int num_b = 0, float* act_scale_out = nullptr) {
  // act_scale_out != nullptr: SwiGLU epilogue - c receives e4m3 bytes [m_rows, n/2], act_scale_out fp32
  // [m_rows, n/256]; b must hold gate and up rows interleaved in 128-row blocks
  const bool swiglu = act_scale_out != nullptr;
  if (swiglu)
    B200_REQUIRE(n > 0 && n % 256 == 0, "%s: the SwiGLU epilogue needs n (= 2 x intermediate size, %d) to be a multiple of 256",
                 who, n);
  if (!b_map) num_b = num_groups;
  B200_REQUIRE(num_b > 0 || num_groups == 0, "%s: num_b must be positive when a group-to-weight map is given", who);
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
  const int block_n = swiglu ? 256 : ((n <= 128 || m_tiles_est * ((n + 255) / 256) < grid) ? 128 : 256);
  // CTA pairs when every pair of SMs gets 256 x 256 tiles (or when forced by the tuning knob)
  bool pair = false;
  if (g_cta_pair_mode == 1) pair = grid >= 2;
  else if (g_cta_pair_mode == -1)
    pair = block_n == 256 && grid >= 2 && (m_rows / 256) * ((n + 255) / 256) >= grid / 2 &&
           m_rows / 256 >= 4ll * num_groups;
  const int b_box_rows = pair ? 128 : block_n;
  CUtensorMap tm_a, tm_b;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(k), static_cast<uint64_t>(m_rows)};
    const uint64_t strides[1] = {static_cast<uint64_t>(k)};
    const uint32_t box[2] = {128, kBlockM};
    int rc = encode_tmap(&tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, "A");
    if (rc) return rc;
  }
  {
    const uint64_t dims[3] = {static_cast<uint64_t>(k), static_cast<uint64_t>(n), static_cast<uint64_t>(num_b)};
    const uint64_t strides[2] = {static_cast<uint64_t>(k), static_cast<uint64_t>(k) * n};
    const uint32_t box[3] = {128, static_cast<uint32_t>(b_box_rows), 1};
    int rc = encode_tmap(&tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, b, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                         "B[G,N,K]");
    if (rc) return rc;
  }
  CUtensorMap tm_c;
  if (swiglu) {
    const uint64_t dims[2] = {static_cast<uint64_t>(n / 2), static_cast<uint64_t>(m_rows)};
    const uint64_t strides[1] = {static_cast<uint64_t>(n / 2)};
    const uint32_t box[2] = {128, 32};
    int rc = encode_tmap(&tm_c, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, c, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                         "act[M, n/2] (e4m3)");
    if (rc) return rc;
  } else {
    const uint64_t dims[2] = {static_cast<uint64_t>(n), static_cast<uint64_t>(m_rows)};
    const uint64_t strides[1] = {static_cast<uint64_t>(n) * 2};
    const uint32_t box[2] = {64, 32};
    int rc = encode_tmap(&tm_c, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, c, dims, strides, box,
                         CU_TENSOR_MAP_SWIZZLE_128B, "C");
    if (rc) return rc;
  }
  if (swiglu) {
    if (pair)
      return launch_fp8_block<256, true, true>(tm_a, tm_b, tm_c, c, a_scale, b_scale, sizes,
                                               sizes_is_i64, num_groups, masked_stride, m_rows, n, k, b_map, num_b, grid,
                                               stream, act_scale_out);
    return launch_fp8_block<256, false, true>(tm_a, tm_b, tm_c, c, a_scale, b_scale, sizes,
                                              sizes_is_i64, num_groups, masked_stride, m_rows, n, k, b_map, num_b, grid,
                                              stream, act_scale_out);
  }
  if (pair)
    return launch_fp8_block<256, true>(tm_a, tm_b, tm_c, c, a_scale, b_scale, sizes, sizes_is_i64, num_groups,
                                       masked_stride, m_rows, n, k, b_map, num_b, grid, stream);
  if (block_n == 256)
    return launch_fp8_block<256, false>(tm_a, tm_b, tm_c, c, a_scale, b_scale, sizes, sizes_is_i64, num_groups,
                                        masked_stride, m_rows, n, k, b_map, num_b, grid, stream);
  return launch_fp8_block<128, false>(tm_a, tm_b, tm_c, c, a_scale, b_scale, sizes, sizes_is_i64, num_groups,
                                      masked_stride, m_rows, n, k, b_map, num_b, grid, stream);
}

}  // namespace b200

extern "C" {

int b200gemm_fp8_m_grouped_block(const void* a, const float* a_scale, const void* b, const float* b_scale, void* c,
                                 const void* sizes, int sizes_is_i64, int num_groups, int64_t m_rows, int n, int k,
                                 int rows_padded, int num_sms, void* stream) {
  return b200::fp8_block_common(a, a_scale, b, b_scale, c, sizes, sizes_is_i64, num_groups, m_rows,
                                rows_padded ? -1 : 0, n, k, num_sms, stream, "b200gemm_fp8_m_grouped_block");
}

int b200gemm_fp8_m_grouped_block_mapped(const void* a, const float* a_scale, const void* b, const float* b_scale,
                                        void* c, const void* sizes, int sizes_is_i64, int num_groups,
                                        const int* group_to_b, int num_b, int64_t m_rows, int n, int k, int num_sms,
                                        void* stream) {
  if (!group_to_b)
    return b200::set_error(b200::kErrInvalidArgument, "b200gemm_fp8_m_grouped_block_mapped: group_to_b is null");
  return b200::fp8_block_common(a, a_scale, b, b_scale, c, sizes, sizes_is_i64, num_groups, m_rows, 0, n, k, num_sms,
                                stream, "b200gemm_fp8_m_grouped_block_mapped", group_to_b, num_b);
}

int b200gemm_fp8_m_grouped_block_swiglu(const void* a, const float* a_scale, const void* b, const float* b_scale,
                                        void* act, float* act_scale, const void* sizes, int sizes_is_i64,
                                        int num_groups, const int* group_to_b, int num_b, int64_t m_rows,
                                        int masked_stride, int n, int k, int num_sms, void* stream) {
  const char* who = "b200gemm_fp8_m_grouped_block_swiglu";
  if (!act_scale) return b200::set_error(b200::kErrInvalidArgument, "%s: act_scale is null", who);
  if (masked_stride < 0) return b200::set_error(b200::kErrInvalidArgument, "%s: masked_stride must be >= 0", who);
  if (reinterpret_cast<uintptr_t>(act) & 15)
    return b200::set_error(b200::kErrInvalidArgument, "%s: act must be 16-byte aligned", who);
  return b200::fp8_block_common(a, a_scale, b, b_scale, act, sizes, sizes_is_i64, num_groups, m_rows, masked_stride, n,
                                k, num_sms, stream, who, group_to_b, group_to_b ? num_b : 0, act_scale);
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
