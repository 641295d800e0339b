// BF16 / FP16 K-grouped GEMM (expert weight gradient) for sm_100a:
//   C[g] = A[gs:ge, :]^T * B[gs:ge, :],  A [K_total, M_DIM], B [K_total, N_DIM], C [G, M_DIM, N_DIM]
// The grouping runs along the contraction (token) axis, so both operands are MN-major in
// shared memory: a k-block is 64 token rows, each row 128 bytes of one 64-column chunk
// (128-byte swizzle), and the UMMA descriptors carry the "MN-major" bit for A and B.
//
// Same warp roles as the M-grouped kernel (TMA producer / MMA issuer / 4 epilogue warps,
// double-buffered TMEM accumulator).  Tiles are numbered g * tiles_per_group + local, and the
// token range of a group comes from a running prefix over the device-resident sizes.
// The last k-block of a group may hold rows of the next group (TMA cannot clip in the
// middle of a tensor): the MMA warp zeroes those rows in shared memory up to the next
// multiple of 16 and issues only as many K=16 steps as the group has rows for.
// An empty group writes zeros (the reference's TMA kernel stores its zero accumulator,
// gemm/BF16/k_grouped_gemm_TMA.py:141,167-170).
//
// Tile cost is proportional to the group's token count, which differs by 10x between experts,
// so a fixed round-robin assignment leaves SMs idle at the end.  With a scratch buffer the
// kernel runs BALANCED: a one-block plan kernel writes, per group, the first token row, the
// token count and the groups' order by decreasing token count, and zeroes a tile counter;
// the producer warp of every CTA then claims tiles with atomicAdd in that order (long tiles
// first) and hands each claimed tile - id, group, token count, first token row - to the CTA's
// other warps through a small shared-memory ring, so that only the producer pays the latency of
// the atomic and of the plan look-ups, and it pays it one tile ahead, in steps spread over the
// k-blocks of the tile it is loading.  Without scratch (workspace == NULL) tiles are assigned
// round-robin.
#include <mutex>

#include "../../include/b200gemm.h"
#include "common.cuh"
#include "gemm_tile.cuh"

namespace b200 {

template <int kBlockN, int kStages>
struct KGroupedSmem {
  static constexpr int kABytes = kBlockM * kBlockK * 2;  // 2 chunks of [64 tokens][64 m]
  static constexpr int kBBytes = kBlockN * kBlockK * 2;  // kBlockN/64 chunks of [64 tokens][64 n]
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kEpiOffset = kStages * kStageBytes;  // 4 warps x 2 x 4 KB store staging
  static constexpr int kBarOffset = kEpiOffset + 4 * kEpiStageBytesPerWarp;
  static constexpr int kSchedDepth = 4;                     // tile-id ring of the balanced scheduler
  static constexpr int kNumBars = 2 * kStages + 4 + 2 * kSchedDepth;
  static constexpr int kTotal = kBarOffset + kNumBars * 8 + 16 + kSchedDepth * 16;  // ring of int4 entries
  static constexpr int kDynamicBytes = kTotal + 1024;
};

// Token range of a group: either explicit int32 [start, end) arrays, or a running exclusive
// prefix over the group sizes (`g` only moves forward).
struct TokenRange {
  const void* sizes;
  const int* starts;
  const int* ends;
  int sizes_i64;
  int cur;
  long long start;
  __device__ __forceinline__ long long size_of(int i) const {
    long long v = sizes_i64 ? static_cast<const long long*>(sizes)[i]
                            : static_cast<long long>(static_cast<const int*>(sizes)[i]);
    return v < 0 ? 0 : v;
  }
  __device__ __forceinline__ void init(const void* s, int i64, const int* gs, const int* ge) {
    sizes = s;
    sizes_i64 = i64;
    starts = gs;
    ends = ge;
    cur = 0;
    start = 0;
  }
  // returns the number of tokens of group g; start = first token row of g
  __device__ __forceinline__ long long seek(int g) {
    if (starts) {
      start = starts[g];
      const long long t = static_cast<long long>(ends[g]) - start;
      return t < 0 ? 0 : t;
    }
    while (cur < g) {
      start += size_of(cur);
      ++cur;
    }
    return size_of(g);
  }
};

// Scratch layout (int32 words): [0] tile counter, [1..63] unused, then starts[G], tokens[G], order[G].
__host__ __device__ inline long long k_grouped_scratch_words(int num_groups) {
  return kPlanHeaderWords + 3ll * num_groups;
}

__global__ void __launch_bounds__(1024) k_grouped_plan_kernel(const void* __restrict__ sizes, int sizes_i64,
                                                              const int* __restrict__ group_start,
                                                              const int* __restrict__ group_end, int num_groups,
                                                              int* __restrict__ scratch) {
  int* starts = scratch + kPlanHeaderWords;
  int* tokens = starts + num_groups;
  int* order = tokens + num_groups;
  auto size_of = [&](int g) -> long long {
    long long v;
    if (group_start) v = static_cast<long long>(group_end[g]) - group_start[g];
    else v = sizes_i64 ? static_cast<const long long*>(sizes)[g] : static_cast<long long>(static_cast<const int*>(sizes)[g]);
    return v < 0 ? 0 : v;
  };
  if (threadIdx.x == 0) {
    scratch[0] = 0;  // tile counter
    long long run = 0;
    for (int g = 0; g < num_groups; ++g) {  // G is small (<= 4096): a serial prefix is a few microseconds
      const long long t = size_of(g);
      starts[g] = group_start ? group_start[g] : static_cast<int>(run);
      tokens[g] = static_cast<int>(t);
      run += t;
    }
  }
  __syncthreads();
  // rank of every group in the order "more tokens first, ties by index" (stable)
  for (int g = threadIdx.x; g < num_groups; g += blockDim.x) {
    const int tg = tokens[g];
    int rank = 0;
    for (int h = 0; h < num_groups; ++h) {
      const int th = tokens[h];
      rank += (th > tg) || (th == tg && h < g);
    }
    order[rank] = g;
  }
}

// kFp8 = false: 16-bit A [K_total, M_DIM], B [K_total, N_DIM] (MN-major operands, 64 tokens
//               per k-block, `in_fmt`: 0 = f16, 1 = bf16).
// kFp8 = true:  8-bit X [M, K_total], Y [N, K_total] (K-major operands, 128 tokens per
//               k-block, `in_fmt` = x_fmt | y_fmt << 4 with 0 = e4m3, 1 = e5m2); the epilogue
//               applies x_scale[g*M+m] * y_scale[g*N+n]; token counts are multiples of 128
//               with zero padding (gemm/FP8/k_grouped_gemm_channel_expert.py:64-140).
template <int kBlockN, int kStages, bool kFp8, bool kBalanced>
__global__ void __launch_bounds__(kNumThreads, 1)
k_grouped_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                 const __grid_constant__ CUtensorMap tm_c, void* __restrict__ c_ptr, const void* __restrict__ sizes, int sizes_i64,
                 const int* __restrict__ group_start, const int* __restrict__ group_end, int num_groups, int m_dim,
                 int n_dim, long long k_total, int in_fmt, int out_fp16, const float* __restrict__ a_scale,
                 const float* __restrict__ b_scale, int* __restrict__ scratch, unsigned* status) {
  constexpr int kTokensPerKb = kFp8 ? 128 : kBlockK;
  using L = KGroupedSmem<kBlockN, kStages>;
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
  auto sched_full_bar = [&](int i) { return bar_base + 8u * (2 * kStages + 4 + i); };
  auto sched_empty_bar = [&](int i) { return bar_base + 8u * (2 * kStages + 4 + L::kSchedDepth + i); };
  volatile int4* sched_info = reinterpret_cast<volatile int4*>(smem + L::kBarOffset + L::kNumBars * 8 + 16);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_tiles = (m_dim + kBlockM - 1) / kBlockM;
  const int n_tiles = (n_dim + kBlockN - 1) / kBlockN;
  const int tiles_per_group = m_tiles * n_tiles;
  const long long num_tiles = static_cast<long long>(tiles_per_group) * num_groups;
  constexpr uint32_t kTmemCols = 2 * kBlockN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tmem_full_bar(a), 1);
      mbar_init(tmem_empty_bar(a), 4);
    }
    for (int i = 0; i < L::kSchedDepth; ++i) {
      mbar_init(sched_full_bar(i), 1);
      mbar_init(sched_empty_bar(i), 5);  // MMA warp + 4 epilogue warps
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

  // tile -> (group slot, m tile, n tile): n fastest, so CTAs running side by side share A chunks.
  // Balanced mode visits the groups in the plan's order (most tokens first).
  const int* plan_starts = scratch + kPlanHeaderWords;
  const int* plan_tokens = plan_starts + num_groups;
  const int* plan_order = plan_tokens + num_groups;
  struct TileInfo {
    long long tile;  // -1: no more work (or a wait ran out)
    int g;
    long long tokens, start;
  };
  auto split_tile = [&](long long tile, int& slot, int& mt, int& nt) {
    slot = static_cast<int>(tile / tiles_per_group);
    const int local = static_cast<int>(tile - static_cast<long long>(slot) * tiles_per_group);
    mt = local / n_tiles;
    nt = local - mt * n_tiles;
  };
  // i-th tile of this CTA for a consumer role (MMA / epilogue): static round-robin with the
  // role's own running prefix over the sizes, or the entry the producer warp published.
  auto consumer_tile = [&](uint32_t i, unsigned role_bit, TokenRange& tr) -> TileInfo {
    TileInfo ti;
    if constexpr (!kBalanced) {
      const long long t = blockIdx.x + static_cast<long long>(i) * gridDim.x;
      ti.tile = t < num_tiles ? t : -1;
      if (ti.tile >= 0) {
        ti.g = static_cast<int>(t / tiles_per_group);
        ti.tokens = tr.seek(ti.g);
        ti.start = tr.start;
      }
    } else {
      const int slot = i % L::kSchedDepth;
      ti.tile = -1;
      if (!wait_bounded(sched_full_bar(slot), (i / L::kSchedDepth) & 1u, abort_flag, status, role_bit)) return ti;
      const int t = sched_info[slot].x;
      ti.g = sched_info[slot].y;
      ti.tokens = sched_info[slot].z;
      ti.start = sched_info[slot].w;
      __syncwarp();
      if (lane == 0) mbar_arrive(sched_empty_bar(slot));
      ti.tile = t < num_tiles ? t : -1;
    }
    return ti;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    TokenRange tr;
    tr.init(sizes, sizes_i64, group_start, group_end);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    // Balanced mode: the claim of the next tile (an atomic, ~1 us) and its two dependent plan
    // look-ups are issued one step per k-block while this tile's loads stream, with volatile
    // instructions so that each sits where it is written and its latency passes before the
    // following step needs the result.
    int nx_t = 0, nx_slot = 0, nx_g = 0, nx_tokens = 0, nx_start = 0, nx_step = 3;
    auto prefetch_step = [&]() {
      if (nx_step == 0) {
        if (lane == 0) asm volatile("atom.global.add.u32 %0, [%1], 1;" : "=r"(nx_t) : "l"(scratch) : "memory");
      } else if (nx_step == 1) {
        nx_t = __shfl_sync(0xFFFFFFFFu, nx_t, 0);
        nx_slot = static_cast<int>(nx_t / tiles_per_group);
        if (nx_t < num_tiles) asm volatile("ld.global.nc.s32 %0, [%1];" : "=r"(nx_g) : "l"(plan_order + nx_slot));
      } else if (nx_step == 2) {
        if (nx_t < num_tiles) {
          asm volatile("ld.global.nc.s32 %0, [%1];" : "=r"(nx_tokens) : "l"(plan_tokens + nx_g));
          asm volatile("ld.global.nc.s32 %0, [%1];" : "=r"(nx_start) : "l"(plan_starts + nx_g));
        }
      }
      ++nx_step;
    };
    if constexpr (kBalanced) nx_step = 0;
    for (uint32_t i = 0; ok; ++i) {
      long long tile;
      int g, mt, nt;
      long long tokens;
      if constexpr (kBalanced) {
        while (nx_step < 3) prefetch_step();  // first tile, or a tile with fewer than three k-blocks
        // publish the claimed tile (also the end marker) to the other warps
        const int slot = i % L::kSchedDepth;
        if (!wait_bounded(sched_empty_bar(slot), ((i / L::kSchedDepth) & 1u) ^ 1u, abort_flag, status,
                          kDevTimeoutProducer))
          break;
        if (lane == 0) {
          sched_info[slot].x = nx_t;
          sched_info[slot].y = nx_g;
          sched_info[slot].z = nx_tokens;
          sched_info[slot].w = nx_start;
          mbar_arrive(sched_full_bar(slot));
        }
        __syncwarp();
        tile = nx_t;
        if (tile >= num_tiles) break;
        int slot_g;
        split_tile(tile, slot_g, mt, nt);
        g = nx_g;
        tokens = nx_tokens;
        tr.start = nx_start;
        nx_step = 0;
      } else {
        tile = blockIdx.x + static_cast<long long>(i) * gridDim.x;
        if (tile >= num_tiles) break;
        split_tile(tile, g, mt, nt);
        tokens = tr.seek(g);
      }
      const int num_kb = static_cast<int>((tokens + kTokensPerKb - 1) / kTokensPerKb);
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!wait_bounded(empty_bar(stage), phase ^ 1u, abort_flag, status, kDevTimeoutProducer)) {
          ok = false;
          break;
        }
        if (lane == 0) {
          const uint32_t a_dst = smem_base + stage * L::kStageBytes;
          const uint32_t b_dst = a_dst + L::kABytes;
          const int krow = static_cast<int>(tr.start + static_cast<long long>(kb) * kTokensPerKb);
          mbar_arrive_expect_tx(full_bar(stage), L::kStageBytes);
          if constexpr (kFp8) {
            tma_load_2d(a_dst, &tm_a, full_bar(stage), krow, mt * kBlockM);
            tma_load_2d(b_dst, &tm_b, full_bar(stage), krow, nt * kBlockN);
          } else {
#pragma unroll
            for (int j = 0; j < kBlockM / 64; ++j)
              tma_load_2d(a_dst + j * (kBlockK * 128), &tm_a, full_bar(stage), mt * kBlockM + j * 64, krow);
#pragma unroll
            for (int j = 0; j < kBlockN / 64; ++j)
              tma_load_2d(b_dst + j * (kBlockK * 128), &tm_b, full_bar(stage), nt * kBlockN + j * 64, krow);
          }
        }
        __syncwarp();
        if constexpr (kBalanced) {
          if (nx_step < 3) prefetch_step();
        }
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    TokenRange tr;
    tr.init(sizes, sizes_i64, group_start, group_end);
    const uint32_t a_fmt = kFp8 ? static_cast<uint32_t>(in_fmt & 0xF) : static_cast<uint32_t>(in_fmt);
    const uint32_t b_fmt = kFp8 ? static_cast<uint32_t>((in_fmt >> 4) & 0xF) : static_cast<uint32_t>(in_fmt);
    const uint32_t mn_major = kFp8 ? 0u : 1u;
    const uint32_t idesc = make_instr_desc(a_fmt, b_fmt, mn_major, mn_major, kBlockM, kBlockN);
    int stage = 0;
    uint32_t phase = 0;
    uint32_t tile_iter = 0;  // counts non-empty tiles only (same rule in the epilogue)
    bool ok = true;
    for (uint32_t i = 0; ok; ++i) {
      const TileInfo ti = consumer_tile(i, kDevTimeoutMma, tr);
      if (ti.tile < 0) break;
      const long long tokens = ti.tokens;
      if (tokens == 0) continue;
      const int num_kb = static_cast<int>((tokens + kTokensPerKb - 1) / kTokensPerKb);
      const uint32_t acc = tile_iter & 1u;
      const uint32_t acc_phase = (tile_iter >> 1) & 1u;
      ++tile_iter;
      if (!wait_bounded(tmem_empty_bar(acc), acc_phase ^ 1u, abort_flag, status, kDevTimeoutMma)) break;
      tc_fence_after_sync();
      const uint32_t d_tmem = tmem_base + acc * kBlockN;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!wait_bounded(full_bar(stage), phase, abort_flag, status, kDevTimeoutMma)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t a_addr = smem_base + stage * L::kStageBytes;
        int k16_steps = kBlockK / kUmmaK;
        if (!kFp8 && kb == num_kb - 1) {
          const int valid = static_cast<int>(tokens - static_cast<long long>(kb) * kBlockK);  // 1..64
          k16_steps = (valid + kUmmaK - 1) / kUmmaK;
          const int zero_rows = k16_steps * kUmmaK - valid;  // rows [valid, valid + zero_rows)
          if (zero_rows > 0) {
            // every chunk (A: 2, B: kBlockN/64) is [64 token rows][128 bytes]; a token row keeps
            // its own 128 bytes under the swizzle, so clearing whole rows is layout-agnostic
            constexpr int kChunks = (kBlockM + kBlockN) / 64;
            const int vec_per_chunk = zero_rows * 8;  // 16-byte vectors
            uint8_t* stage_ptr = smem + stage * L::kStageBytes;
            for (int i = lane; i < kChunks * vec_per_chunk; i += 32) {
              const int ch = i / vec_per_chunk;
              const int v = i - ch * vec_per_chunk;
              *reinterpret_cast<uint4*>(stage_ptr + ch * (kBlockK * 128) + valid * 128 + v * 16) =
                  make_uint4(0, 0, 0, 0);
            }
            fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core
          }
          __syncwarp();
        }
        if (lane == 0) {
          const uint32_t b_addr = a_addr + L::kABytes;
          for (int k16 = 0; k16 < k16_steps; ++k16) {
            // MN-major: a K step is 16 token rows of 128 bytes; K-major (fp8): 32 bytes in a row
            const uint32_t step = kFp8 ? 32u : kUmmaK * 128u;
            const uint32_t lbo = kFp8 ? 16u : kBlockK * 128u;
            const uint64_t a_desc = make_smem_desc(a_addr + k16 * step, lbo, 1024, kSwizzle128);
            const uint64_t b_desc = make_smem_desc(b_addr + k16 * step, lbo, 1024, kSwizzle128);
            umma<1, kFp8>(d_tmem, a_desc, b_desc, idesc, (kb | k16) != 0 ? 1u : 0u);
          }
          umma_commit_1cta(empty_bar(stage));
        }
        __syncwarp();
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (ok && lane == 0) umma_commit_1cta(tmem_full_bar(acc));
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    TokenRange tr;
    tr.init(sizes, sizes_i64, group_start, group_end);
    const int quarter = warp & 3;
    uint8_t* epi_stage = smem + L::kEpiOffset + quarter * kEpiStageBytesPerWarp;
    int epi_sel = 0;
    uint32_t tile_iter = 0;
    for (uint32_t i = 0;; ++i) {
      const TileInfo ti = consumer_tile(i, kDevTimeoutEpilogue, tr);
      if (ti.tile < 0) break;
      int slot_g, mt, nt;
      split_tile(ti.tile, slot_g, mt, nt);
      const int g = ti.g;
      const long long tokens = ti.tokens;
      const int row = mt * kBlockM + quarter * 32 + lane;
      const bool row_ok = row < m_dim;
      uint16_t* c_row = static_cast<uint16_t*>(c_ptr) +
                        (static_cast<long long>(g) * m_dim + row) * static_cast<long long>(n_dim);
      if (tokens == 0) {
        store_zero_row_16bit<kBlockN>(c_row, row_ok, nt * kBlockN, n_dim);
        continue;
      }
      const uint32_t acc = tile_iter & 1u;
      const uint32_t acc_phase = (tile_iter >> 1) & 1u;
      ++tile_iter;
      if (!wait_bounded(tmem_full_bar(acc), acc_phase, abort_flag, status, kDevTimeoutEpilogue)) break;
      tc_fence_after_sync();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kBlockN;
      float rs = 1.0f;
      const float* cs = nullptr;
      if constexpr (kFp8) {
        rs = row_ok ? __ldg(a_scale + static_cast<long long>(g) * m_dim + row) : 0.f;
        cs = b_scale + static_cast<long long>(g) * n_dim;
      }
      const int row_w0 = mt * kBlockM + quarter * 32;
      if (row_w0 + 32 <= m_dim)
        store_acc_warp_tma<kBlockN, kFp8>(t_addr, &tm_c, epi_stage, epi_sel, row_w0, g, nt * kBlockN, n_dim, out_fp16,
                                          lane, rs, cs);
      else
        store_acc_row_16bit<kBlockN, kFp8>(t_addr, c_row, row_ok, nt * kBlockN, n_dim, out_fp16, rs, cs);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty_bar(acc));
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

template <int kBlockN, int kStages, bool kFp8>
static int launch_k_grouped(const CUtensorMap& tm_a, const CUtensorMap& tm_b, const CUtensorMap& tm_c, void* c,
                            const void* sizes, int sizes_is_i64, const int* gs, const int* ge, int num_groups,
                            int m_dim, int n_dim, long long k_total, int in_fmt, int out_fp16, const float* a_scale,
                            const float* b_scale, int* scratch, int grid, cudaStream_t stream) {
  using L = KGroupedSmem<kBlockN, kStages>;
  unsigned* status = device_status_ptr();
  if (scratch) {
    // balanced: plan (starts, token counts, longest-first order, zeroed tile counter), then the GEMM
    auto kern = k_grouped_kernel<kBlockN, kStages, kFp8, true>;
    B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes));
    k_grouped_plan_kernel<<<1, 1024, 0, stream>>>(sizes, sizes_is_i64, gs, ge, num_groups, scratch);
    B200_CUDA(cudaGetLastError());
    kern<<<grid, kNumThreads, L::kDynamicBytes, stream>>>(tm_a, tm_b, tm_c, c, sizes, sizes_is_i64, gs, ge, num_groups,
                                                          m_dim, n_dim, k_total, in_fmt, out_fp16, a_scale, b_scale,
                                                          scratch, status);
  } else {
    auto kern = k_grouped_kernel<kBlockN, kStages, kFp8, false>;
    B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes));
    kern<<<grid, kNumThreads, L::kDynamicBytes, stream>>>(tm_a, tm_b, tm_c, c, sizes, sizes_is_i64, gs, ge, num_groups,
                                                          m_dim, n_dim, k_total, in_fmt, out_fp16, a_scale, b_scale,
                                                          nullptr, status);
  }
  B200_CUDA(cudaGetLastError());
  return 0;
}

constexpr int kMaxBalancedGroups = 4096;

// validates a caller-provided scratch buffer for the balanced scheduler; nullptr = round-robin
static int check_scratch(void* workspace, long long workspace_bytes, int num_groups, const char* who, int** out) {
  *out = nullptr;
  if (!workspace) return 0;
  B200_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 3) == 0, "%s: workspace must be 4-byte aligned", who);
  B200_REQUIRE(num_groups <= kMaxBalancedGroups, "%s: the balanced scheduler supports at most %d groups (got %d)", who,
               kMaxBalancedGroups, num_groups);
  const long long need = k_grouped_scratch_words(num_groups) * 4;
  B200_REQUIRE(workspace_bytes >= need, "%s: workspace of %lld bytes is too small, %lld needed", who, workspace_bytes,
               need);
  *out = static_cast<int*>(workspace);
  return 0;
}

// CTA pairs (256 x 256 tiles, gemm_k_pair.cu) need the balanced scheduler's scratch and enough
// tiles for every pair of SMs; the tuning knob can force them on or off
static bool want_k_pair(const int* scratch, int num_groups, int m_dim, int n_dim, int grid) {
  if (!scratch || grid < 2 || g_cta_pair_mode == 0) return false;
  if (g_cta_pair_mode == 1) return true;
  const long long tiles = static_cast<long long>(num_groups) * ((m_dim + 255) / 256) * ((n_dim + 255) / 256);
  return m_dim >= 256 && n_dim >= 256 && tiles >= grid;
}

static int launch_plan(const void* sizes, int sizes_is_i64, const int* gs, const int* ge, int num_groups, int* scratch,
                       cudaStream_t stream) {
  k_grouped_plan_kernel<<<1, 1024, 0, stream>>>(sizes, sizes_is_i64, gs, ge, num_groups, scratch);
  B200_CUDA(cudaGetLastError());
  return 0;
}

// for the other K-grouped translation units: validate a workspace and queue the plan kernel
// (starts, token counts, longest-first order) on it; *out = nullptr when no workspace was given
int k_grouped_plan_into(void* workspace, long long workspace_bytes, const void* sizes, int sizes_is_i64,
                        int num_groups, const char* who, int** out, cudaStream_t stream) {
  int rc = check_scratch(workspace, workspace_bytes, num_groups, who, out);
  if (rc || !*out) return rc;
  return launch_plan(sizes, sizes_is_i64, nullptr, nullptr, num_groups, *out, stream);
}

// tile width: 256 output columns unless that leaves SMs without a tile
static int pick_block_n(int num_groups, int m_dim, int n_dim, int grid) {
  const long long m_tiles = static_cast<long long>(num_groups) * ((m_dim + 127) / 128);
  if (n_dim <= 64 || m_tiles * ((n_dim + 127) / 128) < grid) return 64;
  if (n_dim <= 128 || m_tiles * ((n_dim + 255) / 256) < grid) return 128;
  return 256;
}

}  // namespace b200

extern "C" long long b200gemm_k_grouped_workspace_bytes(int num_groups) {
  return num_groups < 0 ? 0 : b200::k_grouped_scratch_words(num_groups) * 4;
}

namespace b200 {
static int k_grouped_bf16(const void* a, const void* b, void* c, const void* sizes, int sizes_is_i64,
                          const int* group_start, const int* group_end, int num_groups, int64_t k_total, int m_dim,
                          int n_dim, int dtype, int* scratch, int num_sms, void* stream_v, const char* who) {
  B200_REQUIRE(dtype == 0 || dtype == 1, "%s: dtype must be 0 (bf16) or 1 (fp16), got %d", who, dtype);
  B200_REQUIRE(num_groups >= 0 && k_total >= 0 && m_dim >= 0 && n_dim >= 0, "%s: negative dimension", who);
  if (num_groups == 0 || m_dim == 0 || n_dim == 0) return 0;
  B200_REQUIRE(c && (sizes || (group_start && group_end)), "%s: null pointer", who);
  B200_REQUIRE((group_start == nullptr) == (group_end == nullptr), "%s: pass both group_start and group_end or neither",
               who);
  B200_REQUIRE(m_dim % 8 == 0, "%s: A row stride must be 16-byte aligned (M_DIM=%d)", who, m_dim);
  B200_REQUIRE(n_dim % 8 == 0, "%s: B row stride must be 16-byte aligned (N_DIM=%d)", who, n_dim);
  B200_REQUIRE(k_total < (1ll << 31), "%s: K_TOTAL must fit in int32", who);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(a) & 15) == 0 && (reinterpret_cast<uintptr_t>(b) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(c) & 15) == 0,
               "%s: base pointers must be 16-byte aligned", who);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const int sms = sm_count();
  B200_REQUIRE(sms > 0, "%s: no CUDA device", who);
  const int grid = (num_sms > 0 && num_sms < sms) ? num_sms : sms;

  // With no tokens at all there is nothing to load: tensor maps need a non-empty tensor, so
  // point them at the (never dereferenced) output instead.
  const void* a_base = (k_total > 0 && a) ? a : c;
  const void* b_base = (k_total > 0 && b) ? b : c;
  B200_REQUIRE(k_total == 0 || (a && b), "%s: null pointer", who);
  const uint64_t rows = k_total > 0 ? static_cast<uint64_t>(k_total) : 1;
  const CUtensorMapDataType dt = dtype == 1 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tm_a, tm_b;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(m_dim), rows};
    const uint64_t strides[1] = {static_cast<uint64_t>(m_dim) * 2};
    const uint32_t box[2] = {64, kBlockK};
    int rc = encode_tmap(&tm_a, dt, 2, a_base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, "A[K_TOTAL,M_DIM]");
    if (rc) return rc;
  }
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(n_dim), rows};
    const uint64_t strides[1] = {static_cast<uint64_t>(n_dim) * 2};
    const uint32_t box[2] = {64, kBlockK};
    int rc = encode_tmap(&tm_b, dt, 2, b_base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, "B[K_TOTAL,N_DIM]");
    if (rc) return rc;
  }
  CUtensorMap tm_c;
  {
    const uint64_t dims[3] = {static_cast<uint64_t>(n_dim), static_cast<uint64_t>(m_dim),
                              static_cast<uint64_t>(num_groups)};
    const uint64_t strides[2] = {static_cast<uint64_t>(n_dim) * 2, static_cast<uint64_t>(n_dim) * m_dim * 2};
    const uint32_t box[3] = {64, 32, 1};
    int rc = encode_tmap(&tm_c, dt, 3, c, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, "C[G,M_DIM,N_DIM]");
    if (rc) return rc;
  }
  const int in_fmt = dtype == 1 ? 0 : 1;  // UMMA kind::f16 operand format: 0 = f16, 1 = bf16
  if (want_k_pair(scratch, num_groups, m_dim, n_dim, grid)) {
    int rc = launch_plan(sizes, sizes_is_i64, group_start, group_end, num_groups, scratch, stream);
    if (rc) return rc;
    return launch_k_grouped_pair<false>(tm_a, tm_b, tm_c, c, num_groups, m_dim, n_dim, in_fmt, dtype, nullptr, nullptr,
                                        scratch, grid, stream);
  }
  const int bn = pick_block_n(num_groups, m_dim, n_dim, grid);
#define B200_LAUNCH_K(BN, ST)                                                                                     \
  launch_k_grouped<BN, ST, false>(tm_a, tm_b, tm_c, c, sizes, sizes_is_i64, group_start, group_end, num_groups, m_dim,  \
                                  n_dim, k_total, in_fmt, dtype, nullptr, nullptr, scratch, grid, stream)
  if (bn == 64) return B200_LAUNCH_K(64, 8);
  if (bn == 128) return B200_LAUNCH_K(128, 6);
  return B200_LAUNCH_K(256, 4);
#undef B200_LAUNCH_K
}
}  // namespace b200

extern "C" int b200gemm_k_grouped(const void* a, const void* b, void* c, const void* sizes, int sizes_is_i64,
                                  const int* group_start, const int* group_end, int num_groups, int64_t k_total,
                                  int m_dim, int n_dim, int dtype, void* workspace, int64_t workspace_bytes,
                                  int num_sms, void* stream) {
  int* scratch = nullptr;
  int rc = b200::check_scratch(workspace, workspace_bytes, num_groups, "b200gemm_k_grouped", &scratch);
  if (rc) return rc;
  return b200::k_grouped_bf16(a, b, c, sizes, sizes_is_i64, group_start, group_end, num_groups, k_total, m_dim, n_dim,
                              dtype, scratch, num_sms, stream, "b200gemm_k_grouped");
}

extern "C" int b200gemm_fp8_k_grouped_rowcol(const void* x, const float* x_scale, const void* y, const float* y_scale,
                                             void* out, const void* tokens_per_expert, int sizes_is_i64,
                                             int num_groups, int64_t k_total, int m_dim, int n_dim, int fmt_x,
                                             int fmt_y, void* workspace, int64_t workspace_bytes, int num_sms,
                                             void* stream_v) {
  using namespace b200;
  const char* who = "b200gemm_fp8_k_grouped_rowcol";
  int* scratch = nullptr;
  {
    int rc = check_scratch(workspace, workspace_bytes, num_groups, who, &scratch);
    if (rc) return rc;
  }
  B200_REQUIRE((fmt_x == 0 || fmt_x == 1) && (fmt_y == 0 || fmt_y == 1), "%s: fp8 format must be 0 (e4m3) or 1 (e5m2)",
               who);
  B200_REQUIRE(num_groups >= 0 && k_total >= 0 && m_dim >= 0 && n_dim >= 0, "%s: negative dimension", who);
  if (num_groups == 0 || m_dim == 0 || n_dim == 0) return 0;
  B200_REQUIRE(x && y && out && tokens_per_expert && x_scale && y_scale, "%s: null pointer", who);
  B200_REQUIRE(k_total > 0 && k_total % 16 == 0, "%s: K_total (%lld) must be a positive multiple of 16", who,
               (long long)k_total);
  B200_REQUIRE(n_dim % 8 == 0, "%s: N must be a multiple of 8 (N=%d)", who, n_dim);
  B200_REQUIRE(k_total < (1ll << 31), "%s: K_total must fit in int32", who);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(out) & 15) == 0 && (reinterpret_cast<uintptr_t>(y_scale) & 15) == 0,
               "%s: x, y, out and y_scale must be 16-byte aligned", who);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const int sms = sm_count();
  B200_REQUIRE(sms > 0, "%s: no CUDA device", who);
  const int grid = (num_sms > 0 && num_sms < sms) ? num_sms : sms;
  const bool pair = want_k_pair(scratch, num_groups, m_dim, n_dim, grid);
  const int bn = pair ? 128 : pick_block_n(num_groups, m_dim, n_dim, grid);  // pair: 128 rows of Y per CTA
  CUtensorMap tm_x, tm_y;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(k_total), static_cast<uint64_t>(m_dim)};
    const uint64_t strides[1] = {static_cast<uint64_t>(k_total)};
    const uint32_t box[2] = {128, kBlockM};
    int rc = encode_tmap(&tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, x, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                         "X[M,K_TOTAL]");
    if (rc) return rc;
  }
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(k_total), static_cast<uint64_t>(n_dim)};
    const uint64_t strides[1] = {static_cast<uint64_t>(k_total)};
    const uint32_t box[2] = {128, static_cast<uint32_t>(bn)};
    int rc = encode_tmap(&tm_y, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, y, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                         "Y[N,K_TOTAL]");
    if (rc) return rc;
  }
  CUtensorMap tm_c;
  {
    const uint64_t dims[3] = {static_cast<uint64_t>(n_dim), static_cast<uint64_t>(m_dim),
                              static_cast<uint64_t>(num_groups)};
    const uint64_t strides[2] = {static_cast<uint64_t>(n_dim) * 2, static_cast<uint64_t>(n_dim) * m_dim * 2};
    const uint32_t box[3] = {64, 32, 1};
    int rc = encode_tmap(&tm_c, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, out, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, "C[G,M_DIM,N_DIM]");
    if (rc) return rc;
  }
  const int in_fmt = fmt_x | (fmt_y << 4);
  if (pair) {
    int rc = launch_plan(tokens_per_expert, sizes_is_i64, nullptr, nullptr, num_groups, scratch, stream);
    if (rc) return rc;
    return launch_k_grouped_pair<true>(tm_x, tm_y, tm_c, out, num_groups, m_dim, n_dim, in_fmt, /*out bf16*/ 0, x_scale,
                                       y_scale, scratch, grid, stream);
  }
#define B200_LAUNCH_K8(BN, ST)                                                                                  \
  launch_k_grouped<BN, ST, true>(tm_x, tm_y, tm_c, out, tokens_per_expert, sizes_is_i64, nullptr, nullptr, num_groups, \
                                 m_dim, n_dim, k_total, in_fmt, /*out bf16*/ 0, x_scale, y_scale, scratch, grid, stream)
  if (bn == 64) return B200_LAUNCH_K8(64, 8);
  if (bn == 128) return B200_LAUNCH_K8(128, 6);
  return B200_LAUNCH_K8(256, 4);
#undef B200_LAUNCH_K8
}

// ------------------------------------------------------------------ balanced K-grouped GEMM without caller scratch
// Some hosts of this library cannot hand it device memory: a serving runtime that reserved the
// whole HBM for its own pools at start-up (a later cudaMalloc fails or is forbidden by policy),
// or a latency-critical loop in which cudaMalloc's implicit device-wide synchronisation is not
// acceptable, called from C where the framework's caching allocator is out of reach.  For them
// the scheduler's scratch lives in this fixed array, which every GPU that loads the library
// carries until the process exits: (64 + 3 * 1024) * 4 bytes = 12.5 KB.
namespace b200 {

constexpr int kStaticScratchMaxGroups = 1024;
static __device__ __align__(256) int g_k_grouped_static_scratch[kPlanHeaderWords + 3 * kStaticScratchMaxGroups];

// Device address of the array on the current device.  In host code the array's name is only a
// handle for the runtime, never a pointer a kernel may dereference, so the address is looked up
// with cudaGetSymbolAddress - once per device, with that device current - and cached.
static int static_scratch_address(int** out, const char* who) {
  static std::mutex mu;
  static int* cached[64] = {nullptr};
  int dev = 0;
  B200_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return set_error(kErrUnsupported, "%s: device index %d out of range", who, dev);
  std::lock_guard<std::mutex> lock(mu);
  if (!cached[dev]) {
    int* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_k_grouped_static_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return set_error(kErrCuda, "%s: cudaGetSymbolAddress failed for the static scratch: %s", who,
                       cudaGetErrorString(e));
    cached[dev] = ptr;
  }
  *out = cached[dev];
  return 0;
}

}  // namespace b200

extern "C" int b200gemm_k_grouped_static_scratch(const void* a, const void* b, void* c, const void* sizes,
                                                 int sizes_is_i64, const int* group_start, const int* group_end,
                                                 int num_groups, int64_t k_total, int m_dim, int n_dim, int dtype,
                                                 int num_sms, void* stream) {
  using namespace b200;
  const char* who = "b200gemm_k_grouped_static_scratch";
  B200_REQUIRE(num_groups <= kStaticScratchMaxGroups,
               "%s: %d groups exceed the %d the built-in scratch holds; use b200gemm_k_grouped with a workspace", who,
               num_groups, kStaticScratchMaxGroups);
  int* scratch = nullptr;
  int rc = static_scratch_address(&scratch, who);
  if (rc) return rc;
  // The plan kernel launched inside rewrites every word it later reads (tile counter, starts,
  // token counts, order), so whatever the previous call left in the array is harmless.
  return k_grouped_bf16(a, b, c, sizes, sizes_is_i64, group_start, group_end, num_groups, k_total, m_dim, n_dim, dtype,
                        scratch, num_sms, stream, who);
}
