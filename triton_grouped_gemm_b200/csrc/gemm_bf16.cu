// BF16 / FP16 M-grouped and masked M-grouped GEMM for sm_100a.
//
// One persistent CTA per SM.  Warp roles:
//   warp 0      TMA producer: walks the group sizes once, loads A / B_g tiles into a
//               multi-stage shared-memory ring (128-byte swizzle)
//   warp 1      MMA issuer: one lane issues tcgen05.mma (128 x BLOCK_N x 16) into one of two
//               TMEM accumulators, commits ring slots back to the producer
//   warps 2..5  epilogue: tcgen05.ld the finished accumulator (one TMEM lane quarter per
//               warp), round once to the output type, masked 16-byte stores
// The accumulator is double buffered so the epilogue of tile i overlaps the main loop of
// tile i+1.  Tile numbering is "padded tile space" (each group owns ceil(rows/128) row
// tiles); nothing is precomputed on the host and nothing is synchronised.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../../include/b200gemm.h"
#include "common.cuh"
#include "gemm_tile.cuh"

namespace b200 {

template <int kBlockN, int kStages>
struct MGroupedSmem {
  static constexpr int kABytes = kBlockM * kBlockK * 2;
  static constexpr int kBBytes = kBlockN * kBlockK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kEpiOffset = kStages * kStageBytes;  // 4 warps x 2 x 4 KB store staging
  static constexpr int kBarOffset = kEpiOffset + 4 * kEpiStageBytesPerWarp;
  // full[kStages], empty[kStages], tmem_full[2], tmem_empty[2], then tmem ptr + abort flag
  static constexpr int kNumBars = 2 * kStages + 4;
  static constexpr int kTotal = kBarOffset + kNumBars * 8 + 16;
  static constexpr int kDynamicBytes = kTotal + 1024;  // slack for manual 1024-byte alignment
};

// kFp8 = false: 16-bit operands (`in_fmt`: 0 = f16, 1 = bf16), kBlockK = 64 elements.
// kFp8 = true:  8-bit operands (`in_fmt` = a_fmt | b_fmt << 4, 0 = e4m3, 1 = e5m2), 128
//               elements per k-block, and the epilogue applies a_scale[row] * b_scale[g*n+col]
//               (per-row activation x per-expert-per-channel weight scales, the reference's
//               gemm/FP8/m_grouped_gemm_channel_expert.py:119-136).  A k-block is 128 bytes
//               per row either way, so the shared-memory ring is identical.
template <int kBlockN, int kStages, bool kBMnMajor, bool kFp8>
__global__ void __launch_bounds__(kNumThreads, 1)
m_grouped_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                 const __grid_constant__ CUtensorMap tm_c, void* __restrict__ c_ptr, const void* __restrict__ sizes, int sizes_i64, int num_groups,
                 int masked_stride, long long m_rows, int n, int k, int in_fmt, int out_fp16,
                 const float* __restrict__ a_scale, const float* __restrict__ b_scale, unsigned* status) {
  static_assert(!(kFp8 && kBMnMajor), "fp8 operands are K-major only");
  constexpr int kElemsPerKb = kFp8 ? 128 : 64;
  using L = MGroupedSmem<kBlockN, kStages>;
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
  const int num_kb = (k + kElemsPerKb - 1) / kElemsPerKb;
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

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    GroupWalker w;
    w.init(sizes, sizes_i64, num_groups, masked_stride, kBlockM, m_rows);
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
          const uint32_t b_dst = a_dst + L::kABytes;
          mbar_arrive_expect_tx(full_bar(stage), L::kStageBytes);
          tma_load_2d(a_dst, &tm_a, full_bar(stage), kb * kElemsPerKb, row0);
          if constexpr (!kBMnMajor) {
            tma_load_3d(b_dst, &tm_b, full_bar(stage), kb * kElemsPerKb, nt * kBlockN, g);
          } else {
#pragma unroll
            for (int j = 0; j < kBlockN / 64; ++j)
              tma_load_3d(b_dst + j * (kBlockK * 128), &tm_b, full_bar(stage), nt * kBlockN + j * 64, kb * kBlockK, g);
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
    // ------------------------------------------------------------ MMA issuer
    GroupWalker w;
    w.init(sizes, sizes_i64, num_groups, masked_stride, kBlockM, m_rows);
    const uint32_t a_fmt = kFp8 ? static_cast<uint32_t>(in_fmt & 0xF) : static_cast<uint32_t>(in_fmt);
    const uint32_t b_fmt = kFp8 ? static_cast<uint32_t>((in_fmt >> 4) & 0xF) : static_cast<uint32_t>(in_fmt);
    const uint32_t idesc = make_instr_desc(a_fmt, b_fmt, 0u, kBMnMajor ? 1u : 0u, kBlockM, kBlockN);
    int stage = 0;
    uint32_t phase = 0;
    uint32_t tile_iter = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok; tile += gridDim.x, ++tile_iter) {
      const int mt = tile / n_tiles;
      if (!w.seek(mt)) break;
      const uint32_t acc = tile_iter & 1u;
      const uint32_t acc_phase = (tile_iter >> 1) & 1u;
      if (!wait_bounded(tmem_empty_bar(acc), acc_phase ^ 1u, abort_flag, status, kDevTimeoutMma)) break;
      tc_fence_after_sync();
      const uint32_t d_tmem = tmem_base + acc * kBlockN;
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
          for (int k16 = 0; k16 < kBlockK / kUmmaK; ++k16) {
            const uint64_t a_desc = make_smem_desc(a_addr + k16 * (kUmmaK * 2), 16, 1024, kSwizzle128);
            const uint64_t b_desc =
                kBMnMajor ? make_smem_desc(b_addr + k16 * (kUmmaK * 128), kBlockK * 128, 1024, kSwizzle128)
                          : make_smem_desc(b_addr + k16 * (kUmmaK * 2), 16, 1024, kSwizzle128);
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
    GroupWalker w;
    w.init(sizes, sizes_i64, num_groups, masked_stride, kBlockM, m_rows);
    const int quarter = warp & 3;  // TMEM lane quarter this warp may read
    uint8_t* epi_stage = smem + L::kEpiOffset + quarter * kEpiStageBytesPerWarp;
    int epi_sel = 0;
    uint32_t tile_iter = 0;
    for (int tile = blockIdx.x;; tile += gridDim.x, ++tile_iter) {
      const int mt = tile / n_tiles;
      const int nt = tile - mt * n_tiles;
      if (!w.seek(mt)) break;
      const long long row = w.tile_row0(mt) + quarter * 32 + lane;
      const bool row_ok = row < w.group_row_end();
      const uint32_t acc = tile_iter & 1u;
      const uint32_t acc_phase = (tile_iter >> 1) & 1u;
      if (!wait_bounded(tmem_full_bar(acc), acc_phase, abort_flag, status, kDevTimeoutEpilogue)) break;
      tc_fence_after_sync();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * kBlockN;
      uint16_t* c_row = static_cast<uint16_t*>(c_ptr) + row * static_cast<long long>(n);
      // warps whose 32 rows all belong to the group take the staged TMA-store path; a warp
      // that straddles the end of its group falls back to masked per-thread stores
      const long long row_w0 = w.tile_row0(mt) + quarter * 32;
      const bool warp_full = row_w0 + 32 <= w.group_row_end();
      float rs = 1.0f;
      const float* cs = nullptr;
      if constexpr (kFp8) {
        rs = row_ok ? __ldg(a_scale + row) : 0.f;
        cs = b_scale + static_cast<long long>(w.g) * n;
      }
      if (warp_full)
        store_acc_warp_tma<kBlockN, kFp8>(t_addr, &tm_c, epi_stage, epi_sel, static_cast<int>(row_w0), -1,
                                          nt * kBlockN, n, out_fp16, lane, rs, cs);
      else
        store_acc_row_16bit<kBlockN, kFp8>(t_addr, c_row, row_ok, nt * kBlockN, n, out_fp16, rs, cs);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty_bar(acc));
    }
    if (lane == 0) tma_store_wait_all<0>();  // staged stores have left shared memory and landed
    // the sizes added up to more rows than A / C have: the excess was cut off, tell the host
    if (w.overflow && quarter == 0 && lane == 0 && status) atomicOr(status, kDevBadGroupSize);
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    // a role gave up: give copies / MMAs still in flight time to land before the shared
    // memory and TMEM of this CTA are released
    for (int i = 0; i < 64; ++i) __nanosleep(4000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------ host side
template <int kBlockN, int kStages, bool kBMnMajor, bool kFp8>
static int launch_m_grouped(const CUtensorMap& tm_a, const CUtensorMap& tm_b, const CUtensorMap& tm_c, void* c,
                            const void* sizes,
                            int sizes_is_i64, int num_groups, int masked_stride, long long m_rows, int n, int k,
                            int in_fmt, int out_fp16, const float* a_scale, const float* b_scale, int grid,
                            cudaStream_t stream) {
  using L = MGroupedSmem<kBlockN, kStages>;
  auto kern = m_grouped_kernel<kBlockN, kStages, kBMnMajor, kFp8>;
  B200_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamicBytes));
  unsigned* status = device_status_ptr();
  kern<<<grid, kNumThreads, L::kDynamicBytes, stream>>>(tm_a, tm_b, tm_c, c, sizes, sizes_is_i64, num_groups, masked_stride,
                                                        m_rows, n, k, in_fmt, out_fp16, a_scale, b_scale, status);
  B200_CUDA(cudaGetLastError());
  return 0;
}

// 0 = choose the tile width from the problem size; 64 / 128 / 256 force one variant
static int g_forced_block_n = 0;
int g_cta_pair_mode = -1;

// The CTA-pair kernel pays off when every pair of SMs gets 256 x 256 tiles to work on.
static bool want_pair(long long m_rows, int num_groups, int n, int grid, int block_n) {
  if (g_cta_pair_mode == 0 || grid < 2) return false;
  if (g_cta_pair_mode == 1) return true;
  if (block_n != 256 || g_forced_block_n) return false;
  const long long pair_tiles = (m_rows / 256) * ((n + 255) / 256);
  return pair_tiles >= grid / 2 && m_rows / 256 >= 4ll * num_groups;
}

static int m_grouped_common(const void* a, const void* b, void* c, const void* sizes, int sizes_is_i64,
                            int num_groups, int64_t m_rows, int masked_stride, int n, int k, int trans_b, int dtype,
                            int num_sms, void* stream_v, const char* who) {
  B200_REQUIRE(dtype == 0 || dtype == 1, "%s: dtype must be 0 (bf16) or 1 (fp16), got %d", who, dtype);
  B200_REQUIRE(num_groups >= 0 && m_rows >= 0 && n >= 0 && k >= 0, "%s: negative dimension", who);
  if (num_groups == 0 || m_rows == 0 || n == 0) return 0;
  B200_REQUIRE(k > 0, "%s: k must be positive", who);
  B200_REQUIRE(a && b && c && sizes, "%s: null pointer", who);
  B200_REQUIRE(k % 8 == 0, "%s: TMA required 16-byte alignment: k*2 bytes (k=%d)", who, k);
  B200_REQUIRE(n % 8 == 0, "%s: TMA required 16-byte alignment: n*2 bytes (n=%d)", who, n);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(a) & 15) == 0 && (reinterpret_cast<uintptr_t>(b) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(c) & 15) == 0,
               "%s: base pointers must be 16-byte aligned", who);
  B200_REQUIRE(m_rows < (1ll << 31), "%s: m_rows must fit in int32", who);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const int sms = sm_count();
  B200_REQUIRE(sms > 0, "%s: no CUDA device", who);
  const int grid = (num_sms > 0 && num_sms < sms) ? num_sms : sms;

  // Tile width: 256 columns unless the problem is too small to give every SM a tile.
  const long long m_tiles_est = (m_rows + kBlockM - 1) / kBlockM;
  int block_n = 256;
  if (n <= 64 || m_tiles_est * ((n + 127) / 128) < grid) block_n = 64;
  else if (n <= 128 || m_tiles_est * ((n + 255) / 256) < grid) block_n = 128;
  if (g_forced_block_n) block_n = g_forced_block_n;
  // masked layout: every slot ends in a partial row tile, and a 256-row pair tile wastes twice what
  // a 128-row tile does there (measured: 1221 against 1182 TFLOP/s on 128 slots of ~880 valid rows)
  const bool pair = (masked_stride > 0 && g_cta_pair_mode != 1) ? false : want_pair(m_rows, num_groups, n, grid, block_n);
  if (pair) block_n = 128;  // per-CTA slice of the 256-wide pair tile (tensor-map box rows)

  const CUtensorMapDataType dt = dtype == 1 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap tm_a, tm_b;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(k), static_cast<uint64_t>(m_rows)};
    const uint64_t strides[1] = {static_cast<uint64_t>(k) * 2};
    const uint32_t box[2] = {kBlockK, kBlockM};
    int rc = encode_tmap(&tm_a, dt, 2, a, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, "A");
    if (rc) return rc;
  }
  if (trans_b) {
    const uint64_t dims[3] = {static_cast<uint64_t>(k), static_cast<uint64_t>(n), static_cast<uint64_t>(num_groups)};
    const uint64_t strides[2] = {static_cast<uint64_t>(k) * 2, static_cast<uint64_t>(k) * n * 2};
    const uint32_t box[3] = {kBlockK, static_cast<uint32_t>(block_n), 1};
    int rc = encode_tmap(&tm_b, dt, 3, b, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, "B[G,N,K]");
    if (rc) return rc;
  } else {
    const uint64_t dims[3] = {static_cast<uint64_t>(n), static_cast<uint64_t>(k), static_cast<uint64_t>(num_groups)};
    const uint64_t strides[2] = {static_cast<uint64_t>(n) * 2, static_cast<uint64_t>(k) * n * 2};
    const uint32_t box[3] = {64, kBlockK, 1};
    int rc = encode_tmap(&tm_b, dt, 3, b, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, "B[G,K,N]");
    if (rc) return rc;
  }

  CUtensorMap tm_c;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(n), static_cast<uint64_t>(m_rows)};
    const uint64_t strides[1] = {static_cast<uint64_t>(n) * 2};
    const uint32_t box[2] = {64, 32};
    int rc = encode_tmap(&tm_c, dt, 2, c, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, "C");
    if (rc) return rc;
  }
  const int in_fmt = dtype == 1 ? 0 : 1;  // UMMA kind::f16 operand format: 0 = f16, 1 = bf16
  if (pair) {
    const int want = (num_sms > 0 && num_sms < sms) ? num_sms : 0;
    return trans_b ? launch_m_grouped_pair<false, false>(tm_a, tm_b, tm_c, c, sizes, sizes_is_i64, num_groups,
                                                         masked_stride, m_rows, n, k, in_fmt, dtype, nullptr, nullptr, want,
                                                         stream)
                   : launch_m_grouped_pair<true, false>(tm_a, tm_b, tm_c, c, sizes, sizes_is_i64, num_groups,
                                                        masked_stride, m_rows, n, k, in_fmt, dtype, nullptr, nullptr, want,
                                                        stream);
  }
#define B200_LAUNCH(BN, ST)                                                                                          \
  (trans_b ? launch_m_grouped<BN, ST, false, false>(tm_a, tm_b, tm_c, c, sizes, sizes_is_i64, num_groups, masked_stride, m_rows, n, \
                                                    k, in_fmt, dtype, nullptr, nullptr, grid, stream)                \
           : launch_m_grouped<BN, ST, true, false>(tm_a, tm_b, tm_c, c, sizes, sizes_is_i64, num_groups, masked_stride, m_rows, n,  \
                                                   k, in_fmt, dtype, nullptr, nullptr, grid, stream))
  if (block_n == 256) return B200_LAUNCH(256, 4);
  if (block_n == 128) return B200_LAUNCH(128, 6);
  return B200_LAUNCH(64, 8);
#undef B200_LAUNCH
}

// FP8 operands with per-row activation scales and per-expert-per-channel weight scales.
static int fp8_rowcol_m_grouped(const void* a, const float* a_scale, const void* b, const float* b_scale, void* c,
                                const void* sizes, int sizes_is_i64, int num_groups, int64_t m_rows, int n, int k,
                                int fmt_a, int fmt_b, int out_dtype, int num_sms, void* stream_v) {
  const char* who = "b200gemm_fp8_m_grouped_rowcol";
  B200_REQUIRE((fmt_a == 0 || fmt_a == 1) && (fmt_b == 0 || fmt_b == 1), "%s: fp8 format must be 0 (e4m3) or 1 (e5m2)",
               who);
  B200_REQUIRE(out_dtype == 0 || out_dtype == 1, "%s: out_dtype must be 0 (bf16) or 1 (fp16)", who);
  B200_REQUIRE(num_groups >= 0 && m_rows >= 0 && n >= 0 && k >= 0, "%s: negative dimension", who);
  if (num_groups == 0 || m_rows == 0 || n == 0) return 0;
  B200_REQUIRE(k > 0, "%s: k must be positive", who);
  B200_REQUIRE(a && b && c && sizes && a_scale && b_scale, "%s: null pointer", who);
  B200_REQUIRE(k % 16 == 0, "%s: TMA required 16-byte alignment: k bytes (k=%d)", who, k);
  B200_REQUIRE(n % 8 == 0, "%s: n must be a multiple of 8 (n=%d)", who, n);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(a) & 15) == 0 && (reinterpret_cast<uintptr_t>(b) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(c) & 15) == 0 && (reinterpret_cast<uintptr_t>(b_scale) & 15) == 0,
               "%s: a, b, c and b_scale must be 16-byte aligned", who);
  B200_REQUIRE(m_rows < (1ll << 31), "%s: m_rows must fit in int32", who);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const int sms = sm_count();
  B200_REQUIRE(sms > 0, "%s: no CUDA device", who);
  const int grid = (num_sms > 0 && num_sms < sms) ? num_sms : sms;
  const long long m_tiles_est = (m_rows + kBlockM - 1) / kBlockM;
  int block_n = 256;
  if (n <= 64 || m_tiles_est * ((n + 127) / 128) < grid) block_n = 64;
  else if (n <= 128 || m_tiles_est * ((n + 255) / 256) < grid) block_n = 128;
  if (g_forced_block_n) block_n = g_forced_block_n;
  const bool pair = want_pair(m_rows, num_groups, n, grid, block_n);
  if (pair) block_n = 128;
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
    int rc = encode_tmap(&tm_c, (out_dtype == 1 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16), 2, c, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, "C");
    if (rc) return rc;
  }
  const int in_fmt = fmt_a | (fmt_b << 4);
  if (pair)
    return launch_m_grouped_pair<false, true>(tm_a, tm_b, tm_c, c, sizes, sizes_is_i64, num_groups, 0, m_rows, n, k, in_fmt,
                                              out_dtype, a_scale, b_scale,
                                              (num_sms > 0 && num_sms < sms) ? num_sms : 0, stream);
#define B200_LAUNCH8(BN, ST)                                                                                        \
  launch_m_grouped<BN, ST, false, true>(tm_a, tm_b, tm_c, c, sizes, sizes_is_i64, num_groups, 0, m_rows, n, k, in_fmt, out_dtype, \
                                        a_scale, b_scale, grid, stream)
  if (block_n == 256) return B200_LAUNCH8(256, 4);
  if (block_n == 128) return B200_LAUNCH8(128, 6);
  return B200_LAUNCH8(64, 8);
#undef B200_LAUNCH8
}

}  // namespace b200

extern "C" {

int b200gemm_fp8_m_grouped_rowcol(const void* a, const float* a_scale, const void* b, const float* b_scale, void* c,
                                  const void* sizes, int sizes_is_i64, int num_groups, int64_t m_rows, int n, int k,
                                  int fmt_a, int fmt_b, int out_dtype, int num_sms, void* stream) {
  return b200::fp8_rowcol_m_grouped(a, a_scale, b, b_scale, c, sizes, sizes_is_i64, num_groups, m_rows, n, k, fmt_a,
                                    fmt_b, out_dtype, num_sms, stream);
}

int b200gemm_set_block_n(int block_n) {
  if (block_n != 0 && block_n != 64 && block_n != 128 && block_n != 256)
    return b200::set_error(b200::kErrInvalidArgument, "b200gemm_set_block_n: block_n must be 0, 64, 128 or 256");
  b200::g_forced_block_n = block_n;
  return 0;
}

int b200gemm_set_cta_pair(int mode) {
  if (mode < -1 || mode > 1)
    return b200::set_error(b200::kErrInvalidArgument, "b200gemm_set_cta_pair: mode must be -1 (auto), 0 or 1");
  b200::g_cta_pair_mode = mode;
  return 0;
}

int b200gemm_cta_pair_grid(void) { return b200::pair_kernel_grid(); }

int b200gemm_m_grouped(const void* a, const void* b, void* c, const void* sizes, int sizes_is_i64, int num_groups,
                       int64_t m_rows, int n, int k, int trans_b, int dtype, int num_sms, void* stream) {
  return b200::m_grouped_common(a, b, c, sizes, sizes_is_i64, num_groups, m_rows, /*masked_stride=*/0, n, k, trans_b,
                                dtype, num_sms, stream, "b200gemm_m_grouped");
}

int b200gemm_m_grouped_padded(const void* a, const void* b, void* c, const void* sizes, int sizes_is_i64,
                              int num_groups, int64_t m_rows, int n, int k, int trans_b, int dtype, int num_sms,
                              void* stream) {
  return b200::m_grouped_common(a, b, c, sizes, sizes_is_i64, num_groups, m_rows, /*padded rows*/ -1, n, k, trans_b,
                                dtype, num_sms, stream, "b200gemm_m_grouped_padded");
}

int b200gemm_m_grouped_masked(const void* lhs, const void* rhs, void* out, const void* masked_m, int sizes_is_i64,
                              int num_groups, int expected_m, int n, int k, int trans_b, int dtype, int num_sms,
                              void* stream) {
  if (expected_m <= 0)
    return b200::set_error(b200::kErrInvalidArgument, "b200gemm_m_grouped_masked: expected_m must be positive");
  return b200::m_grouped_common(lhs, rhs, out, masked_m, sizes_is_i64, num_groups,
                                static_cast<int64_t>(num_groups) * expected_m, expected_m, n, k, trans_b, dtype,
                                num_sms, stream, "b200gemm_m_grouped_masked");
}

}  // extern "C"
