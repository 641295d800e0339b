// Row movement around the expert GEMMs of an MoE layer (HBM-bound, no arithmetic on the
// gather side): gather rows into expert-major order for dispatch, and the router-weighted sum
// of each token's top-k expert outputs for combine.  The reference ships equivalents only in
// its vendored baseline extension (grouped_gemm/csrc/permute.cu:40-297); these are written for
// sm_100a: 16-byte vector accesses, one warp per row, several rows in flight per warp.
#include <cuda_bf16.h>

#include "../../include/b200gemm.h"
#include "common.cuh"
#include "quant_math.cuh"

namespace b200 {

constexpr int kMoeThreads = 256;

// dst[i, :] = src[idx[i], :] for i < rows; row_vecs = row bytes / 16.  An index outside
// [0, src_rows) (e.g. the -1 the routing plan gives a pair with a bad expert id) is skipped and
// flagged: the destination row keeps its contents.
__global__ void __launch_bounds__(kMoeThreads)
gather_rows_kernel(const uint4* __restrict__ src, const long long* __restrict__ idx, uint4* __restrict__ dst,
                   long long rows, int row_vecs, long long src_rows, unsigned* status) {
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * kMoeThreads + threadIdx.x) >> 5;
  const long long warps = (static_cast<long long>(gridDim.x) * kMoeThreads) >> 5;
  for (long long r = warp; r < rows; r += warps) {
    const long long sr = idx[r];
    if (sr < 0 || sr >= src_rows) {
      if (lane == 0 && status) atomicOr(status, kDevBadRowIndex);
      continue;
    }
    const uint4* s = src + sr * row_vecs;
    uint4* d = dst + r * row_vecs;
    int v = lane;
    for (; v + 96 < row_vecs; v += 128) {  // four independent 16-byte loads in flight per lane
      const uint4 a = __ldg(s + v), b = __ldg(s + v + 32), c = __ldg(s + v + 64), e = __ldg(s + v + 96);
      d[v] = a;
      d[v + 32] = b;
      d[v + 64] = c;
      d[v + 96] = e;
    }
    for (; v < row_vecs; v += 32) d[v] = __ldg(s + v);
  }
}

// out[t, :] = bf16( sum_k w[t,k] * y[pos[t,k], :] ), fp32 accumulation in k order.
// kTopK > 0: top_k known at compile time - the k rows' loads of a 16-byte column chunk are all
// issued before the first multiply-add, so a lane keeps kTopK loads in flight instead of one (the
// kernel is bound by bytes in flight, not by arithmetic); kTopK == 0: any top_k, one load at a
// time.  Same operations in the same order either way, so the results are identical.
template <int kTopK>
__global__ void __launch_bounds__(kMoeThreads)
combine_topk_kernel(const uint4* __restrict__ y, const long long* __restrict__ pos, const float* __restrict__ w,
                    uint4* __restrict__ out, long long tokens, int top_k_rt, int row_vecs, long long y_rows,
                    unsigned* status) {
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * kMoeThreads + threadIdx.x) >> 5;
  const long long warps = (static_cast<long long>(gridDim.x) * kMoeThreads) >> 5;
  const int top_k = kTopK > 0 ? kTopK : top_k_rt;
  for (long long t = warp; t < tokens; t += warps) {
    if constexpr (kTopK > 0) {
      long long yr[kTopK];
      float wk[kTopK];
      bool bad = false;
#pragma unroll
      for (int k = 0; k < kTopK; ++k) {
        yr[k] = pos[t * kTopK + k];
        wk[k] = w[t * kTopK + k];
        if (yr[k] < 0 || yr[k] >= y_rows) {  // a pair the routing plan rejected: it contributes nothing
          yr[k] = -1;
          bad = true;
        }
      }
      if (bad && lane == 0 && status) atomicOr(status, kDevBadRowIndex);
      for (int v = lane; v < row_vecs; v += 32) {
        uint4 q[kTopK];
#pragma unroll
        for (int k = 0; k < kTopK; ++k) q[k] = yr[k] >= 0 ? __ldg(y + yr[k] * row_vecs + v) : make_uint4(0, 0, 0, 0);
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
        for (int k = 0; k < kTopK; ++k) {
          if (yr[k] < 0) continue;
          const uint32_t p[4] = {q[k].x, q[k].y, q[k].z, q[k].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            acc[2 * e] = fmaf(wk[k], __uint_as_float(p[e] << 16), acc[2 * e]);
            acc[2 * e + 1] = fmaf(wk[k], __uint_as_float(p[e] & 0xFFFF0000u), acc[2 * e + 1]);
          }
        }
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
          o[e] = *reinterpret_cast<uint32_t*>(&h);
        }
        out[t * row_vecs + v] = make_uint4(o[0], o[1], o[2], o[3]);
      }
    } else {
      for (int v = lane; v < row_vecs; v += 32) {
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.f;
        for (int k = 0; k < top_k; ++k) {
          const long long yr = pos[t * top_k + k];
          if (yr < 0 || yr >= y_rows) {
            if (v == lane && lane == 0 && status) atomicOr(status, kDevBadRowIndex);
            continue;
          }
          const uint4 q = __ldg(y + yr * row_vecs + v);
          const float wk = w[t * top_k + k];
          const uint32_t p[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            acc[2 * e] = fmaf(wk, __uint_as_float(p[e] << 16), acc[2 * e]);
            acc[2 * e + 1] = fmaf(wk, __uint_as_float(p[e] & 0xFFFF0000u), acc[2 * e + 1]);
          }
        }
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
          o[e] = *reinterpret_cast<uint32_t*>(&h);
        }
        out[t * row_vecs + v] = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
}

// ---- routing plan: counting sort of the (token, k) pairs by expert --------------------------
// expert[i] in [0, num_experts) for i < n.  Produces counts[e], order (pair indices grouped by
// expert: expert e's pairs occupy [start_e, start_e + counts[e])) and pos = order^-1.  The order
// inside an expert's range is not specified (rows of a group are independent in the GEMM), which
// allows atomics: a block histograms its slice in shared memory, reserves one range per expert
// with a single global atomic each, and hands out positions from shared-memory counters.
constexpr int kPlanThreads = 256;
constexpr int kPlanItems = 8;        // pairs per thread
constexpr int kPlanMaxExperts = 1024;

__global__ void __launch_bounds__(kPlanThreads)
route_count_kernel(const long long* __restrict__ expert, long long n, int num_experts,
                   const long long* __restrict__ key_table, int* __restrict__ counts) {
  __shared__ int hist[kPlanMaxExperts];
  for (int e = threadIdx.x; e < num_experts; e += kPlanThreads) hist[e] = 0;
  __syncthreads();
  const long long base = static_cast<long long>(blockIdx.x) * kPlanThreads * kPlanItems;
#pragma unroll
  for (int j = 0; j < kPlanItems; ++j) {
    const long long i = base + j * kPlanThreads + threadIdx.x;
    if (i < n) {
      long long e = expert[i];
      if (e >= 0 && e < num_experts) {
        if (key_table) e = key_table[e];  // sort by a permutation of the expert ids instead
        atomicAdd(&hist[e], 1);
      }
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < num_experts; e += kPlanThreads)
    if (hist[e]) atomicAdd(&counts[e], hist[e]);
}

// one block: cursor[e] = exclusive prefix of counts (the start of expert e's range)
__global__ void __launch_bounds__(kPlanMaxExperts)
route_scan_kernel(const int* __restrict__ counts, int num_experts, int* __restrict__ cursor) {
  __shared__ int tmp[kPlanMaxExperts];
  const int e = threadIdx.x;
  tmp[e] = e < num_experts ? counts[e] : 0;
  __syncthreads();
  for (int off = 1; off < kPlanMaxExperts; off <<= 1) {
    const int v = e >= off ? tmp[e - off] : 0;
    __syncthreads();
    tmp[e] += v;
    __syncthreads();
  }
  if (e < num_experts) cursor[e] = tmp[e] - counts[e];
}

__global__ void __launch_bounds__(kPlanThreads)
route_scatter_kernel(const long long* __restrict__ expert, long long n, int num_experts,
                     const long long* __restrict__ key_table, int* __restrict__ cursor,
                     long long* __restrict__ order, long long* __restrict__ pos, unsigned* status) {
  __shared__ int hist[kPlanMaxExperts];   // first: this block's count per expert; then: next free position
  for (int e = threadIdx.x; e < num_experts; e += kPlanThreads) hist[e] = 0;
  __syncthreads();
  const long long base = static_cast<long long>(blockIdx.x) * kPlanThreads * kPlanItems;
  long long ex[kPlanItems];
#pragma unroll
  for (int j = 0; j < kPlanItems; ++j) {
    const long long i = base + j * kPlanThreads + threadIdx.x;
    ex[j] = -1;
    if (i < n) {
      long long e = expert[i];
      if (e >= 0 && e < num_experts) {
        if (key_table) e = key_table[e];
        ex[j] = e;
        atomicAdd(&hist[e], 1);
      } else if (status) {
        atomicOr(status, kDevBadRowIndex);
      }
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < num_experts; e += kPlanThreads) {
    const int c = hist[e];
    hist[e] = c ? atomicAdd(&cursor[e], c) : 0;  // start of this block's range inside expert e's range
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < kPlanItems; ++j) {
    const long long i = base + j * kPlanThreads + threadIdx.x;
    if (ex[j] >= 0) {
      const long long p = atomicAdd(&hist[ex[j]], 1);
      order[p] = i;
      pos[i] = p;
    } else if (i < n) {
      pos[i] = -1;  // rejected pair: the row movers skip negative indices
    }
  }
}

// ---- the same two movers over several buffers: one per rank of an expert-parallel group, the
// other ranks' buffers being peer memory mapped into this process.  The dispatch kernel stores
// each row straight into the owning rank's receive buffer at its final position and the combine
// kernel loads each (token, k) result from the rank that computed it, so a step needs no
// all-to-all, no send-side gather and no staging copy of the returned rows; the bytes cross
// NVLink once, as plain stores / loads issued by these kernels.  Every access is bounds-checked
// (rank < world, row < capacity): a bad index sets a status bit and is skipped, it cannot fault
// a peer.
constexpr int kMaxPeers = 16;
struct PeerBases {
  void* base[kMaxPeers];
};

// bases[rank[i]][row[i], :] = src[src_idx[i], :]
__global__ void __launch_bounds__(1024)
scatter_rows_multi_kernel(const uint4* __restrict__ src, const long long* __restrict__ src_idx, PeerBases bases,
                          const int* __restrict__ rank, const long long* __restrict__ row, long long rows,
                          int row_vecs, int world, long long capacity_rows, long long src_rows, unsigned* status) {
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long r = warp; r < rows; r += warps) {
    const int dst_rank = rank[r];
    const long long dst_row = row[r];
    const long long sr = src_idx[r];
    if (dst_rank < 0 || dst_rank >= world || dst_row < 0 || dst_row >= capacity_rows || sr < 0 || sr >= src_rows) {
      if (lane == 0 && status) atomicOr(status, kDevBadRowIndex);
      continue;
    }
    const uint4* s = src + sr * row_vecs;
    uint4* d = static_cast<uint4*>(bases.base[dst_rank]) + dst_row * row_vecs;
    int v = lane;
    for (; v + 96 < row_vecs; v += 128) {
      const uint4 a = __ldg(s + v), b = __ldg(s + v + 32), c = __ldg(s + v + 64), e = __ldg(s + v + 96);
      d[v] = a;
      d[v + 32] = b;
      d[v + 64] = c;
      d[v + 96] = e;
    }
    for (; v < row_vecs; v += 32) d[v] = __ldg(s + v);
  }
}

// Quantise-on-dispatch: pair i (first <= i < first + count, send order) takes the 16-bit row of
// token token_of_pair[i], quantises it 1x128 exactly like quant_act_1x128_kernel (same operation
// order, so bytes and scales equal per_token_cast_to_fp8 followed by a row scatter), and stores
// the e4m3 row, its hidden/128 fp32 scales and the pair's return address (i, my_rank) into the
// owning rank's three buffers at row dst_row[i].  One warp per pair; 16 lanes share a 128-wide
// block (8 elements each), so a warp does two blocks per step, four steps in flight.
constexpr int kDqUnroll = 4;

__global__ void __launch_bounds__(1024)
dispatch_quant_rows_multi_kernel(const uint4* __restrict__ x, const long long* __restrict__ token_of_pair,
                                 PeerBases rows8, PeerBases scales, PeerBases meta, const int* __restrict__ rank,
                                 const long long* __restrict__ row, long long first, long long count,
                                 long long tokens, int hidden, int is_fp16, int world, long long capacity_rows,
                                 int my_rank, unsigned* status) {
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const int chunks = hidden >> 3;   // 8-element chunks per row (a multiple of 16: hidden % 128 == 0)
  const int nb = hidden >> 7;       // 1x128 blocks per row (<= 64)
  const int steps = (chunks + 31) >> 5;
  for (long long p = warp; p < count; p += warps) {
    const long long i = first + p;
    const int dst_rank = rank[i];
    const long long dst_row = row[i];
    const long long t = token_of_pair[i];
    if (dst_rank < 0 || dst_rank >= world || dst_row < 0 || dst_row >= capacity_rows || t < 0 || t >= tokens) {
      if (lane == 0 && status) atomicOr(status, kDevBadRowIndex);
      continue;
    }
    const uint4* src = x + t * chunks;
    uint2* d8 = reinterpret_cast<uint2*>(static_cast<uint8_t*>(rows8.base[dst_rank]) + dst_row * hidden);
    float* ds = static_cast<float*>(scales.base[dst_rank]) + dst_row * nb;
    float s_lo = 0.f, s_hi = 0.f;  // lane L ends up holding the scales of blocks L and L + 32
    for (int st0 = 0; st0 < steps; st0 += kDqUnroll) {
      uint4 v[kDqUnroll];
#pragma unroll
      for (int u = 0; u < kDqUnroll; ++u) {
        const int c = (st0 + u) * 32 + lane;
        v[u] = (st0 + u < steps && c < chunks) ? __ldg(src + c) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < kDqUnroll; ++u) {
        const int st = st0 + u;
        if (st >= steps) break;  // uniform over the warp
        float amax = abs_max8(v[u], is_fp16);
#pragma unroll
        for (int o = 8; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
        amax = fmaxf(amax, 1e-4f);
        const int c = st * 32 + lane;
        if (c < chunks) d8[c] = quant8_e4m3(v[u], inv_scale_448(amax), is_fp16);
        // blocks 2 st (lanes 0..15) and 2 st + 1 (lanes 16..31): lane L keeps the scale of block L mod 32
        const float sc = __shfl_sync(0xFFFFFFFFu, __fdiv_rn(amax, 448.0f), (lane & 1) << 4);
        if ((lane >> 1) == (st & 15)) {
          if (st < 16) s_lo = sc;
          else s_hi = sc;
        }
      }
    }
    if (lane < nb) ds[lane] = s_lo;
    if (lane + 32 < nb) ds[lane + 32] = s_hi;
    if (lane == 0)
      *reinterpret_cast<longlong2*>(static_cast<long long*>(meta.base[dst_rank]) + 2 * dst_row) =
          make_longlong2(i, static_cast<long long>(my_rank));
  }
}

// Quantise-and-permute on one GPU: token t's 16-bit row is quantised 1x128 ONCE and its e4m3 row
// and scales are written to every row pos[t * top_k + j] of the expert-major buffers - the
// activation quantiser and the permute in one pass (read T rows, write T * top_k rows; the fp8
// copy of x is never read back).  One warp per token; the quantised row stays in registers (one
// 8-byte chunk per lane and step; kQsMaxSteps = 16 serves hidden <= 4096, 32 hidden <= 8192)
// between the k stores.
template <int kQsMaxSteps>
__global__ void __launch_bounds__(256, kQsMaxSteps <= 16 ? 2 : 1)
quant_scatter_rows_kernel(const uint4* __restrict__ x, const long long* __restrict__ pos, uint8_t* __restrict__ dst8,
                          float* __restrict__ dst_scales, long long tokens, int top_k, int hidden, int is_fp16,
                          long long dst_rows, unsigned* status) {
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const int chunks = hidden >> 3;   // 8-element chunks per row (a multiple of 16: hidden % 128 == 0)
  const int nb = hidden >> 7;       // 1x128 blocks per row (<= 64)
  const int steps = (chunks + 31) >> 5;
  for (long long t = warp; t < tokens; t += warps) {
    const uint4* src = x + t * chunks;
    uint2 q[kQsMaxSteps];
    float s_lo = 0.f, s_hi = 0.f;  // lane L ends up holding the scales of blocks L and L + 32
#pragma unroll
    for (int st0 = 0; st0 < kQsMaxSteps; st0 += kDqUnroll) {
      if (st0 < steps) {  // uniform over the warp
        uint4 v[kDqUnroll];
#pragma unroll
        for (int u = 0; u < kDqUnroll; ++u) {
          const int c = (st0 + u) * 32 + lane;
          v[u] = (st0 + u < steps && c < chunks) ? __ldg(src + c) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < kDqUnroll; ++u) {
          const int st = st0 + u;
          if (st < steps) {
            float amax = abs_max8(v[u], is_fp16);
#pragma unroll
            for (int o = 8; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
            amax = fmaxf(amax, 1e-4f);
            q[st] = quant8_e4m3(v[u], inv_scale_448(amax), is_fp16);
            // blocks 2 st (lanes 0..15) and 2 st + 1 (lanes 16..31): lane L keeps the scale of block L mod 32
            const float sc = __shfl_sync(0xFFFFFFFFu, __fdiv_rn(amax, 448.0f), (lane & 1) << 4);
            if ((lane >> 1) == (st & 15)) {
              if (st < 16) s_lo = sc;
              else s_hi = sc;
            }
          }
        }
      }
    }
    for (int j = 0; j < top_k; ++j) {
      const long long r = __ldg(pos + t * top_k + j);
      if (r < 0 || r >= dst_rows) {
        if (lane == 0 && status) atomicOr(status, kDevBadRowIndex);
        continue;
      }
      uint2* d8 = reinterpret_cast<uint2*>(dst8 + r * hidden);
#pragma unroll
      for (int st = 0; st < kQsMaxSteps; ++st) {
        const int c = st * 32 + lane;
        if (st < steps && c < chunks) d8[c] = q[st];
      }
      float* ds = dst_scales + r * nb;
      if (lane < nb) ds[lane] = s_lo;
      if (lane + 32 < nb) ds[lane + 32] = s_hi;
    }
  }
}

// The same dispatch for rows that are already quantised (x8 [tokens, hidden] bytes, xs [tokens,
// hidden/128] fp32): the pair's row, its scales and its return address in one pass - one launch
// per chunk instead of one scatter per payload.  hidden % 16 == 0.
__global__ void __launch_bounds__(1024)
dispatch_rows_multi_kernel(const uint4* __restrict__ x8, const float* __restrict__ xs,
                           const long long* __restrict__ token_of_pair, PeerBases rows8, PeerBases scales,
                           PeerBases meta, const int* __restrict__ rank, const long long* __restrict__ row,
                           long long first, long long count, long long tokens, int hidden, int nb, int world,
                           long long capacity_rows, int my_rank, unsigned* status) {
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const int row_vecs = hidden >> 4;
  for (long long p = warp; p < count; p += warps) {
    const long long i = first + p;
    const int dst_rank = rank[i];
    const long long dst_row = row[i];
    const long long t = token_of_pair[i];
    if (dst_rank < 0 || dst_rank >= world || dst_row < 0 || dst_row >= capacity_rows || t < 0 || t >= tokens) {
      if (lane == 0 && status) atomicOr(status, kDevBadRowIndex);
      continue;
    }
    const uint4* s = x8 + t * row_vecs;
    uint4* d = reinterpret_cast<uint4*>(static_cast<uint8_t*>(rows8.base[dst_rank]) + dst_row * hidden);
    int v = lane;
    for (; v + 96 < row_vecs; v += 128) {
      const uint4 a = __ldg(s + v), b = __ldg(s + v + 32), c = __ldg(s + v + 64), e = __ldg(s + v + 96);
      d[v] = a;
      d[v + 32] = b;
      d[v + 64] = c;
      d[v + 96] = e;
    }
    for (; v < row_vecs; v += 32) d[v] = __ldg(s + v);
    const float* ss = xs + t * nb;
    float* ds = static_cast<float*>(scales.base[dst_rank]) + dst_row * nb;
    for (int j = lane; j < nb; j += 32) ds[j] = __ldg(ss + j);
    if (lane == 0)
      *reinterpret_cast<longlong2*>(static_cast<long long*>(meta.base[dst_rank]) + 2 * dst_row) =
          make_longlong2(i, static_cast<long long>(my_rank));
  }
}

// The way back: dst[meta[r].rank][meta[r].row, :] = src[r, :] for r < rows, meta [rows, 2] int64 being
// the return addresses the dispatch kernel left beside the rows (row in the owner's return
// buffer, owner rank).
__global__ void __launch_bounds__(1024)
return_rows_multi_kernel(const uint4* __restrict__ src, const longlong2* __restrict__ meta, PeerBases bases,
                         long long rows, int row_vecs, int world, long long capacity_rows, unsigned* status) {
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long r = warp; r < rows; r += warps) {
    const longlong2 m = meta[r];
    const long long dst_row = m.x, dst_rank = m.y;
    if (dst_rank < 0 || dst_rank >= world || dst_row < 0 || dst_row >= capacity_rows) {
      if (lane == 0 && status) atomicOr(status, kDevBadRowIndex);
      continue;
    }
    const uint4* s = src + r * row_vecs;
    uint4* d = static_cast<uint4*>(bases.base[dst_rank]) + dst_row * row_vecs;
    int v = lane;
    for (; v + 96 < row_vecs; v += 128) {
      const uint4 a = s[v], b = s[v + 32], c = s[v + 64], e = s[v + 96];
      d[v] = a;
      d[v + 32] = b;
      d[v + 64] = c;
      d[v + 96] = e;
    }
    for (; v < row_vecs; v += 32) d[v] = s[v];
  }
}

// out[t, :] = bf16( sum_k w[t,k] * bases[rank[t,k]][row[t,k], :] ), fp32 accumulation in k order
__global__ void __launch_bounds__(kMoeThreads)
combine_topk_multi_kernel(PeerBases bases, const int* __restrict__ rank, const long long* __restrict__ row,
                          const float* __restrict__ w, uint4* __restrict__ out, long long tokens, int top_k,
                          int row_vecs, int world, long long capacity_rows, unsigned* status) {
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * kMoeThreads + threadIdx.x) >> 5;
  const long long warps = (static_cast<long long>(gridDim.x) * kMoeThreads) >> 5;
  for (long long t = warp; t < tokens; t += warps) {
    for (int v = lane; v < row_vecs; v += 32) {
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
      for (int k = 0; k < top_k; ++k) {
        const int src_rank = rank[t * top_k + k];
        const long long src_row = row[t * top_k + k];
        if (src_rank < 0 || src_rank >= world || src_row < 0 || src_row >= capacity_rows) {
          if (v == lane && lane == 0 && status) atomicOr(status, kDevBadRowIndex);
          continue;
        }
        // peer memory is not read-only for the whole grid's lifetime in general: plain loads
        const uint4 q = *(static_cast<const uint4*>(bases.base[src_rank]) + src_row * row_vecs + v);
        const float wk = w[t * top_k + k];
        const uint32_t p[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          acc[2 * e] = fmaf(wk, __uint_as_float(p[e] << 16), acc[2 * e]);
          acc[2 * e + 1] = fmaf(wk, __uint_as_float(p[e] & 0xFFFF0000u), acc[2 * e + 1]);
        }
      }
      uint32_t o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
        o[e] = *reinterpret_cast<uint32_t*>(&h);
      }
      out[t * row_vecs + v] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// ---- plan of the peer-memory exchange, on the device -----------------------------------------
// After the all-gather of every rank's per-key pair counts (keys = a fixed permutation of the
// global expert ids that makes the send order chunk-major), one block derives what this rank needs
// to address the other ranks' buffers, which are laid out [local expert][source rank]:
//   dst_start[key]   first row, in the owning rank's buffers, of THIS rank's pairs with that key
//   send_start[key]  first position of that key in this rank's send order
//   size_per_group[l]  rows of local expert l here, all sources together
__global__ void __launch_bounds__(1024)
peer_layout_kernel(const int* __restrict__ counts_all /* [world, E] by key */, const int* __restrict__ expert_of_key,
                   const long long* __restrict__ key_of_expert, int world, int me, int e_loc, int num_experts,
                   long long* __restrict__ dst_start, long long* __restrict__ send_start,
                   long long* __restrict__ size_per_group) {
  for (int key = threadIdx.x; key < num_experts; key += blockDim.x) {
    const int e = expert_of_key[key];
    const int d = e / e_loc, l = e - d * e_loc;
    long long before = 0;
    for (int l2 = 0; l2 <= l; ++l2) {
      const long long k2 = key_of_expert[d * e_loc + l2];
      const int s_end = l2 < l ? world : me;  // whole earlier experts, then the lower source ranks of this one
      for (int s = 0; s < s_end; ++s) before += counts_all[static_cast<long long>(s) * num_experts + k2];
    }
    dst_start[key] = before;
    long long mine = 0;
    for (int k2 = 0; k2 < key; ++k2) mine += counts_all[static_cast<long long>(me) * num_experts + k2];
    send_start[key] = mine;
  }
  for (int l = threadIdx.x; l < e_loc; l += blockDim.x) {
    const long long k2 = key_of_expert[me * e_loc + l];
    long long rows = 0;
    for (int s = 0; s < world; ++s) rows += counts_all[static_cast<long long>(s) * num_experts + k2];
    size_per_group[l] = rows;
  }
}

// per position i of the send order: the pair's token, owning rank and row in the owner's buffers
// (a slot of the order that holds -1 - a rejected pair - becomes token -1, which the movers skip)
__global__ void __launch_bounds__(256)
peer_pairs_kernel(const long long* __restrict__ order, const long long* __restrict__ expert,
                  const long long* __restrict__ key_of_expert, const long long* __restrict__ dst_start,
                  const long long* __restrict__ send_start, long long n, int top_k, int e_loc, int num_experts,
                  long long* __restrict__ token_of_pair, int* __restrict__ dst_rank, long long* __restrict__ dst_row) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long long p = order[i];
  long long e = p >= 0 && p < n ? expert[p] : -1;
  if (e < 0 || e >= num_experts) {
    token_of_pair[i] = -1;
    dst_rank[i] = -1;
    dst_row[i] = -1;
    return;
  }
  const long long key = key_of_expert[e];
  token_of_pair[i] = p / top_k;
  dst_rank[i] = static_cast<int>(e / e_loc);
  dst_row[i] = dst_start[key] + (i - send_start[key]);
}

static int fill_bases(PeerBases* out, const void* const* bases, int world, const char* who) {
  B200_REQUIRE(world >= 1 && world <= kMaxPeers, "%s: world (%d) must be in [1, %d]", who, world, kMaxPeers);
  B200_REQUIRE(bases, "%s: null pointer table", who);
  for (int i = 0; i < kMaxPeers; ++i) out->base[i] = nullptr;
  for (int i = 0; i < world; ++i) {
    B200_REQUIRE(bases[i] && (reinterpret_cast<uintptr_t>(bases[i]) & 15) == 0,
                 "%s: buffer of rank %d is null or not 16-byte aligned", who, i);
    out->base[i] = const_cast<void*>(bases[i]);
  }
  return 0;
}

}  // namespace b200

extern "C" {

static int route_plan_impl(const int64_t* expert, int64_t n, int num_experts, const int64_t* key_table, int* counts,
                           int* cursor, int64_t* order, int64_t* pos, void* stream_v, const char* who);

int b200moe_route_plan(const int64_t* expert, int64_t n, int num_experts, int* counts, int* cursor, int64_t* order,
                       int64_t* pos, void* stream_v) {
  return route_plan_impl(expert, n, num_experts, nullptr, counts, cursor, order, pos, stream_v, "b200moe_route_plan");
}

int b200moe_route_plan_mapped(const int64_t* expert, int64_t n, int num_experts, const int64_t* key_table, int* counts,
                              int* cursor, int64_t* order, int64_t* pos, void* stream_v) {
  if (!key_table) return b200::set_error(b200::kErrInvalidArgument, "b200moe_route_plan_mapped: key_table is null");
  return route_plan_impl(expert, n, num_experts, key_table, counts, cursor, order, pos, stream_v,
                         "b200moe_route_plan_mapped");
}

int b200moe_peer_plan(const int* counts_all, const int* expert_of_key, const int64_t* key_of_expert, int world, int me,
                      int num_experts, const int64_t* order, const int64_t* expert, int64_t n, int top_k,
                      int64_t* dst_start, int64_t* send_start, int64_t* size_per_group, int64_t* token_of_pair,
                      int* dst_rank, int64_t* dst_row, void* stream_v) {
  using namespace b200;
  const char* who = "b200moe_peer_plan";
  B200_REQUIRE(world >= 1 && world <= kMaxPeers && me >= 0 && me < world, "%s: bad world / rank (%d, %d)", who, world, me);
  B200_REQUIRE(num_experts > 0 && num_experts <= kPlanMaxExperts && num_experts % world == 0,
               "%s: num_experts (%d) must be a multiple of world, at most %d", who, num_experts, kPlanMaxExperts);
  B200_REQUIRE(n >= 0 && top_k > 0, "%s: bad pair count / top_k", who);
  B200_REQUIRE(counts_all && expert_of_key && key_of_expert && dst_start && send_start && size_per_group,
               "%s: null pointer", who);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const int e_loc = num_experts / world;
  peer_layout_kernel<<<1, 1024, 0, stream>>>(counts_all, expert_of_key, reinterpret_cast<const long long*>(key_of_expert),
                                             world, me, e_loc, num_experts, reinterpret_cast<long long*>(dst_start),
                                             reinterpret_cast<long long*>(send_start),
                                             reinterpret_cast<long long*>(size_per_group));
  if (n > 0) {
    B200_REQUIRE(order && expert && token_of_pair && dst_rank && dst_row, "%s: null pointer", who);
    const long long blocks = (n + 255) / 256;
    B200_REQUIRE(blocks < (1ll << 31), "%s: too many pairs", who);
    peer_pairs_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(
        reinterpret_cast<const long long*>(order), reinterpret_cast<const long long*>(expert),
        reinterpret_cast<const long long*>(key_of_expert), reinterpret_cast<const long long*>(dst_start),
        reinterpret_cast<const long long*>(send_start), n, top_k, e_loc, num_experts,
        reinterpret_cast<long long*>(token_of_pair), dst_rank, reinterpret_cast<long long*>(dst_row));
  }
  B200_CUDA(cudaGetLastError());
  return 0;
}

static int route_plan_impl(const int64_t* expert, int64_t n, int num_experts, const int64_t* key_table, int* counts,
                           int* cursor, int64_t* order, int64_t* pos, void* stream_v, const char* who) {
  using namespace b200;
  B200_REQUIRE(n >= 0 && num_experts > 0 && num_experts <= kPlanMaxExperts, "%s: num_experts (%d) must be in [1, %d]",
               who, num_experts, kPlanMaxExperts);
  B200_REQUIRE(counts && cursor, "%s: null pointer", who);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  B200_CUDA(cudaMemsetAsync(counts, 0, sizeof(int) * num_experts, stream));
  if (n > 0) {
    B200_REQUIRE(expert && order && pos, "%s: null pointer", who);
    // pairs with an expert id outside [0, num_experts) get no slot: the slots left over at the end
    // of `order` then read -1, which every row mover skips
    B200_CUDA(cudaMemsetAsync(order, 0xFF, sizeof(int64_t) * static_cast<size_t>(n), stream));
    const long long per_block = static_cast<long long>(kPlanThreads) * kPlanItems;
    const long long blocks = (n + per_block - 1) / per_block;
    B200_REQUIRE(blocks < (1ll << 31), "%s: too many pairs", who);
    route_count_kernel<<<static_cast<int>(blocks), kPlanThreads, 0, stream>>>(
        reinterpret_cast<const long long*>(expert), n, num_experts, reinterpret_cast<const long long*>(key_table), counts);
    route_scan_kernel<<<1, kPlanMaxExperts, 0, stream>>>(counts, num_experts, cursor);
    route_scatter_kernel<<<static_cast<int>(blocks), kPlanThreads, 0, stream>>>(
        reinterpret_cast<const long long*>(expert), n, num_experts, reinterpret_cast<const long long*>(key_table), cursor,
        reinterpret_cast<long long*>(order),
        reinterpret_cast<long long*>(pos), device_status_ptr());
  } else {
    route_scan_kernel<<<1, kPlanMaxExperts, 0, stream>>>(counts, num_experts, cursor);
  }
  B200_CUDA(cudaGetLastError());
  return 0;
}

// grid of a multi-buffer mover: `blocks` > 0 = that many 1024-thread blocks (at most one per SM),
// for running beside a persistent GEMM that was given the other SMs; otherwise fill the GPU
static void mover_grid(int blocks_arg, long long rows, int sms, int* blocks, int* threads) {
  if (blocks_arg > 0) {
    *threads = 1024;
    *blocks = blocks_arg < sms ? blocks_arg : sms;
    return;
  }
  long long b = (rows + b200::kMoeThreads / 32 - 1) / (b200::kMoeThreads / 32);
  if (b > 16ll * sms) b = 16ll * sms;
  *threads = b200::kMoeThreads;
  *blocks = static_cast<int>(b);
}

int b200moe_scatter_rows_multi(const void* src, const int64_t* src_idx, void* const* dst_bases, const int* dst_rank,
                               const int64_t* dst_row, int64_t rows, int64_t row_bytes, int world,
                               int64_t capacity_rows, int64_t src_rows, int blocks_arg, void* stream) {
  using namespace b200;
  const char* who = "b200moe_scatter_rows_multi";
  B200_REQUIRE(rows >= 0 && row_bytes >= 0 && capacity_rows >= 0 && src_rows >= 0, "%s: negative size", who);
  if (rows == 0 || row_bytes == 0) return 0;
  B200_REQUIRE(src && src_idx && dst_rank && dst_row, "%s: null pointer", who);
  B200_REQUIRE(row_bytes % 16 == 0 && row_bytes / 16 < (1ll << 30), "%s: row_bytes (%lld) must be a multiple of 16", who,
               (long long)row_bytes);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(src) & 15) == 0, "%s: src must be 16-byte aligned", who);
  PeerBases pb;
  int rc = fill_bases(&pb, const_cast<const void* const*>(dst_bases), world, who);
  if (rc) return rc;
  const int sms = sm_count();
  B200_REQUIRE(sms > 0, "%s: no CUDA device", who);
  int blocks, threads;
  mover_grid(blocks_arg, rows, sms, &blocks, &threads);
  scatter_rows_multi_kernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), reinterpret_cast<const long long*>(src_idx), pb, dst_rank,
      reinterpret_cast<const long long*>(dst_row), rows, static_cast<int>(row_bytes / 16), world, capacity_rows,
      src_rows, device_status_ptr());
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_dispatch_quant_rows_multi(const void* x, const int64_t* token_of_pair, void* const* row_bases,
                                      void* const* scale_bases, void* const* meta_bases, const int* dst_rank,
                                      const int64_t* dst_row, int64_t first_pair, int64_t num_pairs, int64_t tokens,
                                      int hidden, int dtype, int world, int64_t capacity_rows, int my_rank,
                                      int blocks_arg, void* stream) {
  using namespace b200;
  const char* who = "b200moe_dispatch_quant_rows_multi";
  B200_REQUIRE(first_pair >= 0 && num_pairs >= 0 && tokens >= 0 && capacity_rows >= 0, "%s: negative size", who);
  B200_REQUIRE(dtype == 0 || dtype == 1, "%s: dtype must be 0 (bf16) or 1 (fp16)", who);
  B200_REQUIRE(hidden > 0 && hidden % 128 == 0 && hidden <= 8192,
               "%s: hidden (%d) must be a multiple of 128, at most 8192", who, hidden);
  B200_REQUIRE(my_rank >= 0 && my_rank < world, "%s: my_rank (%d) outside [0, world)", who, my_rank);
  if (num_pairs == 0) return 0;
  B200_REQUIRE(x && token_of_pair && dst_rank && dst_row, "%s: null pointer", who);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0, "%s: x must be 16-byte aligned", who);
  PeerBases pr, ps, pm;
  int rc = fill_bases(&pr, const_cast<const void* const*>(row_bases), world, who);
  if (rc) return rc;
  rc = fill_bases(&ps, const_cast<const void* const*>(scale_bases), world, who);
  if (rc) return rc;
  rc = fill_bases(&pm, const_cast<const void* const*>(meta_bases), world, who);
  if (rc) return rc;
  const int sms = sm_count();
  B200_REQUIRE(sms > 0, "%s: no CUDA device", who);
  int blocks, threads;
  mover_grid(blocks_arg, num_pairs, sms, &blocks, &threads);
  dispatch_quant_rows_multi_kernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), reinterpret_cast<const long long*>(token_of_pair), pr, ps, pm, dst_rank,
      reinterpret_cast<const long long*>(dst_row), first_pair, num_pairs, tokens, hidden, dtype, world, capacity_rows,
      my_rank, device_status_ptr());
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_quant_scatter_rows(const void* x, int dtype, int64_t tokens, int hidden, const int64_t* pos, int top_k,
                               void* dst8, float* dst_scales, int64_t dst_rows, void* stream) {
  using namespace b200;
  const char* who = "b200moe_quant_scatter_rows";
  B200_REQUIRE(tokens >= 0 && dst_rows >= 0 && top_k >= 0, "%s: negative size", who);
  B200_REQUIRE(dtype == 0 || dtype == 1, "%s: dtype must be 0 (bf16) or 1 (fp16)", who);
  B200_REQUIRE(hidden > 0 && hidden % 128 == 0 && hidden <= 8192,
               "%s: hidden (%d) must be a multiple of 128, at most 8192", who, hidden);
  if (tokens == 0 || top_k == 0) return 0;
  B200_REQUIRE(x && pos && dst8 && dst_scales, "%s: null pointer", who);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(dst8) & 7) == 0,
               "%s: x must be 16-byte aligned, dst8 8-byte aligned", who);
  const int sms = sm_count();
  B200_REQUIRE(sms > 0, "%s: no CUDA device", who);
  const long long want = (tokens + 7) / 8;  // 8 warps per block
  const int blocks = static_cast<int>(want < 16ll * sms ? want : 16ll * sms);
  auto kern = hidden <= 4096 ? quant_scatter_rows_kernel<16> : quant_scatter_rows_kernel<32>;
  kern<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), reinterpret_cast<const long long*>(pos), static_cast<uint8_t*>(dst8), dst_scales,
      tokens, top_k, hidden, dtype, dst_rows, device_status_ptr());
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_dispatch_rows_multi(const void* x8, const float* x_scales, const int64_t* token_of_pair,
                                void* const* row_bases, void* const* scale_bases, void* const* meta_bases,
                                const int* dst_rank, const int64_t* dst_row, int64_t first_pair, int64_t num_pairs,
                                int64_t tokens, int hidden, int world, int64_t capacity_rows, int my_rank,
                                int blocks_arg, void* stream) {
  using namespace b200;
  const char* who = "b200moe_dispatch_rows_multi";
  B200_REQUIRE(first_pair >= 0 && num_pairs >= 0 && tokens >= 0 && capacity_rows >= 0, "%s: negative size", who);
  B200_REQUIRE(hidden > 0 && hidden % 128 == 0, "%s: hidden (%d) must be a multiple of 128", who, hidden);
  B200_REQUIRE(my_rank >= 0 && my_rank < world, "%s: my_rank (%d) outside [0, world)", who, my_rank);
  if (num_pairs == 0) return 0;
  B200_REQUIRE(x8 && x_scales && token_of_pair && dst_rank && dst_row, "%s: null pointer", who);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(x8) & 15) == 0, "%s: x8 must be 16-byte aligned", who);
  PeerBases pr, ps, pm;
  int rc = fill_bases(&pr, const_cast<const void* const*>(row_bases), world, who);
  if (rc) return rc;
  rc = fill_bases(&ps, const_cast<const void* const*>(scale_bases), world, who);
  if (rc) return rc;
  rc = fill_bases(&pm, const_cast<const void* const*>(meta_bases), world, who);
  if (rc) return rc;
  const int sms = sm_count();
  B200_REQUIRE(sms > 0, "%s: no CUDA device", who);
  int blocks, threads;
  mover_grid(blocks_arg, num_pairs, sms, &blocks, &threads);
  dispatch_rows_multi_kernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x8), x_scales, reinterpret_cast<const long long*>(token_of_pair), pr, ps, pm, dst_rank,
      reinterpret_cast<const long long*>(dst_row), first_pair, num_pairs, tokens, hidden, hidden / 128, world,
      capacity_rows, my_rank, device_status_ptr());
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_return_rows_multi(const void* src, const int64_t* meta, void* const* dst_bases, int64_t rows,
                              int64_t row_bytes, int world, int64_t capacity_rows, int blocks_arg, void* stream) {
  using namespace b200;
  const char* who = "b200moe_return_rows_multi";
  B200_REQUIRE(rows >= 0 && row_bytes >= 0 && capacity_rows >= 0, "%s: negative size", who);
  if (rows == 0 || row_bytes == 0) return 0;
  B200_REQUIRE(src && meta, "%s: null pointer", who);
  B200_REQUIRE(row_bytes % 16 == 0 && row_bytes / 16 < (1ll << 30), "%s: row_bytes (%lld) must be a multiple of 16", who,
               (long long)row_bytes);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(src) & 15) == 0 && (reinterpret_cast<uintptr_t>(meta) & 15) == 0,
               "%s: src and meta must be 16-byte aligned", who);
  PeerBases pb;
  int rc = fill_bases(&pb, const_cast<const void* const*>(dst_bases), world, who);
  if (rc) return rc;
  const int sms = sm_count();
  B200_REQUIRE(sms > 0, "%s: no CUDA device", who);
  int blocks, threads;
  mover_grid(blocks_arg, rows, sms, &blocks, &threads);
  return_rows_multi_kernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), reinterpret_cast<const longlong2*>(meta), pb, rows,
      static_cast<int>(row_bytes / 16), world, capacity_rows, device_status_ptr());
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_combine_topk_multi(const void* const* src_bases, const int* pair_rank, const int64_t* pair_row,
                               const float* weights, void* out, int64_t tokens, int top_k, int hidden, int world,
                               int64_t capacity_rows, void* stream) {
  using namespace b200;
  const char* who = "b200moe_combine_topk_multi";
  B200_REQUIRE(tokens >= 0 && top_k > 0 && hidden >= 0 && capacity_rows >= 0, "%s: bad size", who);
  if (tokens == 0 || hidden == 0) return 0;
  B200_REQUIRE(pair_rank && pair_row && weights && out, "%s: null pointer", who);
  B200_REQUIRE(hidden % 8 == 0, "%s: hidden (%d) must be a multiple of 8", who, hidden);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(out) & 15) == 0, "%s: out must be 16-byte aligned", who);
  PeerBases pb;
  int rc = fill_bases(&pb, src_bases, world, who);
  if (rc) return rc;
  const int sms = sm_count();
  B200_REQUIRE(sms > 0, "%s: no CUDA device", who);
  long long blocks = (tokens + kMoeThreads / 32 - 1) / (kMoeThreads / 32);
  if (blocks > 16ll * sms) blocks = 16ll * sms;
  combine_topk_multi_kernel<<<static_cast<int>(blocks), kMoeThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      pb, pair_rank, reinterpret_cast<const long long*>(pair_row), weights, static_cast<uint4*>(out), tokens, top_k,
      hidden / 8, world, capacity_rows, device_status_ptr());
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_gather_rows(const void* src, const int64_t* idx, void* dst, int64_t rows, int64_t row_bytes,
                        int64_t src_rows, void* stream) {
  using namespace b200;
  B200_REQUIRE(rows >= 0 && row_bytes >= 0 && src_rows >= 0, "b200moe_gather_rows: negative size");
  if (rows == 0 || row_bytes == 0) return 0;
  B200_REQUIRE(src && idx && dst, "b200moe_gather_rows: null pointer");
  B200_REQUIRE(row_bytes % 16 == 0 && row_bytes / 16 < (1ll << 30), "b200moe_gather_rows: row_bytes (%lld) must be a multiple of 16",
               (long long)row_bytes);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(src) & 15) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0,
               "b200moe_gather_rows: src and dst must be 16-byte aligned");
  const int sms = sm_count();
  B200_REQUIRE(sms > 0, "b200moe_gather_rows: no CUDA device");
  long long blocks = (rows + kMoeThreads / 32 - 1) / (kMoeThreads / 32);
  if (blocks > 16ll * sms) blocks = 16ll * sms;
  gather_rows_kernel<<<static_cast<int>(blocks), kMoeThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), reinterpret_cast<const long long*>(idx), static_cast<uint4*>(dst), rows,
      static_cast<int>(row_bytes / 16), src_rows, device_status_ptr());
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200moe_combine_topk(const void* y, const int64_t* pos, const float* weights, void* out, int64_t tokens, int top_k,
                         int hidden, int64_t y_rows, void* stream) {
  using namespace b200;
  B200_REQUIRE(tokens >= 0 && top_k > 0 && hidden >= 0 && y_rows >= 0, "b200moe_combine_topk: bad size");
  if (tokens == 0 || hidden == 0) return 0;
  B200_REQUIRE(y && pos && weights && out, "b200moe_combine_topk: null pointer");
  B200_REQUIRE(hidden % 8 == 0, "b200moe_combine_topk: hidden (%d) must be a multiple of 8", hidden);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(y) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0,
               "b200moe_combine_topk: y and out must be 16-byte aligned");
  const int sms = sm_count();
  B200_REQUIRE(sms > 0, "b200moe_combine_topk: no CUDA device");
  long long blocks = (tokens + kMoeThreads / 32 - 1) / (kMoeThreads / 32);
  if (blocks > 16ll * sms) blocks = 16ll * sms;
#define B200_COMBINE(K)                                                                                              \
  combine_topk_kernel<K><<<static_cast<int>(blocks), kMoeThreads, 0, static_cast<cudaStream_t>(stream)>>>(           \
      static_cast<const uint4*>(y), reinterpret_cast<const long long*>(pos), weights, static_cast<uint4*>(out), tokens, \
      top_k, hidden / 8, y_rows, device_status_ptr())
  switch (top_k) {
    case 1: B200_COMBINE(1); break;
    case 2: B200_COMBINE(2); break;
    case 4: B200_COMBINE(4); break;
    case 6: B200_COMBINE(6); break;
    case 8: B200_COMBINE(8); break;
    default: B200_COMBINE(0); break;
  }
#undef B200_COMBINE
  B200_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
