// Per-block FP8 (e4m3) quantisers, HBM-bound, bit-exact with the reference's torch code:
//   act_1x128        one scale per 1x128 block along K           (activations)
//   w_128x128        one scale per 128x128 block                 (weights, batched over experts)
//   trans_expand     128x128 blocks, transposed output, each expert padded to 128 rows
// All arithmetic that decides a byte or a scale is IEEE fp32 with explicit round-to-nearest
// intrinsics (no fast-math, no reciprocal-multiply where the reference divides).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "../../include/b200gemm.h"
#include "common.cuh"
#include "quant_math.cuh"

namespace b200 {

// ------------------------------------------------------------------ 1x128 (activations)
// Follows per_token_cast_to_fp8 (gemm/FP8/m_grouped_gemm_channel_expert.py:217-222):
//   amax = max|x| over the block, clamped below at 1e-4
//   q    = e4m3( fp32(x) * (rcp(amax) * 448) ),  scale = amax / 448
// 16 lanes own one block (8 elements = 16 bytes each): coalesced 16-byte loads, 8-byte stores.
constexpr int kActThreads = 256;
constexpr int kActUnroll = 4;

__global__ void __launch_bounds__(kActThreads)
quant_act_1x128_kernel(const uint4* __restrict__ x, uint2* __restrict__ q, float* __restrict__ s,
                       long long num_chunks /* 8-element chunks */, int is_fp16) {
  const long long stride = static_cast<long long>(gridDim.x) * kActThreads;
  long long i = static_cast<long long>(blockIdx.x) * kActThreads + threadIdx.x;
  // The loop bound is taken at the warp's first chunk so that all 32 lanes run the same trip
  // count and the shuffles below always see a full warp; lanes past the end carry zeros.
  for (; i - (threadIdx.x & 31) < num_chunks; i += stride * kActUnroll) {
    uint4 v[kActUnroll];
    bool live[kActUnroll];
#pragma unroll
    for (int u = 0; u < kActUnroll; ++u) {
      const long long idx = i + u * stride;
      live[u] = idx < num_chunks;
      v[u] = live[u] ? __ldg(x + idx) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < kActUnroll; ++u) {
      float amax = abs_max8(v[u], is_fp16);
#pragma unroll
      for (int o = 8; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
      amax = fmaxf(amax, 1e-4f);
      const float inv = inv_scale_448(amax);
      const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
      uint32_t out[2];
#pragma unroll
      for (int p = 0; p < 2; ++p) {
        const float f0 = __fmul_rn(to_f32(static_cast<uint16_t>(w[2 * p] & 0xFFFFu), is_fp16), inv);
        const float f1 = __fmul_rn(to_f32(static_cast<uint16_t>(w[2 * p] >> 16), is_fp16), inv);
        const float f2 = __fmul_rn(to_f32(static_cast<uint16_t>(w[2 * p + 1] & 0xFFFFu), is_fp16), inv);
        const float f3 = __fmul_rn(to_f32(static_cast<uint16_t>(w[2 * p + 1] >> 16), is_fp16), inv);
        out[p] = cvt_e4m3x2(f0, f1) | (cvt_e4m3x2(f2, f3) << 16);
      }
      if (live[u]) {
        const long long idx = i + u * stride;
        q[idx] = make_uint2(out[0], out[1]);
        if ((threadIdx.x & 15) == 0) s[idx >> 4] = __fdiv_rn(amax, 448.0f);
      }
    }
  }
}

// ------------------------------------------------------------------ SwiGLU + 1x128 (between the two expert GEMMs)
// h [rows, 2*inter] holds gate | up (the gate+up GEMM's output).  act = bf16(silu(gate) * up)
// with silu(x) = x / (1 + exp(-x)) evaluated in fp32 (fast exponential and quotient) from the
// 16-bit inputs; act is then quantised exactly like act_1x128 above (same bytes and scales as
// running per_token_cast_to_fp8 on the rounded activation).  Saves writing and re-reading act.

__global__ void __launch_bounds__(kActThreads)
quant_swiglu_1x128_kernel(const uint16_t* __restrict__ h, uint2* __restrict__ q, float* __restrict__ s,
                          long long rows, int inter) {
  const long long chunks_per_row = inter / 8;
  const long long num_chunks = rows * chunks_per_row;
  const long long stride = static_cast<long long>(gridDim.x) * kActThreads;
  long long i = static_cast<long long>(blockIdx.x) * kActThreads + threadIdx.x;
  // (row, chunk in row) of chunk i, advanced by the constant stride with a carry instead of a
  // 64-bit division per chunk
  long long r = i / chunks_per_row;
  long long c = i - r * chunks_per_row;
  const long long dr = stride / chunks_per_row;
  const long long dc = stride - dr * chunks_per_row;
  // loop bound taken at the warp's first chunk: all lanes run the same trip count for the shuffles
  for (; i - (threadIdx.x & 31) < num_chunks; i += stride) {
    const bool live = i < num_chunks;
    float f[8];
    if (live) {
      const uint16_t* row_ptr = h + r * 2 * inter + c * 8;
      const uint4 gv = __ldg(reinterpret_cast<const uint4*>(row_ptr));
      const uint4 uv = __ldg(reinterpret_cast<const uint4*>(row_ptr + inter));
      const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        f[2 * e] = silu_mul_round_bf16(__uint_as_float(gw[e] << 16), __uint_as_float(uw[e] << 16));
        f[2 * e + 1] = silu_mul_round_bf16(__uint_as_float(gw[e] & 0xFFFF0000u), __uint_as_float(uw[e] & 0xFFFF0000u));
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = 0.f;
    }
    r += dr;
    c += dc;
    if (c >= chunks_per_row) {
      c -= chunks_per_row;
      ++r;
    }
    float amax = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(f[e]));
#pragma unroll
    for (int o = 8; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    amax = fmaxf(amax, 1e-4f);
    const float inv = inv_scale_448(amax);
    uint32_t out[2];
#pragma unroll
    for (int p = 0; p < 2; ++p)
      out[p] = cvt_e4m3x2(__fmul_rn(f[4 * p], inv), __fmul_rn(f[4 * p + 1], inv)) |
               (cvt_e4m3x2(__fmul_rn(f[4 * p + 2], inv), __fmul_rn(f[4 * p + 3], inv)) << 16);
    if (live) {
      q[i] = make_uint2(out[0], out[1]);
      if ((threadIdx.x & 15) == 0) s[i >> 4] = __fdiv_rn(amax, 448.0f);
    }
  }
}

// ------------------------------------------------------------------ 128x128 (weights)
// Follows per_block_cast_to_fp8 (gemm/FP8/m_grouped_gemm_channel_expert.py:237-245), batched
// over a leading expert dimension.  One CTA per 128x128 block; the block stays in registers
// between the amax pass and the scaling pass, so HBM is read once.
constexpr int kBlkThreads = 256;

__device__ __forceinline__ float block_max_256(float v, float* red) {
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  __syncthreads();  // protects `red` against the previous use
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float m = red[0];
#pragma unroll
  for (int i = 1; i < kBlkThreads / 32; ++i) m = fmaxf(m, red[i]);
  return m;
}

__global__ void __launch_bounds__(kBlkThreads)
quant_w_128x128_kernel(const uint16_t* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ s, int rows,
                       int cols, int row_blocks, int col_blocks, long long num_blocks, int is_fp16) {
  __shared__ float red[kBlkThreads / 32];
  const int tr = threadIdx.x >> 4;        // 0..15: row inside a 16-row pass
  const int tc = (threadIdx.x & 15) * 8;  // first of this thread's 8 columns
  const bool vec_ok = (cols % 8) == 0;
  for (long long blk = blockIdx.x; blk < num_blocks; blk += gridDim.x) {
    const int cb = static_cast<int>(blk % col_blocks);
    const long long t = blk / col_blocks;
    const int rb = static_cast<int>(t % row_blocks);
    const long long e = t / row_blocks;
    const uint16_t* xe = x + e * static_cast<long long>(rows) * cols;
    uint8_t* qe = q + e * static_cast<long long>(rows) * cols;
    const int c0 = cb * 128 + tc;
    uint4 v[8];
    float amax = 0.f;
#pragma unroll
    for (int p = 0; p < 8; ++p) {
      const int r = rb * 128 + p * 16 + tr;
      v[p] = make_uint4(0, 0, 0, 0);
      if (r < rows) {
        const uint16_t* src = xe + static_cast<long long>(r) * cols + c0;
        if (vec_ok && c0 + 8 <= cols) {
          v[p] = __ldg(reinterpret_cast<const uint4*>(src));
        } else {
          uint16_t tmp[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) tmp[i] = (c0 + i < cols) ? src[i] : uint16_t(0);
          v[p] = make_uint4(tmp[0] | (uint32_t(tmp[1]) << 16), tmp[2] | (uint32_t(tmp[3]) << 16),
                            tmp[4] | (uint32_t(tmp[5]) << 16), tmp[6] | (uint32_t(tmp[7]) << 16));
        }
      }
      amax = fmaxf(amax, abs_max8(v[p], is_fp16));
    }
    amax = fmaxf(block_max_256(amax, red), 1e-4f);
    const float inv = inv_scale_448(amax);
    if (threadIdx.x == 0) s[blk] = __fdiv_rn(amax, 448.0f);
#pragma unroll
    for (int p = 0; p < 8; ++p) {
      const int r = rb * 128 + p * 16 + tr;
      if (r >= rows) continue;
      const uint32_t w[4] = {v[p].x, v[p].y, v[p].z, v[p].w};
      uint32_t out[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float f0 = __fmul_rn(to_f32(static_cast<uint16_t>(w[2 * h] & 0xFFFFu), is_fp16), inv);
        const float f1 = __fmul_rn(to_f32(static_cast<uint16_t>(w[2 * h] >> 16), is_fp16), inv);
        const float f2 = __fmul_rn(to_f32(static_cast<uint16_t>(w[2 * h + 1] & 0xFFFFu), is_fp16), inv);
        const float f3 = __fmul_rn(to_f32(static_cast<uint16_t>(w[2 * h + 1] >> 16), is_fp16), inv);
        out[h] = cvt_e4m3x2(f0, f1) | (cvt_e4m3x2(f2, f3) << 16);
      }
      uint8_t* dst = qe + static_cast<long long>(r) * cols + c0;
      if (vec_ok && c0 + 8 <= cols) {
        *reinterpret_cast<uint2*>(dst) = make_uint2(out[0], out[1]);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (c0 + i < cols) dst[i] = static_cast<uint8_t>((out[i >> 2] >> (8 * (i & 3))) & 0xFFu);
      }
    }
  }
}

// ------------------------------------------------------------------ transposing 128x128 with expansion
// Follows per_block_trans_quant_expand_torch (quant/trans_per_block_quant_expand_128x.py:216-273):
// per expert, rows are padded with zeros to a multiple of 128; per 128x128 block
//   scale = clamp(amax / 448, 1e-12, 3e38),  q = e4m3( clamp(fp32(x) / scale, +-448) )
// and the block is written transposed: out[n, pad_start_g + local_row].  Columns and scales
// past the last padded expert (up to m_expand) are zero.  The clamp of the scale is the one the
// reference's shipped operator applies (its Triton kernel, same file :124-126); the torch helper
// has none and turns an all-zero block (zero gradients, a dead column) into scale 0 and NaN
// bytes, which would poison every product that consumes them.  With the clamp such a block
// gives zero bytes and scale 1e-12; blocks whose amax / 448 is at least 1e-12 are bit for bit
// what the torch helper produces.  (The block maximum ignores NaN elements, as a reduction
// with max.f32 does; a NaN element itself becomes the byte 0xff.)
constexpr int kTqPitch = 132;  // bytes per staged row: 33 words -> conflict-free column reads

// Largest |x| of eight 16-bit floats as raw bits (sign cleared).  For bf16 and fp16 alike the
// magnitude order of non-NaN values is the unsigned order of these bits, and every NaN pattern
// sorts above infinity, so one integer maximum also tells whether a NaN or Inf was present.
__device__ __forceinline__ uint32_t abs_bits_max8(const uint4& v, uint32_t m) {
  constexpr uint32_t kAbs = 0x7FFF7FFFu;
  m = __vimax3_u16x2(m, v.x & kAbs, v.y & kAbs);
  return __vimax3_u16x2(m, v.z & kAbs, v.w & kAbs);
}

// Slow, always-exact form of one 8-element chunk: IEEE division per element.
// torch.clamp propagates NaN; the host's 0/0 is the negative quiet NaN -> byte 0xff.
__device__ __noinline__ uint2 trans_quant_chunk_exact(uint4 v, float scale, int is_fp16) {
  const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
  uint32_t out[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float f[4];
    f[0] = to_f32(static_cast<uint16_t>(wv[2 * h] & 0xFFFFu), is_fp16);
    f[1] = to_f32(static_cast<uint16_t>(wv[2 * h] >> 16), is_fp16);
    f[2] = to_f32(static_cast<uint16_t>(wv[2 * h + 1] & 0xFFFFu), is_fp16);
    f[3] = to_f32(static_cast<uint16_t>(wv[2 * h + 1] >> 16), is_fp16);
    uint32_t b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float d = __fdiv_rn(f[i], scale);
      b[i] = (d != d) ? 0xFFu : (cvt_e4m3x2(fminf(fmaxf(d, -448.0f), 448.0f), 0.f) & 0xFFu);
    }
    out[h] = b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24);
  }
  return make_uint2(out[0], out[1]);
}

// Fast form of one chunk, used when the block holds no NaN/Inf and its scale is far from the
// ends of the fp32 range.  With r = RN(1/scale) computed once per block,
//   q0 = RN(x * r),  e = RN(x - scale * q0),  q1 = RN(q0 + e * r)      (two fused multiply-adds)
// is the correctly rounded quotient RN(x / scale): checked exhaustively on the host for every
// pair of 8-bit (bf16) and 11-bit (fp16) significands of x and of the block maximum that
// `scale = RN(amax / 448)` derives from (tests/test_trans_quant_division.py); rounding
// depends on the significands only while nothing underflows, which the caller's range check
// guarantees for every quotient that does not convert to zero anyway.  The saturating
// conversion then equals the reference's clamp + cast.
template <bool kFp16>
__device__ __forceinline__ uint2 trans_quant_chunk_fast(const uint4& v, float scale, float r) {
  const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
  const float neg_scale = -scale;
  uint32_t out[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float q[4];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const uint32_t w = wv[2 * h + i];
      float x0, x1;
      if (kFp16) {
        const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w));
        x0 = t.x;
        x1 = t.y;
      } else {
        x0 = __uint_as_float(w << 16);
        x1 = __uint_as_float(w & 0xFFFF0000u);
      }
      const float a0 = __fmul_rn(x0, r), a1 = __fmul_rn(x1, r);
      q[2 * i] = __fmaf_rn(__fmaf_rn(neg_scale, a0, x0), r, a0);
      q[2 * i + 1] = __fmaf_rn(__fmaf_rn(neg_scale, a1, x1), r, a1);
    }
    // x = -0 gives q1 = +0 (the residual of a negative zero is +0); the reference keeps the sign,
    // so take every byte's sign bit from x (bit 15 / 31 of the 16-bit inputs; a no-op otherwise)
    const uint32_t signs = __byte_perm(wv[2 * h], wv[2 * h + 1], 0x7531) & 0x80808080u;
    out[h] = cvt_e4m3x2(q[0], q[1]) | (cvt_e4m3x2(q[2], q[3]) << 16) | signs;
  }
  return make_uint2(out[0], out[1]);
}

template <bool kFp16>
__global__ void __launch_bounds__(kBlkThreads)
quant_trans_expand_kernel(const uint16_t* __restrict__ x, const void* __restrict__ sizes, int sizes_i64,
                          int num_groups, uint8_t* __restrict__ q, float* __restrict__ s,
                          long long* __restrict__ padded_sizes_out, long long m_rows, int n, long long m_expand) {
  __shared__ uint32_t red[kBlkThreads / 32];
  __shared__ __align__(16) uint8_t stage[128 * kTqPitch];
  const int n_tiles = n / 128;
  const int m_tiles_total = static_cast<int>(m_expand / 128);
  const int scale_cols = m_tiles_total;
  const int tr = threadIdx.x >> 4;
  const int tc = (threadIdx.x & 15) * 8;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr uint32_t kInfBits = kFp16 ? 0x7C00u : 0x7F80u;

  if (padded_sizes_out && blockIdx.x == 0) {
    for (int g = threadIdx.x; g < num_groups; g += kBlkThreads) {
      long long v = sizes_i64 ? static_cast<const long long*>(sizes)[g]
                              : static_cast<long long>(static_cast<const int*>(sizes)[g]);
      if (v < 0) v = 0;
      padded_sizes_out[g] = (v + 127) / 128 * 128;
    }
  }

  GroupWalker w;
  w.init(sizes, sizes_i64, num_groups, 0, 128, m_rows);  // no row of x at or past m_rows is read
  bool in_groups = true;
  for (long long tile = blockIdx.x; tile < static_cast<long long>(m_tiles_total) * n_tiles; tile += gridDim.x) {
    const int mt = static_cast<int>(tile / n_tiles);
    const int nt = static_cast<int>(tile - static_cast<long long>(mt) * n_tiles);
    if (in_groups) in_groups = w.seek(mt);
    const long long col0 = static_cast<long long>(mt) * 128;  // output column of local row 0
    if (!in_groups) {
      // expansion tail: zero bytes and zero scales
      for (int i = threadIdx.x; i < 128 * 8; i += kBlkThreads) {
        const int r = i >> 3, c = (i & 7) * 16;
        *reinterpret_cast<uint4*>(q + (static_cast<long long>(nt) * 128 + r) * m_expand + col0 + c) =
            make_uint4(0, 0, 0, 0);
      }
      if (threadIdx.x == 0) s[static_cast<long long>(nt) * scale_cols + mt] = 0.f;
      continue;
    }
    const long long row0 = w.tile_row0(mt);
    const long long row_end = w.group_row_end();
    uint4 v[8];
    uint32_t mx2 = 0;
#pragma unroll
    for (int p = 0; p < 8; ++p) {
      const long long r = row0 + p * 16 + tr;
      v[p] = (r < row_end) ? __ldg(reinterpret_cast<const uint4*>(x + r * n + nt * 128 + tc)) : make_uint4(0, 0, 0, 0);
      mx2 = abs_bits_max8(v[p], mx2);
    }
    // block maximum of the raw magnitude bits
    uint32_t mx = __reduce_max_sync(0xFFFFFFFFu, max(mx2 & 0xFFFFu, mx2 >> 16));
    __syncthreads();  // protects `red` and `stage` against the previous tile
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = red[0];
#pragma unroll
    for (int i = 1; i < kBlkThreads / 32; ++i) mx = max(mx, red[i]);

    uint32_t* dst0 = reinterpret_cast<uint32_t*>(stage + tr * kTqPitch + tc);
    const float amax_fast = to_f32(static_cast<uint16_t>(mx), kFp16);
    // fast block: no NaN/Inf anywhere, scale and its reciprocal far from the ends of the range
    if (mx < kInfBits && amax_fast >= 0x1p-30f && amax_fast <= 0x1p100f) {
      const float scale = __fdiv_rn(amax_fast, 448.0f);
      if (threadIdx.x == 0) s[static_cast<long long>(nt) * scale_cols + mt] = scale;
      const float r = __frcp_rn(scale);
#pragma unroll
      for (int p = 0; p < 8; ++p) {
        const uint2 o = trans_quant_chunk_fast<kFp16>(v[p], scale, r);
        uint32_t* dst = dst0 + p * 16 * (kTqPitch / 4);
        dst[0] = o.x;
        dst[1] = o.y;
      }
    } else {
      // NaN/Inf in the block, an all-zero block or an extreme scale (any block whose scale the
      // clamp could touch lands here): per-element IEEE division
      // with the fp32 maximum taken by fmaxf
      float amax = 0.f;
#pragma unroll
      for (int p = 0; p < 8; ++p) amax = fmaxf(amax, abs_max8(v[p], kFp16));
#pragma unroll
      for (int o = 16; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
      __shared__ float redf[kBlkThreads / 32];
      if (lane == 0) redf[warp] = amax;
      __syncthreads();
      amax = redf[0];
#pragma unroll
      for (int i = 1; i < kBlkThreads / 32; ++i) amax = fmaxf(amax, redf[i]);
      float scale = __fdiv_rn(amax, 448.0f);
      scale = fminf(fmaxf(scale, 1e-12f), 3e38f);  // the shipped operator's clamp
      if (threadIdx.x == 0) s[static_cast<long long>(nt) * scale_cols + mt] = scale;
#pragma unroll
      for (int p = 0; p < 8; ++p) {
        const uint2 o = trans_quant_chunk_exact(v[p], scale, kFp16);
        uint32_t* dst = dst0 + p * 16 * (kTqPitch / 4);
        dst[0] = o.x;
        dst[1] = o.y;
      }
    }
    __syncthreads();
    // transposed write-out: lane (a = lane%8, b = lane/8) gathers a 4x4 byte block
    // (rows 4a..4a+3 of a 32-row quarter, columns 4(q0+b)..+3), transposes it with byte
    // permutes and stores one 32-bit word per output row: 8 lanes -> one 32-byte sector.
    const int a = lane & 7, bq = lane >> 3;
    for (int it = warp; it < 32; it += kBlkThreads / 32) {
      const int mq = it & 3;           // 32-row quarter of the tile
      const int q0 = (it >> 2) * 4;    // first 4-column group
      const int m_local = mq * 32 + 4 * a;
      const int n4 = (q0 + bq) * 4;
      uint32_t r0 = *reinterpret_cast<const uint32_t*>(stage + (m_local + 0) * kTqPitch + n4);
      uint32_t r1 = *reinterpret_cast<const uint32_t*>(stage + (m_local + 1) * kTqPitch + n4);
      uint32_t r2 = *reinterpret_cast<const uint32_t*>(stage + (m_local + 2) * kTqPitch + n4);
      uint32_t r3 = *reinterpret_cast<const uint32_t*>(stage + (m_local + 3) * kTqPitch + n4);
      // 4x4 byte transpose
      const uint32_t t0 = __byte_perm(r0, r1, 0x5140);  // r0.b0 r1.b0 r0.b1 r1.b1
      const uint32_t t1 = __byte_perm(r2, r3, 0x5140);
      const uint32_t t2 = __byte_perm(r0, r1, 0x7362);  // r0.b2 r1.b2 r0.b3 r1.b3
      const uint32_t t3 = __byte_perm(r2, r3, 0x7362);
      const uint32_t c0 = __byte_perm(t0, t1, 0x5410);  // column n4+0: r0.b0 r1.b0 r2.b0 r3.b0
      const uint32_t c1 = __byte_perm(t0, t1, 0x7632);
      const uint32_t c2 = __byte_perm(t2, t3, 0x5410);
      const uint32_t c3 = __byte_perm(t2, t3, 0x7632);
      uint8_t* o = q + (static_cast<long long>(nt) * 128 + n4) * m_expand + col0 + m_local;
      *reinterpret_cast<uint32_t*>(o) = c0;
      *reinterpret_cast<uint32_t*>(o + m_expand) = c1;
      *reinterpret_cast<uint32_t*>(o + 2 * m_expand) = c2;
      *reinterpret_cast<uint32_t*>(o + 3 * m_expand) = c3;
    }
  }
}

static int grid_for(long long work_items, int per_sm) {
  const int sms = sm_count();
  long long g = static_cast<long long>(sms > 0 ? sms : 1) * per_sm;
  if (g > work_items) g = work_items;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

}  // namespace b200

extern "C" {

int b200quant_act_1x128(const void* x, void* q, float* scales, int64_t rows, int64_t k, int dtype, void* stream) {
  using namespace b200;
  B200_REQUIRE(dtype == 0 || dtype == 1, "b200quant_act_1x128: dtype must be 0 (bf16) or 1 (fp16)");
  B200_REQUIRE(rows >= 0 && k >= 0, "b200quant_act_1x128: negative dimension");
  B200_REQUIRE(k % 128 == 0, "b200quant_act_1x128: k (%lld) must be a multiple of 128", (long long)k);
  if (rows == 0 || k == 0) return 0;
  B200_REQUIRE(x && q && scales, "b200quant_act_1x128: null pointer");
  B200_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(q) & 7) == 0,
               "b200quant_act_1x128: x must be 16-byte and q 8-byte aligned");
  const long long chunks = rows * k / 8;
  const int grid = grid_for((chunks + kActThreads - 1) / kActThreads, 16);
  quant_act_1x128_kernel<<<grid, kActThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), static_cast<uint2*>(q), scales, chunks, dtype);
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200quant_swiglu_act_1x128(const void* h, void* q, float* scales, int64_t rows, int64_t inter, void* stream) {
  using namespace b200;
  B200_REQUIRE(rows >= 0 && inter >= 0, "b200quant_swiglu_act_1x128: negative dimension");
  B200_REQUIRE(inter % 128 == 0, "b200quant_swiglu_act_1x128: inter (%lld) must be a multiple of 128", (long long)inter);
  if (rows == 0 || inter == 0) return 0;
  B200_REQUIRE(h && q && scales, "b200quant_swiglu_act_1x128: null pointer");
  B200_REQUIRE((reinterpret_cast<uintptr_t>(h) & 15) == 0 && (reinterpret_cast<uintptr_t>(q) & 7) == 0,
               "b200quant_swiglu_act_1x128: h must be 16-byte and q 8-byte aligned");
  const long long chunks = rows * inter / 8;
  const int grid = grid_for((chunks + kActThreads - 1) / kActThreads, 16);
  quant_swiglu_1x128_kernel<<<grid, kActThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t*>(h), static_cast<uint2*>(q), scales, rows, static_cast<int>(inter));
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200quant_w_128x128(const void* x, void* q, float* scales, int64_t batch, int rows, int cols, int dtype,
                        void* stream) {
  using namespace b200;
  B200_REQUIRE(dtype == 0 || dtype == 1, "b200quant_w_128x128: dtype must be 0 (bf16) or 1 (fp16)");
  B200_REQUIRE(batch >= 0 && rows >= 0 && cols >= 0, "b200quant_w_128x128: negative dimension");
  if (batch == 0 || rows == 0 || cols == 0) return 0;
  B200_REQUIRE(x && q && scales, "b200quant_w_128x128: null pointer");
  B200_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(q) & 7) == 0,
               "b200quant_w_128x128: x must be 16-byte and q 8-byte aligned");
  const int rb = (rows + 127) / 128, cb = (cols + 127) / 128;
  const long long blocks = batch * rb * cb;
  const int grid = grid_for(blocks, 8);
  quant_w_128x128_kernel<<<grid, kBlkThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t*>(x), static_cast<uint8_t*>(q), scales, rows, cols, rb, cb, blocks, dtype);
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200quant_trans_expand_128x(const void* x, const void* sizes, int sizes_is_i64, int num_groups, void* q,
                                float* scales, int64_t* padded_sizes_out, int64_t m_rows, int n, int64_t m_expand,
                                int dtype, void* stream) {
  using namespace b200;
  B200_REQUIRE(dtype == 0 || dtype == 1, "b200quant_trans_expand_128x: dtype must be 0 (bf16) or 1 (fp16)");
  B200_REQUIRE(num_groups > 0 && m_rows >= 0 && n > 0, "b200quant_trans_expand_128x: bad dimension");
  B200_REQUIRE(n % 128 == 0, "b200quant_trans_expand_128x: n (%d) must be a multiple of 128", n);
  B200_REQUIRE(m_expand % 128 == 0 && m_expand >= 128, "b200quant_trans_expand_128x: m_expand must be a multiple of 128");
  B200_REQUIRE(x && sizes && q && scales, "b200quant_trans_expand_128x: null pointer");
  B200_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(q) & 15) == 0,
               "b200quant_trans_expand_128x: x and q must be 16-byte aligned");
  B200_REQUIRE(m_expand / 128 < (1ll << 30), "b200quant_trans_expand_128x: m_expand too large");
  const long long tiles = (m_expand / 128) * (n / 128);
  const int grid = grid_for(tiles, 4);
  if (dtype == 1)
    quant_trans_expand_kernel<true><<<grid, kBlkThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(x), sizes, sizes_is_i64, num_groups, static_cast<uint8_t*>(q), scales,
        reinterpret_cast<long long*>(padded_sizes_out), m_rows, n, m_expand);
  else
    quant_trans_expand_kernel<false><<<grid, kBlkThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(x), sizes, sizes_is_i64, num_groups, static_cast<uint8_t*>(q), scales,
        reinterpret_cast<long long*>(padded_sizes_out), m_rows, n, m_expand);
  B200_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
