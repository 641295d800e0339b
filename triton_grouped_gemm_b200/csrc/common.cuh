// Host/device helpers shared by every translation unit of the library: error reporting,
// the device status word, tensor-map encoding, bounded mbarrier waits and the one-pass
// group walker that replaces the reference's host-built tile metadata
// (gemm/BF16/m_grouped_gemm_TMA.py:297-326 in the reference).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "ptx.cuh"

namespace b200 {

// ------------------------------------------------------------------ status codes (C ABI return values)
enum : int {
  kOk = 0,
  kErrInvalidArgument = -1,
  kErrUnsupported = -2,
  kErrCuda = -3,
  kErrDriverEntry = -4,
};

// bits of the device status word (b200gemm_device_status)
enum : unsigned {
  kDevTimeoutProducer = 1u << 0,
  kDevTimeoutMma = 1u << 1,
  kDevTimeoutEpilogue = 1u << 2,
  kDevTimeoutPromote = 1u << 3,
  kDevBadGroupSize = 1u << 4,
  kDevBadRowIndex = 1u << 5,  // a row mover was given a rank or row outside its buffers (access skipped)
};

// implemented in api.cu
int set_error(int code, const char* fmt, ...);
int check_cuda(cudaError_t e, const char* what);
// device address of the per-device status word (set-up on first use, per device)
unsigned* device_status_ptr();
int sm_count();
// cuTensorMapEncodeTiled through cudaGetDriverEntryPoint (no link-time libcuda dependency)
int encode_tmap(CUtensorMap* out, CUtensorMapDataType dtype, int rank, const void* base, const uint64_t* dims,
                const uint64_t* strides_bytes /* rank-1 entries */, const uint32_t* box, CUtensorMapSwizzle swz,
                const char* what);

#define B200_REQUIRE(cond, ...)                                   \
  do {                                                            \
    if (!(cond)) return ::b200::set_error(::b200::kErrInvalidArgument, __VA_ARGS__); \
  } while (0)

#define B200_CUDA(expr)                                          \
  do {                                                           \
    int _rc = ::b200::check_cuda((expr), #expr);                 \
    if (_rc != 0) return _rc;                                    \
  } while (0)

// ------------------------------------------------------------------ bounded waits
// Every spin on an mbarrier gives up after kWaitLimitNs; the waiting role then raises the
// CTA-wide abort flag, records which role timed out in the device status word and leaves
// its loop, so a protocol error ends in an error code instead of a hung GPU.
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // 2 s

__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                             unsigned* status, unsigned role_bit) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 63u) == 0u) {
      if (*abort_flag) return false;
      if (global_timer_ns() - t0 > kWaitLimitNs) {
        *abort_flag = 1;
        if (status) atomicOr(status, role_bit);
        return false;
      }
    }
  }
  return true;
}

// Polling variant (mbarrier.test_wait, no hardware suspend) for handshakes whose wake-up
// latency is on the critical path; same bound, same abort protocol.
__device__ __forceinline__ bool wait_bounded_spin(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                  unsigned* status, unsigned role_bit) {
  uint32_t spins = 0;
  uint64_t t0 = 0;
  while (!mbar_test_wait(bar, parity)) {
    if ((++spins & 1023u) == 0u) {
      if (*abort_flag) return false;
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > kWaitLimitNs) {
        *abort_flag = 1;
        if (status) atomicOr(status, role_bit);
        return false;
      }
    }
  }
  return true;
}

// same, for barriers that the peer CTA of a pair arrives on (cluster-scope acquire)
__device__ __forceinline__ bool wait_bounded_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                     unsigned* status, unsigned role_bit) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait_cluster(bar, parity)) {
    if ((++spins & 63u) == 0u) {
      if (*abort_flag) return false;
      if (global_timer_ns() - t0 > kWaitLimitNs) {
        *abort_flag = 1;
        if (status) atomicOr(status, role_bit);
        return false;
      }
    }
  }
  return true;
}

// ------------------------------------------------------------------ group walker
// Tiles are numbered in "padded tile space": group g owns ceil(size_g / kTileRows)
// consecutive row tiles.  A walker is advanced monotonically to the row tile a role is about
// to process; all lanes of a warp run it redundantly (uniform loads, no divergence).
// stride == 0 : compact rows (group g starts at the sum of the earlier sizes)
// stride  > 0 : masked layout (group g starts at g * stride, only sizes[g] rows are valid)
// stride == -1: padded rows (group g starts at the sum of the earlier sizes, each rounded up
//               to a multiple of 128; rows between size and the padded size are skipped)
struct GroupWalker {
  const void* sizes;
  int sizes_i64;
  int num_groups;
  int stride;        // see above
  int tile_rows;
  int g;             // current group
  int tile_begin;    // first padded tile of group g
  int ntiles;        // tiles of group g
  int size;          // rows of group g (after clamping, see enter())
  bool overflow;     // some group's rows ran past row_limit and were cut off
  long long row_begin;  // first row of group g (contiguous kind)
  long long row_limit;  // rows the A / C tensors really have: no row >= row_limit is ever touched

  // Loads the size of group i, whose first row is already in row_begin.  Negative sizes count as
  // zero, masked sizes are clamped to the slot, and in the contiguous layouts a group is cut off
  // at row_limit: a size vector whose sum exceeds the tensors' row count (a bad routing vector)
  // must neither write past the end of C nor read scales past their end, and it must not
  // stretch the persistent loop either.  The cut is remembered in `overflow`.
  __device__ __forceinline__ void enter(int i) {
    long long v = sizes_i64 ? static_cast<const long long*>(sizes)[i]
                            : static_cast<long long>(static_cast<const int*>(sizes)[i]);
    if (v < 0) v = 0;
    if (stride > 0) {
      if (v > stride) v = stride;
    } else {
      long long room = row_limit - row_begin;
      if (room < 0) room = 0;
      if (v > room) {
        v = room;
        overflow = true;
      }
    }
    size = static_cast<int>(v);
    ntiles = (size + tile_rows - 1) / tile_rows;
  }

  // row_limit_: number of rows of the row-grouped tensors (m_rows; G * stride in the masked layout)
  __device__ __forceinline__ void init(const void* sizes_, int sizes_i64_, int num_groups_, int stride_,
                                       int tile_rows_, long long row_limit_) {
    sizes = sizes_;
    sizes_i64 = sizes_i64_;
    num_groups = num_groups_;
    stride = stride_;
    tile_rows = tile_rows_;
    row_limit = row_limit_;
    overflow = false;
    g = 0;
    tile_begin = 0;
    row_begin = 0;
    size = 0;
    ntiles = 0;
    if (num_groups > 0) enter(0);
  }

  // Move to padded row tile `t` (t must not decrease between calls).  false = past the end.
  __device__ __forceinline__ bool seek(int t) {
    while (g < num_groups && t >= tile_begin + ntiles) {
      tile_begin += ntiles;
      // padded layout: every group occupies its size rounded up to 128 rows, whatever the tile height
      row_begin += stride < 0 ? (static_cast<long long>(size) + 127) / 128 * 128 : static_cast<long long>(size);
      ++g;
      if (g < num_groups) enter(g);
    }
    return g < num_groups;
  }

  // first row (in the A / C row space) of padded tile t, and one-past-last valid row of the group
  __device__ __forceinline__ long long tile_row0(int t) const {
    long long base = stride > 0 ? static_cast<long long>(g) * stride : row_begin;
    return base + static_cast<long long>(t - tile_begin) * tile_rows;
  }
  __device__ __forceinline__ long long group_row_end() const {
    long long base = stride > 0 ? static_cast<long long>(g) * stride : row_begin;
    return base + size;
  }
};

}  // namespace b200
