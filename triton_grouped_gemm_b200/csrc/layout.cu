// Device-side builders of the integer layouts in gemm/layout.py (the reference builds them with
// host loops over .tolist(), gemm/layout.py:73-120).  The GEMM kernels derive their own tile
// metadata on the fly; these exist for callers that keep using the layout tensors (DeepGEMM-style
// per-row expert ids, psum offsets, group starts).  Group counts are small (tens to a few
// thousand), so every block recomputes the prefix it needs from the size vector.
#include "../../include/b200gemm.h"
#include "common.cuh"

namespace b200 {

__device__ __forceinline__ long long layout_size_of(const void* sizes, int i64, int g) {
  const long long v = i64 ? static_cast<const long long*>(sizes)[g]
                          : static_cast<long long>(static_cast<const int*>(sizes)[g]);
  return v < 0 ? 0 : v;
}

// exclusive prefix of (optionally padded) sizes; psum: padded prefix + own size
// mode 0: starts of compact sizes, 1: starts of padded sizes, 2: psum layout
__global__ void __launch_bounds__(256) layout_prefix_kernel(const void* __restrict__ sizes, int i64, int num_groups,
                                                            int block_m, int mode, int* __restrict__ out) {
  // one thread per output, each walks its own prefix (O(G^2) integer adds for G of a few thousand)
  for (int g = blockIdx.x * blockDim.x + threadIdx.x; g < num_groups; g += gridDim.x * blockDim.x) {
    long long run = 0;
    for (int h = 0; h < g; ++h) {
      const long long s = layout_size_of(sizes, i64, h);
      run += mode == 0 ? s : (s + block_m - 1) / block_m * block_m;
    }
    out[g] = static_cast<int>(mode == 2 ? run + layout_size_of(sizes, i64, g) : run);
  }
}

// one int32 per padded row: the group id on real rows, -1 on padding rows; block g fills group g
__global__ void __launch_bounds__(256) layout_rows_kernel(const void* __restrict__ sizes, int i64, int num_groups,
                                                          int block_m, int* __restrict__ out, long long total_rows) {
  for (int g = blockIdx.x; g < num_groups; g += gridDim.x) {
    long long start = 0;
    for (int h = 0; h < g; ++h) start += (layout_size_of(sizes, i64, h) + block_m - 1) / block_m * block_m;
    const long long s = layout_size_of(sizes, i64, g);
    const long long p = (s + block_m - 1) / block_m * block_m;
    for (long long r = threadIdx.x; r < p; r += blockDim.x)
      if (start + r < total_rows) out[start + r] = r < s ? g : -1;
  }
}

}  // namespace b200

extern "C" {

int b200layout_group_starts(const void* sizes, int sizes_is_i64, int num_groups, int padded, int block_m, int* out,
                            void* stream) {
  using namespace b200;
  B200_REQUIRE(num_groups >= 0 && block_m > 0, "b200layout_group_starts: bad argument");
  if (num_groups == 0) return 0;
  B200_REQUIRE(sizes && out, "b200layout_group_starts: null pointer");
  layout_prefix_kernel<<<(num_groups + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      sizes, sizes_is_i64, num_groups, block_m, padded ? 1 : 0, out);
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200layout_psum(const void* sizes, int sizes_is_i64, int num_groups, int block_m, int* out, void* stream) {
  using namespace b200;
  B200_REQUIRE(num_groups >= 0 && block_m > 0, "b200layout_psum: bad argument");
  if (num_groups == 0) return 0;
  B200_REQUIRE(sizes && out, "b200layout_psum: null pointer");
  layout_prefix_kernel<<<(num_groups + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(sizes, sizes_is_i64,
                                                                                                 num_groups, block_m, 2, out);
  B200_CUDA(cudaGetLastError());
  return 0;
}

int b200layout_grouped_rows(const void* sizes, int sizes_is_i64, int num_groups, int block_m, int* out,
                            int64_t total_padded_rows, void* stream) {
  using namespace b200;
  B200_REQUIRE(num_groups >= 0 && block_m > 0 && total_padded_rows >= 0, "b200layout_grouped_rows: bad argument");
  if (num_groups == 0 || total_padded_rows == 0) return 0;
  B200_REQUIRE(sizes && out, "b200layout_grouped_rows: null pointer");
  const int grid = num_groups < 1024 ? num_groups : 1024;
  layout_rows_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(sizes, sizes_is_i64, num_groups, block_m, out,
                                                                         total_padded_rows);
  B200_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"
