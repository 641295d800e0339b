// Library-wide services behind the C ABI: last-error text, the per-device status word,
// the SM count cache and tensor-map encoding through the driver entry point.
#include <cudaTypedefs.h>
#include <stdarg.h>
#include <string.h>

#include <mutex>

#include "../../include/b200gemm.h"
#include "common.cuh"

namespace b200 {

static thread_local char g_last_error[512] = "";

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}

int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return 0;
  return set_error(kErrCuda, "CUDA error %d (%s) in %s", static_cast<int>(e), cudaGetErrorString(e), what);
}

// One status word per device (a __device__ variable exists once per device that loads the
// module).  Kernels OR error bits into it; the host reads it on demand.
__device__ unsigned g_device_status = 0;

constexpr int kMaxDevices = 64;
static std::mutex g_mutex;
static unsigned* g_status_ptr[kMaxDevices] = {nullptr};
static int g_sm_count[kMaxDevices] = {0};

unsigned* device_status_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_status_ptr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
    g_status_ptr[dev] = static_cast<unsigned*>(p);
  }
  return g_status_ptr[dev];
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_sm_count[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    g_sm_count[dev] = n;
  }
  return g_sm_count[dev];
}

static PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  });
  return fn;
}

int encode_tmap(CUtensorMap* out, CUtensorMapDataType dtype, int rank, const void* base, const uint64_t* dims,
                const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swz, const char* what) {
  auto fn = get_encode_fn();
  if (!fn) return set_error(kErrDriverEntry, "cuTensorMapEncodeTiled is not available from this driver");
  // The encode function is a raw driver call and needs a current context.  A host thread that has
  // only inherited "the current device" (e.g. an autograd worker thread) may not have one bound
  // yet; re-selecting the current device binds its primary context to this thread.
  {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaSetDevice(dev);
  }
  cuuint64_t gdim[5];
  cuuint64_t gstr[5];
  cuuint32_t bdim[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estr[i] = 1;
    if (i + 1 < rank) gstr[i] = strides_bytes[i];
  }
  CUresult r = fn(out, dtype, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdim, gstr, bdim, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    return set_error(kErrInvalidArgument,
                     "tensor map for %s rejected by the driver (CUresult %d): base=%p rank=%d dims=[%llu,%llu,%llu] "
                     "box=[%u,%u,%u]",
                     what, static_cast<int>(r), base, rank, (unsigned long long)dims[0],
                     (unsigned long long)(rank > 1 ? dims[1] : 0), (unsigned long long)(rank > 2 ? dims[2] : 0), box[0],
                     rank > 1 ? box[1] : 0, rank > 2 ? box[2] : 0);
  }
  return 0;
}

}  // namespace b200

extern "C" {

int b200gemm_version(void) { return 100; }

const char* b200gemm_last_error(void) { return b200::g_last_error; }

int b200gemm_device_status(unsigned* out_status, int clear) {
  if (!out_status) return b200::set_error(b200::kErrInvalidArgument, "out_status is null");
  unsigned* p = b200::device_status_ptr();
  if (!p) return b200::set_error(b200::kErrCuda, "no CUDA device / status word unavailable");
  // kernels on non-blocking streams (torch's side streams are) do not order with the legacy
  // stream's copy below, so wait for the whole device first
  B200_CUDA(cudaDeviceSynchronize());
  B200_CUDA(cudaMemcpy(out_status, p, sizeof(unsigned), cudaMemcpyDeviceToHost));
  if (clear && *out_status) B200_CUDA(cudaMemset(p, 0, sizeof(unsigned)));
  return 0;
}

int b200gemm_sm_count(void) { return b200::sm_count(); }

}  // extern "C"
