// Buffers that the other ranks of a node can address (CUDA IPC), for the peer-memory exchange
// of the expert-parallel layer.  The owner allocates with cudaMalloc and exports a handle; every
// other process opens the handle WITH ITS OWN DEVICE CURRENT and cudaIpcMemLazyEnablePeerAccess,
// which maps the memory into that device's address space and enables peer access to the owning
// device, so kernels launched on the opening rank's GPU may load and store through the pointer.
// (Opening it with the owning device current instead - what a framework's generic tensor
// sharing does - leaves the opening rank's GPU without access: its kernels fault.)
#include "../../include/b200gemm.h"
#include "common.cuh"

extern "C" {

int b200ipc_alloc(int64_t bytes, void** out) {
  using namespace b200;
  B200_REQUIRE(out && bytes > 0, "b200ipc_alloc: bad argument");
  void* p = nullptr;
  B200_CUDA(cudaMalloc(&p, static_cast<size_t>(bytes)));
  cudaError_t e = cudaMemset(p, 0, static_cast<size_t>(bytes));
  if (e != cudaSuccess) {
    cudaFree(p);
    return check_cuda(e, "cudaMemset");
  }
  *out = p;
  return 0;
}

int b200ipc_free(void* p) {
  using namespace b200;
  if (!p) return 0;
  B200_CUDA(cudaFree(p));
  return 0;
}

int b200ipc_export(const void* p, void* handle64) {
  using namespace b200;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  B200_REQUIRE(p && handle64, "b200ipc_export: null pointer");
  cudaIpcMemHandle_t h;
  B200_CUDA(cudaIpcGetMemHandle(&h, const_cast<void*>(p)));
  memcpy(handle64, &h, sizeof(h));
  return 0;
}

int b200ipc_open(const void* handle64, void** out) {
  using namespace b200;
  B200_REQUIRE(handle64 && out, "b200ipc_open: null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  B200_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *out = p;
  return 0;
}

int b200ipc_close(void* p) {
  using namespace b200;
  if (!p) return 0;
  B200_CUDA(cudaIpcCloseMemHandle(p));
  return 0;
}

// n contiguous device-to-device copies on `stream`, one cudaMemcpyAsync each (the copy engines
// move them, over NVLink when a side is another rank's buffer, without occupying an SM).
int b200ipc_copy_many_async(int n, void* const* dst, const void* const* src, const int64_t* bytes, void* stream) {
  using namespace b200;
  B200_REQUIRE(n >= 0, "b200ipc_copy_many_async: negative count");
  if (n == 0) return 0;
  B200_REQUIRE(dst && src && bytes, "b200ipc_copy_many_async: null pointer");
  for (int i = 0; i < n; ++i) {
    if (bytes[i] == 0) continue;
    B200_REQUIRE(bytes[i] > 0 && dst[i] && src[i], "b200ipc_copy_many_async: copy %d has a null pointer or a negative size", i);
    B200_CUDA(cudaMemcpyAsync(dst[i], src[i], static_cast<size_t>(bytes[i]), cudaMemcpyDeviceToDevice,
                              static_cast<cudaStream_t>(stream)));
  }
  return 0;
}

}  // extern "C"
