// C entry points of the native CUDA-IPC symmetric-memory provider (used by the
// Python package when torch symmetric memory is not wanted or not available).
// Parity: the role of csrc/contrib/symm_mem.cuh:10-59 in the reference
// (allocate, map every peer, zero, synchronise), without NVSHMEM.
#include <cuda_runtime.h>

#include <cstring>
#include <string>

namespace purlin { void setError(const std::string& e); }

extern "C" {

void* purlin_ipc_alloc(size_t bytes) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) { purlin::setError(std::string("cudaMalloc: ") + cudaGetErrorString(e)); return nullptr; }
  e = cudaMemset(p, 0, bytes);
  if (e != cudaSuccess) { purlin::setError(std::string("cudaMemset: ") + cudaGetErrorString(e)); cudaFree(p); return nullptr; }
  cudaDeviceSynchronize();
  return p;
}

int purlin_ipc_free(void* p) { return p ? int(cudaFree(p)) : 0; }

int purlin_ipc_export(void* devicePtr, char* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, devicePtr);
  if (e != cudaSuccess) { purlin::setError(std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(e)); return 1; }
  static_assert(sizeof(h) == 64, "IPC handle size");
  std::memcpy(handle64, &h, sizeof(h));
  return 0;
}

void* purlin_ipc_open(const char* handle64) {
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) { purlin::setError(std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e)); return nullptr; }
  return p;
}

int purlin_ipc_close(void* p) { return p ? int(cudaIpcCloseMemHandle(p)) : 0; }

}  // extern "C"
