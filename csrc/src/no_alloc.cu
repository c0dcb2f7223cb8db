// Allocation-free variant of the MoE routing kernel: its scratch (one counter per expert) is a static device array.
// See csrc/include/purlin/no_alloc.h for who needs this and the rules of use. No counterpart in the reference.
#include <cuda_runtime.h>

#include <mutex>
#include <string>

#include "purlin/moe_route.cuh"
#include "purlin/no_alloc.h"

namespace purlin { void setError(const std::string& e); }

namespace {

constexpr int kThreads = 256;
constexpr int kMaxDevices = 64;

// The scratch itself. In host code this name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) uint32_t g_routeCounters[PURLIN_NOALLOC_MAX_EXPERTS];

// one warp per token; the selection itself is the code the context-based routing kernel runs (moe_route.cuh)
template <int VPL>   // values per lane = experts / 32
__global__ void __launch_bounds__(kThreads) routeNoAllocKernel(const float* logits, int tokens, int experts, int topk, int normalize,
                                                               int32_t* topkIdx, float* topkWeight, int32_t* slot, uint32_t* counters) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= tokens) return;
  int myE; float myW;
  purlin::moe::routeToken<VPL>(logits + size_t(warp) * experts, experts, topk, normalize, lane, myE, myW);
  if (lane < topk) {
    topkIdx[size_t(warp) * topk + lane] = myE;
    topkWeight[size_t(warp) * topk + lane] = myW;
    slot[size_t(warp) * topk + lane] = int32_t(atomicAdd(counters + myE, 1u));
  }
}

// device address of g_routeCounters on each device, resolved on that device's first call
uint32_t* g_scratch[kMaxDevices] = {};
std::mutex g_mutex;

uint32_t* scratchFor(int device) {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_scratch[device] == nullptr) {
    // the caller's current device is `device`: the symbol resolves to that device's copy of the array
    uint32_t* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_routeCounters);
    if (e != cudaSuccess || p == nullptr) {
      purlin::setError(std::string("cudaGetSymbolAddress(route counters): ") + cudaGetErrorString(e));
      return nullptr;
    }
    g_scratch[device] = p;
  }
  return g_scratch[device];
}

}  // namespace

extern "C" int purlin_moe_route_noalloc(const float* logits, int tokens, int experts, int topk, int normalize,
                                        int32_t* topkIdx, float* topkWeight, int32_t* slot, void* stream) {
  if (experts <= 0 || experts % 32 != 0 || experts > PURLIN_NOALLOC_MAX_EXPERTS) {
    purlin::setError("purlin_moe_route_noalloc: experts must be a multiple of 32 and at most " +
                     std::to_string(PURLIN_NOALLOC_MAX_EXPERTS) + " (the size of the built-in scratch array)");
    return 1;
  }
  if (topk < 1 || topk > 8 || topk > experts) { purlin::setError("purlin_moe_route_noalloc: top-k must be 1..8"); return 1; }
  if (tokens < 0 || tokens > (1 << 26) || !logits || !topkIdx || !topkWeight || !slot) { purlin::setError("purlin_moe_route_noalloc: null argument"); return 1; }
  if (tokens == 0) return 0;
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess || device < 0 || device >= kMaxDevices) { purlin::setError("purlin_moe_route_noalloc: cannot identify the current device"); return 1; }
  uint32_t* counters = scratchFor(device);
  if (!counters) return 1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // the array keeps the previous call's counts: every call starts from zero
  e = cudaMemsetAsync(counters, 0, size_t(experts) * sizeof(uint32_t), s);
  if (e != cudaSuccess) { purlin::setError(std::string("purlin_moe_route_noalloc: clearing the counters: ") + cudaGetErrorString(e)); return 1; }
  const int blocks = (tokens * 32 + kThreads - 1) / kThreads;
  switch (experts / 32) {
    case 1: routeNoAllocKernel<1><<<blocks, kThreads, 0, s>>>(logits, tokens, experts, topk, normalize, topkIdx, topkWeight, slot, counters); break;
    case 2: routeNoAllocKernel<2><<<blocks, kThreads, 0, s>>>(logits, tokens, experts, topk, normalize, topkIdx, topkWeight, slot, counters); break;
    case 4: routeNoAllocKernel<4><<<blocks, kThreads, 0, s>>>(logits, tokens, experts, topk, normalize, topkIdx, topkWeight, slot, counters); break;
    case 8: routeNoAllocKernel<8><<<blocks, kThreads, 0, s>>>(logits, tokens, experts, topk, normalize, topkIdx, topkWeight, slot, counters); break;
    case 16: routeNoAllocKernel<16><<<blocks, kThreads, 0, s>>>(logits, tokens, experts, topk, normalize, topkIdx, topkWeight, slot, counters); break;
    default:
      purlin::setError("purlin_moe_route_noalloc: experts / 32 must be 1, 2, 4, 8 or 16");
      return 1;
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) { purlin::setError(std::string("purlin_moe_route_noalloc launch: ") + cudaGetErrorString(e)); return 1; }
  return 0;
}
