// C++ host API: purlin::initialize / allReduce / allGather / reduceScatter / allToAll (alias all2all) and their
// variable-length forms / finalize.
//
// Parity: the public surface of csrc/include/purlin/host.cuh and setup.cuh:126-267 in the reference:
//   auto managed = purlin::initialize(rank, world, stream, Provider{...});
//   purlin::allReduce<__nv_bfloat16>(src, dst, bytes, managed.context(), stream);
//   purlin::finalize(managed, stream);
// The reference's functions are header-only templates over an ARCH parameter; this build targets sm_100a only,
// so ARCH is accepted and ignored, and the templates are thin wrappers over the C entry points of libpurlin_cuda
// (capi.h). One kernel launch per call, no host synchronisation, errors as exceptions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <memory>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <utility>
#include <vector>

#include "capi.h"
#include "constants.hpp"
#include "plan.hpp"
#include "provider.hpp"

namespace purlin {

namespace detail {
inline void check(int rc) { if (rc != 0) throw std::runtime_error(std::string("purlin: ") + purlin_last_error()); }
template <class T> constexpr DType dtypeOf() {
  if constexpr (std::is_same_v<T, __nv_bfloat16>) return DType::bf16;
  else if constexpr (std::is_same_v<T, __half>) return DType::fp16;
  else if constexpr (std::is_same_v<T, float>) return DType::fp32;
  else if constexpr (std::is_same_v<T, __nv_fp8_e4m3>) return DType::fp8e4m3;
  else if constexpr (std::is_same_v<T, __nv_fp8_e5m2>) return DType::fp8e5m2;
  else static_assert(sizeof(T) == 0, "unsupported element type");
}
}  // namespace detail

// A context the caller may pass around by reference; it does not own the symmetric memory.
class ContextRef {
 public:
  ContextRef() = default;
  explicit ContextRef(PurlinHostContext* h) : h_(h) {}
  PurlinHostContext* handle() const { return h_; }
  explicit operator bool() const { return h_ != nullptr; }
  bool hasMulticast() const { return h_ && purlin_context_has_multicast(h_) != 0; }
  // Synchronises the stream; throws if a bounded device wait gave up since the last check.
  void check(cudaStream_t stream) const {
    uint32_t st[4] = {0, 0, 0, 0};
    detail::check(purlin_context_status(h_, st, stream));
    if (st[0]) {
      purlin_context_clear_status(h_, stream);
      throw std::runtime_error("purlin: device wait timed out (code " + std::to_string(st[0]) + ", step " + std::to_string(st[1]) +
                               ", peer " + std::to_string(st[2]) + ", chunk " + std::to_string(st[3]) + ")");
    }
  }
 private:
  PurlinHostContext* h_ = nullptr;
};

// The symmetric block a caller already owns: one base pointer per rank (+ optional multicast alias).
struct WorkspaceMemory {
  std::vector<void*> peers;
  void* multicast = nullptr;
};

inline size_t workspaceBytes(int world, size_t stagingTRSize = kDefaultStagingBytes) {
  size_t ws[8];
  detail::check(purlin_workspace_layout(world, stagingTRSize, ws));
  return ws[6];
}

// Caller-owned memory: the returned context borrows it; finalize(ctx) frees only the library's local state.
inline ContextRef initialize(int rank, int world, const WorkspaceMemory& memory, cudaStream_t stream,
                             size_t stagingTRSize = kDefaultStagingBytes, uint64_t timeoutNs = 0) {
  if (int(memory.peers.size()) != world) throw std::invalid_argument("The provider must return one pointer per rank");
  std::vector<uint64_t> ptrs(world);
  for (int q = 0; q < world; ++q) ptrs[q] = reinterpret_cast<uint64_t>(memory.peers[q]);
  PurlinHostContext* h = purlin_context_create(rank, world, ptrs.data(), reinterpret_cast<uint64_t>(memory.multicast),
                                               stagingTRSize, timeoutNs, stream);
  if (!h) throw std::invalid_argument(std::string("purlin: ") + purlin_last_error());
  return ContextRef(h);
}
inline void finalize(ContextRef& ctx, cudaStream_t stream) {
  if (ctx) { purlin_context_destroy(ctx.handle(), stream); ctx = ContextRef(); }
}

// Owns the provider, its allocation and the context; releases them in the reverse order of creation.
template <class Provider>
class ManagedContext {
 public:
  ManagedContext() = default;
  ManagedContext(int rank, int world, cudaStream_t stream, Provider provider, size_t stagingTRSize = kDefaultStagingBytes)
      : state_(std::make_unique<State>(std::move(provider))) {
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world) throw std::invalid_argument("Invalid Purlin rank or world size");
    if (stagingTRSize < kMinChunkBytes || stagingTRSize > kMaxStagingBytes || stagingTRSize % kAccessAlign)
      throw std::invalid_argument("Invalid Purlin staging size");
    state_->stream = stream;
    state_->allocation = state_->provider.allocate_zeroed(workspaceBytes(world, stagingTRSize), kAccessAlign, stream);
    state_->allocated = true;
    WorkspaceMemory m;
    m.peers = state_->allocation.peers;
    m.multicast = state_->allocation.multicast;
    try {
      state_->ctx = initialize(rank, world, m, stream, stagingTRSize);
    } catch (...) {
      state_->provider.free(state_->allocation);
      state_->allocated = false;
      throw;
    }
  }
  ManagedContext(ManagedContext&&) noexcept = default;
  ManagedContext& operator=(ManagedContext&& o) noexcept { if (this != &o) { reset(); state_ = std::move(o.state_); } return *this; }
  ManagedContext(const ManagedContext&) = delete;
  ManagedContext& operator=(const ManagedContext&) = delete;
  ~ManagedContext() { reset(); }

  ContextRef& context() & {
    if (!state_) throw std::logic_error("The managed context is empty");
    return state_->ctx;
  }
  const ContextRef& context() const& {
    if (!state_) throw std::logic_error("The managed context is empty");
    return state_->ctx;
  }
  ContextRef& context() && = delete;
  bool empty() const { return !state_; }

  // Waits for work in flight on `stream`, frees the library's state, then the provider's memory.
  void reset(cudaStream_t stream) {
    if (!state_) return;
    finalize(state_->ctx, stream);
    if (state_->allocated) { state_->provider.free(state_->allocation); state_->allocated = false; }
    state_.reset();
  }
  void reset() { if (state_) reset(state_->stream); }

 private:
  struct State {
    explicit State(Provider p) : provider(std::move(p)) {}
    Provider provider;
    SymmetricAllocation allocation;
    bool allocated = false;
    ContextRef ctx;
    cudaStream_t stream = nullptr;
  };
  std::unique_ptr<State> state_;
};

template <class Provider>
ManagedContext<Provider> initialize(int rank, int world, cudaStream_t stream, Provider provider, size_t stagingTRSize = kDefaultStagingBytes) {
  return ManagedContext<Provider>(rank, world, stream, std::move(provider), stagingTRSize);
}
template <class Provider>
void finalize(ManagedContext<Provider>& managed, cudaStream_t stream) { managed.reset(stream); }

// ---- collectives. Byte conventions as in the reference: allReduce = whole payload; allGather = bytes per rank in;
// reduceScatter = bytes per rank out; allToAll = bytes per peer slice. Buffers and counts: multiples of 32 bytes.
template <class Element, ReduceOp Op = ReduceOp::add, ReductionMode Mode = ReductionMode::nonDeterministic>
void allReduce(const void* src, void* dst, size_t bytes, const ContextRef& ctx, cudaStream_t stream) {
  detail::check(purlin_all_reduce(ctx.handle(), src, dst, bytes, int(detail::dtypeOf<Element>()), int(Op), int(Mode), stream));
}
template <int ARCH, class Element, ReduceOp Op = ReduceOp::add, ReductionMode Mode = ReductionMode::nonDeterministic>
void allReduce(const void* src, void* dst, size_t bytes, const ContextRef& ctx, cudaStream_t stream) {
  allReduce<Element, Op, Mode>(src, dst, bytes, ctx, stream);
}
inline void allGather(const void* src, void* dst, size_t bytesPerRank, const ContextRef& ctx, cudaStream_t stream) {
  detail::check(purlin_all_gather(ctx.handle(), src, dst, bytesPerRank, stream));
}
inline void allGatherV(const void* src, void* dst, const std::vector<size_t>& bytesList, const ContextRef& ctx, cudaStream_t stream) {
  detail::check(purlin_all_gather_v(ctx.handle(), src, dst, bytesList.data(), stream));
}
template <class Element, ReduceOp Op = ReduceOp::add, ReductionMode Mode = ReductionMode::nonDeterministic>
void reduceScatter(const void* src, void* dst, size_t bytesPerRankOut, const ContextRef& ctx, cudaStream_t stream) {
  detail::check(purlin_reduce_scatter(ctx.handle(), src, dst, bytesPerRankOut, int(detail::dtypeOf<Element>()), int(Op), int(Mode), stream));
}
template <class Element, ReduceOp Op = ReduceOp::add, ReductionMode Mode = ReductionMode::nonDeterministic>
void reduceScatterV(const void* src, void* dst, const std::vector<size_t>& bytesList, const ContextRef& ctx, cudaStream_t stream) {
  detail::check(purlin_reduce_scatter_v(ctx.handle(), src, dst, bytesList.data(), int(detail::dtypeOf<Element>()), int(Op), int(Mode), stream));
}
inline void allToAll(const void* src, void* dst, size_t bytesPerPeer, const ContextRef& ctx, cudaStream_t stream) {
  detail::check(purlin_all_to_all(ctx.handle(), src, dst, bytesPerPeer, stream));
}
inline void allToAllV(const void* src, void* dst, const std::vector<size_t>& inSplits, const std::vector<size_t>& outSplits,
                      const ContextRef& ctx, cudaStream_t stream) {
  detail::check(purlin_all_to_all_v(ctx.handle(), src, dst, inSplits.data(), outSplits.data(), stream));
}
// the reference spells these all2all / all2allV
inline void all2all(const void* src, void* dst, size_t bytesPerPeer, const ContextRef& ctx, cudaStream_t stream) { allToAll(src, dst, bytesPerPeer, ctx, stream); }
inline void all2allV(const void* src, void* dst, const std::vector<size_t>& inSplits, const std::vector<size_t>& outSplits,
                     const ContextRef& ctx, cudaStream_t stream) { allToAllV(src, dst, inSplits, outSplits, ctx, stream); }

// run-time reduction mode -> template argument (csrc/include/purlin/host/reduction.cuh:8-25 in the reference)
template <class F>
decltype(auto) dispatchReductionMode(ReductionMode mode, F&& f) {
  if (mode == ReductionMode::deterministic) return f(std::integral_constant<ReductionMode, ReductionMode::deterministic>{});
  return f(std::integral_constant<ReductionMode, ReductionMode::nonDeterministic>{});
}

}  // namespace purlin
