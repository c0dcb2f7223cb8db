// Symmetric-memory providers for the C++ API.
//
// A provider hands the library one zero-filled block of device memory per rank
// plus a mapping of every peer's block (and optionally an NVLS multicast alias
// of the same range). Parity: the SymmetricMemoryProvider concept of
// csrc/include/purlin/setup.cuh:126-134 and the provider contract of
// csrc/contrib/README.md in the reference. The reference ships an NVSHMEM
// provider; this build has no NVSHMEM dependency and ships:
//   EmulatedMemory  world blocks on one GPU (single-GPU emulation, tests, fault modes)
//   IpcMemory       CUDA IPC peer mappings; handles travel through a caller-supplied all-gather
//   VmmMemory       CUDA virtual-memory blocks with POSIX-fd handles and an NVLS multicast alias (vmm_provider.cu)
// The Python package adds the torch symmetric-memory provider.
#pragma once
#include <cuda_runtime.h>

#include <cstring>
#include <functional>
#include <stdexcept>
#include <string>
#include <vector>

#include "capi.h"
#include "constants.hpp"

namespace purlin {

struct SymmetricAllocation {
  std::vector<void*> peers;   // one pointer per rank; peers[rank] is local
  void* multicast = nullptr;  // NVLS alias of the block, or null
};

// What a provider must offer (C++17 spelling of the concept):
//   SymmetricAllocation allocate_zeroed(size_t bytes, size_t alignment, cudaStream_t stream);
//   void free(SymmetricAllocation&);
// allocate_zeroed is collective over the ranks and returns only when every rank's block is zero.
// A failure must surface on every rank (throw), so that no peer stays blocked.

enum class EmulatedFault { none, shortTable, nullPeer, unalignedPeer, multicast };

// All "ranks" live on the current GPU. Construct one per virtual rank with the same shared state.
class EmulatedMemory {
 public:
  struct Shared {
    int world = 0;
    std::vector<void*> blocks;
    size_t bytes = 0;
    int users = 0;
  };
  EmulatedMemory(Shared* shared, int world, EmulatedFault fault = EmulatedFault::none) : shared_(shared), fault_(fault) { shared_->world = world; }
  SymmetricAllocation allocate_zeroed(size_t bytes, size_t alignment, cudaStream_t stream) {
    if (shared_->blocks.empty()) {
      shared_->bytes = bytes;
      for (int q = 0; q < shared_->world; ++q) {
        void* p = nullptr;
        if (cudaMalloc(&p, bytes + alignment) != cudaSuccess) throw std::runtime_error("EmulatedMemory: cudaMalloc failed");
        cudaMemsetAsync(p, 0, bytes + alignment, stream);
        shared_->blocks.push_back(p);
      }
      cudaStreamSynchronize(stream);
    } else if (bytes != shared_->bytes) {
      throw std::invalid_argument("EmulatedMemory: every rank must ask for the same size");
    }
    ++shared_->users;
    SymmetricAllocation a;
    a.peers = shared_->blocks;
    switch (fault_) {
      case EmulatedFault::shortTable: a.peers.pop_back(); break;
      case EmulatedFault::nullPeer: a.peers.back() = nullptr; break;
      case EmulatedFault::unalignedPeer: a.peers.back() = static_cast<char*>(a.peers.back()) + 8; break;
      case EmulatedFault::multicast: a.multicast = a.peers[0]; break;   // a stand-in alias, for plumbing tests only
      default: break;
    }
    return a;
  }
  void free(SymmetricAllocation& a) {
    a.peers.clear();
    if (--shared_->users == 0) {
      for (void* p : shared_->blocks) cudaFree(p);
      shared_->blocks.clear();
    }
  }
 private:
  Shared* shared_;
  EmulatedFault fault_;
};

// One process per GPU. `allGather(sendBytes, recvBytes[world * n], n)` is supplied by the caller
// (MPI, a torch process group, a file store...) and `barrier()` likewise.
class IpcMemory {
 public:
  using AllGather = std::function<void(const void* send, void* recv, size_t bytesPerRank)>;
  using Barrier = std::function<void()>;
  IpcMemory(int rank, int world, AllGather ag, Barrier barrier) : rank_(rank), world_(world), ag_(std::move(ag)), barrier_(std::move(barrier)) {}
  SymmetricAllocation allocate_zeroed(size_t bytes, size_t /*alignment*/, cudaStream_t stream) {
    if (cudaMalloc(&local_, bytes) != cudaSuccess) throw std::runtime_error("IpcMemory: cudaMalloc failed");
    cudaMemsetAsync(local_, 0, bytes, stream);
    cudaStreamSynchronize(stream);
    cudaIpcMemHandle_t mine;
    if (cudaIpcGetMemHandle(&mine, local_) != cudaSuccess) throw std::runtime_error("IpcMemory: cudaIpcGetMemHandle failed");
    std::vector<cudaIpcMemHandle_t> all(world_);
    ag_(&mine, all.data(), sizeof(mine));
    SymmetricAllocation a;
    a.peers.resize(world_, nullptr);
    for (int q = 0; q < world_; ++q) {
      if (q == rank_) { a.peers[q] = local_; continue; }
      if (cudaIpcOpenMemHandle(&a.peers[q], all[q], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess)
        throw std::runtime_error("IpcMemory: cudaIpcOpenMemHandle failed for rank " + std::to_string(q));
    }
    barrier_();
    return a;
  }
  void free(SymmetricAllocation& a) {
    barrier_();   // nobody still reads this block
    for (int q = 0; q < int(a.peers.size()); ++q)
      if (q != rank_ && a.peers[q]) cudaIpcCloseMemHandle(a.peers[q]);
    if (local_) cudaFree(local_);
    local_ = nullptr;
    a.peers.clear();
  }
 private:
  int rank_, world_;
  AllGather ag_;
  Barrier barrier_;
  void* local_ = nullptr;
};

// One rank per GPU: separate processes, or the threads of one process. Memory comes from cuMemCreate, peers are
// mapped from exported descriptors, and when every rank's device supports it all blocks are bound to one multicast
// object whose mapping is returned as the NVLS alias. `allGather` and `barrier` as for IpcMemory.
class VmmMemory {
 public:
  using AllGather = std::function<void(const void* send, void* recv, size_t bytesPerRank)>;
  using Barrier = std::function<void()>;
  VmmMemory(int rank, int world, int device, AllGather ag, Barrier barrier, bool wantMulticast = true)
      : rank_(rank), world_(world), device_(device), ag_(std::move(ag)), barrier_(std::move(barrier)), wantMulticast_(wantMulticast) {}
  SymmetricAllocation allocate_zeroed(size_t bytes, size_t /*alignment*/, cudaStream_t /*stream*/) {
    block_ = purlin_vmm_create(device_, bytes, rank_, world_);
    // every rank reports success or failure before anyone proceeds, so that a failure surfaces everywhere
    struct Hello { int pid, fd, ok, multicast; } mine{0, -1, block_ ? 1 : 0, 0};
    if (block_) {
      purlin_vmm_local_handle(block_, &mine.pid, &mine.fd);
      mine.multicast = wantMulticast_ && world_ > 1 && purlin_vmm_multicast_supported(device_) == 1 ? 1 : 0;
    }
    std::vector<Hello> all(static_cast<size_t>(world_));
    ag_(&mine, all.data(), sizeof(Hello));
    bool ok = true, multicast = true;
    for (const Hello& h : all) { ok = ok && h.ok; multicast = multicast && h.multicast; }
    if (!ok) { release(); throw std::runtime_error(std::string("VmmMemory: allocation failed on some rank: ") + purlin_last_error()); }
    std::vector<int> pids, fds;
    for (const Hello& h : all) { pids.push_back(h.pid); fds.push_back(h.fd); }
    int good = purlin_vmm_map_peers(block_, pids.data(), fds.data()) == 0 ? 1 : 0;
    if (!agree(good)) { release(); throw std::runtime_error(std::string("VmmMemory: peer mapping failed on some rank: ") + purlin_last_error()); }
    if (multicast) {
      int handle[2] = {0, -1};
      int made = 1;
      if (rank_ == 0) made = purlin_vmm_multicast_create(block_, &handle[0], &handle[1]) == 0 ? 1 : 0;
      std::vector<int> handles(static_cast<size_t>(world_) * 2);
      ag_(handle, handles.data(), sizeof(handle));
      multicast = agree(made);                       // no object: carry on without the alias
      if (multicast) {
        good = purlin_vmm_multicast_join(block_, handles[0], handles[1]) == 0 ? 1 : 0;
        if (!agree(good)) { release(); throw std::runtime_error(std::string("VmmMemory: joining the multicast object failed: ") + purlin_last_error()); }
        good = purlin_vmm_multicast_bind(block_) == 0 ? 1 : 0;
        if (!agree(good)) { release(); throw std::runtime_error(std::string("VmmMemory: binding the multicast object failed: ") + purlin_last_error()); }
      }
    }
    barrier_();
    purlin_vmm_exchange_done();   // every rank has duplicated what it needs: close the descriptor-sharing window
    SymmetricAllocation a;
    for (int q = 0; q < world_; ++q) a.peers.push_back(reinterpret_cast<void*>(purlin_vmm_peer_ptr(block_, q)));
    a.multicast = reinterpret_cast<void*>(purlin_vmm_multicast_ptr(block_));
    return a;
  }
  void free(SymmetricAllocation& a) {
    barrier_();   // nobody still reads or writes this block
    if (block_) purlin_vmm_detach(block_);
    barrier_();   // every alias and peer mapping is gone before any block is released
    release();
    a.peers.clear();
    a.multicast = nullptr;
  }
 private:
  // true when every rank passed 1; doubles as a barrier
  bool agree(int mine) {
    std::vector<int> all(static_cast<size_t>(world_));
    ag_(&mine, all.data(), sizeof(int));
    for (int v : all) if (!v) return false;
    return true;
  }
  void release() { if (block_) { purlin_vmm_destroy(block_); block_ = nullptr; } }
  int rank_, world_, device_;
  AllGather ag_;
  Barrier barrier_;
  bool wantMulticast_;
  PurlinVmmBlock* block_ = nullptr;
};

}  // namespace purlin
