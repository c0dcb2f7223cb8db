// Native symmetric-memory provider on the CUDA virtual-memory API, with an NVLS multicast alias.
//
// Role of csrc/contrib/symm_mem.cuh:10-59 in the reference (allocate a symmetric block, map every peer's block,
// obtain the multicast alias, zero, synchronise), which the reference delegates to NVSHMEM. Here the same is built
// directly on the driver: cuMemCreate with a POSIX-fd shareable handle, cuMemMap of every peer's handle into this
// process, and a cuMulticast object that all ranks' blocks are bound to, whose mapping is the address the
// multimem.* instructions use. No NVSHMEM, no MPI: the handles travel through whatever all-gather the caller has
// (a torch process group, a socket, or shared memory between the threads of one process).
//
// Handles are file descriptors. A peer process duplicates them with pidfd_getfd (ranks of one job run as one
// user); within one process a plain dup suffices. Driver entry points are resolved at run time through
// cudaGetDriverEntryPoint, so the library does not link against libcuda.
//
// Collective protocol (the caller supplies the exchanges between the steps):
//   create  -> all-gather (pid, fd) -> map_peers
//   rank 0: multicast_create -> all-gather (pid, fd) -> multicast_join on every rank -> barrier ->
//   multicast_bind on every rank -> barrier.
// destroy must follow a barrier after the last kernel that touches peer memory.
#include <cuda.h>
#include <cuda_runtime.h>
#include <sys/prctl.h>

#include <cstdlib>
#include <sys/syscall.h>
#include <unistd.h>

#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#include "purlin/constants.hpp"

namespace purlin { void setError(const std::string& e); }

namespace {

struct Driver {
  decltype(&cuMemCreate) memCreate = nullptr;
  decltype(&cuMemRelease) memRelease = nullptr;
  decltype(&cuMemAddressReserve) addressReserve = nullptr;
  decltype(&cuMemAddressFree) addressFree = nullptr;
  decltype(&cuMemMap) memMap = nullptr;
  decltype(&cuMemUnmap) memUnmap = nullptr;
  decltype(&cuMemSetAccess) setAccess = nullptr;
  decltype(&cuMemGetAllocationGranularity) granularity = nullptr;
  decltype(&cuMemExportToShareableHandle) exportHandle = nullptr;
  decltype(&cuMemImportFromShareableHandle) importHandle = nullptr;
  decltype(&cuMulticastCreate) mcCreate = nullptr;
  decltype(&cuMulticastAddDevice) mcAddDevice = nullptr;
  decltype(&cuMulticastBindMem) mcBindMem = nullptr;
  decltype(&cuMulticastUnbind) mcUnbind = nullptr;
  decltype(&cuMulticastGetGranularity) mcGranularity = nullptr;
  decltype(&cuDeviceGetAttribute) deviceAttribute = nullptr;
  decltype(&cuGetErrorString) errorString = nullptr;
  bool ok = false;
};

template <class Fn>
bool resolve(Fn& fn, const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) return false;
  fn = reinterpret_cast<Fn>(p);
  return true;
}

const Driver& driver() {
  static const Driver d = [] {
    Driver x;
    x.ok = resolve(x.memCreate, "cuMemCreate") && resolve(x.memRelease, "cuMemRelease") &&
           resolve(x.addressReserve, "cuMemAddressReserve") && resolve(x.addressFree, "cuMemAddressFree") &&
           resolve(x.memMap, "cuMemMap") && resolve(x.memUnmap, "cuMemUnmap") && resolve(x.setAccess, "cuMemSetAccess") &&
           resolve(x.granularity, "cuMemGetAllocationGranularity") && resolve(x.exportHandle, "cuMemExportToShareableHandle") &&
           resolve(x.importHandle, "cuMemImportFromShareableHandle") && resolve(x.deviceAttribute, "cuDeviceGetAttribute") &&
           resolve(x.errorString, "cuGetErrorString");
    // multicast entry points are optional: an older driver simply has no NVLS alias
    const bool mc = resolve(x.mcCreate, "cuMulticastCreate") && resolve(x.mcAddDevice, "cuMulticastAddDevice") &&
                    resolve(x.mcBindMem, "cuMulticastBindMem") && resolve(x.mcUnbind, "cuMulticastUnbind") &&
                    resolve(x.mcGranularity, "cuMulticastGetGranularity");
    if (!mc) x.mcCreate = nullptr;
    return x;
  }();
  return d;
}

bool fail(const char* what, CUresult r) {
  const char* s = nullptr;
  if (driver().errorString) driver().errorString(r, &s);
  purlin::setError(std::string("vmm provider: ") + what + ": " + (s ? s : "unknown driver error"));
  return false;
}
#define DRV(call, what) do { CUresult r_ = (call); if (r_ != CUDA_SUCCESS) return fail(what, r_) ? 0 : 1; } while (0)

// duplicate a descriptor that lives in process `pid`
int adoptFd(int pid, int fd) {
  if (pid == int(getpid())) return dup(fd);
  const int pidfd = int(syscall(SYS_pidfd_open, pid, 0));
  if (pidfd < 0) return -1;
  const int mine = int(syscall(SYS_pidfd_getfd, pidfd, fd, 0));
  close(pidfd);
  return mine;
}

struct Mapping {
  CUmemGenericAllocationHandle handle = 0;
  CUdeviceptr va = 0;
  bool mapped = false;
};

}  // namespace

struct PurlinVmmBlock {
  int device = 0, rank = 0, world = 0;
  size_t bytes = 0;          // rounded up to the mapping granularity (the same on every rank)
  size_t align = 0;
  Mapping local;
  int localFd = -1;
  std::vector<Mapping> peers;
  CUmemGenericAllocationHandle mcHandle = 0;
  int mcFd = -1;
  bool mcJoined = false, mcBound = false;
  CUdeviceptr mcVa = 0;
  bool mcMapped = false;
};

namespace {

int mapHandle(const PurlinVmmBlock& b, Mapping& m) {
  const Driver& d = driver();
  DRV(d.addressReserve(&m.va, b.bytes, b.align, 0, 0), "cuMemAddressReserve");
  DRV(d.memMap(m.va, b.bytes, 0, m.handle, 0), "cuMemMap");
  m.mapped = true;
  CUmemAccessDesc acc{};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = b.device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  DRV(d.setAccess(m.va, b.bytes, &acc, 1), "cuMemSetAccess");
  return 0;
}

void unmapHandle(const PurlinVmmBlock& b, Mapping& m) {
  const Driver& d = driver();
  if (m.mapped) d.memUnmap(m.va, b.bytes);
  if (m.va) d.addressFree(m.va, b.bytes);
  if (m.handle) d.memRelease(m.handle);
  m = Mapping{};
}

CUmulticastObjectProp multicastProp(int world, size_t bytes) {
  CUmulticastObjectProp p{};
  p.numDevices = unsigned(world);
  p.size = bytes;
  p.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

}  // namespace

extern "C" {

// Ends the window in which peers may duplicate this process's descriptors: back to the kernel's default (ancestors
// only). Call on every rank after the barrier that follows mapping (and multicast binding).
int purlin_vmm_exchange_done(void) {
  if (std::getenv("PURLIN_VMM_NO_PTRACE_RELAX") == nullptr) prctl(PR_SET_PTRACER, 0, 0, 0, 0);
  return 0;
}

// 1 when the device and the driver offer NVLS multicast objects, 0 when not, -1 on error
int purlin_vmm_multicast_supported(int device) {
  const Driver& d = driver();
  if (!d.ok) { purlin::setError("vmm provider: the driver lacks the virtual-memory entry points"); return -1; }
  if (!d.mcCreate) return 0;
  int v = 0;
  if (d.deviceAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, device) != CUDA_SUCCESS) return 0;
  return v ? 1 : 0;
}

// Allocates this rank's zero-filled block on `device` (made current) and exports its handle.
PurlinVmmBlock* purlin_vmm_create(int device, size_t bytes, int rank, int world) {
  const Driver& d = driver();
  if (!d.ok) { purlin::setError("vmm provider: the driver lacks the virtual-memory entry points"); return nullptr; }
  if (world < 1 || world > purlin::kMaxRanks || rank < 0 || rank >= world || bytes == 0) { purlin::setError("vmm provider: invalid arguments"); return nullptr; }
  if (cudaSetDevice(device) != cudaSuccess || cudaFree(nullptr) != cudaSuccess) { purlin::setError("vmm provider: cannot use the device"); return nullptr; }
  // pidfd_getfd needs ptrace access to the exporting process. The relaxation lasts for the handle exchange only:
  // purlin_vmm_exchange_done() restores the default once every rank has mapped what it needs (after the barrier).
  // PURLIN_VMM_NO_PTRACE_RELAX=1 skips it altogether (for hosts where the ranks may read each other anyway).
  if (world > 1 && std::getenv("PURLIN_VMM_NO_PTRACE_RELAX") == nullptr) prctl(PR_SET_PTRACER, PR_SET_PTRACER_ANY, 0, 0, 0);
  auto* b = new PurlinVmmBlock;
  b->device = device; b->rank = rank; b->world = world;
  b->peers.resize(size_t(world));
  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 0;
  CUresult r = d.granularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
  if (r != CUDA_SUCCESS) { fail("cuMemGetAllocationGranularity", r); delete b; return nullptr; }
  if (world > 1 && purlin_vmm_multicast_supported(device) == 1) {
    // the multicast object wants its own granularity; every rank computes the same rounded size
    size_t mcGran = 0;
    CUmulticastObjectProp mp = multicastProp(world, bytes);
    if (d.mcGranularity(&mcGran, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mcGran > gran) gran = mcGran;
  }
  b->align = gran;
  b->bytes = (bytes + gran - 1) / gran * gran;
  r = d.memCreate(&b->local.handle, b->bytes, &prop, 0);
  if (r != CUDA_SUCCESS) { fail("cuMemCreate", r); delete b; return nullptr; }
  if (mapHandle(*b, b->local) != 0) { unmapHandle(*b, b->local); delete b; return nullptr; }
  if (cudaMemset(reinterpret_cast<void*>(b->local.va), 0, b->bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
    purlin::setError("vmm provider: zero-fill failed"); unmapHandle(*b, b->local); delete b; return nullptr;
  }
  r = d.exportHandle(&b->localFd, b->local.handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) { fail("cuMemExportToShareableHandle", r); unmapHandle(*b, b->local); delete b; return nullptr; }
  return b;
}

size_t purlin_vmm_bytes(const PurlinVmmBlock* b) { return b ? b->bytes : 0; }

// what this rank contributes to the all-gather of handles
int purlin_vmm_local_handle(const PurlinVmmBlock* b, int* pid, int* fd) {
  if (!b || b->localFd < 0) { purlin::setError("vmm provider: no exported handle"); return 1; }
  *pid = int(getpid());
  *fd = b->localFd;
  return 0;
}

// pids/fds: one entry per rank (the entry of this rank is ignored)
int purlin_vmm_map_peers(PurlinVmmBlock* b, const int* pids, const int* fds) {
  if (!b) { purlin::setError("vmm provider: null block"); return 1; }
  const Driver& d = driver();
  if (cudaSetDevice(b->device) != cudaSuccess) { purlin::setError("vmm provider: cannot use the device"); return 1; }
  for (int q = 0; q < b->world; ++q) {
    if (q == b->rank || b->peers[size_t(q)].mapped) continue;
    const int fd = adoptFd(pids[q], fds[q]);
    if (fd < 0) { purlin::setError("vmm provider: cannot duplicate the handle of rank " + std::to_string(q) + " (pidfd_getfd refused)"); return 1; }
    Mapping& m = b->peers[size_t(q)];
    const CUresult r = d.importHandle(&m.handle, reinterpret_cast<void*>(uintptr_t(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    close(fd);
    if (r != CUDA_SUCCESS) { fail("cuMemImportFromShareableHandle", r); return 1; }
    if (mapHandle(*b, m) != 0) return 1;
  }
  return 0;
}

uint64_t purlin_vmm_peer_ptr(const PurlinVmmBlock* b, int q) {
  if (!b || q < 0 || q >= b->world) return 0;
  return q == b->rank ? uint64_t(b->local.va) : uint64_t(b->peers[size_t(q)].va);
}

// Rank 0 creates the multicast object and exports it; its (pid, fd) is then broadcast to every rank.
int purlin_vmm_multicast_create(PurlinVmmBlock* b, int* pid, int* fd) {
  if (!b) { purlin::setError("vmm provider: null block"); return 1; }
  const Driver& d = driver();
  if (!d.mcCreate) { purlin::setError("vmm provider: multicast is not offered by this driver"); return 1; }
  if (cudaSetDevice(b->device) != cudaSuccess) { purlin::setError("vmm provider: cannot use the device"); return 1; }
  CUmulticastObjectProp mp = multicastProp(b->world, b->bytes);
  DRV(d.mcCreate(&b->mcHandle, &mp), "cuMulticastCreate");
  DRV(d.exportHandle(&b->mcFd, b->mcHandle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle (multicast)");
  *pid = int(getpid());
  *fd = b->mcFd;
  return 0;
}

// Every rank: import the object (rank 0 already holds it) and add this rank's device to it.
int purlin_vmm_multicast_join(PurlinVmmBlock* b, int pid, int fd) {
  if (!b) { purlin::setError("vmm provider: null block"); return 1; }
  const Driver& d = driver();
  if (!d.mcCreate) { purlin::setError("vmm provider: multicast is not offered by this driver"); return 1; }
  if (cudaSetDevice(b->device) != cudaSuccess) { purlin::setError("vmm provider: cannot use the device"); return 1; }
  if (!b->mcHandle) {
    const int mine = adoptFd(pid, fd);
    if (mine < 0) { purlin::setError("vmm provider: cannot duplicate the multicast handle (pidfd_getfd refused)"); return 1; }
    const CUresult r = d.importHandle(&b->mcHandle, reinterpret_cast<void*>(uintptr_t(mine)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    close(mine);
    if (r != CUDA_SUCCESS) { fail("cuMemImportFromShareableHandle (multicast)", r); return 1; }
  }
  DRV(d.mcAddDevice(b->mcHandle, b->device), "cuMulticastAddDevice");
  b->mcJoined = true;
  return 0;
}

// After every rank joined: bind this rank's block to the object and map the alias.
int purlin_vmm_multicast_bind(PurlinVmmBlock* b) {
  if (!b || !b->mcJoined) { purlin::setError("vmm provider: join the multicast object first"); return 1; }
  const Driver& d = driver();
  if (cudaSetDevice(b->device) != cudaSuccess) { purlin::setError("vmm provider: cannot use the device"); return 1; }
  DRV(d.mcBindMem(b->mcHandle, 0, b->local.handle, 0, b->bytes, 0), "cuMulticastBindMem");
  b->mcBound = true;
  DRV(d.addressReserve(&b->mcVa, b->bytes, b->align, 0, 0), "cuMemAddressReserve (multicast)");
  DRV(d.memMap(b->mcVa, b->bytes, 0, b->mcHandle, 0), "cuMemMap (multicast)");
  b->mcMapped = true;
  CUmemAccessDesc acc{};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = b->device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  DRV(d.setAccess(b->mcVa, b->bytes, &acc, 1), "cuMemSetAccess (multicast)");
  return 0;
}

uint64_t purlin_vmm_multicast_ptr(const PurlinVmmBlock* b) { return b && b->mcMapped ? uint64_t(b->mcVa) : 0; }

// First half of the release: drop the multicast alias and the peers' mappings. Every rank calls it (after the last
// kernel that touches peer memory has finished everywhere), then a barrier, then purlin_vmm_destroy.
int purlin_vmm_detach(PurlinVmmBlock* b) {
  if (!b) return 0;
  const Driver& d = driver();
  cudaSetDevice(b->device);
  cudaDeviceSynchronize();
  if (b->mcMapped) { d.memUnmap(b->mcVa, b->bytes); b->mcMapped = false; }
  if (b->mcVa) { d.addressFree(b->mcVa, b->bytes); b->mcVa = 0; }
  if (b->mcBound) { d.mcUnbind(b->mcHandle, b->device, 0, b->bytes); b->mcBound = false; }
  if (b->mcHandle) { d.memRelease(b->mcHandle); b->mcHandle = 0; }
  if (b->mcFd >= 0) { close(b->mcFd); b->mcFd = -1; }
  for (Mapping& m : b->peers) unmapHandle(*b, m);
  return 0;
}

int purlin_vmm_destroy(PurlinVmmBlock* b) {
  if (!b) return 0;
  purlin_vmm_detach(b);
  unmapHandle(*b, b->local);
  if (b->localFd >= 0) close(b->localFd);
  delete b;
  return 0;
}

}  // extern "C"
