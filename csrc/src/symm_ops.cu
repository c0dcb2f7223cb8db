// Zero-copy all-reduce, reduce-scatter and all-gather on tensors that already live in symmetric memory.
//
// The general all-reduce (collectives.cu) accepts any device pointer, so it must copy the input into the symmetric
// staging buffer and the result back out: four extra passes over local HBM around the NVLink phase. When the caller
// allocates the tensor through the symmetric-memory provider (purlin_b200.symm_empty), those passes disappear: every
// rank lets the NVSwitch reduce its shard straight out of all ranks' tensors (multimem.ld_reduce) and broadcasts the
// result straight back into them (multimem.st), in place. Without a multicast alias the same kernel reads the shard
// from every peer with plain loads (ascending rank order, fp32 accumulation) and stores the result to every peer.
// The reference has no such entry point (its collectives always stage: csrc/include/purlin/snac.cuh:237-373); the
// provider abstraction it defines (setup.cuh:126-134) is what makes this one possible.
//
// reduce-scatter reads the rank's shard of every peer's input tensor (through the switch or with peer loads) straight
// into an ordinary local output; all-gather pushes the rank's slice into every peer's tensor in place (multimem.st, or
// one plain store per peer). Both skip the staging pass the general collectives need for arbitrary pointers.
//
// Protocol: flag words live in a small symmetric block next to the tensor. barrier-in (everyone's input is complete),
// reduce + broadcast of this rank's shard, barrier-out (everyone's shard has landed everywhere). Waits are bounded.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>
#include <string>

#include "purlin/atom.cuh"
#include "purlin/constants.hpp"
#include "purlin/plan.hpp"
#include "purlin/signal.cuh"
#include "purlin/telemetry.hpp"

namespace purlin { void setError(const std::string& e); }
using namespace purlin;

namespace {

constexpr int kThreads = 256;

struct SymmParams {
  unsigned char* data[kMaxRanks];     // every rank's tensor
  unsigned char* mcData;              // multicast alias of the tensor, or null
  uint64_t* flags[kMaxRanks];         // every rank's flag block: [0,W) arrived, [W,2W) done; [2W] epoch; [2W+1] counters; [2W+2] status
  unsigned char* out;                 // reduce-scatter: ordinary local output
  size_t bytes;                       // all-reduce: whole tensor; reduce-scatter / all-gather: bytes per rank
  int rank, world, mmDepth;
  int fusedPair;                      // two ranks: the reduce loop stores its result locally and to the peer in one pass
  uint64_t timeoutNs;
};

PURLIN_D bool waitFlag(const SymmParams& p, const uint64_t* flag, uint64_t value) {
  if (sig::ldAcquireSys(flag) >= value) return true;
  uint32_t* status = reinterpret_cast<uint32_t*>(p.flags[p.rank] + 2 * p.world + 2);
  const uint64_t start = sig::globalTimerNs();
  uint32_t spins = 0;
  while (sig::ldRelaxedSys(flag) < value) {
    if ((++spins & 63u) == 0u) {
      if (sig::ldRelaxedGpu32(status) != 0u) return false;
      if (sig::globalTimerNs() - start > p.timeoutNs) { atomicCAS(status, 0u, uint32_t(kStatusTimeoutSignal)); return false; }
    }
  }
  return sig::ldAcquireSys(flag) >= value;
}

enum { kSymmAllReduce = 0, kSymmReduceScatter = 1, kSymmAllGather = 2 };

template <DType T, ReduceOp Op, int Kind>
__global__ void __launch_bounds__(kThreads, 1) symmKernel(const __grid_constant__ SymmParams p) {
  __shared__ const unsigned char* peers[kMaxRanks];
  __shared__ int lastCta;
  uint64_t* mine = p.flags[p.rank];
  const uint64_t epoch = sig::ldRelaxedSys(mine + 2 * p.world) + 1;
  const int tid = threadIdx.x;
  // barrier-in: this rank's tensor is complete (stream order); tell everyone, wait for everyone
  if (blockIdx.x == 0 && tid < p.world) sig::stReleaseSys(p.flags[tid] + p.rank, epoch);
  int ok = 1;
  if (tid < p.world) ok = waitFlag(p, mine + tid, epoch) ? 1 : 0;
  ok = __syncthreads_and(ok);
  if (ok && Kind == kSymmReduceScatter) {
    // this rank's shard of every rank's input -> local output; inputs are only read
    const Span part = partitionAligned(p.bytes, gridDim.x, blockIdx.x, kAccessAlign);
    const size_t off = size_t(p.rank) * p.bytes + part.offset;
    ReduceArgs a;
    a.world = p.world;
    a.bytes = part.bytes;
    a.dst = p.out + part.offset;
    bool viaSwitch = false;
    if constexpr (MultimemReducible<T, Op>::value) viaSwitch = p.mcData != nullptr && part.bytes % 16 == 0;
    if (viaSwitch) {
      a.mcSrc = p.mcData + off;
    } else {
      if (tid < p.world) peers[tid] = p.data[tid] + off;
      __syncthreads();
      a.srcs = peers;
    }
    if (part.bytes) AtomSm100<>::reduce<T, Op>(a, p.mmDepth);
  } else if (ok && Kind == kSymmAllGather) {
    // this rank's slice -> the same slice of every peer's tensor (own copy is already in place)
    const Span part = partitionAligned(p.bytes, gridDim.x, blockIdx.x, kAccessAlign);
    const size_t off = size_t(p.rank) * p.bytes + part.offset;
    const unsigned char* src = p.data[p.rank] + off;
    if (part.bytes && p.mcData != nullptr && part.bytes % 16 == 0) {
      const size_t n = part.bytes / 16, nt = blockDim.x;
      size_t i = tid;
      for (; i + 3 * nt < n; i += 4 * nt) {      // four loads in flight per thread, then four broadcast stores
        Vec16 v[4];
#pragma unroll
        for (int d = 0; d < 4; ++d) v[d] = ld16(src + (i + size_t(d) * nt) * 16);
#pragma unroll
        for (int d = 0; d < 4; ++d) multimemSt(p.mcData + off + (i + size_t(d) * nt) * 16, v[d]);
      }
      for (; i < n; i += nt) multimemSt(p.mcData + off + i * 16, ld16(src + i * 16));
    } else if (part.bytes) {
      for (int q = 1; q < p.world; ++q) {
        const int peer = (p.rank + q) % p.world;
        AtomSm100<>::copy(p.data[peer] + off, src, part.bytes, 8);
      }
    }
    __threadfence_system();
  } else if (ok) {
    const Span shard = partitionAligned(p.bytes, p.world, p.rank, kAccessAlign);
    const Span part = partitionAligned(shard.bytes, gridDim.x, blockIdx.x, kAccessAlign);
    const size_t off = shard.offset + part.offset;
    ReduceArgs a;
    a.world = p.world;
    a.bytes = part.bytes;
    bool viaSwitch = false;
    if constexpr (MultimemReducible<T, Op>::value) viaSwitch = p.mcData != nullptr && part.bytes % 16 == 0;
    if (viaSwitch) {
      a.mcSrc = p.mcData + off;
      a.mcSeam = p.mcData + off;                 // in place, on every rank at once
      if (part.bytes) AtomSm100<>::reduce<T, Op>(a, p.mmDepth);
    } else {
      if (tid < p.world) peers[tid] = p.data[tid] + off;
      __syncthreads();
      a.srcs = peers;
      a.dst = p.data[p.rank] + off;              // reduce once into own tensor (ranks touch disjoint shards) ...
      const bool fused = p.fusedPair && p.world == 2;
      if (fused) a.seam = p.data[p.rank ^ 1] + off;   // ... and, with a single peer, into the peer's tensor in the same pass
      if (part.bytes) AtomSm100<>::reduce<T, Op>(a, p.mmDepth);
      __syncthreads();
      for (int q = 1; q < p.world && !fused; ++q) {   // ... then store that slice into every peer's tensor
        const int peer = (p.rank + q) % p.world;
        if (part.bytes) AtomSm100<>::copy(p.data[peer] + off, p.data[p.rank] + off, part.bytes, 8);
      }
    }
    __threadfence_system();
  }
  // barrier-out: the last CTA of this rank says "my shard is everywhere"; the call ends when all ranks said so
  __syncthreads();
  uint32_t* counter = reinterpret_cast<uint32_t*>(mine + 2 * p.world + 1);
  if (tid == 0) lastCta = sig::lastArrival(counter, gridDim.x) ? 1 : 0;
  __syncthreads();
  if (lastCta && tid < p.world) sig::stReleaseSys(p.flags[(p.rank + tid) % p.world] + p.world + p.rank, epoch);
  if (blockIdx.x == 0 && ok) {
    if (tid < p.world) waitFlag(p, mine + p.world + tid, epoch);
    __syncthreads();
  }
  if (lastCta && tid == 0) { sig::stRelaxedSys(mine + 2 * p.world, epoch); __threadfence(); }
}

using Fn = void (*)(const SymmParams);
template <DType T, int Kind> Fn byOp(int op) {
  switch (ReduceOp(op)) {
    case ReduceOp::add: return symmKernel<T, ReduceOp::add, Kind>;
    case ReduceOp::mul: return symmKernel<T, ReduceOp::mul, Kind>;
    default: return symmKernel<T, ReduceOp::max, Kind>;
  }
}
template <int Kind> Fn byType(int dtype, int op) {
  switch (DType(dtype)) {
    case DType::bf16: return byOp<DType::bf16, Kind>(op);
    case DType::fp16: return byOp<DType::fp16, Kind>(op);
    case DType::fp8e4m3: return byOp<DType::fp8e4m3, Kind>(op);
    case DType::fp8e5m2: return byOp<DType::fp8e5m2, Kind>(op);
    default: return byOp<DType::fp32, Kind>(op);
  }
}

bool fillParams(SymmParams& p, int rank, int world, const uint64_t* dataPtrs, const uint64_t* flagPtrs, size_t bytes, int mmDepth, uint64_t timeoutNs) {
  if (world < 2 || world > kMaxRanks || rank < 0 || rank >= world) { setError("invalid rank or world size"); return false; }
  if (bytes % kAccessAlign) { setError("byte count must be a multiple of 32"); return false; }
  for (int q = 0; q < world; ++q) {
    if (!dataPtrs[q] || dataPtrs[q] % kAccessAlign || !flagPtrs[q] || flagPtrs[q] % 8) { setError("symmetric pointers must be non-null and aligned"); return false; }
    p.data[q] = reinterpret_cast<unsigned char*>(dataPtrs[q]);
    p.flags[q] = reinterpret_cast<uint64_t*>(flagPtrs[q]);
  }
  p.bytes = bytes; p.rank = rank; p.world = world; p.mmDepth = mmDepth > 0 ? mmDepth : 8;
  p.timeoutNs = timeoutNs ? timeoutNs : 10ull * 1000 * 1000 * 1000;
  return true;
}

int launchSymm(Fn fn, const SymmParams& p, int blocks, const char* what, void* stream) {
  blocks = std::min(std::max(blocks, 1), kMaxCtas);
  fn<<<blocks, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { setError(std::string(what) + " launch: " + cudaGetErrorString(e)); return 1; }
  return 0;
}

}  // namespace

extern "C" {

// bytes of the flag block that must accompany a symmetric tensor (zero-filled, symmetric, 32-byte aligned)
size_t purlin_symm_flag_bytes(int world) { return roundUp(size_t(2 * world + 4) * 8, 256); }

// In-place all-reduce of a symmetric tensor. dataPtrs / flagPtrs: one pointer per rank; multicastPtr: NVLS alias of the
// tensor or 0; mode 1 (deterministic) never uses the switch. Epoch and error status live in the flag block.
int purlin_symm_all_reduce(int rank, int world, const uint64_t* dataPtrs, uint64_t multicastPtr, const uint64_t* flagPtrs,
                           size_t bytes, int dtype, int reduceOp, int mode, int blocks, int mmDepth, uint64_t timeoutNs, void* stream) {
  NvtxRange range("symmAllReduce", bytes);
  SymmParams p{};
  if (!fillParams(p, rank, world, dataPtrs, flagPtrs, bytes, mmDepth, timeoutNs)) return 1;
  if (bytes == 0) return 0;
  // Two ranks: the switch path moves 1.5 x the payload into every GPU (its own broadcast comes back through the link),
  // plain peer loads and stores move 1.0 x. Measured on 2 x B200 at 256 MiB: 670 us through the switch, 410 us without.
  const bool viaSwitch = multicastPtr != 0 && mode != int(ReductionMode::deterministic) && world > 2;
  p.mcData = viaSwitch ? reinterpret_cast<unsigned char*>(multicastPtr) : nullptr;
  static const bool fusedPair = [] { const char* e = std::getenv("PURLIN_SYMM_FUSED_PAIR"); return !e || e[0] != '0'; }();
  p.fusedPair = fusedPair ? 1 : 0;
  // remote loads need many CTAs in flight to fill a link; the switch path saturates with fewer
  if (blocks <= 0) {
    if (viaSwitch) blocks = bytes >= (8u << 20) ? 96 : bytes >= (1u << 20) ? 48 : 16;
    else blocks = bytes >= (2u << 20) ? kMaxCtas : bytes >= (256u << 10) ? 64 : 16;
  }
  return launchSymm(byType<kSymmAllReduce>(dtype, reduceOp), p, blocks, "symmetric all-reduce", stream);
}

// Reduce-scatter out of symmetric input tensors: every rank's tensor holds world x bytesPerRank; rank r receives the
// reduction of slice r of all of them in `out` (any local device pointer). The call ends only when every rank has
// finished reading, so the inputs may be overwritten as soon as it returns in stream order.
int purlin_symm_reduce_scatter(int rank, int world, const uint64_t* dataPtrs, uint64_t multicastPtr, const uint64_t* flagPtrs,
                               void* out, size_t bytesPerRank, int dtype, int reduceOp, int mode, int blocks, int mmDepth,
                               uint64_t timeoutNs, void* stream) {
  NvtxRange range("symmReduceScatter", bytesPerRank);
  SymmParams p{};
  if (!fillParams(p, rank, world, dataPtrs, flagPtrs, bytesPerRank, mmDepth, timeoutNs)) return 1;
  if (bytesPerRank == 0) return 0;
  if (!out || reinterpret_cast<uintptr_t>(out) % kAccessAlign) { setError("the output must be a 32-byte aligned device pointer"); return 1; }
  // through the switch a rank receives only the reduced slice (1/world of what peer loads bring in); with two ranks
  // the switch reduction is slower than loading the one peer slice (445 us against 299 us staged at 2 x 128 MiB)
  const bool viaSwitch = multicastPtr != 0 && mode != int(ReductionMode::deterministic) && world > 2;
  p.mcData = viaSwitch ? reinterpret_cast<unsigned char*>(multicastPtr) : nullptr;
  p.out = static_cast<unsigned char*>(out);
  if (blocks <= 0) {
    if (viaSwitch) blocks = bytesPerRank >= (8u << 20) ? 96 : bytesPerRank >= (1u << 20) ? 48 : 16;
    else blocks = bytesPerRank >= (2u << 20) ? kMaxCtas : bytesPerRank >= (256u << 10) ? 64 : 16;
  }
  return launchSymm(byType<kSymmReduceScatter>(dtype, reduceOp), p, blocks, "symmetric reduce-scatter", stream);
}

// In-place all-gather of a symmetric tensor of world x bytesPerRank: rank r's slice r goes to slice r of every rank.
// viaSwitch > 0: one multimem.st per 16 bytes (the switch replicates); 0 or < 0: one plain store per peer, which is
// also the built-in choice: measured at 2 and 4 x B200 the plain stores are faster at every size (332 us against 400 us
// for 4 x 64 MiB), the switch sends every rank its own slice back through its link.
int purlin_symm_all_gather(int rank, int world, const uint64_t* dataPtrs, uint64_t multicastPtr, const uint64_t* flagPtrs,
                           size_t bytesPerRank, int viaSwitch, int blocks, uint64_t timeoutNs, void* stream) {
  NvtxRange range("symmAllGather", bytesPerRank);
  SymmParams p{};
  if (!fillParams(p, rank, world, dataPtrs, flagPtrs, bytesPerRank, 0, timeoutNs)) return 1;
  if (bytesPerRank == 0) return 0;
  const bool sw = multicastPtr != 0 && viaSwitch > 0;
  p.mcData = sw ? reinterpret_cast<unsigned char*>(multicastPtr) : nullptr;
  if (blocks <= 0) blocks = bytesPerRank >= (8u << 20) ? 64 : bytesPerRank >= (1u << 20) ? 32 : 8;   // remote stores fill a link with few CTAs
  return launchSymm(byType<kSymmAllGather>(int(DType::fp32), int(ReduceOp::add)), p, blocks, "symmetric all-gather", stream);
}

}  // extern "C"
