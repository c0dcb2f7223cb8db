// Zero-copy all-reduce on tensors that already live in symmetric memory.
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

namespace purlin { void setError(const std::string& e); }
using namespace purlin;

namespace {

constexpr int kThreads = 256;

struct SymmParams {
  unsigned char* data[kMaxRanks];     // every rank's tensor
  unsigned char* mcData;              // multicast alias of the tensor, or null
  uint64_t* flags[kMaxRanks];         // every rank's flag block: [0,W) arrived, [W,2W) done; [2W] epoch; [2W+1] counters; [2W+2] status
  size_t bytes;
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

template <DType T, ReduceOp Op>
__global__ void __launch_bounds__(kThreads, 1) symmAllReduceKernel(const __grid_constant__ SymmParams p) {
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
  if (ok) {
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
template <DType T> Fn byOp(int op) {
  switch (ReduceOp(op)) {
    case ReduceOp::add: return symmAllReduceKernel<T, ReduceOp::add>;
    case ReduceOp::mul: return symmAllReduceKernel<T, ReduceOp::mul>;
    default: return symmAllReduceKernel<T, ReduceOp::max>;
  }
}

}  // namespace

extern "C" {

// bytes of the flag block that must accompany a symmetric tensor (zero-filled, symmetric, 32-byte aligned)
size_t purlin_symm_flag_bytes(int world) { return roundUp(size_t(2 * world + 4) * 8, 256); }

// In-place all-reduce of a symmetric tensor. dataPtrs / flagPtrs: one pointer per rank; multicastPtr: NVLS alias of the
// tensor or 0; mode 1 (deterministic) never uses the switch. Epoch and error status live in the flag block.
int purlin_symm_all_reduce(int rank, int world, const uint64_t* dataPtrs, uint64_t multicastPtr, const uint64_t* flagPtrs,
                           size_t bytes, int dtype, int reduceOp, int mode, int blocks, int mmDepth, uint64_t timeoutNs, void* stream) {
  if (world < 2 || world > kMaxRanks || rank < 0 || rank >= world) { setError("invalid rank or world size"); return 1; }
  if (bytes == 0) return 0;
  if (bytes % kAccessAlign) { setError("byte count must be a multiple of 32"); return 1; }
  SymmParams p{};
  for (int q = 0; q < world; ++q) {
    if (!dataPtrs[q] || dataPtrs[q] % kAccessAlign || !flagPtrs[q] || flagPtrs[q] % 8) { setError("symmetric pointers must be non-null and aligned"); return 1; }
    p.data[q] = reinterpret_cast<unsigned char*>(dataPtrs[q]);
    p.flags[q] = reinterpret_cast<uint64_t*>(flagPtrs[q]);
  }
  // Two ranks: the switch path moves 1.5 x the payload into every GPU (its own broadcast comes back through the link),
  // plain peer loads and stores move 1.0 x. Measured on 2 x B200 at 256 MiB: 670 us through the switch, 410 us without.
  const bool viaSwitch = multicastPtr != 0 && mode != int(ReductionMode::deterministic) && world > 2;
  p.mcData = viaSwitch ? reinterpret_cast<unsigned char*>(multicastPtr) : nullptr;
  p.bytes = bytes; p.rank = rank; p.world = world; p.mmDepth = mmDepth > 0 ? mmDepth : 8;
  p.timeoutNs = timeoutNs ? timeoutNs : 10ull * 1000 * 1000 * 1000;
  static const bool fusedPair = [] { const char* e = std::getenv("PURLIN_SYMM_FUSED_PAIR"); return !e || e[0] != '0'; }();
  p.fusedPair = fusedPair ? 1 : 0;
  Fn fn;
  switch (DType(dtype)) {
    case DType::bf16: fn = byOp<DType::bf16>(reduceOp); break;
    case DType::fp16: fn = byOp<DType::fp16>(reduceOp); break;
    case DType::fp8e4m3: fn = byOp<DType::fp8e4m3>(reduceOp); break;
    case DType::fp8e5m2: fn = byOp<DType::fp8e5m2>(reduceOp); break;
    default: fn = byOp<DType::fp32>(reduceOp); break;
  }
  // remote loads need many CTAs in flight to fill a link; the switch path saturates with fewer
  if (blocks <= 0) {
    if (viaSwitch) blocks = bytes >= (8u << 20) ? 96 : bytes >= (1u << 20) ? 48 : 16;
    else blocks = bytes >= (2u << 20) ? kMaxCtas : bytes >= (256u << 10) ? 64 : 16;
  }
  blocks = std::min(std::max(blocks, 1), kMaxCtas);
  fn<<<blocks, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { setError(std::string("symmetric all-reduce launch: ") + cudaGetErrorString(e)); return 1; }
  return 0;
}

}  // extern "C"
