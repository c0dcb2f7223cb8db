// Expert-parallel MoE token exchange: routing, dispatch fused with the token permute, combine fused with the
// gate-weighted sum.
//
// The reference stops at allToAllV (csrc/include/purlin/host/all2all.cuh:293-319); a MoE layer built on it would
// permute tokens into per-destination order, exchange counts, run the variable-length all-to-all, permute again
// into expert order, and mirror all of that on the way back. Here each direction is ONE kernel over peer memory:
//
//   route     softmax over the gating logits, top-k, per-expert slot assignment           (local)
//   dispatch  counts travel to every rank as flagged stores; every CTA derives where each (token, expert) row
//             belongs in the receiver's expert-major buffer and the warps store the rows there directly over
//             NVLink: the permute IS the address computation. A last-arrival flag per destination tells the
//             receiver that all rows of this sender have landed.
//   combine   every rank reads the rows its tokens produced on the experts' GPUs (peer loads), multiplies by the
//             gate weights and accumulates the top-k contributions in fp32: one pass, no intermediate buffer.
//             The kernel ends with a "done reading" handshake so buffers can be reused by the next layer.
// Signalling uses the same primitives as the collectives (release/acquire flags in peer memory, bounded waits).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <string>

#include "purlin/atom.cuh"
#include "purlin/constants.hpp"
#include "purlin/moe.h"
#include "purlin/moe_route.cuh"
#include "purlin/signal.cuh"
#include "purlin/telemetry.hpp"

namespace purlin { void setError(const std::string& e); }
using namespace purlin;

struct PurlinMoeContext {
  int rank = 0, world = 1, maxTokens = 0, hidden = 0, experts = 0, topk = 0, capacityRows = 0;
  unsigned char* peers[kMaxRanks] = {};
  size_t recvOff = 0, outOff = 0, countsOff = 0, flagsOff = 0, total = 0;
  void* local = nullptr;
  uint64_t timeoutNs = 0;
};

namespace {

constexpr int kThreads = 256;
constexpr int kMaxExperts = 512;

struct MoeParams {
  int rank, world, tokens, hiddenBytes, experts, topk, expertsPerRank, capacityRows;
  const unsigned char* x;          // [tokens, hidden] bf16
  const int32_t* topkIdx;          // [tokens, topk]
  const float* topkWeight;         // [tokens, topk]
  const int32_t* slot;             // [tokens, topk] position of the row among this rank's rows of that expert
  const uint32_t* localCounts;     // [experts] rows this rank sends to each expert
  int32_t* sentRow;                // [tokens, topk] row index inside the destination's receive buffer
  int32_t* recvCounts;             // [expertsPerRank + 1] rows received per local expert, then their total
  unsigned char* recvBuf[kMaxRanks];   // every rank's expert-major receive buffer [capacityRows, hidden]
  unsigned char* outBuf[kMaxRanks];    // every rank's expert-output buffer [capacityRows, hidden]
  uint32_t* countsAll[kMaxRanks];      // every rank's copy of the count matrix [world][experts]
  uint64_t* flags[kMaxRanks];          // every rank's flags: [0,W) counts, [W,2W) rows landed, [2W,3W) outputs ready, [3W,4W) done reading
  unsigned char* y;                // combine output [tokens, hidden] bf16
  uint64_t* epoch;                 // device call counters: [0] dispatch, [1] combine
  uint32_t* exitCounter;
  uint32_t* pushCounters;          // [world] last-arrival counters
  uint32_t* status;
  uint64_t timeoutNs;
};

PURLIN_D bool waitFlag(const MoeParams& p, const uint64_t* flag, uint64_t value, uint32_t where, uint32_t peer) {
  if (sig::ldAcquireSys(flag) >= value) return true;
  const uint64_t start = sig::globalTimerNs();
  uint32_t spins = 0;
  while (sig::ldRelaxedSys(flag) < value) {
    if ((++spins & 63u) == 0u) {
      if (sig::ldRelaxedGpu32(p.status) != 0u) return false;
      if (sig::globalTimerNs() - start > p.timeoutNs) {
        if (atomicCAS(p.status, 0u, uint32_t(kStatusTimeoutTile)) == 0u) { p.status[1] = where; p.status[2] = peer; p.status[3] = 0; __threadfence(); }
        return false;
      }
    }
  }
  return sig::ldAcquireSys(flag) >= value;
}

// thread q < world waits on flags[base + q]; the CTA learns whether all arrived
PURLIN_D bool waitAllRanks(const MoeParams& p, int base, uint64_t value, uint32_t where) {
  int ok = 1;
  if (int(threadIdx.x) < p.world) ok = waitFlag(p, p.flags[p.rank] + base + threadIdx.x, value, where, threadIdx.x) ? 1 : 0;
  return __syncthreads_and(ok) != 0;
}

// ---------------------------------------------------------------------------------------------
// route: one warp per token
// ---------------------------------------------------------------------------------------------
template <int VPL>   // values per lane = experts / 32
__global__ void __launch_bounds__(kThreads) routeKernel(const float* logits, int tokens, int experts, int topk, int normalize,
                                                        int32_t* topkIdx, float* topkWeight, int32_t* slot, uint32_t* counts) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= tokens) return;
  int myE; float myW;     // lane k keeps the k-th choice; always a valid expert id (see moe_route.cuh)
  moe::routeToken<VPL>(logits + size_t(warp) * experts, experts, topk, normalize, lane, myE, myW);
  if (lane < topk) {
    topkIdx[size_t(warp) * topk + lane] = myE;
    topkWeight[size_t(warp) * topk + lane] = myW;
    slot[size_t(warp) * topk + lane] = int32_t(atomicAdd(counts + myE, 1u));
  }
}

// ---------------------------------------------------------------------------------------------
// dispatch
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads, 1) dispatchKernel(const __grid_constant__ MoeParams p) {
  __shared__ int32_t rowBase[kMaxExperts];      // first row of (this rank, expert e) inside the destination's buffer
  __shared__ int overflow;
  const uint64_t epoch = sig::ldRelaxedSys(p.epoch) + 1;
  const int tid = threadIdx.x;
  if (tid == 0) overflow = 0;

  // 1. publish this rank's counts on every rank (flagged stores; the flag is released after the data)
  if (blockIdx.x == 0) {
    for (int q = 0; q < p.world; ++q)
      for (int e = tid; e < p.experts; e += blockDim.x) p.countsAll[q][size_t(p.rank) * p.experts + e] = p.localCounts[e];
    __syncthreads();
    if (tid < p.world) sig::stReleaseSys(p.flags[tid] + p.rank, epoch);
  }
  // 2. everyone's counts are here
  const bool ok = waitAllRanks(p, 0, epoch, 1);
  // 3. where my rows go: expert-major on the destination, sources in rank order inside an expert
  const uint32_t* all = p.countsAll[p.rank];
  for (int e = tid; ok && e < p.experts; e += blockDim.x) {
    const int first = e / p.expertsPerRank * p.expertsPerRank;
    int base = 0;
    for (int e2 = first; e2 < e; ++e2)
      for (int s = 0; s < p.world; ++s) base += int(all[size_t(s) * p.experts + e2]);
    for (int s = 0; s < p.rank; ++s) base += int(all[size_t(s) * p.experts + e]);
    rowBase[e] = base;
  }
  // Capacity is judged on the whole count matrix, which every rank holds: if any destination would receive more rows
  // than its buffer has, every rank sees it, every rank reports it and nobody stores a row.
  if (ok && tid < p.world) {
    long total = 0;
    for (int e = tid * p.expertsPerRank; e < (tid + 1) * p.expertsPerRank; ++e)
      for (int s = 0; s < p.world; ++s) total += long(all[size_t(s) * p.experts + e]);
    if (total > long(p.capacityRows)) overflow = 1;
  }
  if (blockIdx.x == 0 && ok) {
    // what this rank receives: rows per local expert and their total
    for (int e = tid; e < p.expertsPerRank; e += blockDim.x) {
      int n = 0;
      for (int s = 0; s < p.world; ++s) n += int(all[size_t(s) * p.experts + p.rank * p.expertsPerRank + e]);
      p.recvCounts[e] = n;
    }
    if (tid == 0) {
      int total = 0;
      for (int e = 0; e < p.expertsPerRank; ++e)
        for (int s = 0; s < p.world; ++s) total += int(all[size_t(s) * p.experts + p.rank * p.expertsPerRank + e]);
      p.recvCounts[p.expertsPerRank] = total;
    }
  }
  __syncthreads();
  if (!ok) {
    // a rank never published its counts: nothing can be placed; the status word already says why
  } else if (overflow) {
    if (tid == 0 && atomicCAS(p.status, 0u, uint32_t(kStatusBadPlan)) == 0u) { p.status[1] = 2; __threadfence(); }
    if (blockIdx.x == 0) for (int e = tid; e <= p.expertsPerRank; e += blockDim.x) p.recvCounts[e] = 0;     // nothing was delivered
  } else {
    // 4. one warp per (token, choice): the row goes straight to its permuted place in the receiver's memory
    const int warp = tid >> 5, lane = tid & 31, warpsPerCta = blockDim.x >> 5;
    const int items = p.tokens * p.topk;
    const int vecs = p.hiddenBytes / 32;
    for (int item = blockIdx.x * warpsPerCta + warp; item < items; item += gridDim.x * warpsPerCta) {
      const int t = item / p.topk;
      const int e = p.topkIdx[item];
      if (e < 0 || e >= p.experts) {     // an id the caller supplied out of range: report it, store nothing
        if (lane == 0 && atomicCAS(p.status, 0u, uint32_t(kStatusBadPlan)) == 0u) { p.status[1] = 7; p.status[2] = uint32_t(item); __threadfence(); }
        continue;
      }
      const int dst = e / p.expertsPerRank;
      const int row = rowBase[e] + p.slot[item];
      if (lane == 0) p.sentRow[item] = row;
      const unsigned char* src = p.x + size_t(t) * p.hiddenBytes;
      unsigned char* out = p.recvBuf[dst] + size_t(row) * p.hiddenBytes;
      for (int i = lane; i < vecs; i += 32 * 8) {
        Vec32 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) if (i + u * 32 < vecs) v[u] = ld32(src + size_t(i + u * 32) * 32);
#pragma unroll
        for (int u = 0; u < 8; ++u) if (i + u * 32 < vecs) st32(out + size_t(i + u * 32) * 32, v[u]);
      }
    }
  }
  // 5. all of this rank's rows are on their way: the last CTA tells every destination
  __shared__ int lastCta;
  __syncthreads();
  if (tid == 0) lastCta = sig::lastArrival(p.pushCounters, gridDim.x) ? 1 : 0;
  __syncthreads();
  if (lastCta && tid < p.world) sig::stReleaseSys(p.flags[(p.rank + tid) % p.world] + p.world + p.rank, epoch);   // one peer per thread
  // 6. this rank's receive buffer is complete when every sender has said so
  if (blockIdx.x == 0 && ok) waitAllRanks(p, p.world, epoch, 3);
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(p.exitCounter, 1u) == gridDim.x - 1) { *p.exitCounter = 0; *p.epoch = epoch; __threadfence(); }
  }
}

// ---------------------------------------------------------------------------------------------
// combine
// ---------------------------------------------------------------------------------------------
PURLIN_D void fmaBf16x2(float& a0, float& a1, uint32_t w, float s) {
  a0 = fmaf(__uint_as_float(w << 16), s, a0);
  a1 = fmaf(__uint_as_float(w & 0xffff0000u), s, a1);
}

template <int TOPK>
__global__ void __launch_bounds__(kThreads, 1) combineKernel(const __grid_constant__ MoeParams p) {
  const uint64_t epoch = sig::ldRelaxedSys(p.epoch + 1) + 1;
  const int tid = threadIdx.x;
  // the expert outputs of this rank are complete (stream order): tell every rank, then wait for theirs
  if (blockIdx.x == 0 && tid < p.world) sig::stReleaseSys(p.flags[tid] + 2 * p.world + p.rank, epoch);
  bool ok = waitAllRanks(p, 2 * p.world, epoch, 4);
  if (ok) {
    const int warp = tid >> 5, lane = tid & 31, warpsPerCta = blockDim.x >> 5;
    const int vecs = p.hiddenBytes / 16;
    for (int t = blockIdx.x * warpsPerCta + warp; t < p.tokens; t += gridDim.x * warpsPerCta) {
      const unsigned char* rows[TOPK];
      float w[TOPK];
#pragma unroll
      for (int k = 0; k < TOPK; ++k) {
        const int item = t * TOPK + k;
        const int e = p.topkIdx[item];
        const int r = p.sentRow[item];
        const bool valid = e >= 0 && e < p.experts && r >= 0 && r < p.capacityRows;
        if (!valid && lane == 0 && atomicCAS(p.status, 0u, uint32_t(kStatusBadPlan)) == 0u) { p.status[1] = 8; p.status[2] = uint32_t(item); __threadfence(); }
        rows[k] = p.outBuf[valid ? e / p.expertsPerRank : p.rank] + size_t(valid ? r : 0) * p.hiddenBytes;
        w[k] = valid ? p.topkWeight[item] : 0.f;
      }
      unsigned char* out = p.y + size_t(t) * p.hiddenBytes;
      for (int i = lane; i < vecs; i += 32) {
        Vec16 v[TOPK];
#pragma unroll
        for (int k = 0; k < TOPK; ++k) v[k] = ld16(rows[k] + size_t(i) * 16);   // TOPK peer loads in flight per lane
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
        for (int k = 0; k < TOPK; ++k)
#pragma unroll
          for (int j = 0; j < 4; ++j) fmaBf16x2(acc[2 * j], acc[2 * j + 1], v[k].x[j], w[k]);
        Vec16 o;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const __nv_bfloat162 b = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
          o.x[j] = *reinterpret_cast<const uint32_t*>(&b);
        }
        st16(out + size_t(i) * 16, o);
      }
    }
  }
  // done reading everyone's outputs: the last CTA says so, then the call waits until every rank is done
  // reading this rank's buffers, so the next layer may overwrite them
  __shared__ int lastCta;
  __syncthreads();
  if (tid == 0) lastCta = sig::lastArrival(p.pushCounters + 1, gridDim.x) ? 1 : 0;
  __syncthreads();
  if (lastCta && tid < p.world) sig::stReleaseSys(p.flags[(p.rank + tid) % p.world] + 3 * p.world + p.rank, epoch);
  if (blockIdx.x == 0 && ok) waitAllRanks(p, 3 * p.world, epoch, 5);
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(p.exitCounter + 1, 1u) == gridDim.x - 1) { p.exitCounter[1] = 0; p.epoch[1] = epoch; __threadfence(); }
  }
}

struct MoeLayout { size_t recv, out, counts, flags, total; };
MoeLayout moeLayout(int world, int capacityRows, int hidden, int experts) {
  MoeLayout l{};
  size_t off = 0;
  const size_t buf = roundUp(size_t(capacityRows) * hidden * 2, 1024);
  l.recv = off; off += buf;
  l.out = off; off += buf;
  l.counts = off; off += roundUp(size_t(world) * experts * 4, 1024);
  l.flags = off; off += roundUp(size_t(4) * world * 8, 1024);
  l.total = off;
  return l;
}

int smCount() {
  int d = 0, v = 148;
  cudaGetDevice(&d);
  cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, d);
  return v;
}

void fillCommon(MoeParams& p, PurlinMoeContext* c, int tokens) {
  unsigned char* lb = static_cast<unsigned char*>(c->local);
  p.rank = c->rank; p.world = c->world; p.tokens = tokens; p.hiddenBytes = c->hidden * 2; p.experts = c->experts; p.topk = c->topk;
  p.expertsPerRank = c->experts / c->world; p.capacityRows = c->capacityRows;
  for (int q = 0; q < c->world; ++q) {
    p.recvBuf[q] = c->peers[q] + c->recvOff;
    p.outBuf[q] = c->peers[q] + c->outOff;
    p.countsAll[q] = reinterpret_cast<uint32_t*>(c->peers[q] + c->countsOff);
    p.flags[q] = reinterpret_cast<uint64_t*>(c->peers[q] + c->flagsOff);
  }
  p.epoch = reinterpret_cast<uint64_t*>(lb);
  p.exitCounter = reinterpret_cast<uint32_t*>(lb + 64);
  p.pushCounters = reinterpret_cast<uint32_t*>(lb + 128);
  p.status = reinterpret_cast<uint32_t*>(lb + 256);
  p.localCounts = reinterpret_cast<uint32_t*>(lb + 1024);
  p.timeoutNs = c->timeoutNs;
}

}  // namespace

extern "C" {

size_t purlin_moe_workspace_bytes(int world, int capacityRows, int hidden, int experts) { return moeLayout(world, capacityRows, hidden, experts).total; }

PurlinMoeContext* purlin_moe_create(int rank, int world, const uint64_t* peerPtrs, int maxTokens, int hidden, int experts, int topk,
                                    int capacityRows, uint64_t timeoutNs, void* stream) {
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world) { setError("invalid rank or world size"); return nullptr; }
  if (experts % world || experts % 32 || experts > kMaxExperts) { setError("experts must be a multiple of 32 and of the world size, at most 512"); return nullptr; }
  if (topk < 1 || topk > 8 || hidden % 16) { setError("top-k must be 1..8 and hidden a multiple of 16"); return nullptr; }
  auto* c = new PurlinMoeContext();
  c->rank = rank; c->world = world; c->maxTokens = maxTokens; c->hidden = hidden; c->experts = experts; c->topk = topk; c->capacityRows = capacityRows;
  const MoeLayout l = moeLayout(world, capacityRows, hidden, experts);
  c->recvOff = l.recv; c->outOff = l.out; c->countsOff = l.counts; c->flagsOff = l.flags; c->total = l.total;
  for (int q = 0; q < world; ++q) {
    if (!peerPtrs[q] || peerPtrs[q] % 1024) { delete c; setError("peer blocks must be non-null and 1024-byte aligned"); return nullptr; }
    c->peers[q] = reinterpret_cast<unsigned char*>(peerPtrs[q]);
  }
  c->timeoutNs = timeoutNs ? timeoutNs : 10ull * 1000 * 1000 * 1000;
  const size_t localBytes = 1024 + size_t(kMaxExperts) * 4;
  if (cudaMalloc(&c->local, localBytes) != cudaSuccess) { delete c; setError("cudaMalloc failed"); return nullptr; }
  cudaMemsetAsync(c->local, 0, localBytes, static_cast<cudaStream_t>(stream));
  cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  return c;
}

int purlin_moe_destroy(PurlinMoeContext* c, void* stream) {
  if (!c) return 0;
  cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (c->local) cudaFree(c->local);
  delete c;
  return 0;
}

int purlin_moe_status(PurlinMoeContext* c, uint32_t* out4, void* stream) {
  cudaMemcpyAsync(out4, static_cast<unsigned char*>(c->local) + 256, 16, cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
  return cudaStreamSynchronize(static_cast<cudaStream_t>(stream)) == cudaSuccess ? 0 : 1;
}
int purlin_moe_clear_status(PurlinMoeContext* c, void* stream) {
  return cudaMemsetAsync(static_cast<unsigned char*>(c->local) + 256, 0, 16, static_cast<cudaStream_t>(stream)) == cudaSuccess ? 0 : 1;
}
void* purlin_moe_recv_buffer(PurlinMoeContext* c) { return c->peers[c->rank] + c->recvOff; }
void* purlin_moe_out_buffer(PurlinMoeContext* c) { return c->peers[c->rank] + c->outOff; }

int purlin_moe_route(PurlinMoeContext* c, const float* logits, int tokens, int normalize, int32_t* topkIdx, float* topkWeight,
                     int32_t* slot, void* stream) {
  NvtxRange range("moeRoute", size_t(tokens));
  if (tokens < 0 || tokens > c->maxTokens || tokens > (1 << 26)) { setError("route: more tokens than the context was created for"); return 1; }
  if (tokens == 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint32_t* counts = reinterpret_cast<uint32_t*>(static_cast<unsigned char*>(c->local) + 1024);
  cudaMemsetAsync(counts, 0, size_t(c->experts) * 4, s);
  const int blocks = (tokens * 32 + kThreads - 1) / kThreads;
  switch (c->experts / 32) {
    case 1: routeKernel<1><<<blocks, kThreads, 0, s>>>(logits, tokens, c->experts, c->topk, normalize, topkIdx, topkWeight, slot, counts); break;
    case 2: routeKernel<2><<<blocks, kThreads, 0, s>>>(logits, tokens, c->experts, c->topk, normalize, topkIdx, topkWeight, slot, counts); break;
    case 4: routeKernel<4><<<blocks, kThreads, 0, s>>>(logits, tokens, c->experts, c->topk, normalize, topkIdx, topkWeight, slot, counts); break;
    case 8: routeKernel<8><<<blocks, kThreads, 0, s>>>(logits, tokens, c->experts, c->topk, normalize, topkIdx, topkWeight, slot, counts); break;
    case 16: routeKernel<16><<<blocks, kThreads, 0, s>>>(logits, tokens, c->experts, c->topk, normalize, topkIdx, topkWeight, slot, counts); break;
    default: setError("experts / 32 must be 1, 2, 4, 8 or 16"); return 1;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

int purlin_moe_dispatch(PurlinMoeContext* c, const void* x, int tokens, const int32_t* topkIdx, const int32_t* slot,
                        int32_t* sentRow, int32_t* recvCounts, int blocks, void* stream) {
  NvtxRange range("moeDispatch", size_t(tokens));
  if (tokens < 0 || tokens > c->maxTokens) { setError("dispatch: more tokens than the context was created for"); return 1; }
  MoeParams p{};
  fillCommon(p, c, tokens);
  p.x = static_cast<const unsigned char*>(x); p.topkIdx = topkIdx; p.slot = slot; p.sentRow = sentRow; p.recvCounts = recvCounts;
  if (blocks <= 0) blocks = smCount();
  dispatchKernel<<<std::min(blocks, smCount()), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { setError(std::string("dispatch launch: ") + cudaGetErrorString(e)); return 1; }
  return 0;
}

int purlin_moe_combine(PurlinMoeContext* c, void* y, int tokens, const int32_t* topkIdx, const float* topkWeight,
                       const int32_t* sentRow, int blocks, void* stream) {
  NvtxRange range("moeCombine", size_t(tokens));
  if (tokens < 0 || tokens > c->maxTokens) { setError("combine: more tokens than the context was created for"); return 1; }
  MoeParams p{};
  fillCommon(p, c, tokens);
  p.y = static_cast<unsigned char*>(y); p.topkIdx = topkIdx; p.topkWeight = topkWeight; p.sentRow = const_cast<int32_t*>(sentRow);
  if (blocks <= 0) blocks = smCount();
  blocks = std::min(blocks, smCount());
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (c->topk) {
    case 1: combineKernel<1><<<blocks, kThreads, 0, s>>>(p); break;
    case 2: combineKernel<2><<<blocks, kThreads, 0, s>>>(p); break;
    case 4: combineKernel<4><<<blocks, kThreads, 0, s>>>(p); break;
    case 6: combineKernel<6><<<blocks, kThreads, 0, s>>>(p); break;
    case 8: combineKernel<8><<<blocks, kThreads, 0, s>>>(p); break;
    default: setError("top-k must be 1, 2, 4, 6 or 8"); return 1;
  }
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { setError(std::string("combine launch: ") + cudaGetErrorString(e)); return 1; }
  return 0;
}

}  // extern "C"
