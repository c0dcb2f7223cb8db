// Expert-parallel MoE token exchange: routing, dispatch fused with the token permute, combine fused with the
// gate-weighted sum. Every token crosses NVLink ONCE per destination GPU, whatever number of that GPU's experts it
// was routed to.
//
// The reference stops at allToAllV (csrc/include/purlin/host/all2all.cuh:293-319); a MoE layer built on it would
// permute tokens into per-destination order, exchange counts, run the variable-length all-to-all, permute again
// into expert order, and mirror all of that on the way back. Here each direction is ONE kernel over peer memory:
//
//   route     softmax over the gating logits and top-k (moe_route.cuh), then a plan step: the slot of every
//             (token, expert) pair among this rank's rows of that expert, and one position per (token, destination
//             GPU) in that destination's send list                                                          (local)
//   dispatch  counts travel to every rank as flagged stores. Sender CTAs walk the send lists in chunks of 64 rows:
//             a token's row is stored once into the destination's staging area together with a 64-byte record that
//             names its rows in the destination's expert-major buffer and its gate weights; the chunk's flag is
//             released when its rows are on their way. Receiver CTAs of the same kernel wait on those chunk flags
//             and copy every staged row to its expert rows (local HBM traffic): the permute is that address
//             computation. Rows for this rank's own experts skip the staging area.
//   combine   pusher CTAs on the experts' GPU form, for every staged row, the gate-weighted sum of its expert
//             outputs (fp32) and store ONE row into the token's home GPU, chunk flags as above; finisher CTAs on
//             the home GPU add the rows of a token's destinations as their chunks arrive.
//
// Buffer reuse needs no extra handshake as long as dispatch and combine alternate on one stream (they are two halves
// of a layer): a rank writes into a peer's staging or combine buffers only after it has seen that peer's counts of the
// same dispatch, which the peer publishes after its previous combine has finished (stream order). Both kernels check
// the alternation on the device and report kStatusBadPlan instead of running out of order.
// Signalling uses the same primitives as the collectives (release/acquire flags in peer memory, bounded waits).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
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
  int rank = 0, world = 1, maxTokens = 0, hidden = 0, experts = 0, topk = 0, capacityRows = 0, maxChunks = 0;
  unsigned char* peers[kMaxRanks] = {};
  size_t stageOff = 0, metaOff = 0, recvOff = 0, outOff = 0, cbufOff = 0, countsOff = 0, flagsOff = 0, total = 0;
  void* local = nullptr;
  size_t sendListOff = 0, posOff = 0, countsLocalOff = 0;
  const int32_t* topkIdx = nullptr;      // routing of the current layer (device pointers the caller owns)
  const float* topkWeight = nullptr;
  const int32_t* slot = nullptr;
  uint64_t timeoutNs = 0;
  bool timing = false;                   // PURLIN_MOE_TIMING=1: the kernels stamp their phases (purlin_moe_timing)
};

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kDispatchCtasPerSm = 2;   // the dispatch is bound by memory latency and light on registers: two CTAs of eight warps per SM
constexpr int kCombineCtasPerSm = 1;    // the weighted sums keep 8 x 32 bytes per lane in flight and need the registers
constexpr int kMaxExperts = 512;
constexpr int kChunkRows = 64;          // rows per flag
constexpr int kRecvRows = 16;           // rows per receiver item of the dispatch (a part of a chunk)
constexpr int kMetaWords = 16;          // per staged row: 8 destination rows, 8 gate weights

struct MoeParams {
  int rank, world, tokens, maxTokens, hiddenBytes, experts, topk, expertsPerRank, capacityRows, maxChunks, senders;
  const unsigned char* x;          // [tokens, hidden] bf16
  const int32_t* topkIdx;          // [tokens, topk]
  const float* topkWeight;         // [tokens, topk]
  const int32_t* slot;             // [tokens, topk] position of the row among this rank's rows of that expert
  const int32_t* pos;              // [tokens, topk] position of the token in the send list of that expert's GPU
  const int32_t* sendList;         // [world][maxTokens] token ids in position order
  const uint32_t* localCounts;     // [experts + world] rows per expert, then distinct tokens per destination rank
  int32_t* sentRow;                // optional output [tokens, topk]: row inside the destination's expert-major buffer
  int32_t* recvCounts;             // [expertsPerRank + 1] rows received per local expert, then their total
  unsigned char* stage[kMaxRanks];     // every rank's staging area [world sources][maxTokens][hidden]
  int32_t* meta[kMaxRanks];            // every rank's records [world sources][maxTokens][16]
  unsigned char* cbuf[kMaxRanks];      // every rank's combine buffer [world expert ranks][maxTokens][hidden]
  unsigned char* recvBuf;              // this rank's expert-major receive buffer [capacityRows, hidden]
  unsigned char* outBuf;               // this rank's expert-output buffer [capacityRows, hidden]
  uint32_t* countsAll[kMaxRanks];      // every rank's copy of the count matrix [world][experts + world]
  uint64_t* flags[kMaxRanks];          // every rank's flags: [0, W) counts; then [W][maxChunks] dispatch chunks; then [W][maxChunks] combine chunks
  unsigned char* y;                // combine output [tokens, hidden] bf16
  uint64_t* epoch;                 // device call counters: [0] dispatch, [1] combine
  uint32_t* exitCounter;
  uint32_t* work;                  // next item of {dispatch senders, dispatch receivers, combine pushers}; the last CTA out clears them
  unsigned long long* timing;      // optional (PURLIN_MOE_TIMING=1): per kernel {first start, last sender end, last receiver end, first sender end} in ns
  uint32_t* status;
  uint64_t timeoutNs;
};

PURLIN_D void reportBad(const MoeParams& p, uint32_t where, uint32_t detail) {
  if (atomicCAS(p.status, 0u, uint32_t(kStatusBadPlan)) == 0u) { p.status[1] = where; p.status[2] = detail; p.status[3] = 0; __threadfence(); }
}

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

PURLIN_D uint64_t* dispatchFlag(const MoeParams& p, int onRank, int src, int chunk) { return p.flags[onRank] + p.world + size_t(src) * p.maxChunks + chunk; }
PURLIN_D uint64_t* combineFlag(const MoeParams& p, int onRank, int from, int chunk) { return p.flags[onRank] + p.world + size_t(p.world + from) * p.maxChunks + chunk; }

// Device-side phase times of one kernel (diagnostics; off unless the context was created with PURLIN_MOE_TIMING=1):
// every CTA folds its start and the end of its role into four words with atomics.
PURLIN_D void stampStart(const MoeParams& p, int base) {
  if (p.timing && threadIdx.x == 0) atomicMin(p.timing + base, (unsigned long long)sig::globalTimerNs());
}
PURLIN_D void stampEnd(const MoeParams& p, int base, bool sender) {
  if (p.timing && threadIdx.x == 0) {
    const unsigned long long now = sig::globalTimerNs();
    atomicMax(p.timing + base + (sender ? 1 : 2), now);
    if (sender) atomicMin(p.timing + base + 3, now);
  }
}

// ---------------------------------------------------------------------------------------------
// route: one warp per token
// ---------------------------------------------------------------------------------------------
template <int VPL>   // values per lane = experts / 32
__global__ void __launch_bounds__(kThreads) routeKernel(const float* logits, int tokens, int experts, int topk, int normalize,
                                                        int32_t* topkIdx, float* topkWeight) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= tokens) return;
  int myE; float myW;     // lane k keeps the k-th choice; always a valid expert id (see moe_route.cuh)
  moe::routeToken<VPL>(logits + size_t(warp) * experts, experts, topk, normalize, lane, myE, myW);
  if (lane < topk) {
    topkIdx[size_t(warp) * topk + lane] = myE;
    topkWeight[size_t(warp) * topk + lane] = myW;
  }
}

// plan: slots per expert, one send-list position per (token, destination rank). One warp per token.
// An expert id outside [0, experts) (possible when the caller supplies the routing) is reported and the pair dropped.
__global__ void __launch_bounds__(kThreads) planKernel(const int32_t* topkIdx, int tokens, int maxTokens, int experts, int topk, int expertsPerRank,
                                                       int32_t* slot, int32_t* pos, int32_t* sendList, uint32_t* counts, uint32_t* status) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= tokens) return;
  int e = -1;
  if (lane < topk) {
    e = topkIdx[size_t(warp) * topk + lane];
    if (e < 0 || e >= experts) {
      if (atomicCAS(status, 0u, uint32_t(kStatusBadPlan)) == 0u) { status[1] = 7; status[2] = uint32_t(warp); status[3] = uint32_t(lane); __threadfence(); }
      e = -1;
    }
  }
  const int dst = e >= 0 ? e / expertsPerRank : -1 - lane;            // inactive lanes get values nobody shares
  const unsigned same = __match_any_sync(0xffffffffu, dst);
  const int leader = __ffs(same) - 1;
  int p = -1;
  if (e >= 0 && lane == leader) {
    p = int(atomicAdd(counts + experts + dst, 1u));
    sendList[size_t(dst) * maxTokens + p] = warp;
  }
  p = __shfl_sync(0xffffffffu, p, leader);
  if (lane < topk) {
    slot[size_t(warp) * topk + lane] = e >= 0 ? int32_t(atomicAdd(counts + e, 1u)) : -1;
    pos[size_t(warp) * topk + lane] = e >= 0 ? p : -1;
  }
}

// copy one row (hiddenBytes, a multiple of 32) with the whole warp, 8 accesses in flight per lane
PURLIN_D void copyRow(unsigned char* dst, const unsigned char* src, int vecs, int lane) {
  for (int i = lane; i < vecs; i += 32 * 8) {
    Vec32 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) if (i + u * 32 < vecs) v[u] = ld32(src + size_t(i + u * 32) * 32);
#pragma unroll
    for (int u = 0; u < 8; ++u) if (i + u * 32 < vecs) st32(dst + size_t(i + u * 32) * 32, v[u]);
  }
}

// ---------------------------------------------------------------------------------------------
// dispatch
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads, kDispatchCtasPerSm) dispatchKernel(const __grid_constant__ MoeParams p) {
  __shared__ int32_t rowBase[kMaxExperts];      // first row of (this rank, expert e) inside the destination's buffer
  __shared__ int32_t colTotal[kMaxExperts];     // rows of expert e over all ranks
  __shared__ int32_t sendCount[kMaxRanks], recvFrom[kMaxRanks];
  __shared__ int bad, nextItem;
  const uint64_t epoch = sig::ldRelaxedSys(p.epoch) + 1;
  stampStart(p, 0);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int W = p.world, stride = p.experts + W;
  if (tid == 0) bad = 0;
  __syncthreads();
  // dispatch n may only follow combine n - 1; a call out of order does nothing and is not counted
  const bool outOfOrder = sig::ldRelaxedSys(p.epoch + 1) + 1 != epoch;
  if (outOfOrder && tid == 0) { bad = 1; reportBad(p, 9, 0); }

  // 1. publish this rank's counts on every rank (flagged stores; the flag is released after the data)
  if (blockIdx.x == 0 && !outOfOrder) {
    for (int q = 0; q < W; ++q)
      for (int e = tid; e < stride; e += blockDim.x) p.countsAll[q][size_t(p.rank) * stride + e] = p.localCounts[e];
    __syncthreads();
    if (tid < W) sig::stReleaseSys(p.flags[tid] + p.rank, epoch);
  }
  // 2. everyone's counts are here
  int okI = outOfOrder ? 0 : 1;
  if (!outOfOrder && tid < W) okI = waitFlag(p, p.flags[p.rank] + tid, epoch, 1, tid) ? 1 : 0;
  bool ok = __syncthreads_and(okI) != 0;
  // 3. where my rows go: expert-major on the destination, sources in rank order inside an expert
  const uint32_t* all = p.countsAll[p.rank];
  int before = 0;
  for (int e = tid; ok && e < p.experts; e += blockDim.x) {
    int tot = 0;
    for (int s = 0; s < W; ++s) { const int c = int(all[size_t(s) * stride + e]); tot += c; if (s < p.rank) before += c; }
    colTotal[e] = tot;
  }
  if (ok && tid < W) { sendCount[tid] = int(p.localCounts[p.experts + tid]); recvFrom[tid] = int(all[size_t(tid) * stride + p.experts + p.rank]); }
  __syncthreads();
  for (int e = tid; ok && e < p.experts; e += blockDim.x) {
    // (with experts <= blockDim.x a thread owns one expert, so `before` belongs to e; with more it is recomputed)
    int b = 0;
    if (p.experts > int(blockDim.x)) { for (int s = 0; s < p.rank; ++s) b += int(all[size_t(s) * stride + e]); } else b = before;
    const int first = e / p.expertsPerRank * p.expertsPerRank;
    for (int e2 = first; e2 < e; ++e2) b += colTotal[e2];
    rowBase[e] = b;
  }
  // Capacity is judged on the whole count matrix, which every rank holds: if any destination would receive more rows
  // than its buffer has, every rank sees it, every rank reports it and nobody stores a row.
  if (ok && tid < W) {
    long total = 0;
    for (int e = tid * p.expertsPerRank; e < (tid + 1) * p.expertsPerRank; ++e) total += long(colTotal[e]);
    if (total > long(p.capacityRows)) { bad = 1; reportBad(p, 2, uint32_t(tid)); }
    if (sendCount[tid] > p.maxTokens || recvFrom[tid] > p.maxTokens) { bad = 1; reportBad(p, 3, uint32_t(tid)); }
  }
  __syncthreads();
  if (blockIdx.x == 0 && ok) {
    // what this rank receives: rows per local expert and their total
    for (int e = tid; e < p.expertsPerRank; e += blockDim.x) p.recvCounts[e] = bad ? 0 : colTotal[p.rank * p.expertsPerRank + e];
    if (tid == 0) {
      int total = 0;
      for (int e = 0; e < p.expertsPerRank; ++e) total += colTotal[p.rank * p.expertsPerRank + e];
      p.recvCounts[p.expertsPerRank] = bad ? 0 : total;
    }
  }
  const int vecs = p.hiddenBytes / 32;
  const size_t rowBytes = size_t(p.hiddenBytes);
  if (ok && !bad) {
    const int senders = W == 1 ? 0 : (p.senders < int(gridDim.x) ? p.senders : int(gridDim.x) - 1);
    // the rows and gate weights of token t on rank d, as lanes 0..7 (rows) and 8..15 (weights) of a 16-word record
    auto recordOf = [&](int t, int d, int& row) {
      row = -1; float w = 0.f;
      if (lane < p.topk) {
        const int e = p.topkIdx[size_t(t) * p.topk + lane];
        if (e >= 0 && e < p.experts && e / p.expertsPerRank == d) {
          row = rowBase[e] + p.slot[size_t(t) * p.topk + lane];
          w = p.topkWeight[size_t(t) * p.topk + lane];
          if (p.sentRow) p.sentRow[size_t(t) * p.topk + lane] = row;
        }
      }
      const int wBits = __shfl_sync(0xffffffffu, __float_as_int(w), lane & 7);
      return lane < 8 ? row : (lane < 16 && (lane - 8) < p.topk ? wBits : 0);
    };
    // Items (a chunk of one peer's list) are handed out through a counter, in list order: a CTA that finishes early takes
    // the next one, so the CTAs of a role end together whatever the number of items per CTA would have been (with a
    // static split of 174 items over 32 CTAs the last CTA ran a fifth longer than the first, and everybody waited).
    // `want` is the same in every thread of the CTA and only grows, so the walk over the items below is done once.
    auto grab = [&](uint32_t* counter) {
      __syncthreads();
      if (tid == 0) nextItem = int(atomicAdd(counter, 1u));
      __syncthreads();
      return nextItem;
    };
    if (int(blockIdx.x) < senders) {
      // 4a. sender: chunks of the send lists of the other ranks, destinations interleaved so that every link is busy.
      // A token's row crosses NVLink once per destination, with the record that tells the receiver where it belongs.
      int item = 0, want = grab(p.work + 0);
      for (int c = 0; c < p.maxChunks; ++c) {
        for (int dd = 0; dd + 1 < W; ++dd) {
          const int d = (p.rank + 1 + dd) % W;
          if (c * kChunkRows >= sendCount[d]) continue;
          if (item++ != want) continue;
          const int end = min((c + 1) * kChunkRows, sendCount[d]);
          for (int pp = c * kChunkRows + warp; pp < end; pp += kWarps) {
            const int t = p.sendList[size_t(d) * p.maxTokens + pp];
            int row;
            const int rec = recordOf(t, d, row);
            if (lane < kMetaWords) p.meta[d][(size_t(p.rank) * p.maxTokens + pp) * kMetaWords + lane] = rec;
            copyRow(p.stage[d] + (size_t(p.rank) * p.maxTokens + pp) * rowBytes, p.x + size_t(t) * rowBytes, vecs, lane);
          }
          want = grab(p.work + 0);      // (its first barrier also orders the rows before the flag)
          // the release waits for this CTA's remote stores; only thread 0's warp waits with it
          if (tid == 0) sig::stReleaseSys(dispatchFlag(p, d, p.rank, c), epoch);
        }
      }
    } else {
      // 4b. receiver: every row that belongs on this rank goes to its expert rows (local traffic). Rows of this rank's
      // own tokens come straight from x; a peer's rows are copied out of the staging area as its chunks land.
      int item = 0, want = grab(p.work + 1);
      for (int c = 0; c < p.maxChunks && ok; ++c) {
        for (int ss = 0; ss < W && ok; ++ss) {
          const int s = (p.rank + W - ss) % W;          // own rows first, then the rank that serves this one first
          const int count = s == p.rank ? sendCount[s] : recvFrom[s];
          if (c * kChunkRows >= count) continue;
          // A receiver's item is a part of a chunk (kRecvRows rows, two per warp): a whole chunk per CTA left most CTAs
          // without work (4096 local rows are 64 chunks for 296 CTAs) and made the last chunk to land a 50 us tail.
          for (int part = 0; part < kChunkRows / kRecvRows && ok; ++part) {
            const int begin = c * kChunkRows + part * kRecvRows;
            if (begin >= count) break;
            if (item++ != want) continue;
            if (s != p.rank) {
              int good = 1;
              if (tid == 0) good = waitFlag(p, dispatchFlag(p, p.rank, s, c), epoch, 3, s) ? 1 : 0;
              ok = __syncthreads_and(good) != 0;
              if (!ok) break;
            }
            const int end = min(begin + kRecvRows, count);
            for (int pp = begin + warp; pp < end; pp += kWarps) {
              const size_t at = size_t(s) * p.maxTokens + pp;
              int row;
              const unsigned char* src;
              if (s == p.rank) {
                const int t = p.sendList[size_t(s) * p.maxTokens + pp];
                const int rec = recordOf(t, s, row);
                if (lane < kMetaWords) p.meta[s][at * kMetaWords + lane] = rec;      // the combine reads it like a peer's
                src = p.x + size_t(t) * rowBytes;
              } else {
                row = lane < 8 ? p.meta[p.rank][at * kMetaWords + lane] : -1;
                src = p.stage[p.rank] + at * rowBytes;
              }
              // the row is read once and written to each of its expert rows
              unsigned char* dst[8];
              unsigned mask = 0;
  #pragma unroll
              for (int k = 0; k < 8; ++k) {
                const int r = __shfl_sync(0xffffffffu, row, k);
                const bool valid = r >= 0 && r < p.capacityRows;
                dst[k] = p.recvBuf + size_t(valid ? r : 0) * rowBytes;
                if (valid) mask |= 1u << k;
              }
              for (int i = lane; i < vecs; i += 32 * 8) {
                Vec32 v[8];
  #pragma unroll
                for (int u = 0; u < 8; ++u) if (i + u * 32 < vecs) v[u] = ld32(src + size_t(i + u * 32) * 32);
  #pragma unroll
                for (int k = 0; k < 8; ++k)
                  if ((mask >> k) & 1u) {
  #pragma unroll
                    for (int u = 0; u < 8; ++u) if (i + u * 32 < vecs) st32(dst[k] + size_t(i + u * 32) * 32, v[u]);
                  }
              }
            }
            want = grab(p.work + 1);
          }
        }
      }
    }
  }
  __syncthreads();
  stampEnd(p, 0, p.world > 1 && int(blockIdx.x) < (p.senders < int(gridDim.x) ? p.senders : int(gridDim.x) - 1));
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(p.exitCounter, 1u) == gridDim.x - 1) { *p.exitCounter = 0; p.work[0] = 0; p.work[1] = 0; if (!outOfOrder) *p.epoch = epoch; __threadfence(); }
  }
}

// ---------------------------------------------------------------------------------------------
// combine
// ---------------------------------------------------------------------------------------------
PURLIN_D void fmaBf16x2(float& a0, float& a1, uint32_t w, float s) {
  a0 = fmaf(__uint_as_float(w << 16), s, a0);
  a1 = fmaf(__uint_as_float(w & 0xffff0000u), s, a1);
}
PURLIN_D uint32_t packBf16x2(float lo, float hi) {
  const __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&b);
}

// out = sum of w[k] * rows[k] over the first n of R rows (fp32 accumulate). 32-byte accesses, P positions of every row
// in flight per lane: R x P = 8 loads of 32 bytes, whatever the number of rows, because the sum is latency-bound
// otherwise (16 in flight spilled).
// n is the same in every lane, so the branches are uniform and the arrays stay in registers. rowBytes % 32 == 0.
template <int R, int P>
PURLIN_D void weightedSum(unsigned char* out, const unsigned char* const (&rows)[8], const float (&w)[8], int n, int vecs32, int lane) {
  for (int i = lane; i < vecs32; i += 32 * P) {
    Vec32 v[P][R];
#pragma unroll
    for (int h = 0; h < P; ++h)
#pragma unroll
      for (int k = 0; k < R; ++k)
        if (k < n && i + 32 * h < vecs32) v[h][k] = ld32(rows[k] + size_t(i + 32 * h) * 32);
#pragma unroll
    for (int h = 0; h < P; ++h) {
      if (i + 32 * h >= vecs32) break;
      float acc[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) acc[j] = 0.f;
#pragma unroll
      for (int k = 0; k < R; ++k)
        if (k < n) {
#pragma unroll
          for (int j = 0; j < 8; ++j) fmaBf16x2(acc[2 * j], acc[2 * j + 1], v[h][k].x[j], w[k]);
        }
      Vec32 o;
#pragma unroll
      for (int j = 0; j < 8; ++j) o.x[j] = packBf16x2(acc[2 * j], acc[2 * j + 1]);
      st32(out + size_t(i + 32 * h) * 32, o);
    }
  }
}
// the rows of a sum arrive in arbitrary lanes; few rows take many positions each, many rows few
PURLIN_D void weightedSumAny(unsigned char* out, const unsigned char* const (&rows)[8], const float (&w)[8], int n, int vecs32, int lane) {
  if (n <= 2) weightedSum<2, 4>(out, rows, w, n, vecs32, lane);
  else if (n <= 4) weightedSum<4, 2>(out, rows, w, n, vecs32, lane);
  else weightedSum<8, 1>(out, rows, w, n, vecs32, lane);
}

__global__ void __launch_bounds__(kThreads, kCombineCtasPerSm) combineKernel(const __grid_constant__ MoeParams p) {
  __shared__ int32_t recvFrom[kMaxRanks];
  __shared__ int bad, nextItem;
  const uint64_t epoch = sig::ldRelaxedSys(p.epoch + 1) + 1;
  stampStart(p, 4);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int W = p.world, stride = p.experts + W;
  if (tid == 0) bad = 0;
  __syncthreads();
  // combine n follows dispatch n; a call out of order does nothing and is not counted
  const bool outOfOrder = sig::ldRelaxedSys(p.epoch) != epoch;
  if (outOfOrder && tid == 0) { bad = 1; reportBad(p, 10, 0); }
  if (tid < W) recvFrom[tid] = int(p.countsAll[p.rank][size_t(tid) * stride + p.experts + p.rank]);
  __syncthreads();
  const bool ok = __syncthreads_and(!bad && sig::ldRelaxedGpu32(p.status) == 0u) != 0;   // one answer for the whole CTA: the roles below hold barriers
  const int vecs32 = p.hiddenBytes / 32;
  const size_t rowBytes = size_t(p.hiddenBytes);
  const int senders = p.senders < int(gridDim.x) ? p.senders : int(gridDim.x) - 1;
  if (ok && int(blockIdx.x) < senders) {
    // A. pusher: for every row staged here by rank s, the gate-weighted sum of its expert outputs goes home as ONE row.
    // Items (one chunk of one source) are handed out through a counter in chunk order: the pushers end together, and the
    // chunks complete in the order in which the finishers at home need them (a static split of 232 items over 98 CTAs
    // had the last pusher end at 313 us and the first at 187 us, and left a third of the finishers' work for the end).
    auto grab = [&]() {
      __syncthreads();
      if (tid == 0) nextItem = int(atomicAdd(p.work + 2, 1u));
      __syncthreads();
      return nextItem;
    };
    int item = 0, want = grab();
    for (int c = 0; c < p.maxChunks; ++c) {
      for (int ss = 0; ss < W; ++ss) {
        const int s = (p.rank + 1 + ss) % W;
        if (c * kChunkRows >= recvFrom[s]) continue;
        if (item++ != want) continue;
        const int end = min((c + 1) * kChunkRows, recvFrom[s]);
        for (int pp = c * kChunkRows + warp; pp < end; pp += kWarps) {
          const size_t at = size_t(s) * p.maxTokens + pp;
          const int rec = lane < kMetaWords ? p.meta[p.rank][at * kMetaWords + lane] : 0;
          // lanes 0..7 hold the expert-output rows of this staged row, lanes 8..15 their gate weights; the valid ones are
          // gathered to the front (j-th valid row = the lane of the j-th set bit)
          const bool mine = lane < 8 && rec >= 0 && rec < p.capacityRows;
          const unsigned valid = __ballot_sync(0xffffffffu, mine) & 0xffu;
          const int n = __popc(valid);
          const unsigned char* rows[8];
          float w[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int from = j < n ? int(__fns(valid, 0, j + 1)) : 0;
            const int r = __shfl_sync(0xffffffffu, rec, from);
            w[j] = __int_as_float(__shfl_sync(0xffffffffu, rec, 8 + from));
            rows[j] = p.outBuf + size_t(j < n ? r : 0) * rowBytes;
          }
          weightedSumAny(p.cbuf[s] + (size_t(p.rank) * p.maxTokens + pp) * rowBytes, rows, w, n, vecs32, lane);
        }
        want = grab();                  // (its first barrier also orders the rows before the flag)
        if (tid == 0) sig::stReleaseSys(combineFlag(p, s, p.rank, c), epoch);
      }
    }
  } else if (ok) {
    // B. finisher: a token's result is the sum of one row per destination GPU, added as their chunks arrive
    const int nFin = int(gridDim.x) - senders, me = int(blockIdx.x) - senders;
    for (int t = me * kWarps + warp; t < p.tokens; t += nFin * kWarps) {
      int d = -1 - lane, pos = -1;
      if (lane < p.topk) {
        const int e = p.topkIdx[size_t(t) * p.topk + lane];
        pos = p.pos[size_t(t) * p.topk + lane];
        if (e >= 0 && e < p.experts && pos >= 0) d = e / p.expertsPerRank;
      }
      const unsigned same = __match_any_sync(0xffffffffu, d);
      const bool leader = d >= 0 && (__ffs(same) - 1) == lane;
      int good = 1;
      if (leader) good = waitFlag(p, combineFlag(p, p.rank, d, pos / kChunkRows), epoch, 4, d) ? 1 : 0;
      if (!__all_sync(0xffffffffu, good)) break;
      __syncwarp();
      const unsigned leaders = __ballot_sync(0xffffffffu, leader) & 0xffu;
      const int n = __popc(leaders);
      const unsigned char* rows[8];
      float w[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int from = j < n ? int(__fns(leaders, 0, j + 1)) : 0;
        const int dk = __shfl_sync(0xffffffffu, d, from), pk = __shfl_sync(0xffffffffu, pos, from);
        rows[j] = p.cbuf[p.rank] + (size_t(j < n ? dk : 0) * p.maxTokens + (j < n ? pk : 0)) * rowBytes;
        w[j] = 1.f;
      }
      weightedSumAny(p.y + size_t(t) * rowBytes, rows, w, n, vecs32, lane);
    }
  }
  __syncthreads();
  stampEnd(p, 4, int(blockIdx.x) < senders);
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(p.exitCounter + 1, 1u) == gridDim.x - 1) { p.exitCounter[1] = 0; p.work[2] = 0; if (!outOfOrder) p.epoch[1] = epoch; __threadfence(); }
  }
}

struct MoeLayout { size_t stage, meta, recv, out, cbuf, counts, flags, total; };
MoeLayout moeLayout(int world, int maxTokens, int capacityRows, int hidden, int experts) {
  MoeLayout l{};
  size_t off = 0;
  const int chunks = (maxTokens + kChunkRows - 1) / kChunkRows;
  const size_t perSource = roundUp(size_t(world) * maxTokens * hidden * 2, 1024);
  const size_t buf = roundUp(size_t(capacityRows) * hidden * 2, 1024);
  l.stage = off; off += world > 1 ? perSource : 1024;
  l.meta = off; off += roundUp(size_t(world) * maxTokens * kMetaWords * 4, 1024);
  l.recv = off; off += buf;
  l.out = off; off += buf;
  l.cbuf = off; off += perSource;
  l.counts = off; off += roundUp(size_t(world) * (experts + world) * 4, 1024);
  l.flags = off; off += roundUp(size_t(world + 2 * world * chunks) * 8, 1024);
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
  p.rank = c->rank; p.world = c->world; p.tokens = tokens; p.maxTokens = c->maxTokens; p.hiddenBytes = c->hidden * 2;
  p.experts = c->experts; p.topk = c->topk; p.expertsPerRank = c->experts / c->world; p.capacityRows = c->capacityRows; p.maxChunks = c->maxChunks;
  for (int q = 0; q < c->world; ++q) {
    p.stage[q] = c->peers[q] + c->stageOff;
    p.meta[q] = reinterpret_cast<int32_t*>(c->peers[q] + c->metaOff);
    p.cbuf[q] = c->peers[q] + c->cbufOff;
    p.countsAll[q] = reinterpret_cast<uint32_t*>(c->peers[q] + c->countsOff);
    p.flags[q] = reinterpret_cast<uint64_t*>(c->peers[q] + c->flagsOff);
  }
  p.recvBuf = c->peers[c->rank] + c->recvOff;
  p.outBuf = c->peers[c->rank] + c->outOff;
  p.epoch = reinterpret_cast<uint64_t*>(lb);
  p.exitCounter = reinterpret_cast<uint32_t*>(lb + 64);
  p.work = reinterpret_cast<uint32_t*>(lb + 128);
  p.status = reinterpret_cast<uint32_t*>(lb + 256);
  p.timing = c->timing ? reinterpret_cast<unsigned long long*>(lb + 512) : nullptr;
  p.localCounts = reinterpret_cast<uint32_t*>(lb + c->countsLocalOff);
  p.sendList = reinterpret_cast<int32_t*>(lb + c->sendListOff);
  p.pos = reinterpret_cast<int32_t*>(lb + c->posOff);
  p.topkIdx = c->topkIdx; p.topkWeight = c->topkWeight; p.slot = c->slot;
  p.timeoutNs = c->timeoutNs;
}

int planOn(PurlinMoeContext* c, const int32_t* topkIdx, const float* topkWeight, int tokens, int32_t* slot, cudaStream_t s) {
  unsigned char* lb = static_cast<unsigned char*>(c->local);
  uint32_t* counts = reinterpret_cast<uint32_t*>(lb + c->countsLocalOff);
  if (cudaMemsetAsync(counts, 0, size_t(c->experts + c->world) * 4, s) != cudaSuccess) { setError("route: clearing the counters failed"); return 1; }
  const int blocks = (tokens * 32 + kThreads - 1) / kThreads;
  if (blocks > 0)
    planKernel<<<blocks, kThreads, 0, s>>>(topkIdx, tokens, c->maxTokens, c->experts, c->topk, c->experts / c->world, slot,
                                           reinterpret_cast<int32_t*>(lb + c->posOff), reinterpret_cast<int32_t*>(lb + c->sendListOff), counts,
                                           reinterpret_cast<uint32_t*>(lb + 256));
  c->topkIdx = topkIdx; c->topkWeight = topkWeight; c->slot = slot;
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

}  // namespace

extern "C" {

size_t purlin_moe_workspace_bytes(int world, int maxTokens, int capacityRows, int hidden, int experts) {
  return moeLayout(world, maxTokens, capacityRows, hidden, experts).total;
}

PurlinMoeContext* purlin_moe_create(int rank, int world, const uint64_t* peerPtrs, int maxTokens, int hidden, int experts, int topk,
                                    int capacityRows, uint64_t timeoutNs, void* stream) {
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world) { setError("invalid rank or world size"); return nullptr; }
  if (experts % world || experts % 32 || experts > kMaxExperts) { setError("experts must be a multiple of 32 and of the world size, at most 512"); return nullptr; }
  if (topk < 1 || topk > 8 || topk > experts || hidden % 16) { setError("top-k must be 1..8 and hidden a multiple of 16"); return nullptr; }
  if (maxTokens < 1 || maxTokens > (1 << 24) || capacityRows < 1) { setError("maxTokens must be 1..2^24 and the capacity positive"); return nullptr; }
  auto* c = new PurlinMoeContext();
  c->rank = rank; c->world = world; c->maxTokens = maxTokens; c->hidden = hidden; c->experts = experts; c->topk = topk; c->capacityRows = capacityRows;
  c->maxChunks = (maxTokens + kChunkRows - 1) / kChunkRows;
  const MoeLayout l = moeLayout(world, maxTokens, capacityRows, hidden, experts);
  c->stageOff = l.stage; c->metaOff = l.meta; c->recvOff = l.recv; c->outOff = l.out; c->cbufOff = l.cbuf; c->countsOff = l.counts; c->flagsOff = l.flags; c->total = l.total;
  for (int q = 0; q < world; ++q) {
    if (!peerPtrs[q] || peerPtrs[q] % 1024) { delete c; setError("peer blocks must be non-null and 1024-byte aligned"); return nullptr; }
    c->peers[q] = reinterpret_cast<unsigned char*>(peerPtrs[q]);
  }
  c->timeoutNs = timeoutNs ? timeoutNs : 10ull * 1000 * 1000 * 1000;
  // local block: [0] epochs, [64] exit counters, [256] status, then counters, send lists, positions
  c->countsLocalOff = 1024;
  c->sendListOff = roundUp(c->countsLocalOff + size_t(kMaxExperts + kMaxRanks) * 4, 1024);
  c->posOff = c->sendListOff + roundUp(size_t(world) * maxTokens * 4, 1024);
  const size_t localBytes = c->posOff + roundUp(size_t(maxTokens) * topk * 4, 1024);
  if (cudaMalloc(&c->local, localBytes) != cudaSuccess) { delete c; setError("cudaMalloc failed"); return nullptr; }
  cudaMemsetAsync(c->local, 0, localBytes, static_cast<cudaStream_t>(stream));
  if (const char* t = std::getenv("PURLIN_MOE_TIMING"); t && t[0] != '0') {
    c->timing = true;
    const unsigned long long fresh[8] = {~0ull, 0, 0, ~0ull, ~0ull, 0, 0, ~0ull};
    cudaMemcpyAsync(static_cast<unsigned char*>(c->local) + 512, fresh, sizeof(fresh), cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream));
  }
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
// Phase times of the last dispatch and combine in nanoseconds since each kernel's first CTA started:
// out8 = {dispatch: last sender end, last receiver end, first sender end, 0, combine: last pusher end, last finisher end,
// first pusher end, 0}. Synchronises the stream and re-arms the words. Returns 1 when the context was created without
// PURLIN_MOE_TIMING=1.
int purlin_moe_timing(PurlinMoeContext* c, uint64_t* out8, void* stream) {
  if (!c || !c->timing) { setError("timing is off: create the context with PURLIN_MOE_TIMING=1"); return 1; }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  unsigned long long raw[8];
  unsigned char* at = static_cast<unsigned char*>(c->local) + 512;
  if (cudaMemcpyAsync(raw, at, sizeof(raw), cudaMemcpyDeviceToHost, s) != cudaSuccess || cudaStreamSynchronize(s) != cudaSuccess) { setError("reading the timing words failed"); return 1; }
  for (int k = 0; k < 2; ++k) {
    const unsigned long long t0 = raw[k * 4];
    out8[k * 4 + 0] = raw[k * 4 + 1] > t0 ? raw[k * 4 + 1] - t0 : 0;
    out8[k * 4 + 1] = raw[k * 4 + 2] > t0 ? raw[k * 4 + 2] - t0 : 0;
    out8[k * 4 + 2] = raw[k * 4 + 3] != ~0ull && raw[k * 4 + 3] > t0 ? raw[k * 4 + 3] - t0 : 0;
    out8[k * 4 + 3] = 0;
  }
  const unsigned long long fresh[8] = {~0ull, 0, 0, ~0ull, ~0ull, 0, 0, ~0ull};
  if (cudaMemcpyAsync(at, fresh, sizeof(fresh), cudaMemcpyHostToDevice, s) != cudaSuccess || cudaStreamSynchronize(s) != cudaSuccess) { setError("re-arming the timing words failed"); return 1; }
  return 0;
}
int purlin_moe_clear_status(PurlinMoeContext* c, void* stream) {
  return cudaMemsetAsync(static_cast<unsigned char*>(c->local) + 256, 0, 16, static_cast<cudaStream_t>(stream)) == cudaSuccess ? 0 : 1;
}
void* purlin_moe_recv_buffer(PurlinMoeContext* c) { return c->peers[c->rank] + c->recvOff; }
void* purlin_moe_out_buffer(PurlinMoeContext* c) { return c->peers[c->rank] + c->outOff; }

int purlin_moe_route(PurlinMoeContext* c, const float* logits, int tokens, int normalize, int32_t* topkIdx, float* topkWeight,
                     int32_t* slot, void* stream) {
  NvtxRange range("moeRoute", size_t(tokens));
  if (tokens < 0 || tokens > c->maxTokens) { setError("route: more tokens than the context was created for"); return 1; }
  if (tokens == 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int blocks = (tokens * 32 + kThreads - 1) / kThreads;
  switch (c->experts / 32) {
    case 1: routeKernel<1><<<blocks, kThreads, 0, s>>>(logits, tokens, c->experts, c->topk, normalize, topkIdx, topkWeight); break;
    case 2: routeKernel<2><<<blocks, kThreads, 0, s>>>(logits, tokens, c->experts, c->topk, normalize, topkIdx, topkWeight); break;
    case 4: routeKernel<4><<<blocks, kThreads, 0, s>>>(logits, tokens, c->experts, c->topk, normalize, topkIdx, topkWeight); break;
    case 8: routeKernel<8><<<blocks, kThreads, 0, s>>>(logits, tokens, c->experts, c->topk, normalize, topkIdx, topkWeight); break;
    case 16: routeKernel<16><<<blocks, kThreads, 0, s>>>(logits, tokens, c->experts, c->topk, normalize, topkIdx, topkWeight); break;
    default: setError("experts / 32 must be 1, 2, 4, 8 or 16"); return 1;
  }
  if (cudaGetLastError() != cudaSuccess) { setError("route launch failed"); return 1; }
  return planOn(c, topkIdx, topkWeight, tokens, slot, s);
}

int purlin_moe_plan(PurlinMoeContext* c, const int32_t* topkIdx, const float* topkWeight, int tokens, int32_t* slot, void* stream) {
  NvtxRange range("moePlan", size_t(tokens));
  if (tokens < 0 || tokens > c->maxTokens) { setError("plan: more tokens than the context was created for"); return 1; }
  if (!topkIdx || !topkWeight || !slot) { setError("plan: null argument"); return 1; }
  return planOn(c, topkIdx, topkWeight, tokens, slot, static_cast<cudaStream_t>(stream));
}

int purlin_moe_dispatch(PurlinMoeContext* c, const void* x, int tokens, const int32_t* topkIdx, const int32_t* slot,
                        int32_t* sentRow, int32_t* recvCounts, int blocks, void* stream) {
  NvtxRange range("moeDispatch", size_t(tokens));
  if (tokens < 0 || tokens > c->maxTokens) { setError("dispatch: more tokens than the context was created for"); return 1; }
  if (!c->topkIdx || topkIdx != c->topkIdx || slot != c->slot) { setError("dispatch: the routing must come from purlin_moe_route or purlin_moe_plan on this context"); return 1; }
  MoeParams p{};
  fillCommon(p, c, tokens);
  p.x = static_cast<const unsigned char*>(x); p.sentRow = sentRow; p.recvCounts = recvCounts;
  const int grid = smCount() * kDispatchCtasPerSm;
  // remote stores fill the links with far fewer CTAs (about 32 GB/s each) than the local fan-out needs for HBM; the
  // receivers end last (4 GPUs, 296 CTAs: 32 senders 352 us, 48 senders 357 - 372 us, 64 senders 363 us)
  p.senders = blocks > 0 ? std::min(blocks, grid - 1) : std::max(std::min(grid / 3, 32), 1);
  dispatchKernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { setError(std::string("dispatch launch: ") + cudaGetErrorString(e)); return 1; }
  return 0;
}

int purlin_moe_combine(PurlinMoeContext* c, void* y, int tokens, const int32_t* topkIdx, const float* topkWeight,
                       const int32_t* sentRow, int blocks, void* stream) {
  NvtxRange range("moeCombine", size_t(tokens));
  (void)topkWeight; (void)sentRow;   // the gate weights travelled with the rows at dispatch
  if (tokens < 0 || tokens > c->maxTokens) { setError("combine: more tokens than the context was created for"); return 1; }
  if (!c->topkIdx || topkIdx != c->topkIdx) { setError("combine: the routing must be the one the matching dispatch used"); return 1; }
  MoeParams p{};
  fillCommon(p, c, tokens);
  p.y = static_cast<unsigned char*>(y);
  const int grid = smCount() * kCombineCtasPerSm;
  // The pushers read every expert output row, the finishers add at most `world` rows per token, and it is the finishers
  // that end last: measured at 4 GPUs (4096 tokens, hidden 7168, top-8 of 256), 80 pushers of 148 CTAs 343 us, 98 pushers
  // 366 us, 110 pushers 392 us.
  p.senders = blocks > 0 ? std::min(blocks, grid - 1) : std::max(grid * 54 / 100, 1);
  combineKernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { setError(std::string("combine launch: ") + cudaGetErrorString(e)); return 1; }
  return 0;
}

}  // extern "C"
