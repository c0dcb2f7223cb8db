// tcgen05 GEMM for sm_100a and the two tensor-parallel kernels fused with their collective.
//
//   C[M,N] = A[M,K] * B[N,K]^T      bf16 in, fp32 accumulate in TMEM, bf16 out
//
// The reference contains no GEMM and no tensor-core code; it only says a collective "could be fused into a
// larger kernel" (csrc/examples/ar/ar.cu:81). These kernels are that fusion, built on the same device-side
// signalling primitives as the collectives (release/acquire flags in peer memory, bounded waits).
//
// One persistent CTA per SM, warp-specialised:
//   warp 0      TMA producer   cp.async.bulk.tensor (no cluster multicast) into a ring of 128B-swizzled stages
//   warp 1      MMA issuer     one thread issues tcgen05.mma (128 x bn x 16) into one of two TMEM accumulators
//   warps 2-5   epilogue       tcgen05.ld -> registers -> fused epilogue -> global / peer memory
//   warps 6-9   communication  (all-gather variant) push this rank's activation rows into every peer's buffer
//
// Variants (template COMM):
//   kCommNone  plain GEMM
//   kCommAG    all-gather -> GEMM: A rows of other ranks arrive in a local buffer through the peers' comm warps
//              while tiles over rows that are already here are computed; the producer waits on a per-row-block
//              flag before it loads a block that came over NVLink.
//   kCommRS    GEMM -> reduce-scatter: tiles whose rows belong to another rank are stored straight into that
//              rank's memory from the epilogue registers and flagged; tiles of this rank's own rows are computed
//              last and their epilogue adds the partial tiles received from every peer (ascending rank order).
// Epilogues (template EPI): plain store, or SwiGLU over interleaved gate/up columns (silu(g) * u).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "purlin/atom.cuh"
#include "purlin/constants.hpp"
#include "purlin/gemm.h"
#include "purlin/layout.hpp"
#include "purlin/tc_sm100.cuh"
#include "purlin/telemetry.hpp"

namespace purlin { void setError(const std::string& e); }
using namespace purlin;

namespace {

constexpr int kBM = 128, kBK = 64, kMaxBN = 256;
constexpr int kAccStride = 256;                // TMEM columns between the two accumulators
constexpr int kTmemCols = 512;
constexpr int kABytes = kBM * kBK * 2;         // 16 KiB
constexpr int kEpiWarps = 4, kCommWarps = 4;
constexpr int kThreadsPlain = 32 * (2 + kEpiWarps);
constexpr int kThreadsComm = 32 * (2 + kEpiWarps + kCommWarps);
constexpr int kSmemLimit = 227 * 1024;
constexpr int kBarrierBytes = 256;
constexpr int kMaxStages = 8;
constexpr int kScratchPitch = 272;              // bytes per row of the epilogue's transpose scratch (256 + 16: conflict-free)
constexpr int kScratchBytes = kEpiWarps * 32 * kScratchPitch;   // reduce-scatter variant only

enum { kEpiStore = 0, kEpiSwiglu = 1 };
enum { kCommNone = 0, kCommAG = 1, kCommRS = 2 };

struct Params {
  int M, N, K, bn, stages;
  int tilesM, tilesN;
  __nv_bfloat16* C;
  int ldc;
  uint32_t* status;
  uint64_t timeoutNs;
  // tensor parallel
  int rank, world, blocksPerRank;      // blocksPerRank = rows per rank / 128
  uint64_t* epoch;                     // device call counter (flag values and buffer parity derive from it)
  uint32_t* exitCounter;
  // all-gather -> GEMM
  const __nv_bfloat16* localA;         // this rank's rows [M / world, K]
  __nv_bfloat16* gatherBuf[kMaxRanks]; // every rank's gather buffer of this call's parity, [M, K]
  uint64_t* rowReady[kMaxRanks];       // every rank's flags, [tilesM]
  uint32_t* pushCounters;              // local last-arrival counters, [(world - 1) * blocksPerRank]
  int pushParts;                       // pieces one 128-row block is split into for pushing
  int commWarps;                       // how many of a CTA's communication warps take part (1..4): paces the pushes
  size_t gatherParityBytes;            // bytes between the gather buffers of even and odd calls
  // GEMM -> reduce-scatter
  __nv_bfloat16* partialBuf[kMaxRanks];// every rank's receive buffers: 2 parities x [world slots][M / world, N]
  uint64_t* tileReady[kMaxRanks];      // every rank's flags, [world][blocksPerRank][tilesN][4 row quarters]
  size_t partialParityStride;          // elements between the two parities
  int epiPipe;                         // 1: the epilogue overlaps the next chunk's TMEM load with the current chunk's arithmetic
  int rsScratch;                       // 1: remote tiles leave through a shared-memory transpose (long contiguous runs per row)
};

struct alignas(64) Maps { CUtensorMap a, b, aLocal, a1; };   // a1: gather buffer of odd calls (all-gather variant)

PURLIN_D void recordTimeout(const Params& p, uint32_t where, uint32_t a, uint32_t b) {
  if (p.status && atomicCAS(p.status, 0u, uint32_t(kStatusTimeoutBarrier)) == 0u) { p.status[1] = where; p.status[2] = a; p.status[3] = b; __threadfence(); }
}
PURLIN_D bool waitFlag(const uint64_t* flag, uint64_t value, volatile int* abortWord, uint64_t timeoutNs) {
  if (sig::ldAcquireSys(flag) >= value) return true;
  const uint64_t start = sig::globalTimerNs();
  uint32_t spins = 0;
  while (sig::ldRelaxedSys(flag) < value) {
    if ((++spins & 63u) == 0u) {
      if (*abortWord) return false;
      if (sig::globalTimerNs() - start > timeoutNs) { *abortWord = 1; return false; }
    }
  }
  return sig::ldAcquireSys(flag) >= value;
}

PURLIN_D uint32_t packBf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
PURLIN_D float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
PURLIN_D float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
PURLIN_D float silu(float x) { return x / (1.f + __expf(-x)); }

PURLIN_D void stShared16(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
PURLIN_D Vec16 ldShared16(uint32_t addr) {
  Vec16 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x[0]), "=r"(v.x[1]), "=r"(v.x[2]), "=r"(v.x[3]) : "r"(addr) : "memory");
  return v;
}

// 32 fp32 accumulator values of one row -> bf16 -> global (or peer) memory. Two 32-byte stores when the row pitch
// keeps them aligned (whole sectors, and NVLink-friendly when `out` is peer memory), 16-byte stores otherwise.
PURLIN_D void storeChunkBf16(__nv_bfloat16* out, const uint32_t (&r)[32], int col, int N, bool wide) {
  uint32_t o[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i] = packBf16(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
  if (wide && col + 32 <= N) {
    st32(out, Vec32{{o[0], o[1], o[2], o[3], o[4], o[5], o[6], o[7]}});
    st32(out + 16, Vec32{{o[8], o[9], o[10], o[11], o[12], o[13], o[14], o[15]}});
  } else {
#pragma unroll
    for (int g = 0; g < 4; ++g)
      if (col + g * 8 + 8 <= N) st16(out + g * 8, Vec16{{o[4 * g], o[4 * g + 1], o[4 * g + 2], o[4 * g + 3]}});
  }
}

// order in which (CTAS x 128)-row blocks are visited
template <int COMM>
PURLIN_D int rowBlockOf(const Params& p, int mIdx) {
  if constexpr (COMM == kCommAG) {
    // own rows first, then the rows of rank-1, rank-2, ... (the order in which peers push to this rank)
    const int src = (p.rank - mIdx / p.blocksPerRank + p.world) % p.world;
    return src * p.blocksPerRank + mIdx % p.blocksPerRank;
  } else if constexpr (COMM == kCommRS) {
    // rows of rank+1 first, ..., own rows last (their epilogue needs every peer's partial tile)
    const int dst = (p.rank + 1 + mIdx / p.blocksPerRank) % p.world;
    return dst * p.blocksPerRank + mIdx % p.blocksPerRank;
  } else {
    return mIdx;
  }
}

// Tile t -> (row-block index, column block). Tiles are walked in bands of kGroupM row blocks, rows fastest inside a
// band, so the tiles in flight at one time share a few A blocks and a few B blocks and the working set stays in L2.
constexpr int kGroupM = 8;
template <int COMM>
PURLIN_D void tileCoord(const Params& p, int t, int& mIdx, int& nBlk) {
  if constexpr (COMM == kCommNone) {
    const int perBand = kGroupM * p.tilesN;
    const int band = t / perBand, within = t - band * perBand;
    const int first = band * kGroupM;
    const int rows = p.tilesM - first < kGroupM ? p.tilesM - first : kGroupM;
    mIdx = first + within % rows;
    nBlk = within / rows;
  } else {
    // the same banding inside one rank's rows (a rank's row blocks become usable together: they arrive, or are
    // owed, as one phase), phases in the order rowBlockOf() gives them
    const int perRank = p.blocksPerRank * p.tilesN;
    const int seg = t / perRank, u = t - seg * perRank;
    const int perBand = kGroupM * p.tilesN;
    const int band = u / perBand, within = u - band * perBand;
    const int first = band * kGroupM;
    const int rows = p.blocksPerRank - first < kGroupM ? p.blocksPerRank - first : kGroupM;
    mIdx = seg * p.blocksPerRank + first + within % rows;
    nBlk = within / rows;
  }
}


// CTAS = 1: every CTA owns 128 x bn tiles. CTAS = 2: a cluster of two CTAs owns 256 x bn tiles; each CTA loads its
// 128 rows of A and its half of B's columns, CTA 0 issues one 256-row MMA for the pair (cta_group::2), so every
// byte of B crosses L2 -> shared memory once per 256 rows instead of once per 128.
template <int EPI, int COMM, int CTAS>
__global__ void __launch_bounds__(COMM == kCommAG ? kThreadsComm : kThreadsPlain, 1)
gemmKernel(const __grid_constant__ Maps maps, const __grid_constant__ Params p) {
  extern __shared__ unsigned char smemRaw[];
  const uint32_t rawAddr = tc::smemAddr(smemRaw);
  const uint32_t base = (rawAddr + 1023u) & ~1023u;          // swizzled tiles need 1024-byte alignment
  unsigned char* smem = smemRaw + (base - rawAddr);
  const int bnLocal = p.bn / CTAS;                           // B columns this CTA keeps in shared memory
  const int stageBytes = kABytes + bnLocal * kBK * 2;
  const uint32_t barBase = base + uint32_t(p.stages) * stageBytes;
  // barrier block: full[stages], empty[stages], tmemFull[2], tmemEmpty[2], then the TMEM base word and the abort word
  auto fullBar = [&](int s) { return barBase + 8u * s; };
  auto emptyBar = [&](int s) { return barBase + 8u * (p.stages + s); };
  auto tmemFullBar = [&](int a) { return barBase + 8u * (2 * p.stages + a); };
  auto tmemEmptyBar = [&](int a) { return barBase + 8u * (2 * p.stages + 2 + a); };
  uint32_t* words = reinterpret_cast<uint32_t*>(smem + size_t(p.stages) * stageBytes + 8 * (2 * p.stages + 4));
  volatile uint32_t* tmemBaseWord = words;
  volatile int* abortWord = reinterpret_cast<volatile int*>(words + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t ctaRank = CTAS == 2 ? tc::clusterCtaRank() : 0u;
  const int pairIdx = blockIdx.x / CTAS, numPairs = gridDim.x / CTAS;
  const uint64_t epoch = (COMM != kCommNone) ? sig::ldRelaxedSys(p.epoch) + 1 : 1;
  const int parity = int(epoch & 1);

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) { tc::mbarInit(fullBar(s), 1); tc::mbarInit(emptyBar(s), 1); }
    for (int a = 0; a < 2; ++a) { tc::mbarInit(tmemFullBar(a), 1); tc::mbarInit(tmemEmptyBar(a), kEpiWarps * CTAS); }
    *abortWord = 0;
    tc::mbarFenceInit();
    tc::tmaPrefetchDescriptor(&maps.a);
    tc::tmaPrefetchDescriptor(&maps.b);
  }
  if (warp == 1) {
    if constexpr (CTAS == 2) { tc::tmemAllocPair(tc::smemAddr(words), kTmemCols); tc::tmemRelinquishPair(); }
    else { tc::tmemAlloc(tc::smemAddr(words), kTmemCols); tc::tmemRelinquish(); }
  }
  tc::fenceBeforeThreadSync();
  if constexpr (CTAS == 2) tc::clusterSync(); else __syncthreads();   // the pair's barriers exist before any remote arrival
  tc::fenceAfterThreadSync();
  const uint32_t tmemBase = *tmemBaseWord;
  // the barrier block of CTA 0 and of CTA 1 as seen from this CTA (cluster addresses)
  const uint32_t leaderBars = CTAS == 2 ? tc::mapToCta(barBase, 0) : barBase;
  const uint32_t peerBars = CTAS == 2 ? tc::mapToCta(barBase, 1) : barBase;
  (void)peerBars;

  const int numTiles = p.tilesM * p.tilesN;                  // tilesM counts (CTAS x 128)-row blocks
  const int kBlocks = (p.K + kBK - 1) / kBK;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      uint32_t st = 0, ph = 0;          // ring position and its phase
      uint64_t seenReady = 0;           // row blocks whose arrival flag this thread has already acquired
      bool ok = true;
      for (int t = pairIdx; t < numTiles && ok; t += numPairs) {
        int mIdx, nBlk;
        tileCoord<COMM>(p, t, mIdx, nBlk);
        const int mBlk = rowBlockOf<COMM>(p, mIdx) * CTAS + int(ctaRank);      // this CTA's 128-row block
        const int bRow = nBlk * p.bn + int(ctaRank) * bnLocal;
        const CUtensorMap* aMap = &maps.a;
        int aRow = mBlk * kBM;
        if constexpr (COMM == kCommAG) {
          if (parity) aMap = &maps.a1;
          const int perRank = p.blocksPerRank * CTAS;
          if (mBlk / perRank == p.rank) {
            aMap = &maps.aLocal;                       // own rows come straight from the caller's tensor
            aRow = (mBlk % perRank) * kBM;
          } else {
            // rows pushed by a peer: wait for the block's flag, then order those generic-proxy writes
            // before this thread's async-proxy reads (TMA)
            if (mBlk >= 64 || !((seenReady >> mBlk) & 1ull)) {   // a block seen once stays ready for the whole call
              ok = waitFlag(p.rowReady[p.rank] + mBlk, epoch, abortWord, p.timeoutNs);
              if (!ok) { recordTimeout(p, 4, mBlk, 0); break; }
              tc::fenceProxyAsync();
              if (mBlk < 64) seenReady |= 1ull << mBlk;
            }
          }
        }
        for (int kb = 0; kb < kBlocks; ++kb) {
          ok = tc::mbarWait(emptyBar(st), ph ^ 1, abortWord, p.timeoutNs);
          if (!ok) { recordTimeout(p, 1, t, kb); break; }
          const uint32_t sA = base + st * uint32_t(stageBytes), sB = sA + kABytes;
          if constexpr (CTAS == 2) {
            // both CTAs' bytes are credited to CTA 0's barrier; CTA 0 announces the total
            const uint32_t leaderFull = leaderBars + 8u * st;
            if (ctaRank == 0) tc::mbarExpectTx(fullBar(st), uint32_t(2 * stageBytes));
            tc::tmaLoad2dPair(sA, aMap, kb * kBK, aRow, leaderFull);
            tc::tmaLoad2dPair(sB, &maps.b, kb * kBK, bRow, leaderFull);
          } else {
            tc::mbarExpectTx(fullBar(st), uint32_t(stageBytes));
            tc::tmaLoad2d(sA, aMap, kb * kBK, aRow, fullBar(st));
            tc::tmaLoad2d(sB, &maps.b, kb * kBK, bRow, fullBar(st));
          }
          if (++st == uint32_t(p.stages)) { st = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (CTA 0 of a pair) -------------------------------
    if (lane == 0 && ctaRank == 0) {
      const uint32_t idesc = tc::instrDescBf16(uint32_t(p.bn), uint32_t(kBM * CTAS));
      // descriptors differ only in their 14-bit start address: keep the constant halves out of the loop
      const uint64_t descA0 = tc::smemDescSw128(base), descB0 = tc::smemDescSw128(base + kABytes);
      const uint32_t stageStep = uint32_t(stageBytes) >> 4;
      uint32_t st = 0, ph = 0, accIt = 0;
      bool ok = true;
      for (int t = pairIdx; t < numTiles && ok; t += numPairs, ++accIt) {
        const int a = accIt & 1;
        const uint32_t aph = (accIt >> 1) & 1;
        ok = tc::mbarWait(tmemEmptyBar(a), aph ^ 1, abortWord, p.timeoutNs);   // epilogues drained this accumulator
        if (!ok) { recordTimeout(p, 2, t, 0); break; }
        tc::fenceAfterThreadSync();
        const uint32_t tmemD = tmemBase + uint32_t(a) * kAccStride;
        for (int kb = 0; kb < kBlocks; ++kb) {
          ok = tc::mbarWait(fullBar(st), ph, abortWord, p.timeoutNs);
          if (!ok) { recordTimeout(p, 3, t, kb); break; }
          tc::fenceAfterThreadSync();
          const uint64_t da = descA0 + uint64_t(st * stageStep), db = descB0 + uint64_t(st * stageStep);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            if constexpr (CTAS == 2) tc::mmaPair(tmemD, da + 2 * k, db + 2 * k, idesc, uint32_t((kb | k) != 0));
            else tc::mma(tmemD, da + 2 * k, db + 2 * k, idesc, uint32_t((kb | k) != 0));
          }
          // the stage is free (in both CTAs) once these MMAs have read it
          if constexpr (CTAS == 2) { tc::mmaCommitPair(leaderBars + 8u * (p.stages + st)); tc::mmaCommitPair(peerBars + 8u * (p.stages + st)); }
          else tc::mmaCommit(emptyBar(st));
          if (++st == uint32_t(p.stages)) { st = 0; ph ^= 1; }
        }
        if (ok) {   // the accumulator is complete once every MMA of the tile is done
          if constexpr (CTAS == 2) { tc::mmaCommitPair(leaderBars + 8u * (2 * p.stages + a)); tc::mmaCommitPair(peerBars + 8u * (2 * p.stages + a)); }
          else tc::mmaCommit(tmemFullBar(a));
        }
      }
    }
  } else if (warp < 2 + kEpiWarps) {
    // ------------------------------- epilogue -------------------------------
    const int quarter = warp & 3;                // a warp may only touch TMEM lanes [32 * (warp % 4), +32)
    const int perRank = p.blocksPerRank * CTAS;  // 128-row blocks per rank
    uint32_t accIt = 0;
    bool ok = true;
    for (int t = pairIdx; t < numTiles && ok; t += numPairs, ++accIt) {
      const int a = accIt & 1;
      const uint32_t aph = (accIt >> 1) & 1;
      int mIdx, nBlk;
      tileCoord<COMM>(p, t, mIdx, nBlk);
      const int mBlk = rowBlockOf<COMM>(p, mIdx) * CTAS + int(ctaRank);
      const int n0 = nBlk * p.bn;
      ok = tc::mbarWait(tmemFullBar(a), aph, abortWord, p.timeoutNs);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { if (lane == 0) recordTimeout(p, 5, t, 0); break; }
      tc::fenceAfterThreadSync();
      const uint32_t taddr = tmemBase + (uint32_t(quarter * 32) << 16) + uint32_t(a) * kAccStride;
      const int rowInTile = quarter * 32 + lane;
      const int row = mBlk * kBM + rowInTile;

      int dstRank = p.rank, rowInShard = row;
      const __nv_bfloat16* partialBase = nullptr;   // slot 0 of this row inside the receive buffer
      size_t slotStride = 0;
      bool reduceOwn = false;
      if constexpr (COMM == kCommRS) {
        dstRank = mBlk / perRank;
        rowInShard = row - dstRank * perRank * kBM;
        reduceOwn = dstRank == p.rank && p.world > 1;
        if (reduceOwn) {
          // every peer's partial tile (this row quarter) must have landed
          int good = 1;
          if (lane < p.world && lane != p.rank) {
            const uint64_t* f = p.tileReady[p.rank] + ((size_t(lane) * perRank + (mBlk % perRank)) * p.tilesN + nBlk) * 4 + quarter;
            good = waitFlag(f, epoch, abortWord, p.timeoutNs) ? 1 : 0;
          }
          ok = __all_sync(0xffffffffu, good);
          if (!ok) { if (lane == 0) recordTimeout(p, 6, t, 0); break; }
          slotStride = size_t(perRank) * kBM * p.N;
          partialBase = p.partialBuf[p.rank] + size_t(parity) * p.partialParityStride + size_t(rowInShard) * p.N;
        }
      }

      bool viaScratch = false;
      if constexpr (COMM == kCommRS && EPI == kEpiStore) {
        viaScratch = p.rsScratch && dstRank != p.rank && p.bn % 128 == 0 && n0 + p.bn <= p.N;
        if (viaScratch) {
          // Rows of a remote tile leave as 128-byte runs: the 32 lanes hold 32 different rows (64 bytes each per TMEM
          // load), so a direct store would put 32 separate 32-byte sectors on NVLink per instruction. Through the
          // scratch each store instruction writes 4 rows x 128 contiguous bytes.
          const uint32_t scratch = barBase + kBarrierBytes + uint32_t(warp - 2) * 32u * kScratchPitch;
          __nv_bfloat16* tileOut = p.partialBuf[dstRank] + size_t(parity) * p.partialParityStride +
                                   (size_t(p.rank) * perRank * kBM + size_t(rowInShard - lane)) * p.N + n0;   // row of lane 0
          for (int h0 = 0; h0 < p.bn; h0 += 128) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t r[32];
              tc::tmemLoad32(taddr + uint32_t(h0 + c * 32), r);
              tc::tmemLoadWait();
              const uint32_t rowAddr = scratch + uint32_t(lane) * kScratchPitch + uint32_t(c) * 64u;
#pragma unroll
              for (int g = 0; g < 4; ++g)
                stShared16(rowAddr + g * 16, packBf16(__uint_as_float(r[8 * g]), __uint_as_float(r[8 * g + 1])), packBf16(__uint_as_float(r[8 * g + 2]), __uint_as_float(r[8 * g + 3])),
                           packBf16(__uint_as_float(r[8 * g + 4]), __uint_as_float(r[8 * g + 5])), packBf16(__uint_as_float(r[8 * g + 6]), __uint_as_float(r[8 * g + 7])));
            }
            __syncwarp();
            const int rowInGroup = lane >> 3, piece = lane & 7;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int rr = 4 * i + rowInGroup;
              const uint32_t src = scratch + uint32_t(rr) * kScratchPitch + uint32_t(piece) * 16u;
              const Vec16 lo = ldShared16(src), hi = ldShared16(src + 128);
              __nv_bfloat16* o = tileOut + size_t(rr) * p.N + h0;
              st16(o + piece * 8, lo);
              st16(o + 64 + piece * 8, hi);
            }
            __syncwarp();
          }
        }
      }
      // One 32-column chunk of this warp's rows: convert (and activate) the accumulators and store them.
      auto emitChunk = [&](const uint32_t (&r)[32], int c0) {
        const int col = n0 + c0;
        if constexpr (EPI == kEpiSwiglu) {
          // columns [c0, c0+16) are gate, [c0+16, c0+32) are up, both for output columns (n0 + c0) / 2 + [0, 16)
          if (row < p.M) {
            uint32_t o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float g0 = __uint_as_float(r[2 * i]), g1 = __uint_as_float(r[2 * i + 1]);
              const float u0 = __uint_as_float(r[16 + 2 * i]), u1 = __uint_as_float(r[16 + 2 * i + 1]);
              o[i] = packBf16(silu(g0) * u0, silu(g1) * u1);
            }
            __nv_bfloat16* out = p.C + size_t(row) * p.ldc + col / 2;
            if (col / 2 + 16 <= p.ldc) {
              if ((reinterpret_cast<uintptr_t>(out) & 31u) == 0) st32(out, Vec32{{o[0], o[1], o[2], o[3], o[4], o[5], o[6], o[7]}});
              else { st16(out, Vec16{{o[0], o[1], o[2], o[3]}}); st16(out + 8, Vec16{{o[4], o[5], o[6], o[7]}}); }
            }
          }
        } else if constexpr (COMM == kCommRS) {
          if (reduceOwn) {
            // ascending rank order; own accumulator takes this rank's place in the sum. All peers' copies of the
            // 32 columns are requested before any is consumed (up to 8 peers x 64 bytes in flight per thread).
            float acc[32];
#pragma unroll
            for (int e = 0; e < 32; ++e) acc[e] = 0.f;
            const bool full = col + 32 <= p.N;
            for (int q0 = 0; q0 < p.world; q0 += 8) {
              Vec16 v[8][4];
#pragma unroll
              for (int b = 0; b < 8; ++b)
                if (q0 + b < p.world && q0 + b != p.rank) {
                  const __nv_bfloat16* src = partialBase + size_t(q0 + b) * slotStride + col;
#pragma unroll
                  for (int g = 0; g < 4; ++g)
                    if (full || col + g * 8 + 8 <= p.N) v[b][g] = ld16(src + g * 8);
                }
#pragma unroll
              for (int b = 0; b < 8; ++b) {
                if (q0 + b >= p.world) break;
                if (q0 + b == p.rank) {
#pragma unroll
                  for (int e = 0; e < 32; ++e) acc[e] += __uint_as_float(r[e]);
                } else {
#pragma unroll
                  for (int g = 0; g < 4; ++g)
                    if (full || col + g * 8 + 8 <= p.N) {
#pragma unroll
                      for (int e = 0; e < 4; ++e) { acc[g * 8 + 2 * e] += bf16lo(v[b][g].x[e]); acc[g * 8 + 2 * e + 1] += bf16hi(v[b][g].x[e]); }
                    }
                }
              }
            }
            uint32_t accBits[32];
#pragma unroll
            for (int e = 0; e < 32; ++e) accBits[e] = __float_as_uint(acc[e]);
            __nv_bfloat16* out = p.C + size_t(rowInShard) * p.ldc + col;
            storeChunkBf16(out, accBits, col, p.N, (p.N % 16) == 0 && (reinterpret_cast<uintptr_t>(out) & 31u) == 0);
          } else {
            __nv_bfloat16* out = (dstRank == p.rank)
                ? p.C + size_t(rowInShard) * p.ldc + col      // world of one: plain store
                : p.partialBuf[dstRank] + size_t(parity) * p.partialParityStride + (size_t(p.rank) * perRank * kBM + rowInShard) * p.N + col;
            storeChunkBf16(out, r, col, p.N, (p.N % 16) == 0 && (reinterpret_cast<uintptr_t>(out) & 31u) == 0);
          }
        } else {
          if (row < p.M) {
            __nv_bfloat16* out = p.C + size_t(row) * p.ldc + col;
            storeChunkBf16(out, r, col, p.N, (reinterpret_cast<uintptr_t>(out) & 31u) == 0);
          }
        }
      };
      if (!viaScratch) {
        if (p.epiPipe && COMM != kCommRS) {
          // software-pipelined: the next chunk's TMEM load is in flight while this chunk is converted and stored
          uint32_t ra[32], rb[32];
          tc::tmemLoad32(taddr, ra);
          for (int c0 = 0; c0 < p.bn; c0 += 64) {
            tc::tmemLoadWaitFor(ra);
            const bool second = c0 + 32 < p.bn;
            if (second) tc::tmemLoad32(taddr + uint32_t(c0 + 32), rb);
            emitChunk(ra, c0);
            if (second) {
              tc::tmemLoadWaitFor(rb);
              if (c0 + 64 < p.bn) tc::tmemLoad32(taddr + uint32_t(c0 + 64), ra);
              emitChunk(rb, c0 + 32);
            }
          }
        } else {
          for (int c0 = 0; c0 < p.bn; c0 += 32) {
            uint32_t r[32];
            tc::tmemLoad32(taddr + uint32_t(c0), r);
            tc::tmemLoadWait();
            emitChunk(r, c0);
          }
        }
      }
      // hand the accumulator back to the MMA warp (of CTA 0)
      tc::fenceBeforeThreadSync();
      __syncwarp();
      if (lane == 0) {
        if constexpr (CTAS == 2) tc::mbarArriveCluster(leaderBars + 8u * (2 * p.stages + 2 + a));
        else tc::mbarArrive(tmemEmptyBar(a));
      }
      if constexpr (COMM == kCommRS) {
        if (dstRank != p.rank) {
          // this warp's 32 rows of the tile are in the peer's memory: publish them
          __syncwarp();
          if (lane == 0) {
            uint64_t* f = p.tileReady[dstRank] + ((size_t(p.rank) * perRank + (mBlk % perRank)) * p.tilesN + nBlk) * 4 + quarter;
            sig::stReleaseSys(f, epoch);
          }
        }
      }
    }
  } else {
    // ------------------------------- communication warps (all-gather push) -------------------------------
    if constexpr (COMM == kCommAG) {
      const int ct = threadIdx.x - 32 * (2 + kEpiWarps), cn = 32 * p.commWarps;   // p.commWarps of the 4 warps push
      if (ct < cn) {
      const int perRank = p.blocksPerRank * CTAS;
      const size_t blockBytes = size_t(kBM) * p.K * 2;
      const int items = (p.world - 1) * perRank * p.pushParts;
      for (int item = blockIdx.x; item < items; item += gridDim.x) {
        const int unit = item / p.pushParts, part = item % p.pushParts;
        const int peer = (p.rank + 1 + unit / perRank) % p.world, b = unit % perRank;
        const Span sp = partitionAligned(blockBytes, p.pushParts, part, kAccessAlign);
        const unsigned char* src = reinterpret_cast<const unsigned char*>(p.localA) + size_t(b) * blockBytes + sp.offset;
        unsigned char* dst = reinterpret_cast<unsigned char*>(p.gatherBuf[peer]) + size_t(parity) * p.gatherParityBytes + (size_t(p.rank) * perRank + b) * blockBytes + sp.offset;
        const size_t n = sp.bytes / 32;
        size_t i = ct;
        for (; i + 3 * size_t(cn) < n; i += 4 * size_t(cn)) {
          Vec32 v[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) v[u] = ld32(src + (i + size_t(u) * cn) * 32);
#pragma unroll
          for (int u = 0; u < 4; ++u) st32(dst + (i + size_t(u) * cn) * 32, v[u]);
        }
        for (; i < n; i += cn) st32(dst + i * 32, ld32(src + i * 32));
        asm volatile("bar.sync 1, %0;" ::"r"(cn) : "memory");
        if (ct == 0 && sig::lastArrival(p.pushCounters + unit, uint32_t(p.pushParts)))
          sig::stReleaseSys(p.rowReady[peer] + size_t(p.rank) * perRank + b, epoch);
      }
      }
    }
  }

  // ------------------------------- teardown -------------------------------
  if (*abortWord) __nanosleep(20000);   // let copies already in flight land before shared memory and TMEM go away
  tc::fenceBeforeThreadSync();
  if constexpr (CTAS == 2) tc::clusterSync(); else __syncthreads();   // neither CTA frees TMEM the pair's MMA still writes
  if (warp == 1) {
    if constexpr (CTAS == 2) tc::tmemDeallocPair(tmemBase, kTmemCols);
    else tc::tmemDealloc(tmemBase, kTmemCols);
  }
  if constexpr (COMM != kCommNone) {
    if (threadIdx.x == 0) {
      __threadfence();
      if (atomicAdd(p.exitCounter, 1u) == gridDim.x - 1) { *p.exitCounter = 0; *p.epoch = epoch; __threadfence(); }
    }
  }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encodeFn() {
  static EncodeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
    return reinterpret_cast<EncodeFn>(p);
  }();
  return fn;
}

// [rows, cols] bf16 row-major; box = boxRows x 64 columns, 128-byte swizzle
bool makeMap(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint32_t boxRows) {
  EncodeFn fn = encodeFn();
  if (!fn) { setError("cuTensorMapEncodeTiled is not available from this driver"); return false; }
  if (reinterpret_cast<uintptr_t>(ptr) % 16 || (cols * 2) % 16) { setError("TMA operands need 16-byte aligned base and row pitch"); return false; }
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {uint32_t(kBK), boxRows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { setError("cuTensorMapEncodeTiled failed with code " + std::to_string(int(r))); return false; }
  return true;
}

int smCount() {
  static int n = [] { int d = 0, v = 148; cudaGetDevice(&d); cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, d); return v; }();
  return n;
}

// tile width: fewest idle SMs in the last wave, then the widest tile
int chooseBn(int M, int N, int epilogue) {
  const int tilesM = (M + kBM - 1) / kBM, sms = smCount();
  int best = 256; double bestScore = -1;
  for (int bn : {256, 224, 192, 160, 128}) {
    if (epilogue == kEpiSwiglu && bn % 32) continue;
    if (N % bn && N > bn) continue;             // keep tiles whole when the problem allows it
    const long tiles = long(tilesM) * ((N + bn - 1) / bn);
    const long waves = (tiles + sms - 1) / sms;
    double score = double(tiles) / double(waves * sms);
    // measured on B200: narrower tiles re-read the A tile more often and lose tensor-pipe utilisation
    score *= bn == 256 ? 1.0 : bn == 224 ? 0.86 : bn == 192 ? 0.80 : bn == 160 ? 0.70 : 0.55;
    if (score > bestScore + 1e-9) { bestScore = score; best = bn; }
  }
  return best;
}

// a CTA pair per 256-row block when the rows allow it (and PURLIN_GEMM_SINGLE_CTA is not set)
int ctasFor(int M, int rowsPerRank) {
  static const bool single = std::getenv("PURLIN_GEMM_SINGLE_CTA") != nullptr;
  if (single) return 1;
  return (rowsPerRank % (2 * kBM) == 0 && M >= 2 * kBM) ? 2 : 1;
}

bool fillShape(Params& p, int M, int N, int K, int epilogue, int bn, int ctas, int scratchBytes = 0) {
  if (M <= 0 || N <= 0 || K <= 0) { setError("GEMM dimensions must be positive"); return false; }
  if (K % 8 || N % 8) { setError("N and K must be multiples of 8"); return false; }
  if (bn == 0) bn = chooseBn(M, N, epilogue);
  if (bn % 16 || bn < 16 || bn > kMaxBN || (epilogue == kEpiSwiglu && bn % 32)) { setError("tile width must be a multiple of 16 (32 for SwiGLU) up to 256"); return false; }
  p.M = M; p.N = N; p.K = K; p.bn = bn;
  static const bool epiPipe = [] { const char* e = std::getenv("PURLIN_GEMM_EPI_PIPE"); return !e || e[0] != '0'; }();
  p.epiPipe = epiPipe ? 1 : 0;
  if (ctas == 2 && (bn / 2) % 8) { setError("a CTA pair needs a tile width that is a multiple of 16"); return false; }
  p.tilesM = (M + kBM * ctas - 1) / (kBM * ctas); p.tilesN = (N + bn - 1) / bn;
  const int stageBytes = kABytes + (bn / ctas) * kBK * 2;
  p.stages = std::min((kSmemLimit - kBarrierBytes - 1024 - scratchBytes) / stageBytes, kMaxStages);
  return true;
}
size_t smemFor(const Params& p, int ctas) { return size_t(p.stages) * (kABytes + (p.bn / ctas) * kBK * 2) + kBarrierBytes + 1024 + (p.rsScratch ? kScratchBytes : 0); }

template <int EPI, int COMM, int CTAS>
int launchImpl(const Maps& maps, const Params& p, cudaStream_t stream) {
  auto kernel = gemmKernel<EPI, COMM, CTAS>;
  constexpr int threads = COMM == kCommAG ? kThreadsComm : kThreadsPlain;
  // shared-memory opt-in and cluster occupancy belong to the device's copy of the kernel: resolve them once per device
  static int perDevice[64];
  static bool seen[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) { setError("GEMM launch: no current device"); return 1; }
  int& maxClusters = perDevice[device];
  if (!seen[device]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit) != cudaSuccess) { setError("cannot opt in to 227 KiB of shared memory"); return 1; }
    seen[device] = true;
    maxClusters = smCount() / CTAS;
    if (CTAS == 2) {
      // pairs must sit on SMs of one GPC: ask how many pairs the device can hold at once
      cudaLaunchConfig_t q{};
      cudaLaunchAttribute qa[1];
      qa[0].id = cudaLaunchAttributeClusterDimension; qa[0].val.clusterDim.x = 2; qa[0].val.clusterDim.y = 1; qa[0].val.clusterDim.z = 1;
      q.gridDim = dim3(smCount() / 2 * 2); q.blockDim = dim3(threads); q.dynamicSmemBytes = kSmemLimit; q.attrs = qa; q.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kernel, &q) == cudaSuccess && n > 0) maxClusters = std::min(maxClusters, n);
    }
  }
  const int pairs = std::min(p.tilesM * p.tilesN, maxClusters);
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension; attr[0].val.clusterDim.x = CTAS; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.gridDim = dim3(pairs * CTAS); cfg.blockDim = dim3(threads); cfg.dynamicSmemBytes = smemFor(p, CTAS); cfg.stream = stream;
  cfg.attrs = attr; cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, maps, p);
  if (e != cudaSuccess) { setError(std::string("GEMM launch: ") + cudaGetErrorString(e)); return 1; }
  return 0;
}
template <int EPI, int COMM>
int launch(const Maps& maps, const Params& p, int ctas, cudaStream_t stream) {
  return ctas == 2 ? launchImpl<EPI, COMM, 2>(maps, p, stream) : launchImpl<EPI, COMM, 1>(maps, p, stream);
}

}  // namespace

struct PurlinTpContext {
  int rank = 0, world = 1, M = 0, kAg = 0, nRs = 0;
  unsigned char* peers[kMaxRanks] = {};
  size_t gatherOff[2] = {0, 0}, partialOff = 0, rowReadyOff = 0, tileReadyOff = 0, total = 0;
  size_t partialParityStride = 0;
  void* local = nullptr;     // epoch words, exit counters, status, push counters
  uint64_t timeoutNs = 0;
};

namespace {
struct TpLayout { size_t gather[2], partial, rowReady, tileReady, total, partialParityStride; };
TpLayout tpLayout(int world, int M, int kAg, int nRs) {
  TpLayout l{};
  size_t off = 0;
  const size_t g = roundUp(size_t(M) * kAg * 2, 1024);
  l.gather[0] = off; off += g;
  l.gather[1] = off; off += g;
  const size_t part = roundUp(size_t(M) * nRs * 2, 1024);    // [world slots][M / world rows][nRs]
  l.partial = off; off += 2 * part;
  l.partialParityStride = part / 2;                           // in elements
  l.rowReady = off; off += roundUp(size_t((M + kBM - 1) / kBM) * 8, 1024);
  const size_t tilesNmax = size_t(nRs + 15) / 16;             // narrowest tile
  l.tileReady = off; off += roundUp(size_t((M + kBM - 1) / kBM) * tilesNmax * 4 * 8, 1024);
  l.total = off;
  (void)world;
  return l;
}
}  // namespace

extern "C" {

int purlin_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int epilogue, int bn, uint32_t* status, void* stream) {
  NvtxRange range(epilogue == kEpiSwiglu ? "gemmSwiglu" : "gemm", size_t(M) * size_t(N) * 2);
  Params p{};
  const int ctas = ctasFor(M, M);
  if (!fillShape(p, M, N, K, epilogue, bn, ctas)) return 1;
  Maps maps{};
  if (!makeMap(&maps.a, A, uint64_t(M), uint64_t(K), kBM)) return 1;
  if (!makeMap(&maps.b, B, uint64_t(N), uint64_t(K), uint32_t(p.bn / ctas))) return 1;
  maps.aLocal = maps.a;
  p.C = static_cast<__nv_bfloat16*>(C);
  p.ldc = epilogue == kEpiSwiglu ? N / 2 : N;
  p.status = status;
  p.timeoutNs = 2ull * 1000 * 1000 * 1000;
  p.rank = 0; p.world = 1; p.blocksPerRank = p.tilesM;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return epilogue == kEpiSwiglu ? launch<kEpiSwiglu, kCommNone>(maps, p, ctas, s) : launch<kEpiStore, kCommNone>(maps, p, ctas, s);
}

size_t purlin_tp_workspace_bytes(int world, int M, int kAg, int nRs) { return tpLayout(world, M, kAg, nRs).total; }

PurlinTpContext* purlin_tp_create(int rank, int world, const uint64_t* peerPtrs, int M, int kAg, int nRs, uint64_t timeoutNs, void* stream) {
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world) { setError("invalid rank or world size"); return nullptr; }
  if (M % (world * kBM)) { setError("rows per rank must be a multiple of 128"); return nullptr; }
  auto* c = new PurlinTpContext();
  c->rank = rank; c->world = world; c->M = M; c->kAg = kAg; c->nRs = nRs;
  const TpLayout l = tpLayout(world, M, kAg, nRs);
  c->gatherOff[0] = l.gather[0]; c->gatherOff[1] = l.gather[1]; c->partialOff = l.partial;
  c->rowReadyOff = l.rowReady; c->tileReadyOff = l.tileReady; c->total = l.total; c->partialParityStride = l.partialParityStride;
  for (int q = 0; q < world; ++q) {
    if (!peerPtrs[q] || peerPtrs[q] % 1024) { delete c; setError("peer blocks must be non-null and 1024-byte aligned"); return nullptr; }
    c->peers[q] = reinterpret_cast<unsigned char*>(peerPtrs[q]);
  }
  c->timeoutNs = timeoutNs ? timeoutNs : 10ull * 1000 * 1000 * 1000;
  const size_t localBytes = 4096 + size_t(kMaxRanks) * ((M + kBM - 1) / kBM) * 4;
  if (cudaMalloc(&c->local, localBytes) != cudaSuccess) { delete c; setError("cudaMalloc failed"); return nullptr; }
  cudaMemsetAsync(c->local, 0, localBytes, static_cast<cudaStream_t>(stream));
  cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  return c;
}

int purlin_tp_destroy(PurlinTpContext* c, void* stream) {
  if (!c) return 0;
  cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (c->local) cudaFree(c->local);
  delete c;
  return 0;
}

// local block: [0] AG epoch, [64] AG exit counter, [128] RS epoch, [192] RS exit counter, [256] status[4], [4096...] push counters
int purlin_tp_status(PurlinTpContext* c, uint32_t* out4, void* stream) {
  cudaMemcpyAsync(out4, static_cast<unsigned char*>(c->local) + 256, 16, cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
  return cudaStreamSynchronize(static_cast<cudaStream_t>(stream)) == cudaSuccess ? 0 : 1;
}
int purlin_tp_clear_status(PurlinTpContext* c, void* stream) {
  return cudaMemsetAsync(static_cast<unsigned char*>(c->local) + 256, 0, 16, static_cast<cudaStream_t>(stream)) == cudaSuccess ? 0 : 1;
}

int purlin_tp_ag_gemm(PurlinTpContext* c, const void* xLocal, const void* W, void* out, int M, int N, int K, int epilogue, void* stream) {
  NvtxRange range(epilogue == kEpiSwiglu ? "allGatherGemmSwiglu" : "allGatherGemm", size_t(M) * size_t(K) * 2);   // gathered bytes
  if (M > c->M || K > c->kAg || M % (c->world * kBM)) { setError("all-gather GEMM shape exceeds the workspace or rows per rank are not a multiple of 128"); return 1; }
  Params p{};
  const int ctas = ctasFor(M, M / c->world);
  if (!fillShape(p, M, N, K, epilogue, 0, ctas)) return 1;
  unsigned char* lb = static_cast<unsigned char*>(c->local);
  p.rank = c->rank; p.world = c->world; p.blocksPerRank = M / c->world / (kBM * ctas);
  p.epoch = reinterpret_cast<uint64_t*>(lb); p.exitCounter = reinterpret_cast<uint32_t*>(lb + 64);
  p.status = reinterpret_cast<uint32_t*>(lb + 256); p.timeoutNs = c->timeoutNs;
  p.pushCounters = reinterpret_cast<uint32_t*>(lb + 4096);
  p.pushParts = 8;
  {
    // Few pushing warps per CTA pace the remote stores: a saturated NVLink store queue stalls every memory
    // instruction of its SM, the epilogue's included. PURLIN_AG_COMM_WARPS overrides (1..4).
    const char* e = std::getenv("PURLIN_AG_COMM_WARPS");
    p.commWarps = e ? std::min(std::max(std::atoi(e), 1), kCommWarps) : 1;
    if (const char* pp = std::getenv("PURLIN_AG_PUSH_PARTS")) p.pushParts = std::min(std::max(std::atoi(pp), 1), 64);
  }
  p.localA = static_cast<const __nv_bfloat16*>(xLocal);
  p.C = static_cast<__nv_bfloat16*>(out); p.ldc = epilogue == kEpiSwiglu ? N / 2 : N;
  // the host cannot know the device epoch (graph replays advance it): pass the maps of both gather buffers
  Maps maps{};
  if (!makeMap(&maps.a, c->peers[c->rank] + c->gatherOff[0], uint64_t(M), uint64_t(K), kBM)) return 1;
  if (!makeMap(&maps.a1, c->peers[c->rank] + c->gatherOff[1], uint64_t(M), uint64_t(K), kBM)) return 1;
  p.gatherParityBytes = c->gatherOff[1] - c->gatherOff[0];
  if (!makeMap(&maps.aLocal, xLocal, uint64_t(M / c->world), uint64_t(K), kBM)) return 1;
  if (!makeMap(&maps.b, W, uint64_t(N), uint64_t(K), uint32_t(p.bn / ctas))) return 1;
  for (int q = 0; q < c->world; ++q) {
    p.gatherBuf[q] = reinterpret_cast<__nv_bfloat16*>(c->peers[q] + c->gatherOff[0]);
    p.rowReady[q] = reinterpret_cast<uint64_t*>(c->peers[q] + c->rowReadyOff);
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return epilogue == kEpiSwiglu ? launch<kEpiSwiglu, kCommAG>(maps, p, ctas, s) : launch<kEpiStore, kCommAG>(maps, p, ctas, s);
}

int purlin_tp_gemm_rs(PurlinTpContext* c, const void* A, const void* W, void* out, int M, int N, int K, void* stream) {
  NvtxRange range("gemmReduceScatter", size_t(M) * size_t(N) * 2);   // bytes of the tensor that is reduce-scattered
  if (M > c->M || N > c->nRs || M % (c->world * kBM)) { setError("GEMM reduce-scatter shape exceeds the workspace or rows per rank are not a multiple of 128"); return 1; }
  Params p{};
  const int ctas = ctasFor(M, M / c->world);
  const int scratch = std::getenv("PURLIN_RS_DIRECT_STORES") ? 0 : 1;
  if (!fillShape(p, M, N, K, kEpiStore, 0, ctas, scratch ? kScratchBytes : 0)) return 1;
  p.rsScratch = scratch;
  unsigned char* lb = static_cast<unsigned char*>(c->local);
  p.rank = c->rank; p.world = c->world; p.blocksPerRank = M / c->world / (kBM * ctas);
  p.epoch = reinterpret_cast<uint64_t*>(lb + 128); p.exitCounter = reinterpret_cast<uint32_t*>(lb + 192);
  p.status = reinterpret_cast<uint32_t*>(lb + 256); p.timeoutNs = c->timeoutNs;
  p.C = static_cast<__nv_bfloat16*>(out); p.ldc = N;
  p.partialParityStride = c->partialParityStride;
  Maps maps{};
  if (!makeMap(&maps.a, A, uint64_t(M), uint64_t(K), kBM)) return 1;
  maps.aLocal = maps.a;
  if (!makeMap(&maps.b, W, uint64_t(N), uint64_t(K), uint32_t(p.bn / ctas))) return 1;
  for (int q = 0; q < c->world; ++q) {
    p.partialBuf[q] = reinterpret_cast<__nv_bfloat16*>(c->peers[q] + c->partialOff);
    p.tileReady[q] = reinterpret_cast<uint64_t*>(c->peers[q] + c->tileReadyOff);
  }
  return launch<kEpiStore, kCommRS>(maps, p, ctas, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
