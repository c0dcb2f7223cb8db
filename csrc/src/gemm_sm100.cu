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
//   warp 1      MMA issuer     one thread issues tcgen05.mma (128 x bn x 16) into the TMEM accumulators
//                              ACCS = 1: tiles alternate between two accumulators (epilogue of tile t under tile t+1)
//                              ACCS = 2: a tile is two accumulators tall (two blocks of A rows against one block of B):
//                                        a third fewer operand bytes per flop, and consecutive MMAs alternate between
//                                        the accumulators while they share the B operand, which the tensor pipe rewards
//                                        (measured on B200: +13 % over back-to-back MMAs into one accumulator)
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
// The epilogue's staging tiles: every epilogue warp owns kStageTiles tiles of 32 rows x 64 output columns (bf16, 128-byte rows,
// 128-byte swizzle), filled from its TMEM lanes and drained row-contiguously: by a TMA store, by coalesced stores into
// a peer's memory, or by the owner's sum over the peers' partial tiles.
constexpr int kStageTileBytes = 32 * 128;
constexpr int kStageTiles = 4;                  // per warp: up to three TMA stores in flight while the fourth tile is filled
constexpr int kStagingBytes = kEpiWarps * kStageTiles * kStageTileBytes;   // 64 KiB

enum { kEpiStore = 0, kEpiSwiglu = 1 };
enum { kCommNone = 0, kCommAG = 1, kCommRS = 2 };

struct Params {
  int M, N, K, bn, stages;             // bn: columns of a tile (one MMA); a tile is ACCS x CTAS x 128 rows tall
  int tilesM, tilesN;
  int items, fullItems;                // work items: tiles [0, fullItems) whole, then the remaining tiles as single-accumulator halves
  __nv_bfloat16* C;
  int ldc;
  uint32_t* status;
  uint64_t timeoutNs;
  // tensor parallel
  int rank, world, blocksPerRank;      // blocksPerRank = rows per rank / rows per tile
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
};

struct alignas(64) Maps { CUtensorMap a, b, aLocal, a1, c; };   // a1: gather buffer of odd calls (all-gather variant); c: output, 64 x 32 boxes

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
PURLIN_D float silu(float x) { return __fdividef(x, 1.f + __expf(-x)); }

PURLIN_D void stShared16(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
PURLIN_D Vec16 ldShared16(uint32_t addr) {
  Vec16 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x[0]), "=r"(v.x[1]), "=r"(v.x[2]), "=r"(v.x[3]) : "r"(addr) : "memory");
  return v;
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


// The owner's sum over one staging tile: this rank's own partial (bf16, in shared memory) and every peer's partial tile
// (in this GPU's receive buffer), added in ascending rank order in fp32. A lane handles 16 bytes of a row; an access of
// the warp covers four rows x 128 contiguous bytes. ROWS row groups (of the 8) are in flight at a time.
template <int ROWS, int QMAX>
PURLIN_D void ownerSum(uint32_t buf, const __nv_bfloat16* peer0, size_t slotStride, int ldPartial, __nv_bfloat16* out0, int ldo,
                       int rank, int world, int rowInGroup, int piece, bool colOk) {
#pragma unroll 1
  for (int i = 0; i < 8; i += ROWS) {
    Vec16 own[ROWS], v[ROWS][QMAX];
#pragma unroll
    for (int h = 0; h < ROWS; ++h) {
      const int rr = 4 * (i + h) + rowInGroup;
      own[h] = ldShared16(buf + uint32_t(rr) * 128u + (uint32_t(piece ^ (rr & 7)) << 4));
#pragma unroll
      for (int q = 0; q < QMAX; ++q)
        if (q < world && q != rank && colOk) v[h][q] = ld16(peer0 + size_t(q) * slotStride + size_t(rr) * ldPartial);
    }
#pragma unroll
    for (int h = 0; h < ROWS; ++h) {
      const int rr = 4 * (i + h) + rowInGroup;
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
      for (int q = 0; q < QMAX; ++q) {
        if (q < world) {
          const Vec16 w = q == rank ? own[h] : v[h][q];
#pragma unroll
          for (int e = 0; e < 4; ++e) { acc[2 * e] += bf16lo(w.x[e]); acc[2 * e + 1] += bf16hi(w.x[e]); }
        }
      }
      if (colOk) st16(out0 + size_t(rr) * ldo, Vec16{{packBf16(acc[0], acc[1]), packBf16(acc[2], acc[3]), packBf16(acc[4], acc[5]), packBf16(acc[6], acc[7])}});
    }
  }
}

// Work item i -> tile and the accumulators (row blocks) of it that the item covers. With two accumulators per tile the
// tiles of a small last wave are issued as halves (one accumulator each): the tail costs half a wave instead of a whole one.
template <int ACCS>
PURLIN_D void itemOf(const Params& p, int i, int& tile, int& first, int& count) {
  if (ACCS == 1 || i < p.fullItems) { tile = i; first = 0; count = ACCS; }
  else { const int j = i - p.fullItems; tile = p.fullItems + (j >> 1); first = j & 1; count = 1; }
}

// CTAS = 1: every CTA owns 128 x bn tiles. CTAS = 2: a cluster of two CTAs owns 256-row tiles; each CTA loads its
// 128 rows of A and its half of B's columns, CTA 0 issues one 256-row MMA for the pair (cta_group::2), so every
// byte of B crosses L2 -> shared memory once per 256 rows instead of once per 128.
// ACCS = 2 (pairs only): the tile is 2 x 256 rows tall; each k-block of B meets two blocks of A, one per accumulator.
template <int EPI, int COMM, int CTAS, int ACCS>
__global__ void __launch_bounds__(COMM == kCommAG ? kThreadsComm : kThreadsPlain, 1)
gemmKernel(const __grid_constant__ Maps maps, const __grid_constant__ Params p) {
  extern __shared__ unsigned char smemRaw[];
  const uint32_t rawAddr = tc::smemAddr(smemRaw);
  const uint32_t base = (rawAddr + 1023u) & ~1023u;          // swizzled tiles need 1024-byte alignment
  unsigned char* smem = smemRaw + (base - rawAddr);
  const int bnLocal = p.bn / CTAS;                           // B columns of one accumulator this CTA keeps in shared memory
  const int bBytes = bnLocal * kBK * 2;
  const int stageBytes = ACCS * kABytes + bBytes;            // [A block 0][A block 1][B]
  const int perRank128 = p.blocksPerRank * ACCS * CTAS;      // 128-row blocks per rank
  const uint32_t stagingAll = base + uint32_t(p.stages) * stageBytes;     // 1024-byte aligned: stages are multiples of 8 KiB
  const uint32_t barBase = stagingAll + kStagingBytes;
  // barrier block: full[stages], empty[stages], tmemFull[2], tmemEmpty[2], then the TMEM base word and the abort word
  auto fullBar = [&](int s) { return barBase + 8u * s; };
  auto emptyBar = [&](int s) { return barBase + 8u * (p.stages + s); };
  auto tmemFullBar = [&](int a) { return barBase + 8u * (2 * p.stages + a); };
  auto tmemEmptyBar = [&](int a) { return barBase + 8u * (2 * p.stages + 2 + a); };
  uint32_t* words = reinterpret_cast<uint32_t*>(smem + size_t(p.stages) * stageBytes + kStagingBytes + 8 * (2 * p.stages + 4));
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

  const int numItems = p.items;                              // tiles count (CTAS x 128)-row blocks
  const int kBlocks = (p.K + kBK - 1) / kBK;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      uint32_t st = 0, ph = 0;          // ring position and its phase
      uint64_t seenReady = 0;           // row blocks whose arrival flag this thread has already acquired
      bool ok = true;
      // operand coordinates of a work item: which map A comes from, the first row of this CTA's first A block, B's first row
      struct Coords { const CUtensorMap* aMap; int aRow, bRow, accCount, mBlk, tile; bool remote; };
      auto coordsOf = [&](int it) {
        Coords c;
        int accFirst, mIdx, nBlk;
        itemOf<ACCS>(p, it, c.tile, accFirst, c.accCount);
        tileCoord<COMM>(p, c.tile, mIdx, nBlk);
        // this CTA's 128-row block of the item's first accumulator; the second accumulator's block is CTAS blocks further
        c.mBlk = (rowBlockOf<COMM>(p, mIdx) * ACCS + accFirst) * CTAS + int(ctaRank);
        c.bRow = nBlk * p.bn + int(ctaRank) * bnLocal;
        c.aMap = &maps.a; c.aRow = c.mBlk * kBM; c.remote = false;
        if constexpr (COMM == kCommAG) {
          if (parity) c.aMap = &maps.a1;
          if (c.mBlk / perRank128 == p.rank) { c.aMap = &maps.aLocal; c.aRow = (c.mBlk % perRank128) * kBM; }   // own rows: the caller's tensor
          else c.remote = true;
        }
        return c;
      };
      for (int it = pairIdx; it < numItems && ok; it += numPairs) {
        const Coords c = coordsOf(it);
        if constexpr (COMM == kCommAG) {
          if (c.remote) {
            // rows pushed by a peer: wait for each block's flag, then order those generic-proxy writes
            // before this thread's async-proxy reads (TMA)
            for (int a = 0; a < c.accCount && ok; ++a) {
              const int mBlk = c.mBlk + a * CTAS;
              if (mBlk >= 64 || !((seenReady >> mBlk) & 1ull)) {   // a block seen once stays ready for the whole call
                ok = waitFlag(p.rowReady[p.rank] + mBlk, epoch, abortWord, p.timeoutNs);
                if (!ok) { recordTimeout(p, 4, mBlk, 0); break; }
                tc::fenceProxyAsync();
                if (mBlk < 64) seenReady |= 1ull << mBlk;
              }
            }
            if (!ok) break;
          }
        }
        for (int kb = 0; kb < kBlocks; ++kb) {
          ok = tc::mbarWait(emptyBar(st), ph ^ 1, abortWord, p.timeoutNs);
          if (!ok) { recordTimeout(p, 1, c.tile, kb); break; }
          const uint32_t sA = base + st * uint32_t(stageBytes), sB = sA + ACCS * kABytes;
          if constexpr (CTAS == 2) {
            // both CTAs' bytes are credited to CTA 0's barrier; CTA 0 announces the total
            const uint32_t leaderFull = leaderBars + 8u * st;
            if (ctaRank == 0) tc::mbarExpectTx(fullBar(st), uint32_t(2 * (c.accCount * kABytes + bBytes)));
#pragma unroll
            for (int a = 0; a < ACCS; ++a)
              if (a < c.accCount) tc::tmaLoad2dPair(sA + uint32_t(a * kABytes), c.aMap, kb * kBK, c.aRow + a * CTAS * kBM, leaderFull);
            tc::tmaLoad2dPair(sB, &maps.b, kb * kBK, c.bRow, leaderFull);
          } else {
            tc::mbarExpectTx(fullBar(st), uint32_t(stageBytes));
            tc::tmaLoad2d(sA, c.aMap, kb * kBK, c.aRow, fullBar(st));
            tc::tmaLoad2d(sB, &maps.b, kb * kBK, c.bRow, fullBar(st));
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
      const uint64_t descA0 = tc::smemDescSw128(base), descB0 = tc::smemDescSw128(base + ACCS * kABytes);
      const uint32_t stageStep = uint32_t(stageBytes) >> 4, accStep = uint32_t(kABytes) >> 4;
      uint32_t st = 0, ph = 0;
      uint32_t accIt = 0;
      uint32_t use0 = 0, use1 = 0;          // how often each accumulator slot has been used: barrier phase = uses & 1
      bool ok = true;
      auto releaseStage = [&](uint32_t stg) {   // the stage is free (in both CTAs) once the MMAs issued so far have read it
        if constexpr (CTAS == 2) { tc::mmaCommitPair(leaderBars + 8u * (p.stages + stg)); tc::mmaCommitPair(peerBars + 8u * (p.stages + stg)); }
        else tc::mmaCommit(emptyBar(stg));
      };
      auto accumulatorDone = [&](int a) {      // the accumulator is complete once every MMA issued so far is done
        if constexpr (CTAS == 2) { tc::mmaCommitPair(leaderBars + 8u * (2 * p.stages + a)); tc::mmaCommitPair(peerBars + 8u * (2 * p.stages + a)); }
        else tc::mmaCommit(tmemFullBar(a));
      };
      for (int it = pairIdx; it < numItems && ok; it += numPairs, ++accIt) {
        int t, accFirst, accCount;
        itemOf<ACCS>(p, it, t, accFirst, accCount);
        // ACCS = 1: tiles alternate between the slots. ACCS = 2: slot 0 and slot 1 of one tile (a half tile uses slot 0).
        const int a0 = ACCS == 1 ? int(accIt & 1) : 0;
        const bool two = ACCS == 2 && accCount == 2;
        // the epilogues must have drained the accumulators this item writes
        ok = tc::mbarWait(tmemEmptyBar(a0), ((a0 ? use1 : use0) & 1) ^ 1, abortWord, p.timeoutNs);
        if (ok && two) ok = tc::mbarWait(tmemEmptyBar(1), (use1 & 1) ^ 1, abortWord, p.timeoutNs);
        if (!ok) { recordTimeout(p, 2, t, 0); break; }
        const uint32_t d0 = tmemBase + uint32_t(a0) * kAccStride, d1 = tmemBase + kAccStride;
        for (int kb = 0; kb < kBlocks; ++kb) {
          ok = tc::mbarWait(fullBar(st), ph, abortWord, p.timeoutNs);
          if (!ok) { recordTimeout(p, 3, t, kb); break; }
          tc::fenceAfterThreadSync();
          const uint64_t da = descA0 + uint64_t(st * stageStep), db = descB0 + uint64_t(st * stageStep);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            const uint32_t accumulate = uint32_t((kb | k) != 0);
            if constexpr (CTAS == 2) {
              tc::mmaPair(d0, da + 2 * k, db + 2 * k, idesc, accumulate);
              // the second accumulator: the other block of A rows against the same slice of B
              if constexpr (ACCS == 2) { if (two) tc::mmaPair(d1, da + accStep + 2 * k, db + 2 * k, idesc, accumulate); }
            } else {
              tc::mma(d0, da + 2 * k, db + 2 * k, idesc, accumulate);
            }
          }
          releaseStage(st);
          if (++st == uint32_t(p.stages)) { st = 0; ph ^= 1; }
        }
        if (ok) {
          accumulatorDone(a0);
          if (a0) ++use1; else ++use0;
          if (two) { accumulatorDone(1); ++use1; }
        }
      }
    }
  } else if (warp < 2 + kEpiWarps) {
    // ------------------------------- epilogue -------------------------------
    const int quarter = warp & 3;                // a warp may only touch TMEM lanes [32 * (warp % 4), +32)
    uint32_t accIt = 0;
    uint32_t use0 = 0, use1 = 0;
    uint32_t tileCount = 0;                      // staging tiles this warp has filled: they rotate through its buffers
    bool ok = true;
    for (int it = pairIdx; it < numItems && ok; it += numPairs, ++accIt) {
      int t, accFirst, accCount, mIdx, nBlk;
      itemOf<ACCS>(p, it, t, accFirst, accCount);
      tileCoord<COMM>(p, t, mIdx, nBlk);
      const int rowBlk = rowBlockOf<COMM>(p, mIdx);
      const int n0 = nBlk * p.bn;

#pragma unroll 1
      for (int ai = 0; ai < accCount && ok; ++ai) {
      const int a = ACCS == 1 ? int(accIt & 1) : ai;      // accumulator slot
      const int mBlk = (rowBlk * ACCS + accFirst + ai) * CTAS + int(ctaRank);   // this CTA's 128-row block of the accumulator
      const int rowInTile = quarter * 32 + lane;
      const int row = mBlk * kBM + rowInTile;
      int dstRank = p.rank, rowInShard = row;
      const __nv_bfloat16* partialBase = nullptr;   // slot 0 of this row inside the receive buffer
      size_t slotStride = 0;
      bool reduceOwn = false;
      if constexpr (COMM == kCommRS) {
        dstRank = mBlk / perRank128;
        rowInShard = row - dstRank * perRank128 * kBM;
        reduceOwn = dstRank == p.rank && p.world > 1;
        if (reduceOwn) {
          slotStride = size_t(perRank128) * kBM * p.N;
          partialBase = p.partialBuf[p.rank] + size_t(parity) * p.partialParityStride + size_t(rowInShard) * p.N;
          // every peer's partial of this tile (this row quarter) must have landed
          int good = 1;
          if (lane < p.world && lane != p.rank) {
            const uint64_t* f = p.tileReady[p.rank] + ((size_t(lane) * perRank128 + (mBlk % perRank128)) * p.tilesN + nBlk) * 4 + quarter;
            good = waitFlag(f, epoch, abortWord, p.timeoutNs) ? 1 : 0;
          }
          ok = __all_sync(0xffffffffu, good);
          if (!ok) { if (lane == 0) recordTimeout(p, 6, t, ai); break; }
        }
      }
      ok = tc::mbarWait(tmemFullBar(a), (a ? use1 : use0) & 1, abortWord, p.timeoutNs);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { if (lane == 0) recordTimeout(p, 5, t, ai); break; }
      if (a) ++use1; else ++use0;
      tc::fenceAfterThreadSync();
      const uint32_t taddr = tmemBase + (uint32_t(quarter * 32) << 16) + uint32_t(a) * kAccStride;

      // Where this warp's 32 rows go: `outRow0` is the row of lane 0 at output column 0, `ldo` its pitch in elements.
      constexpr int kOut = EPI == kEpiSwiglu ? 16 : 32;     // output columns per 32 accumulator columns
      constexpr int kPerTile = 64 / kOut;                    // TMEM chunks per staging tile
      const int outBound = EPI == kEpiSwiglu ? p.N / 2 : p.N;
      const int outCol0 = EPI == kEpiSwiglu ? n0 / 2 : n0;
      const int perRank = perRank128;
      const int row0 = row - lane;
      const bool remote = COMM == kCommRS && dstRank != p.rank;
      const int ldo = COMM == kCommRS ? (remote ? p.N : p.ldc) : p.ldc;
      __nv_bfloat16* outRow0;
      if (remote) outRow0 = p.partialBuf[dstRank] + size_t(parity) * p.partialParityStride + (size_t(p.rank) * perRank * kBM + size_t(rowInShard - lane)) * p.N;
      else if (COMM == kCommRS) outRow0 = p.C + size_t(rowInShard - lane) * p.ldc;
      else outRow0 = p.C + size_t(row0) * p.ldc;
      const int rowsValid = COMM == kCommRS ? 32 : (p.M - row0 < 32 ? p.M - row0 : 32);    // rows of this warp inside the output
      const int nChunks = p.bn / 32;

      // 32 accumulator columns of this lane's row -> bf16 (activated) -> chunk `slot` of the staging tile
      const uint32_t stagingWarp = stagingAll + uint32_t(warp - 2) * uint32_t(kStageTiles * kStageTileBytes);
      auto stageChunk = [&](const uint32_t (&r)[32], uint32_t buf, int slot) {
        uint32_t o[kOut / 2];
        if constexpr (EPI == kEpiSwiglu) {
          // columns [0, 16) are gate, [16, 32) are up, both for the same 16 output columns
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float g0 = __uint_as_float(r[2 * i]), g1 = __uint_as_float(r[2 * i + 1]);
            const float u0 = __uint_as_float(r[16 + 2 * i]), u1 = __uint_as_float(r[16 + 2 * i + 1]);
            o[i] = packBf16(silu(g0) * u0, silu(g1) * u1);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = packBf16(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
        }
        const uint32_t rowAddr = buf + uint32_t(lane) * 128u;
#pragma unroll
        for (int j = 0; j < kOut / 8; ++j) {
          const int chunk = slot * (kOut / 8) + j;
          stShared16(rowAddr + (uint32_t(chunk ^ (lane & 7)) << 4), o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
        }
      };

      // Software pipeline over the accumulator: the TMEM load of the next 32 columns is in flight while the current ones
      // are converted and staged; every kPerTile chunks a staging tile is full and is drained.
      uint32_t ra[32], rb[32];
      tc::tmemLoad32(taddr, ra);
#pragma unroll 1
      for (int c0 = 0; c0 < nChunks; c0 += kPerTile) {
        const uint32_t buf = stagingWarp + (tileCount % uint32_t(kStageTiles)) * kStageTileBytes;
        ++tileCount;
        // the TMA store that last read this tile (kStageTiles tiles ago) must be done reading it
        if (lane == 0) tc::bulkWaitGroupRead<kStageTiles - 1>();
        __syncwarp();
        int filled = 0;
#pragma unroll
        for (int sl = 0; sl < kPerTile; ++sl) {
          const int c = c0 + sl;
          if (c < nChunks) {
            if (sl % 2 == 0) {
              tc::tmemLoadWaitFor(ra);
              if (c + 1 < nChunks) tc::tmemLoad32(taddr + uint32_t((c + 1) * 32), rb);
              stageChunk(ra, buf, sl);
            } else {
              tc::tmemLoadWaitFor(rb);
              if (c + 1 < nChunks) tc::tmemLoad32(taddr + uint32_t((c + 1) * 32), ra);
              stageChunk(rb, buf, sl);
            }
            filled = sl + 1;
          }
        }
        // ---- drain the tile: output columns [oc, oc + cols) of the warp's 32 rows ----
        const int oc = outCol0 + (c0 / kPerTile) * 64, cols = filled * kOut;
        if (oc >= outBound || rowsValid <= 0) continue;
        if constexpr (COMM != kCommRS) {
          // a whole tile (or one whose unused columns fall outside the matrix, where the store is clipped) leaves by TMA
          if (cols == 64 || oc + cols >= outBound) {
            tc::fenceProxyAsyncShared();
            __syncwarp();
            if (lane == 0) { tc::tmaStore2d(&maps.c, oc, row0, buf); tc::bulkCommitGroup(); }
            continue;
          }
        }
        __syncwarp();
        const int rowInGroup = lane >> 3, piece = lane & 7;
        const bool colOk = piece * 8 < cols && oc + piece * 8 + 8 <= outBound;
        if (COMM == kCommRS && reduceOwn) {
          const __nv_bfloat16* peer0 = partialBase - size_t(lane) * p.N + oc + piece * 8;     // row of lane 0, slot 0, this lane's columns
          __nv_bfloat16* out0 = outRow0 + oc + piece * 8;
          if (p.world <= 8) ownerSum<2, 8>(buf, peer0, slotStride, p.N, out0, ldo, p.rank, p.world, rowInGroup, piece, colOk);
          else ownerSum<1, kMaxRanks>(buf, peer0, slotStride, p.N, out0, ldo, p.rank, p.world, rowInGroup, piece, colOk);
        } else {
          Vec16 v[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rr = 4 * i + rowInGroup;
            v[i] = ldShared16(buf + uint32_t(rr) * 128u + (uint32_t(piece ^ (rr & 7)) << 4));
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rr = 4 * i + rowInGroup;
            if (colOk && rr < rowsValid) st16(outRow0 + size_t(rr) * ldo + oc + piece * 8, v[i]);
          }
        }
        __syncwarp();
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
          // this warp's 32 rows of these columns are in the peer's memory: publish them
          __syncwarp();
          if (lane == 0) {
            uint64_t* f = p.tileReady[dstRank] + ((size_t(p.rank) * perRank + (mBlk % perRank)) * p.tilesN + nBlk) * 4 + quarter;
            sig::stReleaseSys(f, epoch);
          }
        }
      }
      }   // accumulators of the item
    }
    if (lane == 0) tc::bulkWaitGroup<0>();       // every TMA store of this warp has reached global memory
  } else {
    // ------------------------------- communication warps (all-gather push) -------------------------------
    if constexpr (COMM == kCommAG) {
      const int ct = threadIdx.x - 32 * (2 + kEpiWarps), cn = 32 * p.commWarps;   // p.commWarps of the 4 warps push
      if (ct < cn) {
      const int perRank = perRank128;
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

// [rows, cols] bf16 row-major; box = boxRows x 64 columns (128 bytes), 128-byte swizzle. Operands are loaded through
// such maps (128 or fewer rows per box), the output is stored through one with 32-row boxes (one epilogue warp's rows).
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

// Environment switches, read once per process (they select code paths for experiments, not per-call behaviour).
struct Switches {
  bool singleCta, oneAcc;
  int agCommWarps, agPushParts, rsAccs;
};
const Switches& switches() {
  static const Switches sw = [] {
    Switches v{};
    auto num = [](const char* name, int dflt) { const char* e = std::getenv(name); return e ? std::atoi(e) : dflt; };
    v.singleCta = std::getenv("PURLIN_GEMM_SINGLE_CTA") != nullptr;
    v.oneAcc = std::getenv("PURLIN_GEMM_ONE_ACC") != nullptr;
    // Few pushing warps per CTA pace the remote stores: a saturated NVLink store queue stalls every memory
    // instruction of its SM, the epilogue's included.
    v.agCommWarps = std::min(std::max(num("PURLIN_AG_COMM_WARPS", 1), 1), kCommWarps);
    v.agPushParts = std::min(std::max(num("PURLIN_AG_PUSH_PARTS", 8), 1), 64);
    // GEMM -> reduce-scatter keeps one accumulator per tile: its epilogue (stores into peers' memory, the owner's sum over the
    // peers' partial tiles) is long, and with two TMEM accumulators alternating between tiles it hides behind the next
    // tile's main loop. Measured on 2 x B200, 8192 x 8192 x K: K = 3584 391 us against 541 us with two accumulators per
    // tile, K = 7168 709 us against 783 us. PURLIN_RS_ACCS=2 selects the two-accumulator tile.
    v.rsAccs = num("PURLIN_RS_ACCS", 1);
    return v;
  }();
  return sw;
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
  if (switches().singleCta) return 1;
  return (rowsPerRank % (2 * kBM) == 0 && M >= 2 * kBM) ? 2 : 1;
}

struct Shape { int ctas, accs; };

bool fillShape(Params& p, Shape& sh, int M, int N, int K, int epilogue, int bn, int rowsPerRank, int accsWanted = 0) {
  if (M <= 0 || N <= 0 || K <= 0) { setError("GEMM dimensions must be positive"); return false; }
  if (K % 8 || N % 8) { setError("N and K must be multiples of 8"); return false; }
  const int ctas = ctasFor(M, rowsPerRank);
  if (bn == 0) bn = chooseBn(M, N, epilogue);
  if (bn % 32 || bn < 32 || bn > kMaxBN) { setError("tile width must be a multiple of 32 up to 256"); return false; }
  p.M = M; p.N = N; p.K = K; p.bn = bn;
  if (ctas == 2 && (bn / 2) % 8) { setError("a CTA pair needs a tile width that is a multiple of 16"); return false; }
  // two accumulators per tile (512 rows) whenever the rows allow it: a third fewer operand bytes per flop, and MMAs
  // that alternate between two accumulators while sharing B run faster than a chain into one accumulator
  const int accs = (ctas == 2 && !switches().oneAcc && accsWanted != 1 && 2 * bn <= kTmemCols && rowsPerRank % (4 * kBM) == 0 && M % (4 * kBM) == 0) ? 2 : 1;
  sh.ctas = ctas; sh.accs = accs;
  const int tileRows = kBM * ctas * accs;
  p.tilesM = (M + tileRows - 1) / tileRows; p.tilesN = (N + bn - 1) / bn;
  const int stageBytes = accs * kABytes + (bn / ctas) * kBK * 2;
  p.stages = std::min((kSmemLimit - kBarrierBytes - 1024 - kStagingBytes) / stageBytes, kMaxStages);
  if (p.stages < 2) { setError("GEMM tile does not leave room for two pipeline stages"); return false; }
  return true;
}
size_t smemFor(const Params& p, const Shape& sh) {
  return size_t(p.stages) * (sh.accs * kABytes + (p.bn / sh.ctas) * kBK * 2) + kStagingBytes + kBarrierBytes + 1024;
}

template <int EPI, int COMM, int CTAS, int ACCS>
int launchImpl(const Maps& maps, const Params& p, const Shape& sh, cudaStream_t stream) {
  auto kernel = gemmKernel<EPI, COMM, CTAS, ACCS>;
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
  const int tiles = p.tilesM * p.tilesN;
  const int pairs = std::min(tiles, maxClusters);
  Params q = p;
  q.items = q.fullItems = tiles;
  if (ACCS == 2) {
    // a last wave that fills at most half of the CTA pairs is issued as half tiles: half a wave instead of a whole one
    const int rest = tiles % pairs;
    if (tiles > pairs && rest > 0 && 2 * rest <= pairs) { q.fullItems = tiles - rest; q.items = q.fullItems + 2 * rest; }
  }
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension; attr[0].val.clusterDim.x = CTAS; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.gridDim = dim3(pairs * CTAS); cfg.blockDim = dim3(threads); cfg.dynamicSmemBytes = smemFor(p, sh); cfg.stream = stream;
  cfg.attrs = attr; cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, maps, q);
  if (e != cudaSuccess) { setError(std::string("GEMM launch: ") + cudaGetErrorString(e)); return 1; }
  return 0;
}
template <int EPI, int COMM>
int launch(const Maps& maps, const Params& p, const Shape& sh, cudaStream_t stream) {
  if (sh.ctas == 2) return sh.accs == 2 ? launchImpl<EPI, COMM, 2, 2>(maps, p, sh, stream) : launchImpl<EPI, COMM, 2, 1>(maps, p, sh, stream);
  return launchImpl<EPI, COMM, 1, 1>(maps, p, sh, stream);
}

// Tensor maps are pure functions of (pointer, rows, columns, box rows): encoding one costs about a microsecond of host
// time, and a fused call needs up to four, so each entry point keeps the maps of its last few operand sets.
struct MapKey {
  const void* ptr; uint64_t rows, cols; uint32_t box;
  bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && cols == o.cols && box == o.box; }
};
class MapCache {
 public:
  const CUtensorMap* get(const void* ptr, uint64_t rows, uint64_t cols, uint32_t box) {
    const MapKey k{ptr, rows, cols, box};
    for (int i = 0; i < kSlots; ++i) if (valid_[i] && keys_[i] == k) return &maps_[i];
    const int i = next_; next_ = (next_ + 1) % kSlots;
    valid_[i] = false;
    if (!makeMap(&maps_[i], ptr, rows, cols, box)) return nullptr;
    keys_[i] = k; valid_[i] = true;
    return &maps_[i];
  }
 private:
  static constexpr int kSlots = 16;
  alignas(64) CUtensorMap maps_[kSlots];
  MapKey keys_[kSlots] = {};
  bool valid_[kSlots] = {};
  int next_ = 0;
};

}  // namespace

struct PurlinTpContext {
  int rank = 0, world = 1, M = 0, kAg = 0, nRs = 0;
  unsigned char* peers[kMaxRanks] = {};
  size_t gatherOff[2] = {0, 0}, partialOff = 0, rowReadyOff = 0, tileReadyOff = 0, total = 0;
  size_t partialParityStride = 0;
  void* local = nullptr;     // epoch words, exit counters, status, push counters
  uint64_t timeoutNs = 0;
  MapCache maps;             // tensor maps of recent operand sets (the same tensors come back every step)
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
  Shape sh{};
  if (!fillShape(p, sh, M, N, K, epilogue, bn, M)) return 1;
  static thread_local MapCache cache;
  const CUtensorMap* ma = cache.get(A, uint64_t(M), uint64_t(K), kBM);
  const CUtensorMap* mb = ma ? cache.get(B, uint64_t(N), uint64_t(K), uint32_t(p.bn / sh.ctas)) : nullptr;
  const CUtensorMap* mc = mb ? cache.get(C, uint64_t(M), uint64_t(epilogue == kEpiSwiglu ? N / 2 : N), 32) : nullptr;
  if (!ma || !mb || !mc) return 1;
  Maps maps{};
  maps.a = *ma; maps.b = *mb; maps.aLocal = maps.a; maps.c = *mc;
  p.C = static_cast<__nv_bfloat16*>(C);
  p.ldc = epilogue == kEpiSwiglu ? N / 2 : N;
  p.status = status;
  p.timeoutNs = 2ull * 1000 * 1000 * 1000;
  p.rank = 0; p.world = 1; p.blocksPerRank = p.tilesM;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return epilogue == kEpiSwiglu ? launch<kEpiSwiglu, kCommNone>(maps, p, sh, s) : launch<kEpiStore, kCommNone>(maps, p, sh, s);
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
  Shape sh{};
  if (!fillShape(p, sh, M, N, K, epilogue, 0, M / c->world)) return 1;
  unsigned char* lb = static_cast<unsigned char*>(c->local);
  p.rank = c->rank; p.world = c->world; p.blocksPerRank = M / c->world / (kBM * sh.ctas * sh.accs);
  p.epoch = reinterpret_cast<uint64_t*>(lb); p.exitCounter = reinterpret_cast<uint32_t*>(lb + 64);
  p.status = reinterpret_cast<uint32_t*>(lb + 256); p.timeoutNs = c->timeoutNs;
  p.pushCounters = reinterpret_cast<uint32_t*>(lb + 4096);
  p.pushParts = switches().agPushParts;
  p.commWarps = switches().agCommWarps;
  p.localA = static_cast<const __nv_bfloat16*>(xLocal);
  p.C = static_cast<__nv_bfloat16*>(out); p.ldc = epilogue == kEpiSwiglu ? N / 2 : N;
  // the host cannot know the device epoch (graph replays advance it): pass the maps of both gather buffers
  const CUtensorMap* m0 = c->maps.get(c->peers[c->rank] + c->gatherOff[0], uint64_t(M), uint64_t(K), kBM);
  const CUtensorMap* m1 = m0 ? c->maps.get(c->peers[c->rank] + c->gatherOff[1], uint64_t(M), uint64_t(K), kBM) : nullptr;
  const CUtensorMap* ml = m1 ? c->maps.get(xLocal, uint64_t(M / c->world), uint64_t(K), kBM) : nullptr;
  const CUtensorMap* mb = ml ? c->maps.get(W, uint64_t(N), uint64_t(K), uint32_t(p.bn / sh.ctas)) : nullptr;
  const CUtensorMap* mc = mb ? c->maps.get(out, uint64_t(M), uint64_t(p.ldc), 32) : nullptr;
  if (!mc) return 1;
  Maps maps{};
  maps.a = *m0; maps.a1 = *m1; maps.aLocal = *ml; maps.b = *mb; maps.c = *mc;
  p.gatherParityBytes = c->gatherOff[1] - c->gatherOff[0];
  for (int q = 0; q < c->world; ++q) {
    p.gatherBuf[q] = reinterpret_cast<__nv_bfloat16*>(c->peers[q] + c->gatherOff[0]);
    p.rowReady[q] = reinterpret_cast<uint64_t*>(c->peers[q] + c->rowReadyOff);
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return epilogue == kEpiSwiglu ? launch<kEpiSwiglu, kCommAG>(maps, p, sh, s) : launch<kEpiStore, kCommAG>(maps, p, sh, s);
}

int purlin_tp_gemm_rs(PurlinTpContext* c, const void* A, const void* W, void* out, int M, int N, int K, void* stream) {
  NvtxRange range("gemmReduceScatter", size_t(M) * size_t(N) * 2);   // bytes of the tensor that is reduce-scattered
  if (M > c->M || N > c->nRs || M % (c->world * kBM)) { setError("GEMM reduce-scatter shape exceeds the workspace or rows per rank are not a multiple of 128"); return 1; }
  Params p{};
  Shape sh{};
  if (!fillShape(p, sh, M, N, K, kEpiStore, 0, M / c->world, switches().rsAccs)) return 1;
  unsigned char* lb = static_cast<unsigned char*>(c->local);
  p.rank = c->rank; p.world = c->world; p.blocksPerRank = M / c->world / (kBM * sh.ctas * sh.accs);
  p.epoch = reinterpret_cast<uint64_t*>(lb + 128); p.exitCounter = reinterpret_cast<uint32_t*>(lb + 192);
  p.status = reinterpret_cast<uint32_t*>(lb + 256); p.timeoutNs = c->timeoutNs;
  p.C = static_cast<__nv_bfloat16*>(out); p.ldc = N;
  p.partialParityStride = c->partialParityStride;
  const CUtensorMap* ma = c->maps.get(A, uint64_t(M), uint64_t(K), kBM);
  const CUtensorMap* mb = ma ? c->maps.get(W, uint64_t(N), uint64_t(K), uint32_t(p.bn / sh.ctas)) : nullptr;
  if (!mb) return 1;
  Maps maps{};
  maps.a = *ma; maps.aLocal = maps.a; maps.b = *mb;
  for (int q = 0; q < c->world; ++q) {
    p.partialBuf[q] = reinterpret_cast<__nv_bfloat16*>(c->peers[q] + c->partialOff);
    p.tileReady[q] = reinterpret_cast<uint64_t*>(c->peers[q] + c->tileReadyOff);
  }
  return launch<kEpiStore, kCommRS>(maps, p, sh, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
