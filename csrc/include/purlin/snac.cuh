// Stage, Notify And Consume: the device-side executor of a Plan.
//
// Behavioural parity with csrc/include/purlin/snac.cuh of the reference:
//   stage      (237-373)   copy into own staging, last CTA of a chunk notifies
//   consume    (809-938)   wait for the producer's flag, pull from its staging
//   reduce     (940-1133)  wait for every rank's flag, reduce the same slice of all
//   compose    (1984-2072) reduce into the seam, notify, gather every shard
//   packets    (1163-1955) latency regime: 16-byte flagged packets pushed to peers
//   arrival    (146-191)   variable-length collectives post and await an arrival packet
// What is different: the roles, offsets, chunking and flags come from a Plan
// computed on the host (layout.hpp) instead of template recursion; the same
// code runs production launches (one rank per GPU, context in kernel
// parameters) and single-GPU emulation (one grid row per rank, contexts in
// global memory); every wait is bounded.
#pragma once
#include "atom.cuh"
#include "bulk.cuh"
#include "packet.cuh"
#include "plan.hpp"

namespace purlin {

// What a device-side collective call needs besides the context
// (csrc/include/purlin/snac.cuh "SnacArgs" in the reference).
struct SnacArgs {
  const unsigned char* src;
  unsigned char* dst;
  const Plan* plan;
};

namespace snac {

struct Frame {
  uint64_t seq;
  int half;
  int bIdx;
  const unsigned char* src;
  unsigned char* dst;
  int unroll;
  int mmDepth;
  int bulkDepth;            // > 0: copy roles stream through the bulk-async ring in `smem`
  unsigned char* smem;
};

PURLIN_D size_t chunkLen(const Step& s, uint32_t k) {
  const size_t begin = size_t(k) * s.chunkBytes;
  return s.bytes - begin < s.chunkBytes ? s.bytes - begin : s.chunkBytes;
}
PURLIN_D size_t slotOff(const Step& s, uint32_t k) { return size_t(k % s.slots) * s.chunkBytes; }

// thread 0 waits, the whole CTA learns the outcome
PURLIN_D bool ctaWait(const Context& ctx, const uint64_t* flag, uint64_t value, uint32_t code, int step, int peer, uint32_t k) {
  int ok = 1;
  if (threadIdx.x == 0) ok = sig::waitAtLeast(ctx, flag, value, code, step, peer, k) ? 1 : 0;
  return __syncthreads_and(ok) != 0;
}
// thread q waits on flags[q] for every rank q (optionally skipping self)
PURLIN_D bool ctaWaitAll(const Context& ctx, uint64_t* const* table, int slot, uint64_t value, bool skipSelf,
                         uint32_t code, int step, uint32_t k) {
  int ok = 1;
  const int q = threadIdx.x;
  if (q < ctx.world && !(skipSelf && q == ctx.rank)) ok = sig::waitAtLeast(ctx, table[slot] + q, value, code, step, q, k) ? 1 : 0;
  return __syncthreads_and(ok) != 0;
}

// Thread 0 takes part in the last-arrival count; every thread of the CTA learns whether this CTA was last.
// The two barriers also order every thread's earlier writes before any thread's later flag store, so each
// peer can be signalled by a different thread (a release store to peer memory costs microseconds; W of them
// issued by one thread in sequence would dominate a chunk).
PURLIN_D bool ctaLastArrival(uint32_t* counter, uint32_t expected) {
  __shared__ int lastFlag;
  __syncthreads();
  if (threadIdx.x == 0) lastFlag = sig::lastArrival(counter, expected) ? 1 : 0;
  __syncthreads();
  return lastFlag != 0;
}

// ---------------- copy roles on the bulk-async engine (one driver thread per CTA) ----------------
struct StageHooks {
  const Context& ctx; const Step& s; int si; const Frame& f; unsigned char* staging; int n;
  PURLIN_D const unsigned char* src(uint32_t k, size_t off) const { return f.src + s.srcOff + size_t(k) * s.chunkBytes + off; }
  PURLIN_D unsigned char* dst(uint32_t k, size_t off) const { return staging + slotOff(s, k) + off; }
  PURLIN_D bool beforeLoad(uint32_t) const { return true; }
  PURLIN_D void loaded(uint32_t) const {}
  PURLIN_D bool beforeStore(uint32_t k) const {
    if (!(s.flags & kFlagCyclic) || k < s.slots) return true;
    const uint64_t need = flagValue(f.seq, k - s.slots);      // every reader drained the slot's previous tenant
    if (s.flags & kFlagDrainGather) {
      if (s.peer != ctx.rank) return sig::waitAtLeast(ctx, ctx.gatherSignals[ctx.rank] + s.peer, need, kStatusTimeoutSignal, si, s.peer, k);
      for (int q = 0; q < ctx.world; ++q)
        if (q != ctx.rank && !sig::waitAtLeast(ctx, ctx.consumedSignals[ctx.rank] + q, need, kStatusTimeoutSignal, si, q, k)) return false;
      return true;
    }
    if (s.peer >= 0) return sig::waitAtLeast(ctx, ctx.consumedSignals[ctx.rank] + s.peer, need, kStatusTimeoutSignal, si, s.peer, k);
    for (int q = 0; q < ctx.world; ++q) {
      if (q == ctx.rank && !(s.flags & kFlagDrainSelf)) continue;
      if (!sig::waitAtLeast(ctx, ctx.consumedSignals[ctx.rank] + q, need, kStatusTimeoutSignal, si, q, k)) return false;
    }
    return true;
  }
  PURLIN_D void stored(uint32_t k) const {
    tc::fenceProxyAsync();                                    // bulk (async-proxy) writes before the generic-proxy flag
    if (sig::lastArrival(ctx.counters + s.counterBase + (k % kMaxChunks), n)) {
      const uint64_t v = flagValue(f.seq, k);
      if (s.peer >= 0) sig::stReleaseSys(ctx.signals[s.peer] + ctx.rank, v);
      else {
        __threadfence_system();                               // one fence, then relaxed flag stores to every rank
        for (int q = 0; q < ctx.world; ++q) sig::stRelaxedSys(ctx.signals[(ctx.rank + q) % ctx.world] + ctx.rank, v);
      }
    }
  }
};

struct ConsumeHooks {
  const Context& ctx; const Step& s; int si; const Frame& f; const unsigned char* staging; const uint64_t* flag; int n;
  PURLIN_D const unsigned char* src(uint32_t k, size_t off) const { return staging + slotOff(s, k) + off; }
  PURLIN_D unsigned char* dst(uint32_t k, size_t off) const { return f.dst + s.dstOff + size_t(k) * s.chunkBytes + off; }
  PURLIN_D bool beforeLoad(uint32_t k) const {
    if (!sig::waitAtLeast(ctx, flag, flagValue(f.seq, k), kStatusTimeoutSignal, si, s.peer, k)) return false;
    tc::fenceProxyAsync();                                    // the producer's writes before this thread's bulk reads
    return true;
  }
  PURLIN_D void loaded(uint32_t k) const {
    if ((s.flags & kFlagCyclic) && sig::lastArrival(ctx.counters + s.counterBase + (k % kMaxChunks), n))
      sig::stReleaseSys(ctx.consumedSignals[s.peer] + ctx.rank, flagValue(f.seq, k));
  }
  PURLIN_D bool beforeStore(uint32_t) const { return true; }
  PURLIN_D void stored(uint32_t) const {}
};

struct LocalHooks {
  const Step& s; const Frame& f;
  PURLIN_D const unsigned char* src(uint32_t, size_t off) const { return f.src + s.srcOff + off; }
  PURLIN_D unsigned char* dst(uint32_t, size_t off) const { return f.dst + s.dstOff + off; }
  PURLIN_D bool beforeLoad(uint32_t) const { return true; }
  PURLIN_D void loaded(uint32_t) const {}
  PURLIN_D bool beforeStore(uint32_t) const { return true; }
  PURLIN_D void stored(uint32_t) const {}
};

template <class Hooks>
PURLIN_D bool runBulk(const Context& ctx, const Step& s, const Frame& f, Hooks& h) {
  int ok = 1;
  if (threadIdx.x == 0) {
    bulk::Ring ring;
    ring.init(f.smem, f.bulkDepth, ctx.timeoutNs);
    // a reader of a cyclic window may not run further ahead than the window has slots
    const uint32_t lead = ((s.flags & kFlagCyclic) && s.role != kRoleStage) ? (s.slots > 1 ? s.slots - 1 : 0u) : 0x3fffffffu;
    ok = bulk::stream(ring, s, f.bIdx - s.blockBegin, s.blockCount, lead, h) ? 1 : 0;
    if (!ok && !sig::failed(ctx)) sig::fail(ctx, kStatusTimeoutBarrier, 0, uint32_t(s.peer), 0);
  }
  return __syncthreads_and(ok) != 0;
}

template <class Atom>
PURLIN_D bool stage(const Context& ctx, const Step& s, int si, const Frame& f) {
  const int j = f.bIdx - s.blockBegin, n = s.blockCount;
  unsigned char* staging = ctx.stagingTR[ctx.rank] + size_t(f.half) * ctx.stagingTRSize + s.dstOff;
  if (f.bulkDepth > 0) { StageHooks h{ctx, s, si, f, staging, n}; return runBulk(ctx, s, f, h); }
  for (uint32_t k = 0; k < s.chunks; ++k) {
    if ((s.flags & kFlagCyclic) && k >= s.slots) {
      // back-pressure: every reader of this slot must have drained its previous tenant
      const uint64_t need = flagValue(f.seq, k - s.slots);
      bool ok;
      if (s.flags & kFlagDrainGather) {
        // composed all-reduce: a peer's window is free once that peer has reduced the chunk; this rank's own window
        // (the seam) once every peer has gathered the reduced chunk out of it
        ok = s.peer != ctx.rank
            ? ctaWait(ctx, ctx.gatherSignals[ctx.rank] + s.peer, need, kStatusTimeoutSignal, si, s.peer, k)
            : ctaWaitAll(ctx, ctx.consumedSignals, ctx.rank, need, true, kStatusTimeoutSignal, si, k);
      } else {
        ok = s.peer >= 0
            ? ctaWait(ctx, ctx.consumedSignals[ctx.rank] + s.peer, need, kStatusTimeoutSignal, si, s.peer, k)
            : ctaWaitAll(ctx, ctx.consumedSignals, ctx.rank, need, (s.flags & kFlagDrainSelf) == 0, kStatusTimeoutSignal, si, k);
      }
      if (!ok) return false;
    }
    superCopy<Atom>(staging + slotOff(s, k), f.src + s.srcOff + size_t(k) * s.chunkBytes, chunkLen(s, k), j, n, f.unroll);
    if (ctaLastArrival(ctx.counters + s.counterBase + (k % kMaxChunks), n)) {
      const uint64_t v = flagValue(f.seq, k);
      if (s.peer >= 0) { if (threadIdx.x == 0) sig::stReleaseSys(ctx.signals[s.peer] + ctx.rank, v); }
      else if (int(threadIdx.x) < ctx.world) sig::stReleaseSys(ctx.signals[(ctx.rank + threadIdx.x) % ctx.world] + ctx.rank, v);
    }
  }
  return true;
}

template <class Atom>
PURLIN_D void local(const Context& ctx, const Step& s, const Frame& f) {
  if (f.bulkDepth > 0) { LocalHooks h{s, f}; runBulk(ctx, s, f, h); return; }
  superCopy<Atom>(f.dst + s.dstOff, f.src + s.srcOff, s.bytes, f.bIdx - s.blockBegin, s.blockCount, f.unroll);
}

// consume (copy) and gather share everything but the flag table
template <class Atom>
PURLIN_D bool consume(const Context& ctx, const Step& s, int si, const Frame& f, bool gather) {
  const int j = f.bIdx - s.blockBegin, n = s.blockCount;
  const int from = (s.flags & kFlagLocalSource) ? ctx.rank : s.peer;
  const unsigned char* staging = ctx.stagingTR[from] + size_t(f.half) * ctx.stagingTRSize + s.srcOff;
  uint64_t* const* table = gather ? ctx.gatherSignals : ctx.signals;
  if (f.bulkDepth > 0) { ConsumeHooks h{ctx, s, si, f, staging, table[ctx.rank] + s.peer, n}; return runBulk(ctx, s, f, h); }
  for (uint32_t k = 0; k < s.chunks; ++k) {
    if (!ctaWait(ctx, table[ctx.rank] + s.peer, flagValue(f.seq, k), kStatusTimeoutSignal, si, s.peer, k)) return false;
    superCopy<Atom>(f.dst + s.dstOff + size_t(k) * s.chunkBytes, staging + slotOff(s, k), chunkLen(s, k), j, n, f.unroll);
    if (s.flags & kFlagCyclic) {
      __syncthreads();
      if (threadIdx.x == 0 && sig::lastArrival(ctx.counters + s.counterBase + (k % kMaxChunks), n))
        sig::stReleaseSys(ctx.consumedSignals[s.peer] + ctx.rank, flagValue(f.seq, k));
    }
  }
  return true;
}


template <class Atom, DType T, ReduceOp Op>
PURLIN_D bool reduce(const Context& ctx, const Step& s, int si, const Frame& f, const unsigned char** peerPtr) {
  const int j = f.bIdx - s.blockBegin, n = s.blockCount;
  const size_t halfOff = size_t(f.half) * ctx.stagingTRSize;
  for (uint32_t k = 0; k < s.chunks; ++k) {
    if (!ctaWaitAll(ctx, ctx.signals, ctx.rank, flagValue(f.seq, k), false, kStatusTimeoutSignal, si, k)) return false;
    const Span sp = partitionAligned(chunkLen(s, k), n, j, kAccessAlign);
    const size_t in = halfOff + s.srcOff + slotOff(s, k) + sp.offset;
    if (threadIdx.x < ctx.world) peerPtr[threadIdx.x] = ctx.stagingTR[threadIdx.x] + in;
    __syncthreads();
    ReduceArgs a;
    a.srcs = peerPtr;
    a.world = ctx.world;
    a.bytes = sp.bytes;
    if (s.flags & kFlagMultimemLoad) a.mcSrc = ctx.mcStagingTR + in;
    const size_t lin = size_t(k) * s.chunkBytes + sp.offset;
    if (s.flags & kFlagToDst) a.dst = f.dst + s.dstOff + lin;
    if (s.flags & kFlagToSeam) {
      const size_t so = halfOff + s.seamOff + slotOff(s, k) + sp.offset;
      if (s.flags & kFlagMulticastOut) a.mcSeam = ctx.mcStagingTR + so;
      else a.seam = ctx.stagingTR[ctx.rank] + so;
    }
    if (sp.bytes) Atom::template reduce<T, Op>(a, f.mmDepth);
    if (s.flags & (kFlagNotifyGather | kFlagCyclic)) {
      if (s.flags & kFlagMulticastOut) __threadfence_system();
      if (ctaLastArrival(ctx.counters + s.counterBase + (k % kMaxChunks), n) && int(threadIdx.x) < ctx.world) {
        const uint64_t v = flagValue(f.seq, k);
        const int p = (ctx.rank + 1 + threadIdx.x) % ctx.world;     // one peer per thread
        if ((s.flags & kFlagNotifyGather) && p != ctx.rank) sig::stReleaseSys(ctx.gatherSignals[p] + ctx.rank, v);
        if (s.flags & kFlagCyclic) sig::stReleaseSys(ctx.consumedSignals[p] + ctx.rank, v);
      }
    } else {
      __syncthreads();   // peerPtr is rewritten by the next chunk
    }
  }
  return true;
}

// ---------------- latency regime ----------------
PURLIN_D Packet* slotOf(const Context& ctx, int onRank, int fromRank, int half, bool resultHalf) {
  unsigned char* base = ctx.stagingLR[onRank] + size_t(half) * kPacketEpochBytes + size_t(fromRank) * ctx.packetStride;
  if (resultHalf) base += ctx.packetStride / 2;
  return reinterpret_cast<Packet*>(base);
}
PURLIN_D Packet* slotOfMulticast(const Context& ctx, int fromRank, int half, bool resultHalf) {
  unsigned char* base = ctx.mcStagingLR + size_t(half) * kPacketEpochBytes + size_t(fromRank) * ctx.packetStride;
  if (resultHalf) base += ctx.packetStride / 2;
  return reinterpret_cast<Packet*>(base);
}

PURLIN_D void packetPut(const Context& ctx, const Step& s, const Frame& f) {
  const size_t words = s.bytes / 8, stride = size_t(s.blockCount) * blockDim.x;
  const uint64_t* src = reinterpret_cast<const uint64_t*>(f.src + s.srcOff);
  const uint64_t flag = flagValue(f.seq, 0);
  const size_t first = s.dstOff / 8;
  if (s.flags & kFlagScatter) {
    // every peer gets its own slice: (peer, word) pairs over the threads, one load and one store each
    const size_t pairs = words * size_t(ctx.world - 1);
    for (size_t idx = size_t(f.bIdx - s.blockBegin) * blockDim.x + threadIdx.x; idx < pairs; idx += stride) {
      const size_t i = idx % words;
      const int d = (ctx.rank + 1 + int(idx / words)) % ctx.world;
      pkt::write(slotOf(ctx, d, ctx.rank, f.half, false) + first + i, src[size_t(d) * words + i], flag);
    }
    return;
  }
  if (s.peer < 0 && !(s.flags & kFlagMulticastOut) && ctx.world > 2 && words * size_t(ctx.world - 1) <= 2 * stride) {
    // Peer-striped: with few words and many peers, (word, peer) pairs are spread over the threads, so that every
    // store to a peer is some thread's first and only one instead of the last of W - 1 issued in a row
    // (the one-warp-per-peer latency stage of the reference, csrc/include/purlin/snac.cuh:1672-1688).
    const size_t pairs = words * size_t(ctx.world - 1);
    for (size_t idx = size_t(f.bIdx - s.blockBegin) * blockDim.x + threadIdx.x; idx < pairs; idx += stride) {
      const size_t i = idx % words;
      const int q = 1 + int(idx / words);
      pkt::write(slotOf(ctx, (ctx.rank + q) % ctx.world, ctx.rank, f.half, false) + first + i, src[i], flag);
    }
    return;
  }
  for (size_t i = size_t(f.bIdx - s.blockBegin) * blockDim.x + threadIdx.x; i < words; i += stride) {
    const uint64_t v = src[i];
    if (s.peer >= 0) {
      pkt::write(slotOf(ctx, s.peer, ctx.rank, f.half, false) + first + i, v, flag);
    } else if (s.flags & kFlagMulticastOut) {
      pkt::writeMulticast(slotOfMulticast(ctx, ctx.rank, f.half, false) + first + i, v, flag);
    } else {
      for (int q = 1; q < ctx.world; ++q)
        pkt::write(slotOf(ctx, (ctx.rank + q) % ctx.world, ctx.rank, f.half, false) + first + i, v, flag);
    }
  }
}

PURLIN_D bool packetGet(const Context& ctx, const Step& s, int si, const Frame& f) {
  const size_t words = s.bytes / 8, stride = size_t(s.blockCount) * blockDim.x;
  uint64_t* dst = reinterpret_cast<uint64_t*>(f.dst + s.dstOff);
  const uint64_t flag = flagValue(f.seq, 0);
  bool ok = true;
  if (s.peer < 0) {
    // Every peer's packets in one step: (peer, word) pairs are spread over the threads, so the W - 1 peers are polled at
    // the same time and the step ends with one barrier (the reference polls its peers from separate warps for the same
    // reason, csrc/include/purlin/snac.cuh:1230-1262).
    const size_t pairs = words * size_t(ctx.world - 1);
    const size_t first = s.srcOff / 8;
    for (size_t idx = size_t(f.bIdx - s.blockBegin) * blockDim.x + threadIdx.x; idx < pairs && ok; idx += stride) {
      const size_t i = idx % words;
      const int q = (ctx.rank + 1 + int(idx / words)) % ctx.world;
      uint64_t v;
      ok = pkt::read(ctx, slotOf(ctx, ctx.rank, q, f.half, (s.flags & kFlagResultHalf) != 0) + first + i, flag, v, kStatusTimeoutPacket, si, q);
      if (ok) reinterpret_cast<uint64_t*>(f.dst + s.dstOff + size_t(q) * s.bytes)[i] = v;
    }
    return ok;
  }
  const Packet* slot = slotOf(ctx, ctx.rank, s.peer, f.half, (s.flags & kFlagResultHalf) != 0) + s.srcOff / 8;
  for (size_t i = size_t(f.bIdx - s.blockBegin) * blockDim.x + threadIdx.x; i < words && ok; i += stride) {
    uint64_t v;
    ok = pkt::read(ctx, slot + i, flag, v, kStatusTimeoutPacket, si, s.peer);
    if (ok) dst[i] = v;
  }
  return ok;
}

template <DType T, ReduceOp Op>
PURLIN_D bool packetReduce(const Context& ctx, const Step& s, int si, const Frame& f) {
  const size_t words = s.bytes / 8, stride = size_t(s.blockCount) * blockDim.x;
  const uint64_t* own = reinterpret_cast<const uint64_t*>(f.src + s.seamOff);
  uint64_t* dst = reinterpret_cast<uint64_t*>(f.dst + s.dstOff);
  const uint64_t flag = flagValue(f.seq, 0);
  const size_t first = s.srcOff / 8;
  bool ok = true;
  for (size_t i = size_t(f.bIdx - s.blockBegin) * blockDim.x + threadIdx.x; i < words && ok; i += stride) {
    Acc<T> acc;
#pragma unroll
    for (int e = 0; e < ElemTraits<T>::perWord; ++e) acc.v[e] = identity<Op>();
    const uint64_t mine = own[i];
    // ascending rank order (bit-reproducible); the packets of four ranks are requested before any is looked at, so a
    // word costs a quarter of the memory round trips of a poll per rank
    for (int q0 = 0; q0 < ctx.world && ok; q0 += 4) {
      Packet v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (q0 + u < ctx.world && q0 + u != ctx.rank) v[u] = pkt::load(slotOf(ctx, ctx.rank, q0 + u, f.half, false) + first + i);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int q = q0 + u;
        if (q >= ctx.world || !ok) break;
        uint64_t w = mine;
        if (q != ctx.rank) {
          w = v[u].data;
          if (v[u].flag != flag) ok = pkt::read(ctx, slotOf(ctx, ctx.rank, q, f.half, false) + first + i, flag, w, kStatusTimeoutPacket, si, q);
        }
        if (ok) accumulate<T, Op>(acc, unpack<T>(w));
      }
    }
    if (!ok) break;
    const uint64_t out = pack<T>(acc);
    dst[i] = out;
    if (s.flags & kFlagPublish) {
      if (s.flags & kFlagMulticastOut) {
        pkt::writeMulticast(slotOfMulticast(ctx, ctx.rank, f.half, true) + i, out, flag);
      } else {
        for (int q = 1; q < ctx.world; ++q)
          pkt::write(slotOf(ctx, (ctx.rank + q) % ctx.world, ctx.rank, f.half, true) + i, out, flag);
      }
    }
  }
  return ok;
}

// ---------------- variable-length arrival handshake ----------------
PURLIN_D void postArrival(const Context& ctx, const Frame& f, uint64_t payload) {
  const int q = threadIdx.x;
  if (q < ctx.world) {
    Packet* p = reinterpret_cast<Packet*>(ctx.varLenSignals[q]) + f.half * ctx.world + ctx.rank;
    pkt::write(p, payload, flagValue(f.seq, 0));
  }
}
PURLIN_D bool awaitArrival(const Context& ctx, const Frame& f) {
  int ok = 1;
  const int q = threadIdx.x;
  if (q < ctx.world) {
    uint64_t v;
    const Packet* p = reinterpret_cast<const Packet*>(ctx.varLenSignals[ctx.rank]) + f.half * ctx.world + q;
    ok = pkt::read(ctx, p, flagValue(f.seq, 0), v, kStatusTimeoutArrival, 0, q) ? 1 : 0;
  }
  return __syncthreads_and(ok) != 0;
}

// One CTA's share of a whole collective. `bIdx`/`blocks` are the CTA's index and the
// grid size of this rank (not of the launch: emulation stacks ranks along grid.y).
template <class Atom, DType T, ReduceOp Op, bool Reduces, class PlanType = Plan>
PURLIN_D void run(const Context& ctx, const PlanType& plan, const unsigned char* src, unsigned char* dst,
                  int bIdx, int blocks, const unsigned char** peerPtr, unsigned char* dynSmem) {
  Frame f;
  f.seq = sig::ldRelaxedSys(ctx.seq + (bIdx % kSeqWords));
  f.half = int(f.seq & 1);
  f.bIdx = bIdx;
  f.src = src;
  f.dst = dst;
  f.unroll = plan.unroll;
  f.mmDepth = plan.mmDepth;
  f.bulkDepth = plan.regime == int32_t(Regime::throughput) ? plan.stageDepth : 0;
  f.smem = dynSmem;
  // A context that failed stays quiet until the host clears it. The status word is requested here and looked at after
  // the CTA's first step has issued its own loads, so that its latency overlaps theirs instead of preceding them (a
  // small collective is a chain of a few memory round trips; this removes one). The first step of a latency plan only
  // sends this rank's own input, which is harmless on a failed context.
  const uint32_t statusAtEntry = sig::ldRelaxedGpu32(ctx.status);
  bool ok = true;
  bool checkedStatus = false;
  if (ctx.trace != nullptr && bIdx == 0 && threadIdx.x == 0) {
    // device-side timing: the first CTA stamps the start of call `seq`, the last CTA out stamps its end
    uint64_t* rec = ctx.trace + (f.seq % uint64_t(kTraceSlots)) * 4;
    rec[0] = sig::globalTimerNs();
    rec[2] = plan.payloadBytes;
    rec[3] = uint64_t(uint32_t(plan.collective)) | (uint64_t(uint32_t(blocks)) << 32);
  }
  if (ok && plan.varLenArrival && bIdx == 0) postArrival(ctx, f, plan.payloadBytes);
  for (int si = 0; si < plan.nSteps && ok; ++si) {
    const Step& s = plan.steps[si];
    if (bIdx < s.blockBegin || bIdx >= s.blockBegin + s.blockCount) continue;
    if (!checkedStatus && s.role != kRolePacketPut) { checkedStatus = true; if (statusAtEntry != 0u) { ok = false; break; } }
    switch (s.role) {
      case kRoleStage: ok = stage<Atom>(ctx, s, si, f); break;
      case kRoleLocal: local<Atom>(ctx, s, f); break;
      case kRoleConsume: ok = consume<Atom>(ctx, s, si, f, false); break;
      case kRoleGather: ok = consume<Atom>(ctx, s, si, f, true); break;
      case kRolePacketPut: packetPut(ctx, s, f); break;
      case kRolePacketGet: ok = __syncthreads_and(packetGet(ctx, s, si, f) ? 1 : 0) != 0; break;
      case kRoleReduce:
        if constexpr (Reduces) ok = reduce<Atom, T, Op>(ctx, s, si, f, peerPtr);
        break;
      case kRolePacketReduce:
        if constexpr (Reduces) ok = __syncthreads_and(packetReduce<T, Op>(ctx, s, si, f) ? 1 : 0) != 0;
        break;
      default: break;
    }
  }
  if (ok && plan.varLenArrival && bIdx == 0) ok = awaitArrival(ctx, f);
  // Every CTA advances its share of the sequence words when it leaves; the next launch (stream order) finds them all
  // advanced. Nobody waits for the last CTA. (A traced context also counts the CTAs out: the last one stamps the end.)
  __syncthreads();
  for (int w = bIdx + int(threadIdx.x) * blocks; w < kSeqWords; w += blocks * int(blockDim.x)) ctx.seq[w] = f.seq + 1;
  if (ctx.trace != nullptr && threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(ctx.exitCounter, 1u) == uint32_t(blocks - 1)) {
      *ctx.exitCounter = 0;
      ctx.trace[(f.seq % uint64_t(kTraceSlots)) * 4 + 1] = sig::globalTimerNs();
      __threadfence();
    }
  }
}

}  // namespace snac
}  // namespace purlin
