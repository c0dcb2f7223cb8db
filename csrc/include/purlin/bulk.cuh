// Bulk-asynchronous copy engine for the throughput regime: one elected thread per CTA streams a CTA's share
// of every chunk of a step through a ring of shared-memory tiles with cp.async.bulk (global -> shared, tracked
// by mbarriers; shared -> global, tracked by bulk groups). Loads run depth-1 tiles ahead of stores and do not
// stop at chunk boundaries, so a CTA keeps (depth-1) x 16 KiB in flight for the whole call instead of refilling
// a register pipeline once per chunk.
//
// The reference's copy Atom is a cp.async (16-byte, per-thread) ring (csrc/include/purlin/tendon.cuh:66-115) and
// it carries an unused per-warp bulk-copy variant (ligament.cuh:180-293). This engine is what that variant would
// be on Blackwell if it were used: whole-CTA granularity, bulk groups for the store side, and the flag protocol
// of the step (wait before a chunk's first load, signal after a chunk's last store) folded into the stream.
// No load here uses cluster multicast; sources may be peer memory.
#pragma once
#include "plan.hpp"
#include "tc_sm100.cuh"

namespace purlin {
namespace bulk {

constexpr uint32_t kTileBytes = 16384;
constexpr int kMaxDepth = 13;                     // 13 x 16 KiB = 208 KiB of the 227 KiB a CTA may use
constexpr uint32_t kBarrierBytes = 128;           // kMaxDepth mbarriers + the abort word

PURLIN_HD constexpr size_t smemBytes(int depth) { return size_t(depth) * kTileBytes + kBarrierBytes + 128; }

PURLIN_D void loadTile(uint32_t smemDst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smemDst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
PURLIN_D void storeTile(void* dst, uint32_t smemSrc, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smemSrc), "r"(bytes) : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// all but the most recent store group have finished READING shared memory (their tiles are free)
PURLIN_D void waitStoreReadsButOne() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
PURLIN_D void waitStoresAll() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Walks one CTA's share (part `j` of `n`) of every chunk of a step, 16 KiB at a time.
struct TileWalk {
  const Step* s;
  int j, n;
  uint32_t chunk;
  size_t pos, end, spanOff;
  bool started;
  PURLIN_D void init(const Step& step, int part, int parts) { s = &step; j = part; n = parts; chunk = 0; pos = end = spanOff = 0; started = false; }
  // Next event. bytes == 0 means "this CTA has no bytes in this chunk" (it still takes part in the chunk's protocol).
  PURLIN_D bool next(uint32_t& k, size_t& offInChunk, uint32_t& bytes, bool& first, bool& last) {
    for (;;) {
      if (started && pos < end) {
        k = chunk; offInChunk = spanOff + pos; first = pos == 0;
        const size_t left = end - pos;
        bytes = left < kTileBytes ? uint32_t(left) : kTileBytes;
        pos += bytes; last = pos == end;
        if (last) { ++chunk; started = false; }
        return true;
      }
      if (chunk >= s->chunks) return false;
      const size_t begin = size_t(chunk) * s->chunkBytes;
      const size_t len = s->bytes - begin < s->chunkBytes ? s->bytes - begin : s->chunkBytes;
      const Span sp = partitionAligned(len, n, j, kAccessAlign);
      spanOff = sp.offset; pos = 0; end = sp.bytes; started = true;
      if (end == 0) { k = chunk; offInChunk = spanOff; bytes = 0; first = last = true; ++chunk; started = false; return true; }
    }
  }
};

// The ring. Shared memory: `depth` tiles, then `depth` mbarriers, then the abort word.
struct Ring {
  uint32_t tiles, bars;
  volatile int* abortWord;
  int depth;
  uint64_t timeoutNs;
  PURLIN_D void init(unsigned char* smem, int d, uint64_t timeout) {
    const uint32_t raw = tc::smemAddr(smem);
    const uint32_t aligned = (raw + 127u) & ~127u;
    tiles = aligned; depth = d; timeoutNs = timeout;
    bars = aligned + uint32_t(d) * kTileBytes;
    abortWord = reinterpret_cast<volatile int*>(smem + (aligned - raw) + size_t(d) * kTileBytes + 8 * kMaxDepth);
    for (int i = 0; i < d; ++i) tc::mbarInit(bars + 8u * i, 1);
    *abortWord = 0;
    tc::mbarFenceInit();
  }
};

// Streams a step. Called by ONE thread. `Hooks` supplies:
//   const unsigned char* src(k, off); unsigned char* dst(k, off);
//   bool beforeLoad(k)   first load of chunk k is about to be issued (wait for the producer's flag); false aborts
//   void loaded(k)       every byte this CTA reads of chunk k is in shared memory (report "consumed" for cyclic slots)
//   bool beforeStore(k)  first store of chunk k is about to be issued (wait for a cyclic slot to drain); false aborts
//   void stored(k)       every byte this CTA writes of chunk k is in global memory (last arrival, notify)
// `maxChunkLead`: how many chunks the load side may be ahead of the store side. A reader of a cyclic window must
// stay below the window's slot count, or it would wait for a chunk whose slot it has not yet reported as drained.
template <class Hooks>
PURLIN_D bool stream(Ring& ring, const Step& s, int part, int parts, uint32_t maxChunkLead, Hooks& h) {
  TileWalk lw, sw;
  lw.init(s, part, parts);
  sw.init(s, part, parts);
  uint32_t loads = 0, stores = 0;              // real (non-empty) tiles issued on each side
  const uint32_t depth = uint32_t(ring.depth);
  bool ok = true, moreLoads = true;

  // Issue loads while a tile is free (its previous store has been read out of shared memory: at most depth-1
  // tiles are loaded-but-not-stored, and the store issued last may still be reading) and the lead allows it.
  auto refill = [&]() {
    while (ok && moreLoads && loads + 2 <= stores + depth + (stores == 0 ? 1u : 0u)) {
      if (!lw.started && loads > stores && lw.chunk > sw.chunk + maxChunkLead) return;   // wait for the store side
      uint32_t k, bytes; size_t off; bool first, last;
      if (!lw.next(k, off, bytes, first, last)) { moreLoads = false; return; }
      if (bytes == 0) continue;                // nothing to read; the store side reports the chunk
      if (first && !h.beforeLoad(k)) { ok = false; return; }
      const uint32_t slot = loads % depth;
      tc::mbarExpectTx(ring.bars + 8u * slot, bytes);
      loadTile(ring.tiles + slot * kTileBytes, h.src(k, off), bytes, ring.bars + 8u * slot);
      ++loads;
    }
  };

  refill();
  while (ok) {
    uint32_t k, bytes; size_t off; bool first, last;
    if (!sw.next(k, off, bytes, first, last)) break;
    if (bytes == 0) {                          // this CTA owns no bytes of chunk k: take part in its protocol only
      if (!h.beforeStore(k)) { ok = false; break; }
      h.loaded(k);
      h.stored(k);
      refill();
      continue;
    }
    if (loads == stores) { refill(); if (!ok || loads == stores) { ok = false; break; } }   // nothing in flight: load now
    const uint32_t slot = stores % depth;
    const uint32_t phase = (stores / depth) & 1u;
    if (!tc::mbarWait(ring.bars + 8u * slot, phase, ring.abortWord, ring.timeoutNs)) { ok = false; break; }
    if (last) h.loaded(k);
    if (first && !h.beforeStore(k)) { ok = false; break; }
    storeTile(h.dst(k, off), ring.tiles + slot * kTileBytes, bytes);
    ++stores;
    if (last) { waitStoresAll(); h.stored(k); }   // the chunk is out: drain, then report it
    else waitStoreReadsButOne();                  // the previous store has left shared memory: its tile is free
    refill();
  }
  waitStoresAll();
  return ok;
}

}  // namespace bulk
}  // namespace purlin
