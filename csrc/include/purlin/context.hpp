// Context: every pointer a kernel needs, passed by value as a kernel parameter.
//
// Parity: csrc/include/purlin/context.cuh:10-58 and the workspace layout of
// csrc/include/purlin/setup.cuh:195-239 in the reference. The symmetric block
// keeps the reference's on-device format byte for byte:
//
//   [ 2 x stagingTRSize | 2 x 8 MiB packets | signals[W] | gatherSignals[W] |
//     consumedSignals[W] | pad to 32 B | varLenSignals[2][W] x 16 B ]
//
// What differs: peer pointers live inside the struct (constant-bank reads, no
// dependent load through a device pointer table), one call-sequence number kept in
// kSeqWords identical words (every CTA reads its own and advances its share when it
// leaves, so no CTA waits for another at the end of a call) replaces per-CTA epochs,
// and a status word receives bounded-wait timeouts.
#pragma once
#include "constants.hpp"

namespace purlin {

struct WorkspaceLayout {
  size_t stagingTRSize = 0;   // one half
  size_t lrOffset = 0;        // 2*S
  size_t signalOffset = 0;    // 2*(S + 8 MiB)
  size_t gatherOffset = 0;
  size_t consumedOffset = 0;
  size_t varLenOffset = 0;    // rounded up to 32 B
  size_t totalBytes = 0;
  size_t packetStride = 0;    // bytes of one sender's slot inside one packet half
};

PURLIN_HD inline WorkspaceLayout workspaceLayout(int world, size_t stagingTRSize) {
  WorkspaceLayout w;
  w.stagingTRSize = stagingTRSize;
  w.lrOffset = 2 * stagingTRSize;
  w.signalOffset = 2 * (stagingTRSize + kPacketEpochBytes);
  w.gatherOffset = w.signalOffset + size_t(world) * 8;
  w.consumedOffset = w.signalOffset + 2 * size_t(world) * 8;
  w.varLenOffset = roundUp(w.signalOffset + 3 * size_t(world) * 8, kAccessAlign);
  w.totalBytes = w.varLenOffset + 2 * size_t(world) * kPacketBytes;
  w.packetStride = roundDown(kPacketEpochBytes / size_t(world), kAccessAlign);
  return w;
}

struct Context {
  // symmetric, one entry per rank (entry `rank` is this GPU's own memory)
  unsigned char* stagingTR[kMaxRanks];
  unsigned char* stagingLR[kMaxRanks];
  uint64_t* signals[kMaxRanks];          // signals[p][r]: rank r -> rank p "staged chunk k"
  uint64_t* gatherSignals[kMaxRanks];    // composed all-reduce: "shard reduced"
  uint64_t* consumedSignals[kMaxRanks];  // cyclic back-pressure: "chunk k drained"
  unsigned char* varLenSignals[kMaxRanks];  // [2][W] arrival packets
  unsigned char* mcStagingTR;            // NVLS multicast alias of stagingTR, or null
  unsigned char* mcStagingLR;            // NVLS multicast alias of stagingLR, or null
  // local (not symmetric)
  uint64_t* seq;                         // [kSeqWords] call sequence number, the same in every word between calls; half = seq & 1
  uint32_t* counters;                    // [kCounterSlots] last-arrival counters, self-resetting
  uint32_t* exitCounter;                 // CTAs that finished the running call (used only while tracing: the last one stamps the end)
  uint32_t* status;                      // [4]: code, step, peer, chunk
  uint64_t* trace;                       // optional ring of kTraceSlots x {start ns, end ns, payload bytes, collective}; null = off
  size_t stagingTRSize;
  size_t packetStride;
  uint64_t timeoutNs;                    // time limit of every device wait
  int32_t world;
  int32_t rank;
};

// Variable-length collective sizes, resolved on the host from the caller's lists.
struct VState {
  size_t maxOutBytes = 0;
  size_t maxBytes = 0;
  size_t totalBytes = 0;
  size_t totalOutBytes = 0;
  size_t offset = 0;
  size_t bytes = 0;
};

}  // namespace purlin
