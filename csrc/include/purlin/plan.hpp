// The SNAC plan: a plain-old-data schedule that one generic kernel executes.
//
// The reference derives its Stage-Notify-And-Consume orchestration at compile
// time from template parameters (csrc/include/purlin/snac.cuh:36-78 for the
// topology, 218-1134 for the throughput protocol, 1163-1955 for the latency
// protocol). Here the derivation is a run-time function (layout.hpp) whose
// output is this struct: a list of steps, each bound to a range of CTAs. The
// same plan is executed by the sm_100a kernels (snac.cuh), by the CPU
// interpreter (host_core.cpp) and by the gloo path of the Python package, so the
// protocol can be tested without a GPU.
#pragma once
#include "constants.hpp"

namespace purlin {

enum class DataLayout : int32_t { packed = 0, packedV, scattered, scatteredV, transposed, transposedV };
enum class ConsumeOp : int32_t { copy = 0, reduce = 1 };
enum class Regime : int32_t { latency = 0, throughput = 1 };
enum class MemType : int32_t { unicast = 0, multimem = 1 };
enum class ReduceOp : int32_t { add = 0, mul = 1, max = 2 };
enum class DType : int32_t { bf16 = 0, fp16 = 1, fp8e4m3 = 2, fp8e5m2 = 3, fp32 = 4 };
enum class ReductionMode : int32_t { nonDeterministic = 0, deterministic = 1 };
enum class CollectiveType : int32_t {
  allReduce = 0, allGather, allGatherV, reduceScatter, reduceScatterV, allToAll, allToAllV
};
enum class AllReducePath : int32_t { direct = 0, composed = 1 };

PURLIN_HD constexpr int dtypeBytes(DType t) {
  return t == DType::fp32 ? 4 : (t == DType::bf16 || t == DType::fp16) ? 2 : 1;
}

enum Role : int32_t {
  kRoleStage = 0,     // user src -> own staging, then notify `peer` (-1: every rank)
  kRoleLocal = 1,     // user src -> user dst (the self slice of a copy collective)
  kRoleConsume = 2,   // wait signals[rank][peer]; peer staging -> user dst
  kRoleReduce = 3,    // wait signals[rank][*]; reduce every rank's staging -> dst and/or seam
  kRoleGather = 4,    // composed tail: wait gatherSignals[rank][peer]; peer seam -> user dst
  kRolePacketPut = 5, // latency: user src words -> packets in peer's slot (-1: every peer; with kFlagScatter peer q gets
                      // its own slice, the `bytes` at srcOff + q * bytes)
  kRolePacketGet = 6, // latency: packets from `peer` in own slot -> user dst. peer -1: from every peer q, `bytes` each, to
                      // dstOff + q * bytes (equal slices; seamOff holds this rank's index, whose slice is not touched)
  kRolePacketReduce = 7,  // latency: reduce own words with every peer's packets -> dst (+ publish)
};

enum StepFlags : uint32_t {
  kFlagToSeam = 1u << 0,       // reduce: result is written to own staging (composition head)
  kFlagToDst = 1u << 1,        // reduce: result is written to user dst
  kFlagMultimemLoad = 1u << 2, // reduce: source is the NVLS multicast alias (in-switch reduction)
  kFlagMulticastOut = 1u << 3, // reduce/publish: result broadcast with multimem.st
  kFlagLocalSource = 1u << 4,  // gather/get: read own staging (a multicast result landed there)
  kFlagCyclic = 1u << 5,       // stream longer than its window: slots are reused under back-pressure
  kFlagPublish = 1u << 6,      // packet reduce: publish result packets to every peer
  kFlagResultHalf = 1u << 7,   // packet get: read the result half of the slot
  kFlagNotifyGather = 1u << 8, // reduce: last CTA of a chunk raises gatherSignals on every rank
  kFlagDrainSelf = 1u << 9,    // stage to everyone: this rank's own reducer is a reader of the slot too
  kFlagDrainGather = 1u << 10, // cyclic stage of a composed all-reduce: a peer's window is free again once that peer has
                               // published the reduced chunk (gatherSignals); this rank's own window, which doubles as the
                               // seam, once every peer has gathered the reduced chunk out of it (consumedSignals)
  kFlagScatter = 1u << 11,     // packet put to every peer: peer q receives slice q of the source (equal slices), not the same words
};

struct Step {
  int32_t role;
  int32_t peer;
  int32_t blockBegin;
  int32_t blockCount;
  uint64_t srcOff;      // stage/local/put: offset in user src. consume/reduce/gather/get: offset in a staging half (payload bytes for packets)
  uint64_t dstOff;      // stage: offset in own staging half (put: payload offset in the peer's slot). others: offset in user dst
  uint64_t bytes;       // stream length
  uint64_t chunkBytes;  // bytes per flag; == bytes when not chunked
  uint64_t seamOff;     // reduce: where the result goes in own staging (composition seam). packet reduce: offset of own words in user src
  uint32_t chunks;
  uint32_t slots;       // window = slots * chunkBytes; chunk k lives in slot k % slots
  uint32_t flags;
  uint32_t counterBase; // first last-arrival counter of this step
};

// N = kMaxSteps for the general plan; kCompactSteps for the short plans of the latency regime, which travel as kernel
// parameters in a quarter of the bytes (the header is the same, so the executor is one template over both).
template <int N>
struct PlanT {
  int32_t collective;   // CollectiveType, for reports
  int32_t regime;       // Regime
  int32_t consumeOp;    // ConsumeOp
  int32_t reduceOp;     // ReduceOp
  int32_t dtype;        // DType
  int32_t deterministic;
  int32_t blocks;       // grid size
  int32_t threads;      // block size
  int32_t nSteps;
  int32_t varLenArrival;  // post and await arrival packets (variable-length collectives)
  int32_t mmDepth;        // multimem loads in flight per thread
  int32_t unroll;         // vector accesses in flight per thread in the plain datapath
  int32_t stageDepth;     // stages of the bulk-async ring (0: plain vector datapath)
  int32_t reserved;
  uint64_t smemBytes;
  uint64_t payloadBytes;  // logical bytes for reports
  Step steps[N];
};
using Plan = PlanT<kMaxSteps>;
constexpr int kCompactSteps = 16;
using PlanCompact = PlanT<kCompactSteps>;

// The first steps of a plan that has at most kCompactSteps of them.
inline void compactPlan(const Plan& in, PlanCompact& out) {
  out.collective = in.collective; out.regime = in.regime; out.consumeOp = in.consumeOp; out.reduceOp = in.reduceOp;
  out.dtype = in.dtype; out.deterministic = in.deterministic; out.blocks = in.blocks; out.threads = in.threads;
  out.nSteps = in.nSteps; out.varLenArrival = in.varLenArrival; out.mmDepth = in.mmDepth; out.unroll = in.unroll;
  out.stageDepth = in.stageDepth; out.reserved = in.reserved; out.smemBytes = in.smemBytes; out.payloadBytes = in.payloadBytes;
  for (int i = 0; i < kCompactSteps; ++i) out.steps[i] = in.steps[i];
}

// Aligned even split with the remainder spread over the first parts
// (behaviour of partition<Align>, csrc/include/purlin/partition.cuh:217-247).
struct Span { size_t offset; size_t bytes; };
PURLIN_HD inline Span partitionAligned(size_t bytes, int parts, int index, size_t align) {
  const size_t units = bytes / align;        // whole aligned units
  const size_t tail = bytes - units * align; // goes to the last non-empty part
  const size_t base = units / size_t(parts), rem = units % size_t(parts);
  const size_t i = size_t(index);
  const size_t begin = (i * base + (i < rem ? i : rem)) * align;
  size_t len = (base + (i < rem ? 1 : 0)) * align;
  if (index == parts - 1) len += tail;
  return Span{begin, len};
}

}  // namespace purlin
