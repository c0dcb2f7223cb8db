// Layout engine: from (input layout, output layout, copy-or-reduce) to a SNAC plan.
//
// A collective is named by how its input and output are distributed
// (csrc/include/purlin/collective.cuh:8-58 of the reference):
//
//   reduceScatter   scattered  -> packed      reduce
//   allGather       packed     -> scattered   copy
//   allToAll        scattered  -> transposed  copy
//   allReduce       packed     -> packed      reduce            (direct, one-shot)
//   allReduce       compose(scattered->packed reduce, packed->scattered copy)  (two-shot)
//   ...V            the same with per-rank sizes
//
// The reference turns that triple into block roles, flags and offsets with
// nested `if constexpr` (snac.cuh:36-78, 572-807, 2019-2059). This file does
// the same derivation as ordinary host code that can be unit-tested: first a
// Topology (who stages what for whom, who is notified, who must drain a cyclic
// slot), then a Plan whose steps a generic kernel or the CPU interpreter runs.
#pragma once
#include <algorithm>
#include <cstring>
#include <string>
#include <vector>

#include "context.hpp"
#include "plan.hpp"

namespace purlin { namespace bulk { constexpr int kPlanMaxDepth = 13; constexpr size_t kPlanTileBytes = 16384; } }

namespace purlin {

enum class Notify : int32_t { allPeers = 0, one = 1 };
enum class Drain : int32_t { none = 0, allRanks, single, composed };

// What the layouts alone imply (no sizes, no tuning).
struct Topology {
  bool perDest = false;        // input scattered(V): one staging stream per destination
  bool perStream = false;      // scatteredV copy: protocol chosen per (src, dst) stream
  bool variable = false;       // any V layout
  bool varLenArrival = false;  // arrival handshake needed (a rank may wait on nothing)
  bool selfDirect = false;     // copy collectives move the self slice src -> dst directly
  bool reduceWhole = false;    // packed -> packed reduce: every rank reduces the whole payload
  Notify notify = Notify::allPeers;
  Drain drain = Drain::none;   // who must report "consumed" before a cyclic slot is reused
};

inline bool isVariable(DataLayout l) {
  return l == DataLayout::packedV || l == DataLayout::scatteredV || l == DataLayout::transposedV;
}
inline bool isScattered(DataLayout l) { return l == DataLayout::scattered || l == DataLayout::scatteredV; }
inline bool isPacked(DataLayout l) { return l == DataLayout::packed || l == DataLayout::packedV; }
inline bool isTransposed(DataLayout l) { return l == DataLayout::transposed || l == DataLayout::transposedV; }

// Which (in, out, op) triples are collectives at all.
inline bool validTriple(DataLayout in, DataLayout out, ConsumeOp op) {
  if (isVariable(in) != isVariable(out)) return false;
  if (op == ConsumeOp::copy) return (isPacked(in) && isScattered(out)) || (isScattered(in) && isTransposed(out));
  return (isScattered(in) && isPacked(out)) || (in == DataLayout::packed && out == DataLayout::packed);
}

inline Topology deriveTopology(DataLayout in, DataLayout out, ConsumeOp op, bool cyclic) {
  Topology t;
  t.perDest = isScattered(in);
  t.variable = isVariable(in) || isVariable(out);
  t.perStream = op == ConsumeOp::copy && in == DataLayout::scatteredV;
  t.varLenArrival = t.variable;
  t.selfDirect = op == ConsumeOp::copy;
  t.reduceWhole = op == ConsumeOp::reduce && isPacked(in);
  t.notify = t.perDest ? Notify::one : Notify::allPeers;
  if (cyclic) t.drain = t.perDest ? Drain::single : Drain::allRanks;
  return t;
}

// Largest-remainder apportionment of `total` CTAs over streams by weight; every
// non-empty stream gets at least one (the host-side form of mapWeightedPeerBlock,
// csrc/include/purlin/partition.cuh:97-215). Returns false if total is too small.
inline bool apportion(int total, const std::vector<size_t>& weight, std::vector<int>& out) {
  const size_t n = weight.size();
  out.assign(n, 0);
  int live = 0;
  long double sum = 0;
  for (size_t w : weight) { if (w) { ++live; sum += w; } }
  if (live == 0) return true;
  if (total < live) return false;
  int spare = total - live, given = 0;
  std::vector<std::pair<long double, size_t>> frac;
  for (size_t i = 0; i < n; ++i) {
    if (!weight[i]) continue;
    const long double share = (long double)spare * weight[i] / sum;
    const int whole = (int)share;
    out[i] = 1 + whole;
    given += whole;
    frac.push_back({share - whole, i});
  }
  std::stable_sort(frac.begin(), frac.end(), [](auto& a, auto& b) { return a.first > b.first; });
  for (size_t k = 0; given < spare && k < frac.size(); ++k, ++given) ++out[frac[k].second];
  return true;
}

// Tuning knobs of one launch; the codesign policy (tuning.hpp) fills them per size and world.
struct Policy {
  int32_t regime = int32_t(Regime::throughput);
  int32_t threads = 256;
  int32_t putBlocks = 16;
  int32_t localBlocks = 4;
  int32_t consumeBlocks = 32;   // total over peers
  int32_t gatherBlocks = 16;    // total over peers
  int32_t lrBlocks = 32;
  int32_t memType = int32_t(MemType::unicast);
  int32_t mmDepth = 4;
  int32_t unroll = 4;
  int32_t stageDepth = 0;
  int32_t arPath = int32_t(AllReducePath::composed);
  int32_t lrMulticast = 0;
  int32_t weighted = 1;         // apportion CTAs by stream size in V collectives
  uint64_t chunkBytes = 0;      // 0: one flag per stream
  uint64_t perStreamThreshold = 128ull << 10;
  int32_t maxCtas = 0;          // > 0: the plan may use at most this many CTAs (the collective shares the GPU with other work)
  int32_t reserved = 0;
};

// Shrinks the CTA counts of a policy so that a plan built from it fits `budget` CTAs, given that the plan built from the
// unshrunk policy needed `needed`. The reference caps every collective at 64 CTAs (csrc/include/purlin/constants.cuh:21)
// so that it can run beside compute kernels; here the cap is a knob (0 = the whole GPU).
inline void shrinkToBudget(Policy& p, int needed, int budget, int world) {
  if (budget <= 0 || needed <= budget) return;
  auto scale = [&](int32_t& v, int floorAt) { v = std::max<int32_t>(int32_t(int64_t(v) * budget / needed), floorAt); };
  const int peers = std::max(world - 1, 1);
  scale(p.putBlocks, 1);
  scale(p.localBlocks, 1);
  scale(p.consumeBlocks, peers);
  scale(p.gatherBlocks, peers);
  scale(p.lrBlocks, 1);
}

struct CollectiveSpec {
  CollectiveType type = CollectiveType::allReduce;
  DataLayout in = DataLayout::packed;
  DataLayout out = DataLayout::packed;
  ConsumeOp op = ConsumeOp::reduce;
  ReduceOp reduceOp = ReduceOp::add;
  DType dtype = DType::bf16;
  ReductionMode mode = ReductionMode::nonDeterministic;
  int32_t world = 2;
  int32_t rank = 0;
  // fixed-size collectives: allReduce = whole payload; allGather = bytes per rank in;
  // reduceScatter = bytes per rank out; allToAll = bytes per peer slice.
  size_t bytes = 0;
  // variable-length: allGatherV / reduceScatterV: sizes[q] for every rank q (same list on all ranks);
  // allToAllV: sizes[d] = bytes this rank sends to d, outSizes[q] = bytes it receives from q.
  size_t sizes[kMaxRanks] = {};
  size_t outSizes[kMaxRanks] = {};
  bool multicastAvailable = false;
  bool inPlace = false;         // src and dst are the same buffer
};

inline CollectiveSpec specFor(CollectiveType type) {
  CollectiveSpec s;
  s.type = type;
  switch (type) {
    case CollectiveType::allReduce: s.in = DataLayout::packed; s.out = DataLayout::packed; s.op = ConsumeOp::reduce; break;
    case CollectiveType::allGather: s.in = DataLayout::packed; s.out = DataLayout::scattered; s.op = ConsumeOp::copy; break;
    case CollectiveType::allGatherV: s.in = DataLayout::packedV; s.out = DataLayout::scatteredV; s.op = ConsumeOp::copy; break;
    case CollectiveType::reduceScatter: s.in = DataLayout::scattered; s.out = DataLayout::packed; s.op = ConsumeOp::reduce; break;
    case CollectiveType::reduceScatterV: s.in = DataLayout::scatteredV; s.out = DataLayout::packedV; s.op = ConsumeOp::reduce; break;
    case CollectiveType::allToAll: s.in = DataLayout::scattered; s.out = DataLayout::transposed; s.op = ConsumeOp::copy; break;
    case CollectiveType::allToAllV: s.in = DataLayout::scatteredV; s.out = DataLayout::transposedV; s.op = ConsumeOp::copy; break;
  }
  return s;
}

namespace detail {

struct Builder {
  Plan& plan;
  std::string& err;
  uint32_t nextCounter = 0;
  int nextBlock = 0;

  bool add(Step s) {
    if (s.bytes == 0) return true;                 // empty streams do not exist
    if (plan.nSteps >= kMaxSteps) { err = "plan needs more than kMaxSteps steps"; return false; }
    s.counterBase = nextCounter;
    nextCounter += std::min<uint32_t>(std::max<uint32_t>(s.chunks, 1), kMaxChunks);
    plan.steps[plan.nSteps++] = s;
    return true;
  }
  // reserve a CTA range
  int take(int count) { const int b = nextBlock; nextBlock += count; return b; }
};

// Chunk geometry of one stream: same answer on producer and consumer because it
// depends only on the stream length, the policy chunk and the window.
inline void chunkStream(Step& s, size_t chunkBytes, size_t windowBytes) {
  size_t c = chunkBytes ? std::min<size_t>(chunkBytes, s.bytes) : s.bytes;
  if (s.bytes > windowBytes) {                     // must cycle through the window
    if (c > windowBytes || !chunkBytes) c = std::max<size_t>(roundDown(windowBytes / 4, kAccessAlign), kAccessAlign);
  }
  c = std::max<size_t>(roundUp(c, kAccessAlign), kAccessAlign);
  // flags reserve 2^20 values per call
  while (ceilDiv(s.bytes, c) >= (1u << kSeqShift)) c *= 2;
  for (;;) {
    s.chunkBytes = c;
    s.chunks = uint32_t(ceilDiv(s.bytes, c));
    const size_t fit = std::max<size_t>(windowBytes / c, 1);
    if (s.chunks > fit) {
      s.slots = uint32_t(std::min<size_t>(fit, kMaxChunks));
      s.flags |= kFlagCyclic;
      return;
    }
    // A resident stream has no back-pressure between the CTAs of a step, and its last-arrival counters are indexed
    // k mod kMaxChunks: more chunks than counters would let a CTA that runs ahead share a counter with a chunk still
    // in use. A caller-forced tiny chunk is therefore raised until the stream has at most kMaxChunks chunks.
    if (s.chunks <= uint32_t(kMaxChunks)) { s.slots = s.chunks; return; }
    c = roundUp(c * 2, kAccessAlign);
  }
}

}  // namespace detail

// Compose check (csrc/include/purlin/snac.cuh:1986-2007): the head's output layout must be
// the tail's input layout, both fixed-size, and the head's input must be scattered.
inline bool composable(DataLayout headIn, DataLayout headOut, ConsumeOp headOp,
                       DataLayout tailIn, DataLayout tailOut, ConsumeOp tailOp, std::string& err) {
  if (!validTriple(headIn, headOut, headOp) || !validTriple(tailIn, tailOut, tailOp)) { err = "compose: not a collective"; return false; }
  if (headOut != tailIn) { err = "compose: head output layout differs from tail input layout"; return false; }
  if (isVariable(headIn) || isVariable(headOut) || isVariable(tailOut)) { err = "compose: fixed-size layouts only"; return false; }
  if (headIn != DataLayout::scattered) { err = "compose: head input must be scattered"; return false; }
  return true;
}

inline bool buildThroughputPlan(const CollectiveSpec& spec, const Policy& pol, const WorkspaceLayout& ws,
                                Plan& plan, std::string& err);
inline bool buildLatencyPlan(const CollectiveSpec& spec, const Policy& pol, const WorkspaceLayout& ws,
                             Plan& plan, std::string& err);

inline bool buildPlan(const CollectiveSpec& spec, const Policy& pol, const WorkspaceLayout& ws,
                      Plan& plan, std::string& err) {
  std::memset(&plan, 0, sizeof(plan));
  if (spec.world < 1 || spec.world > kMaxRanks || spec.rank < 0 || spec.rank >= spec.world) { err = "invalid rank or world"; return false; }
  if (!validTriple(spec.in, spec.out, spec.op)) { err = "layout pair is not a collective"; return false; }
  plan.collective = int32_t(spec.type);
  plan.regime = pol.regime;
  plan.consumeOp = int32_t(spec.op);
  plan.reduceOp = int32_t(spec.reduceOp);
  plan.dtype = int32_t(spec.dtype);
  plan.deterministic = int32_t(spec.mode);
  plan.threads = pol.threads;
  plan.mmDepth = pol.mmDepth;
  plan.unroll = pol.unroll;
  plan.stageDepth = std::min(std::max(pol.stageDepth, 0), bulk::kPlanMaxDepth);
  if (plan.stageDepth == 1) plan.stageDepth = 2;   // a ring needs a tile in flight and a tile being stored
  plan.smemBytes = (plan.stageDepth > 0 && pol.regime == int32_t(Regime::throughput)) ? size_t(plan.stageDepth) * bulk::kPlanTileBytes + 256 : 0;
  const bool ok = pol.regime == int32_t(Regime::latency) ? buildLatencyPlan(spec, pol, ws, plan, err)
                                                          : buildThroughputPlan(spec, pol, ws, plan, err);
  if (!ok) return false;
  int blocks = 0;
  for (int i = 0; i < plan.nSteps; ++i) blocks = std::max(blocks, plan.steps[i].blockBegin + plan.steps[i].blockCount);
  plan.blocks = std::max(blocks, 1);
  if (plan.blocks > kMaxCtas) { err = "plan needs more CTAs than the GPU has SMs"; return false; }
  return true;
}

// Sizes of every (source q -> destination d) piece as far as this rank knows them.
struct PieceTable {
  size_t send[kMaxRanks] = {};     // bytes this rank stages for destination d (packed input: same for all d)
  size_t sendOff[kMaxRanks] = {};  // offset of that piece in user src
  size_t recv[kMaxRanks] = {};     // bytes this rank consumes from source q
  size_t recvOff[kMaxRanks] = {};  // offset in user dst where the piece from q lands (copy) / 0 (reduce)
  size_t stageOff[kMaxRanks] = {}; // offset of piece (this -> d) in own staging half
  size_t peerOff[kMaxRanks] = {};  // offset of piece (q -> this) in q's staging half
  size_t window[kMaxRanks] = {};   // bytes of staging the stream (this -> d) may occupy
  size_t peerWindow[kMaxRanks] = {};
  size_t total = 0;                // bytes this rank stages in all
};

inline bool pieceTable(const CollectiveSpec& s, const WorkspaceLayout& ws, AllReducePath arPath,
                       PieceTable& t, std::string& err) {
  const int W = s.world, r = s.rank;
  const size_t S = ws.stagingTRSize;
  auto bad = [&](const char* m) { err = m; return false; };
  if (s.op == ConsumeOp::reduce && isPacked(s.in)) {
    if (arPath == AllReducePath::direct) {
      for (int q = 0; q < W; ++q) { t.send[q] = s.bytes; t.sendOff[q] = 0; t.recv[q] = s.bytes; t.stageOff[q] = 0; t.peerOff[q] = 0; t.window[q] = t.peerWindow[q] = S; }
      t.total = s.bytes;
      return true;
    }
    // composed: shard d of the payload travels to rank d
    for (int d = 0; d < W; ++d) {
      const Span sh = partitionAligned(s.bytes, W, d, kAccessAlign);
      t.send[d] = sh.bytes; t.sendOff[d] = sh.offset; t.stageOff[d] = sh.offset;
    }
    const Span mine = partitionAligned(s.bytes, W, r, kAccessAlign);
    for (int q = 0; q < W; ++q) { t.recv[q] = mine.bytes; t.recvOff[q] = mine.offset; t.peerOff[q] = mine.offset; }
    t.total = s.bytes;
    if (s.bytes <= S) { for (int q = 0; q < W; ++q) t.window[q] = t.peerWindow[q] = S; }
    else {
      // Larger than the staging half: shard d streams through window d of the staging half, chunk by chunk, under
      // back-pressure; the reducer's window doubles as the seam the peers gather from. One launch drives the whole
      // payload (csrc/include/purlin/host/allReduce.cuh:217-260 of the reference: cyclic slots, one region per rank).
      const size_t perDestWindow = roundDown(S / size_t(W), kAccessAlign);
      if (perDestWindow < kAccessAlign) return bad("staging buffer too small for this world size");
      for (int d = 0; d < W; ++d) { t.stageOff[d] = size_t(d) * perDestWindow; t.window[d] = perDestWindow; }
      for (int q = 0; q < W; ++q) { t.peerOff[q] = size_t(r) * perDestWindow; t.peerWindow[q] = perDestWindow; }
    }
    return true;
  }
  if (isPacked(s.in)) {   // all-gather family
    const bool v = s.in == DataLayout::packedV;
    size_t off = 0;
    for (int q = 0; q < W; ++q) {
      const size_t n = v ? s.sizes[q] : s.bytes;
      t.recv[q] = n; t.recvOff[q] = off; off += n; t.peerOff[q] = 0; t.peerWindow[q] = S;
    }
    const size_t mine = v ? s.sizes[r] : s.bytes;
    for (int d = 0; d < W; ++d) { t.send[d] = mine; t.sendOff[d] = 0; t.stageOff[d] = 0; t.window[d] = S; }
    t.total = mine;
    return true;
  }
  // scattered input: reduce-scatter and all-to-all families
  const bool v = s.in == DataLayout::scatteredV;
  const bool a2av = v && s.op == ConsumeOp::copy;
  size_t off = 0, sum = 0;
  for (int d = 0; d < W; ++d) {
    const size_t n = v ? s.sizes[d] : s.bytes;
    t.send[d] = n; t.sendOff[d] = off; off += n; sum += n;
  }
  t.total = sum;
  const size_t perDestWindow = roundDown(S / size_t(W), kAccessAlign);
  // Resident when every rank's whole input fits and every rank can compute every offset.
  // all-to-all-v cannot (a receiver does not know the sender's other splits), so it always
  // uses fixed per-destination windows; so does any payload larger than the staging half.
  const bool windows = a2av || sum > S;
  size_t outOff = 0;
  for (int q = 0; q < W; ++q) {
    size_t n;
    if (s.op == ConsumeOp::reduce) n = v ? s.sizes[r] : s.bytes;
    else n = v ? s.outSizes[q] : s.bytes;
    t.recv[q] = n;
    t.recvOff[q] = s.op == ConsumeOp::reduce ? 0 : outOff;
    outOff += n;
  }
  for (int d = 0; d < W; ++d) {
    t.stageOff[d] = windows ? size_t(d) * perDestWindow : t.sendOff[d];
    t.window[d] = windows ? perDestWindow : S;
  }
  for (int q = 0; q < W; ++q) {
    // where rank q keeps its piece for me: same rule evaluated for destination r
    if (windows) t.peerOff[q] = size_t(r) * perDestWindow;
    else if (v) { size_t o = 0; for (int d = 0; d < r; ++d) o += s.sizes[d]; t.peerOff[q] = o; }
    else t.peerOff[q] = size_t(r) * s.bytes;
    t.peerWindow[q] = windows ? perDestWindow : S;
  }
  if (perDestWindow < kAccessAlign) return bad("staging buffer too small for this world size");
  return true;
}

inline bool buildThroughputPlan(const CollectiveSpec& spec, const Policy& pol, const WorkspaceLayout& ws,
                                Plan& plan, std::string& err) {
  const int W = spec.world, r = spec.rank;
  const bool reduce = spec.op == ConsumeOp::reduce;
  const bool arWhole = reduce && isPacked(spec.in);
  const AllReducePath path = arWhole ? AllReducePath(pol.arPath) : AllReducePath::direct;
  const bool composed = arWhole && path == AllReducePath::composed && W > 1;
  if (composed) {
    std::string why;
    if (!composable(DataLayout::scattered, DataLayout::packed, ConsumeOp::reduce,
                    DataLayout::packed, DataLayout::scattered, ConsumeOp::copy, why)) { err = why; return false; }
  }
  PieceTable pt;
  if (!pieceTable(spec, ws, composed ? AllReducePath::composed : AllReducePath::direct, pt, err)) return false;
  const Topology topo = deriveTopology(composed ? DataLayout::scattered : spec.in, spec.out, spec.op, false);
  plan.varLenArrival = topo.varLenArrival ? 1 : 0;
  const bool perDest = topo.perDest;
  const bool useMultimem = reduce && pol.memType == int32_t(MemType::multimem) && spec.multicastAvailable &&
                           spec.mode == ReductionMode::nonDeterministic;
  detail::Builder b{plan, err};
  const size_t shardChunk = composed && pol.chunkBytes ? std::max<size_t>(roundUp(pol.chunkBytes / size_t(W), kAccessAlign), kAccessAlign) : pol.chunkBytes;

  // ---- stage ----
  if (!perDest) {
    Step s{};
    s.role = kRoleStage; s.peer = -1;
    s.srcOff = 0; s.dstOff = 0; s.bytes = pt.total;
    if (reduce) s.flags |= kFlagDrainSelf;
    detail::chunkStream(s, pol.chunkBytes, pt.window[0]);
    s.blockCount = std::max(pol.putBlocks, 1); s.blockBegin = b.take(s.blockCount);
    if (!b.add(s)) return false;
  } else {
    std::vector<size_t> weight(W, 0);
    for (int d = 0; d < W; ++d) {
      const bool viaPacket = topo.perStream && pt.send[d] <= pol.perStreamThreshold;
      const bool skipSelf = !reduce && d == r;     // copy collectives move the self slice directly
      weight[d] = (viaPacket || skipSelf) ? 0 : (pol.weighted && topo.variable ? pt.send[d] : (pt.send[d] ? 1 : 0));
    }
    int live = 0; for (size_t w : weight) live += w ? 1 : 0;
    std::vector<int> blocks;
    if (!apportion(std::max(pol.putBlocks, live), weight, blocks)) { err = "not enough put CTAs"; return false; }
    for (int k = 0; k < W; ++k) {
      const int d = (r + 1 + k) % W;               // rotate so ranks do not all feed the same peer first
      if (!weight[d]) continue;
      Step s{};
      s.role = kRoleStage; s.peer = d;
      s.srcOff = pt.sendOff[d]; s.dstOff = pt.stageOff[d]; s.bytes = pt.send[d];
      detail::chunkStream(s, shardChunk, pt.window[d]);
      if (composed && (s.flags & kFlagCyclic)) s.flags |= kFlagDrainGather;
      s.blockCount = blocks[d]; s.blockBegin = b.take(s.blockCount);
      if (!b.add(s)) return false;
    }
  }

  // ---- the self slice of a copy collective ----
  if (!reduce && pt.recv[r] && !spec.inPlace) {
    Step s{};
    s.role = kRoleLocal; s.peer = r;
    s.srcOff = perDest ? pt.sendOff[r] : 0; s.dstOff = pt.recvOff[r]; s.bytes = pt.recv[r];
    s.chunkBytes = s.bytes; s.chunks = 1; s.slots = 1;
    s.blockCount = std::max(pol.localBlocks, 1); s.blockBegin = b.take(s.blockCount);
    if (!b.add(s)) return false;
  } else if (!reduce && pt.recv[r] && spec.inPlace && pt.recvOff[r] != (perDest ? pt.sendOff[r] : 0)) {
    err = "in-place copy collective needs the self slice already in position"; return false;
  }

  // ---- consume ----
  if (!reduce) {
    std::vector<size_t> weight(W, 0);
    for (int q = 0; q < W; ++q) {
      const bool viaPacket = topo.perStream && pt.recv[q] <= pol.perStreamThreshold;
      weight[q] = (q == r || viaPacket) ? 0 : (pol.weighted && topo.variable ? pt.recv[q] : (pt.recv[q] ? 1 : 0));
    }
    int live = 0; for (size_t w : weight) live += w ? 1 : 0;
    std::vector<int> blocks;
    if (!apportion(std::max(pol.consumeBlocks, live), weight, blocks)) { err = "not enough consumer CTAs"; return false; }
    for (int k = 1; k < W; ++k) {
      const int q = (r + k) % W;
      if (!weight[q]) continue;
      Step s{};
      s.role = kRoleConsume; s.peer = q;
      s.srcOff = pt.peerOff[q]; s.dstOff = pt.recvOff[q]; s.bytes = pt.recv[q];
      detail::chunkStream(s, pol.chunkBytes, pt.peerWindow[q]);
      s.blockCount = blocks[q]; s.blockBegin = b.take(s.blockCount);
      if (!b.add(s)) return false;
    }
    // short all-to-all-v streams travel as packets through the latency buffer; one CTA range serves them all
    if (topo.perStream) {
      bool any = false;
      for (int q = 0; q < W; ++q) if (q != r && ((pt.send[q] && pt.send[q] <= pol.perStreamThreshold) || (pt.recv[q] && pt.recv[q] <= pol.perStreamThreshold))) any = true;
      if (any) {
        const int n = std::max(pol.localBlocks, 1), begin = b.take(n);
        for (int k = 1; k < W; ++k) {
          const int d = (r + k) % W;
          if (!pt.send[d] || pt.send[d] > pol.perStreamThreshold) continue;
          if (pt.send[d] > ws.packetStride / 2) { err = "per-stream packet threshold exceeds the packet slot"; return false; }
          Step s{}; s.role = kRolePacketPut; s.peer = d; s.srcOff = pt.sendOff[d]; s.dstOff = 0; s.bytes = pt.send[d];
          s.chunkBytes = s.bytes; s.chunks = 1; s.slots = 1; s.blockBegin = begin; s.blockCount = n;
          if (!b.add(s)) return false;
        }
        for (int k = 1; k < W; ++k) {
          const int q = (r + k) % W;
          if (!pt.recv[q] || pt.recv[q] > pol.perStreamThreshold) continue;
          Step s{}; s.role = kRolePacketGet; s.peer = q; s.srcOff = 0; s.dstOff = pt.recvOff[q]; s.bytes = pt.recv[q];
          s.chunkBytes = s.bytes; s.chunks = 1; s.slots = 1; s.blockBegin = begin; s.blockCount = n;
          if (!b.add(s)) return false;
        }
      }
    }
  } else {
    Step s{};
    s.role = kRoleReduce; s.peer = -1;
    s.srcOff = pt.peerOff[r]; s.dstOff = pt.recvOff[r]; s.seamOff = pt.peerOff[r]; s.bytes = pt.recv[r];
    detail::chunkStream(s, composed ? shardChunk : pol.chunkBytes, pt.peerWindow[r]);
    s.flags |= kFlagToDst;
    if (useMultimem && s.bytes % 16 == 0) s.flags |= kFlagMultimemLoad;
    if (composed) {
      const bool cyclicSeam = (s.flags & kFlagCyclic) != 0;
      s.flags |= kFlagToSeam | kFlagNotifyGather;
      // Cyclic: the producers' back-pressure is the gather signal this step raises anyway, and consumedSignals belong
      // to the gatherers (they free the seam slot), so the reducer raises none. The reduced chunk stays in this rank's
      // own window (no switch broadcast: the peers' copies of window r still hold their inputs for this rank).
      if (cyclicSeam) s.flags &= ~uint32_t(kFlagCyclic);
      else if (s.flags & kFlagMultimemLoad) s.flags |= kFlagMulticastOut;
    }
    s.blockCount = std::max(pol.consumeBlocks, 1); s.blockBegin = b.take(s.blockCount);
    if (!b.add(s)) return false;
    if (composed) {
      const bool localGather = (s.flags & kFlagMulticastOut) != 0;
      std::vector<size_t> weight(W, 0);
      for (int q = 0; q < W; ++q) weight[q] = (q == r) ? 0 : (pt.send[q] ? 1 : 0);
      int live = 0; for (size_t w : weight) live += w ? 1 : 0;
      std::vector<int> blocks;
      if (!apportion(std::max(pol.gatherBlocks, live), weight, blocks)) { err = "not enough gather CTAs"; return false; }
      for (int k = 1; k < W; ++k) {
        const int q = (r + k) % W;
        if (!weight[q]) continue;
        Step g{};
        g.role = kRoleGather; g.peer = q;
        g.srcOff = pt.stageOff[q]; g.dstOff = pt.sendOff[q]; g.bytes = pt.send[q];
        detail::chunkStream(g, shardChunk, pt.window[q]);
        if (localGather) g.flags |= kFlagLocalSource;
        g.blockCount = blocks[q]; g.blockBegin = b.take(g.blockCount);
        if (!b.add(g)) return false;
      }
    }
  }
  plan.payloadBytes = pt.total;
  return true;
}

// Latency regime: every CTA walks every step, grid-striding over 8-byte words.
// Behaviour of snac.cuh:1203-1273 (copy), 1583-1813 (one-shot reduce) and
// 1829-1954 (partitioned two-shot reduce) in the reference.
inline bool buildLatencyPlan(const CollectiveSpec& spec, const Policy& pol, const WorkspaceLayout& ws,
                             Plan& plan, std::string& err) {
  const int W = spec.world, r = spec.rank;
  const bool reduce = spec.op == ConsumeOp::reduce;
  const bool arWhole = reduce && isPacked(spec.in);
  const bool composed = arWhole && AllReducePath(pol.arPath) == AllReducePath::composed && W > 1;
  PieceTable pt;
  WorkspaceLayout unbounded = ws; unbounded.stagingTRSize = ~size_t(0) >> 8;  // offsets here are packet offsets, not staging
  if (!pieceTable(spec, unbounded, composed ? AllReducePath::composed : AllReducePath::direct, pt, err)) return false;
  // Fixed-size forms: every rank waits on every peer's packets, which carry their own flags. Variable-length forms keep
  // the arrival handshake here too: a rank whose partition is empty waits on no packet at all and could run two calls
  // ahead, into the packet half a slower rank is still reading (found by the interpreter's overlapped-call schedules).
  plan.varLenArrival = (isVariable(spec.in) || isVariable(spec.out)) ? 1 : 0;
  const size_t slotPayload = ws.packetStride / 2;           // 16-byte packets carry 8 bytes
  const size_t cap = composed ? slotPayload / 2 : slotPayload;
  detail::Builder b{plan, err};
  const int n = std::max(pol.lrBlocks, 1);
  auto one = [&](Step s) { s.chunkBytes = s.bytes; s.chunks = 1; s.slots = 1; s.blockBegin = 0; s.blockCount = n; return b.add(s); };
  const bool mc = pol.lrMulticast && spec.multicastAvailable && spec.mode == ReductionMode::nonDeterministic;
  // Equal slices at q * bytes from a common base (every fixed-size form): the packets of all peers are fetched by ONE step
  // whose (peer, word) pairs are spread over the threads, so a rank polls its W - 1 peers at the same time instead of one
  // after the other with a CTA barrier between them (one memory round trip instead of W - 1).
  auto equalSlices = [&](const size_t* off, const size_t* len) {
    if (plan.varLenArrival || W < 2 || len[r] == 0 || off[r] < size_t(r) * len[r]) return false;
    const size_t base = off[r] - size_t(r) * len[r];
    for (int q = 0; q < W; ++q) if (len[q] != len[r] || off[q] != base + size_t(q) * len[r]) return false;
    return true;
  };

  if (isPacked(spec.in) && !composed) {
    // all-gather family and one-shot all-reduce: the same words go to every peer
    if (pt.total > cap) { err = "payload exceeds the packet slot"; return false; }
    Step p{}; p.role = kRolePacketPut; p.peer = -1; p.srcOff = 0; p.dstOff = 0; p.bytes = pt.total;
    if (mc) p.flags |= kFlagMulticastOut;
    if (!one(p)) return false;
  } else {
    for (int k = 1; k < W; ++k) if (pt.send[(r + k) % W] > cap) { err = "payload exceeds the packet slot"; return false; }
    if (equalSlices(pt.sendOff, pt.send)) {
      // one step sends every peer its slice: a thread loads one word and stores it once, instead of W - 1 steps whose
      // loads wait for the stores of the step before
      Step p{}; p.role = kRolePacketPut; p.peer = -1; p.flags |= kFlagScatter;
      p.srcOff = pt.sendOff[r] - size_t(r) * pt.send[r]; p.dstOff = 0; p.bytes = pt.send[r]; p.seamOff = uint64_t(r);
      if (!one(p)) return false;
    } else {
      for (int k = 1; k < W; ++k) {
        const int d = (r + k) % W;
        Step p{}; p.role = kRolePacketPut; p.peer = d; p.srcOff = pt.sendOff[d]; p.dstOff = 0; p.bytes = pt.send[d];
        if (!one(p)) return false;
      }
    }
  }
  if (!reduce) {
    if (pt.recv[r] && !spec.inPlace) {
      Step l{}; l.role = kRoleLocal; l.peer = r; l.srcOff = isScattered(spec.in) ? pt.sendOff[r] : 0; l.dstOff = pt.recvOff[r]; l.bytes = pt.recv[r];
      if (!one(l)) return false;
    }
    for (int k = 1; k < W; ++k) if (pt.recv[(r + k) % W] > cap) { err = "payload exceeds the packet slot"; return false; }
    if (equalSlices(pt.recvOff, pt.recv)) {
      Step g{}; g.role = kRolePacketGet; g.peer = -1; g.srcOff = 0; g.dstOff = pt.recvOff[r] - size_t(r) * pt.recv[r]; g.bytes = pt.recv[r]; g.seamOff = uint64_t(r);
      if (!one(g)) return false;
    } else {
      for (int k = 1; k < W; ++k) {
        const int q = (r + k) % W;
        Step g{}; g.role = kRolePacketGet; g.peer = q; g.srcOff = 0; g.dstOff = pt.recvOff[q]; g.bytes = pt.recv[q];
        if (!one(g)) return false;
      }
    }
  } else {
    Step red{}; red.role = kRolePacketReduce; red.peer = -1;
    red.srcOff = 0; red.bytes = pt.recv[r]; red.dstOff = pt.recvOff[r];
    red.seamOff = isScattered(spec.in) || composed ? pt.sendOff[r] : 0;   // own contribution inside user src
    red.flags |= kFlagToDst;
    if (composed) { red.flags |= kFlagPublish; if (mc) red.flags |= kFlagMulticastOut; }
    if (!one(red)) return false;
    if (composed && equalSlices(pt.sendOff, pt.send)) {
      Step g{}; g.role = kRolePacketGet; g.peer = -1; g.srcOff = 0; g.dstOff = pt.sendOff[r] - size_t(r) * pt.send[r]; g.bytes = pt.send[r]; g.seamOff = uint64_t(r);
      g.flags |= kFlagResultHalf;
      if (!one(g)) return false;
    } else if (composed) {
      for (int k = 1; k < W; ++k) {
        const int q = (r + k) % W;
        Step g{}; g.role = kRolePacketGet; g.peer = q; g.srcOff = 0; g.dstOff = pt.sendOff[q]; g.bytes = pt.send[q];
        g.flags |= kFlagResultHalf;
        if (!one(g)) return false;
      }
    }
  }
  plan.payloadBytes = pt.total;
  return true;
}

}  // namespace purlin
