// Codesign policy: which regime, variant, chunk size and CTA counts a call gets.
//
// The reference hard-codes about 150 constants per architecture and world size
// as compile-time structs (csrc/include/purlin/host/codesign.cuh:28-792) and
// picks a band with if-chains in each host launcher (host/allReduce.cuh:88-308).
// Here the policy is data: a table of (collective, world, size band) -> Policy
// that is filled from a bandwidth sweep on the machine and cached on disk by the
// Python package; the built-in defaults below are only the starting point of
// that sweep and the fallback when no measured table is loaded.
#pragma once
#include <mutex>
#include <vector>

#include "layout.hpp"

namespace purlin {

struct TuningEntry {
  int32_t collective;   // CollectiveType
  int32_t world;
  uint64_t maxBytes;    // band upper bound (inclusive) on the dispatch size
  Policy policy;
};

// Dispatch size of a call, the quantity bands are keyed on: all-reduce = whole payload,
// all-gather = per-rank input, reduce-scatter = per-rank output, all-to-all = per-peer slice,
// V variants = the largest such piece.
inline uint64_t dispatchBytes(const CollectiveSpec& s) {
  switch (s.type) {
    case CollectiveType::allGatherV:
    case CollectiveType::reduceScatterV: { uint64_t m = 0; for (int q = 0; q < s.world; ++q) m = std::max<uint64_t>(m, s.sizes[q]); return m; }
    case CollectiveType::allToAllV: { uint64_t m = 0; for (int q = 0; q < s.world; ++q) m = std::max<uint64_t>(m, std::max(s.sizes[q], s.outSizes[q])); return m; }
    default: return s.bytes;
  }
}

class TuningTable {
 public:
  static TuningTable& global() { static TuningTable t; return t; }
  void clear() { std::lock_guard<std::mutex> g(mu_); entries_.clear(); }
  void add(const TuningEntry& e) {
    std::lock_guard<std::mutex> g(mu_);
    entries_.push_back(e);
    std::stable_sort(entries_.begin(), entries_.end(), [](const TuningEntry& a, const TuningEntry& b) { return a.maxBytes < b.maxBytes; });
  }
  size_t size() const { return entries_.size(); }
  // The band that holds `bytes`; a payload beyond the largest measured band takes that band's policy (what was measured
  // at 256 MiB is a better guess for 1 GiB than the built-in starting point).
  bool lookup(CollectiveType c, int world, uint64_t bytes, Policy& out) const {
    std::lock_guard<std::mutex> g(mu_);
    const TuningEntry* largest = nullptr;
    for (const TuningEntry& e : entries_) {
      if (e.collective != int32_t(c) || e.world != world) continue;
      if (bytes <= e.maxBytes) { out = e.policy; return true; }
      largest = &e;     // entries are sorted by band
    }
    if (largest) { out = largest->policy; return true; }
    return false;
  }
 private:
  mutable std::mutex mu_;
  std::vector<TuningEntry> entries_;
};

// Built-in starting policy for B200 / NVLink 5 (seeded from the reference's Blackwell
// bands, host/codesign.cuh:193-224,331-371,431-478,546-573, then adjusted to this
// datapath: wider grids, because a B200 has 148 SMs and nothing else is running
// during a standalone collective).
inline Policy defaultPolicy(const CollectiveSpec& s, const WorkspaceLayout& ws) {
  Policy p;
  const int W = s.world;
  const uint64_t n = dispatchBytes(s);
  const uint64_t slotPayload = ws.packetStride / 2;
  p.threads = 256;
  p.unroll = 8;
  p.mmDepth = 4;
  p.weighted = 1;
  p.perStreamThreshold = std::min<uint64_t>(256ull << 10, slotPayload);
  const bool nvls = s.multicastAvailable && s.mode == ReductionMode::nonDeterministic;
  auto lrBlocks = [&](uint64_t bytes) { return int(std::min<uint64_t>(std::max<uint64_t>(ceilDiv(bytes, uint64_t(p.threads) * 8), 1), 128)); };
  switch (s.type) {
    case CollectiveType::allReduce: {
      const uint64_t oneShotMax = W <= 2 ? (1ull << 20) : W <= 4 ? (128ull << 10) : (64ull << 10);
      const uint64_t twoShotMax = W <= 2 ? 0 : std::min<uint64_t>(2ull << 20, (slotPayload / 2) * W);
      if (n <= oneShotMax && n <= slotPayload) {
        p.regime = int32_t(Regime::latency); p.arPath = int32_t(AllReducePath::direct);
        p.lrBlocks = lrBlocks(n); p.lrMulticast = nvls ? 1 : 0;
      } else if (n <= twoShotMax && n % (uint64_t(W) * 32) == 0) {
        p.regime = int32_t(Regime::latency); p.arPath = int32_t(AllReducePath::composed);
        p.lrBlocks = lrBlocks(n / W * 2); p.lrMulticast = nvls ? 1 : 0;
      } else {
        p.regime = int32_t(Regime::throughput);
        p.arPath = int32_t(W <= 2 ? AllReducePath::direct : AllReducePath::composed);
        p.memType = int32_t(nvls && W > 2 ? MemType::multimem : MemType::unicast);
        p.threads = 256;
        p.putBlocks = 32; p.consumeBlocks = p.memType == int32_t(MemType::multimem) ? 32 : 48; p.gatherBlocks = 32;
        p.chunkBytes = n <= (4ull << 20) ? 0 : n <= (64ull << 20) ? (2ull << 20) : (8ull << 20);
      }
      break;
    }
    case CollectiveType::allGather:
    case CollectiveType::allGatherV: {
      const uint64_t lrMax = W <= 2 ? (512ull << 10) : W <= 4 ? (256ull << 10) : (64ull << 10);
      if (n <= lrMax && n <= slotPayload) { p.regime = int32_t(Regime::latency); p.lrBlocks = lrBlocks(n * W); }
      else {
        p.regime = int32_t(Regime::throughput); p.putBlocks = 24; p.localBlocks = 8; p.consumeBlocks = 8 * (W - 1) > 64 ? 64 : 8 * (W - 1);
        if (W == 2) p.consumeBlocks = 32;
        p.chunkBytes = n <= (2ull << 20) ? 0 : (2ull << 20);
      }
      break;
    }
    case CollectiveType::reduceScatter:
    case CollectiveType::reduceScatterV: {
      const uint64_t lrMax = W <= 2 ? (512ull << 10) : W <= 4 ? (256ull << 10) : (128ull << 10);
      if (n <= lrMax && n <= slotPayload) { p.regime = int32_t(Regime::latency); p.lrBlocks = lrBlocks(n * W); }
      else {
        p.regime = int32_t(Regime::throughput); p.putBlocks = std::max(32, W); p.consumeBlocks = 48;
        p.chunkBytes = n <= (2ull << 20) ? 0 : (2ull << 20);
      }
      break;
    }
    case CollectiveType::allToAll: {
      const uint64_t lrMax = W <= 4 ? (256ull << 10) : (128ull << 10);
      if (n <= lrMax && n <= slotPayload) { p.regime = int32_t(Regime::latency); p.lrBlocks = lrBlocks(n * W); }
      else {
        p.regime = int32_t(Regime::throughput); p.putBlocks = std::max(4 * (W - 1), 16); p.localBlocks = 8;
        p.consumeBlocks = std::max(8 * (W - 1), 32) > 64 ? 64 : std::max(8 * (W - 1), 32);
        p.chunkBytes = n <= (2ull << 20) ? 0 : (2ull << 20);
      }
      break;
    }
    case CollectiveType::allToAllV: {
      // no whole-collective latency branch: the packet path is chosen per stream inside the plan
      p.regime = int32_t(Regime::throughput); p.putBlocks = std::max(4 * (W - 1), 16); p.localBlocks = 8;
      p.consumeBlocks = std::max(8 * (W - 1), 32) > 64 ? 64 : std::max(8 * (W - 1), 32);
      p.chunkBytes = 1ull << 20;
      break;
    }
  }
  return p;
}

// The fixed-size collective whose measured bands a variable-length call may borrow.
inline bool fixedSibling(CollectiveType t, CollectiveType& out) {
  switch (t) {
    case CollectiveType::allGatherV: out = CollectiveType::allGather; return true;
    case CollectiveType::reduceScatterV: out = CollectiveType::reduceScatter; return true;
    case CollectiveType::allToAllV: out = CollectiveType::allToAll; return true;
    default: return false;
  }
}

inline Policy selectPolicy(const CollectiveSpec& s, const WorkspaceLayout& ws) {
  Policy p;
  const TuningTable& table = TuningTable::global();
  bool found = table.lookup(s.type, s.world, dispatchBytes(s), p);
  if (!found) {
    // No band measured for a variable-length form: borrow the band its fixed-size sibling measured for the largest
    // stream of this call (CTA counts and chunk size carry over; the switch variants were measured for whole, equal
    // slices only and are dropped). A borrowed policy that does not fit the call falls back like any other (planFor).
    CollectiveType sibling;
    if (fixedSibling(s.type, sibling) && table.lookup(sibling, s.world, dispatchBytes(s), p)) {
      const Policy builtIn = defaultPolicy(s, ws);
      if (s.type == CollectiveType::allToAllV && p.regime != int32_t(Regime::throughput)) return builtIn;   // packets are chosen per stream there
      p.memType = int32_t(MemType::unicast);
      p.lrMulticast = 0;
      p.weighted = 1;
      if (p.perStreamThreshold == 0) p.perStreamThreshold = builtIn.perStreamThreshold;
      found = true;
    }
  }
  if (found) {
    // a measured entry may ask for NVLS; drop it where this call cannot use it
    if (!s.multicastAvailable || s.mode == ReductionMode::deterministic) { p.memType = int32_t(MemType::unicast); p.lrMulticast = 0; }
    return p;
  }
  return defaultPolicy(s, ws);
}

}  // namespace purlin
