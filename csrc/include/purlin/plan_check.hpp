// Static bounds check of a plan: every byte range a step will touch must lie inside the region it addresses.
//
// The reference has no sanitizer hooks and relies on static_asserts inside its templates (for example
// csrc/include/purlin/snac.cuh:55-56,399-400,1181-1182). Here a plan is data, so it can be checked before it is
// launched: user source and destination extents, the staging half, the packet slot (and its input / result halves for
// the composed all-reduce), CTA ranges inside the grid, access alignment, chunk arithmetic, and that the steps' writes
// tile the user's output exactly (no byte left stale, no byte with two writers). The check is host-only
// and costs well under a microsecond per step, so planFor (host_core.cpp) runs it on every plan it hands out: the
// GPU launcher, the CPU interpreter, the gloo executor and purlin_plan_build never see an unchecked plan. Tests
// sweep it over worlds 2-16, sizes around every band boundary and forced policies, and corrupt plans on purpose.
#pragma once
#include <cstdio>
#include <string>

#include "context.hpp"
#include "layout.hpp"
#include "plan.hpp"

namespace purlin {

struct PlanExtents {
  size_t srcBytes = 0;       // user input of this rank
  size_t dstBytes = 0;       // user output of this rank
  bool inPlace = false;      // src and dst are one buffer: the rank's own slice may stay where it is
};

// user buffer extents of one rank for a collective (the byte conventions of the host API)
inline PlanExtents extentsFor(const CollectiveSpec& s) {
  PlanExtents e;
  e.inPlace = s.inPlace;
  size_t sumIn = 0, sumOut = 0;
  for (int q = 0; q < s.world && q < kMaxRanks; ++q) { sumIn += s.sizes[q]; sumOut += s.outSizes[q]; }
  const size_t w = size_t(s.world);
  switch (s.type) {
    case CollectiveType::allReduce: e.srcBytes = s.bytes; e.dstBytes = s.bytes; break;
    case CollectiveType::allGather: e.srcBytes = s.bytes; e.dstBytes = s.bytes * w; break;
    case CollectiveType::allGatherV: e.srcBytes = s.sizes[s.rank]; e.dstBytes = sumIn; break;
    case CollectiveType::reduceScatter: e.srcBytes = s.bytes * w; e.dstBytes = s.bytes; break;
    case CollectiveType::reduceScatterV: e.srcBytes = sumIn; e.dstBytes = s.sizes[s.rank]; break;
    case CollectiveType::allToAll: e.srcBytes = s.bytes * w; e.dstBytes = s.bytes * w; break;
    default: e.srcBytes = sumIn; e.dstBytes = sumOut; break;   // allToAllV
  }
  return e;
}

namespace detail {
inline bool within(size_t off, size_t len, size_t limit) { return off <= limit && len <= limit - off; }
}  // namespace detail

// Every byte of the user's output must be written by exactly one step: the ranges the steps write to `dst` have to
// tile [0, dstBytes) with neither a gap (stale output) nor an overlap (two writers racing). An in-place call may leave
// the rank's own slice untouched, so only overlaps are errors there.
inline std::string checkCoverage(const Plan& plan, int world, const PlanExtents& ext) {
  struct Range { size_t begin, end; int step; };
  Range ranges[kMaxSteps + kMaxRanks];
  int n = 0;
  for (int i = 0; i < plan.nSteps; ++i) {
    const Step& s = plan.steps[i];
    bool writes = false;
    switch (s.role) {
      case kRoleLocal: case kRoleConsume: case kRoleGather: case kRolePacketGet: case kRolePacketReduce: writes = true; break;
      case kRoleReduce: writes = (s.flags & kFlagToDst) != 0; break;
      default: break;
    }
    if (writes && s.bytes && s.role == kRolePacketGet && s.peer < 0) {
      // packets of every peer in one step: slice q lands at dstOff + q * bytes, this rank's own slice is left alone
      for (int q = 0; q < world && n < kMaxSteps + kMaxRanks; ++q)
        if (uint64_t(q) != s.seamOff) ranges[n++] = Range{size_t(s.dstOff + uint64_t(q) * s.bytes), size_t(s.dstOff + uint64_t(q + 1) * s.bytes), i};
      continue;
    }
    if (writes && s.bytes && n < kMaxSteps + kMaxRanks) ranges[n++] = Range{size_t(s.dstOff), size_t(s.dstOff + s.bytes), i};
  }
  for (int a = 1; a < n; ++a)                       // insertion sort: at most kMaxSteps entries
    for (int b = a; b > 0 && ranges[b].begin < ranges[b - 1].begin; --b) { const Range t = ranges[b]; ranges[b] = ranges[b - 1]; ranges[b - 1] = t; }
  char buf[200];
  size_t at = 0;
  for (int k = 0; k < n; ++k) {
    if (ranges[k].begin < at) {
      std::snprintf(buf, sizeof(buf), "steps %d and %d both write the output at byte %zu", ranges[k - 1].step, ranges[k].step, ranges[k].begin);
      return buf;
    }
    if (ranges[k].begin > at && !ext.inPlace) {
      std::snprintf(buf, sizeof(buf), "no step writes the output bytes [%zu, %zu)", at, ranges[k].begin);
      return buf;
    }
    at = ranges[k].end;
  }
  if (at < ext.dstBytes && !ext.inPlace) {
    std::snprintf(buf, sizeof(buf), "no step writes the output bytes [%zu, %zu)", at, ext.dstBytes);
    return buf;
  }
  return std::string();
}

// Returns an empty string when the plan is sound, else a description of the first violation.
inline std::string checkPlan(const Plan& plan, int world, const WorkspaceLayout& ws, const PlanExtents& ext) {
  char buf[256];
  auto bad = [&](int i, const char* what, size_t off, size_t len, size_t limit) {
    std::snprintf(buf, sizeof(buf), "step %d (role %d, peer %d): %s [%zu, +%zu) exceeds %zu", i, int(plan.steps[i].role), int(plan.steps[i].peer),
                  what, off, len, limit);
    return std::string(buf);
  };
  if (plan.nSteps < 0 || plan.nSteps > kMaxSteps) return "step count outside the plan's capacity";
  if (plan.blocks < 1 || plan.blocks > kMaxCtas) return "grid size outside [1, max CTAs]";
  if (plan.threads < 32 || plan.threads > 1024 || plan.threads % 32) return "block size must be a multiple of 32 up to 1024";
  bool composedPackets = false;
  for (int i = 0; i < plan.nSteps; ++i) composedPackets = composedPackets || (plan.steps[i].flags & (kFlagPublish | kFlagResultHalf));
  const size_t slotBytes = composedPackets ? ws.packetStride / 2 : ws.packetStride;   // input half / whole slot
  for (int i = 0; i < plan.nSteps; ++i) {
    const Step& s = plan.steps[i];
    if (s.blockCount < 1 || s.blockBegin < 0 || s.blockBegin + s.blockCount > plan.blocks) {
      std::snprintf(buf, sizeof(buf), "step %d: CTA range [%d, +%d) outside a grid of %d", i, int(s.blockBegin), int(s.blockCount), int(plan.blocks));
      return buf;
    }
    if (s.peer >= world) { std::snprintf(buf, sizeof(buf), "step %d: peer %d outside a world of %d", i, int(s.peer), world); return buf; }
    const bool packet = s.role >= kRolePacketPut;
    if (packet) {
      if (s.bytes % 8) return bad(i, "packet payload not a multiple of 8", 0, s.bytes, 8);
      const size_t words = s.bytes / 8;
      switch (s.role) {
        case kRolePacketPut:
          if ((s.flags & kFlagScatter) && (s.peer >= 0 || s.seamOff >= uint64_t(world))) return bad(i, "scattered put needs peer -1 and the own slice index", s.seamOff, 1, size_t(world));
          if (!detail::within(s.srcOff, (s.flags & kFlagScatter) ? s.bytes * size_t(world) : s.bytes, ext.srcBytes))
            return bad(i, "source", s.srcOff, (s.flags & kFlagScatter) ? s.bytes * size_t(world) : s.bytes, ext.srcBytes);
          if (!detail::within(s.dstOff * 2, words * 16, slotBytes)) return bad(i, "packet slot (put)", s.dstOff * 2, words * 16, slotBytes);
          break;
        case kRolePacketGet:
          if (s.peer < 0 && s.seamOff >= uint64_t(world)) return bad(i, "own slice index of an all-peers get", s.seamOff, 1, size_t(world));
          if (!detail::within(s.dstOff, s.peer < 0 ? s.bytes * size_t(world) : s.bytes, ext.dstBytes))
            return bad(i, "destination", s.dstOff, s.peer < 0 ? s.bytes * size_t(world) : s.bytes, ext.dstBytes);
          if (!detail::within(s.srcOff * 2, words * 16, (s.flags & kFlagResultHalf) ? ws.packetStride / 2 : slotBytes))
            return bad(i, "packet slot (get)", s.srcOff * 2, words * 16, slotBytes);
          break;
        default:   // packet reduce
          if (!detail::within(s.seamOff, s.bytes, ext.srcBytes)) return bad(i, "own words in the source", s.seamOff, s.bytes, ext.srcBytes);
          if (!detail::within(s.dstOff, s.bytes, ext.dstBytes)) return bad(i, "destination", s.dstOff, s.bytes, ext.dstBytes);
          if (!detail::within(s.srcOff * 2, words * 16, slotBytes)) return bad(i, "packet slot (reduce)", s.srcOff * 2, words * 16, slotBytes);
          if ((s.flags & kFlagPublish) && !detail::within(0, words * 16, ws.packetStride / 2)) return bad(i, "result half", 0, words * 16, ws.packetStride / 2);
          break;
      }
      continue;
    }
    if (s.bytes == 0) continue;   // an empty stream touches nothing
    // chunk arithmetic
    if (s.chunkBytes == 0 || s.slots == 0) { std::snprintf(buf, sizeof(buf), "step %d: zero chunk size or slot count", i); return buf; }
    const size_t wantChunks = (s.bytes + s.chunkBytes - 1) / s.chunkBytes;
    if (s.role != kRoleLocal && size_t(s.chunks) != wantChunks) {
      std::snprintf(buf, sizeof(buf), "step %d: %u chunks for %zu bytes in chunks of %zu", i, s.chunks, size_t(s.bytes), size_t(s.chunkBytes));
      return buf;
    }
    if (s.chunks > (1u << kSeqShift) - 1) { std::snprintf(buf, sizeof(buf), "step %d: %u chunks overflow the flag's chunk field", i, s.chunks); return buf; }
    if (s.srcOff % 16 || s.dstOff % 16 || s.seamOff % 16 || (s.chunks > 1 && s.chunkBytes % kAccessAlign)) {
      std::snprintf(buf, sizeof(buf), "step %d: offsets must be 16-byte aligned and chunks a multiple of %d bytes", i, int(kAccessAlign));
      return buf;
    }
    // a window holds min(chunks, slots) chunks; the last chunk may be short
    const size_t live = s.chunks < s.slots ? s.chunks : s.slots;
    const size_t window = live == s.chunks ? s.bytes : live * s.chunkBytes;
    switch (s.role) {
      case kRoleStage:
        if (!detail::within(s.srcOff, s.bytes, ext.srcBytes)) return bad(i, "source", s.srcOff, s.bytes, ext.srcBytes);
        if (!detail::within(s.dstOff, window, ws.stagingTRSize)) return bad(i, "staging window (stage)", s.dstOff, window, ws.stagingTRSize);
        break;
      case kRoleLocal:
        if (!detail::within(s.srcOff, s.bytes, ext.srcBytes)) return bad(i, "source", s.srcOff, s.bytes, ext.srcBytes);
        if (!detail::within(s.dstOff, s.bytes, ext.dstBytes)) return bad(i, "destination", s.dstOff, s.bytes, ext.dstBytes);
        break;
      case kRoleConsume:
      case kRoleGather:
        if (s.peer < 0) { std::snprintf(buf, sizeof(buf), "step %d: a consumer needs a peer", i); return buf; }
        if (!detail::within(s.dstOff, s.bytes, ext.dstBytes)) return bad(i, "destination", s.dstOff, s.bytes, ext.dstBytes);
        if (!detail::within(s.srcOff, window, ws.stagingTRSize)) return bad(i, "staging window (consume)", s.srcOff, window, ws.stagingTRSize);
        break;
      case kRoleReduce:
        if (!detail::within(s.srcOff, window, ws.stagingTRSize)) return bad(i, "staging window (reduce)", s.srcOff, window, ws.stagingTRSize);
        if ((s.flags & kFlagToDst) && !detail::within(s.dstOff, s.bytes, ext.dstBytes)) return bad(i, "destination", s.dstOff, s.bytes, ext.dstBytes);
        if ((s.flags & kFlagToSeam) && !detail::within(s.seamOff, window, ws.stagingTRSize)) return bad(i, "seam", s.seamOff, window, ws.stagingTRSize);
        break;
      default:
        std::snprintf(buf, sizeof(buf), "step %d: unknown role %d", i, int(s.role));
        return buf;
    }
  }
  return checkCoverage(plan, world, ext);
}

}  // namespace purlin
