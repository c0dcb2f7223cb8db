// Host-only half of libpurlin: the layout engine's C entry points, the tuning
// table and a CPU interpreter that executes the same Plan the GPU kernels run.
//
// The reference has no CPU emulation of its protocol (its multi-rank logic is
// only exercised on GPUs: csrc/tests/{ar,ag,rs,a2a}.cu). The interpreter here
// runs every rank of a collective inside one process over host memory, with
// real flag words, packet flags, last-arrival semantics and cyclic
// back-pressure, so protocol errors (a wait nobody satisfies, a slot reused too
// early, a byte produced twice or never) show up without a GPU. A rank can be
// made absent to check that the others report a time-out instead of hanging.
#include <atomic>
#include <cmath>
#include <cstdlib>
#include <cstdio>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "purlin/capi.h"
#include "purlin/layout.hpp"
#include "purlin/moe_route.cuh"
#include "purlin/plan_check.hpp"
#include "purlin/tuning.hpp"

namespace purlin {
thread_local std::string g_lastError;
void setError(const std::string& e) { g_lastError = e; }
}  // namespace purlin

using namespace purlin;

namespace {

bool fillSpec(CollectiveSpec& s, int collective, int world, int rank, size_t bytes, const size_t* sizes, const size_t* outSizes,
              int dtype, int reduceOp, int mode, int multicastAvailable, int inPlace) {
  if (collective < 0 || collective > int(CollectiveType::allToAllV)) { setError("unknown collective"); return false; }
  s = specFor(CollectiveType(collective));
  s.world = world; s.rank = rank; s.bytes = bytes;
  s.dtype = DType(dtype); s.reduceOp = ReduceOp(reduceOp); s.mode = ReductionMode(mode);
  s.multicastAvailable = multicastAvailable != 0; s.inPlace = inPlace != 0;
  if (world < 1 || world > kMaxRanks) { setError("world size must be 1..16"); return false; }
  // In place (src == dst) is sound only where no step overwrites input another step still has to read: the all-reduce
  // orderings and the all-gather whose own slice already sits in position. A reduce-scatter writes dst[0, n), which is
  // the unread input slice of rank 0 on every other rank; an all-to-all writes slice q as soon as q's data arrives,
  // possibly before this rank has staged its own slice q.
  if (s.inPlace && world > 1 && (s.type == CollectiveType::reduceScatter || s.type == CollectiveType::reduceScatterV ||
                                 s.type == CollectiveType::allToAll || s.type == CollectiveType::allToAllV)) {
    setError("reduce-scatter and all-to-all cannot run in place (src == dst): use a separate output buffer");
    return false;
  }
  const bool v = isVariable(s.in);
  if (v) {
    if (!sizes) { setError("variable-length collective needs a size list"); return false; }
    for (int q = 0; q < world; ++q) s.sizes[q] = sizes[q];
    if (s.type == CollectiveType::allToAllV) {
      if (!outSizes) { setError("all-to-all-v needs output splits"); return false; }
      for (int q = 0; q < world; ++q) s.outSizes[q] = outSizes[q];
    }
    for (int q = 0; q < world; ++q)
      if (s.sizes[q] % kAccessAlign || s.outSizes[q] % kAccessAlign) { setError("every size must be a multiple of 32 bytes"); return false; }
  } else if (bytes % kAccessAlign) { setError("byte count must be a multiple of 32"); return false; }
  return true;
}

}  // namespace

namespace purlin {
// shared with the CUDA half
bool makeSpec(CollectiveSpec& s, int collective, int world, int rank, size_t bytes, const size_t* sizes, const size_t* outSizes,
              int dtype, int reduceOp, int mode, int multicastAvailable, int inPlace) {
  return fillSpec(s, collective, world, rank, bytes, sizes, outSizes, dtype, reduceOp, mode, multicastAvailable, inPlace);
}
// build, then bounds-check: no plan leaves this function unchecked
static bool buildChecked(const CollectiveSpec& s, const Policy& p, const WorkspaceLayout& ws, Plan& plan, std::string& err) {
  if (!buildPlan(s, p, ws, plan, err)) return false;
  const std::string violation = checkPlan(plan, s.world, ws, extentsFor(s));
  if (!violation.empty()) { err = "plan check: " + violation; return false; }
  return true;
}

// Process-wide CTA budget of a collective (0 = none): PURLIN_MAX_CTAS in the environment, or purlin_set_max_ctas().
static std::atomic<int> g_maxCtas{-1};
int maxCtasSetting() {
  int v = g_maxCtas.load();
  if (v < 0) {
    const char* e = std::getenv("PURLIN_MAX_CTAS");
    v = e ? std::max(std::atoi(e), 0) : 0;
    g_maxCtas.store(v);
  }
  return v;
}

// build under a CTA budget: shrink the policy's CTA counts until the plan fits (a plan needs a few CTAs per peer at least)
static bool buildWithinBudget(const CollectiveSpec& s, Policy& p, const WorkspaceLayout& ws, Plan& plan, std::string& err) {
  const int budget = p.maxCtas > 0 ? p.maxCtas : maxCtasSetting();
  bool ok = buildChecked(s, p, ws, plan, err);
  for (int attempt = 0; ok && budget > 0 && plan.blocks > budget && attempt < 6; ++attempt) {
    shrinkToBudget(p, plan.blocks, budget - attempt, s.world);
    ok = buildChecked(s, p, ws, plan, err);
  }
  if (ok && budget > 0 && plan.blocks > budget) { err = "the collective cannot run in " + std::to_string(budget) + " CTAs at this world size"; return false; }
  return ok;
}

bool planFor(const CollectiveSpec& s, const WorkspaceLayout& ws, const Policy* forced, Plan& plan, Policy* chosen) {
  std::string err;
  Policy p = forced ? *forced : selectPolicy(s, ws);
  if (!forced && p.regime == int32_t(Regime::latency) && !isVariable(s.in) && !isVariable(s.out) && s.world > 1) {
    // The put and get steps of the fixed-size latency plans spread (peer, word) pairs over the threads. A measured band
    // may name fewer CTAs than one pair per thread needs (at these sizes the sweep that wrote it could not tell 1 CTA
    // from 16: 11 - 12 us either way in stream mode), and then a thread walks its pairs one memory round trip after the
    // other. Up to 16 CTAs, give every pair its own thread.
    const uint64_t pairs = dispatchBytes(s) / 8 * uint64_t(s.world - 1);
    const uint64_t threads = uint64_t(p.threads > 0 ? p.threads : 256);
    const int floorBlocks = int(std::min<uint64_t>(16, (pairs + threads - 1) / threads));
    if (p.lrBlocks < floorBlocks) p.lrBlocks = floorBlocks;
  }
  bool ok = buildWithinBudget(s, p, ws, plan, err);
  if (!ok && !forced) {   // a measured band may not fit this call (uneven V sizes): fall back to built-in choices
    std::string err2;
    p = defaultPolicy(s, ws);
    ok = buildWithinBudget(s, p, ws, plan, err2);
    if (!ok && p.regime == int32_t(Regime::latency)) {
      p.regime = int32_t(Regime::throughput);
      ok = buildWithinBudget(s, p, ws, plan, err2);
    }
    if (!ok) err = err2;
  }
  if (!ok) { setError(err); return false; }
  if (chosen) *chosen = p;
  return true;
}
}  // namespace purlin

extern "C" {

const char* purlin_last_error(void) { return g_lastError.c_str(); }
int purlin_version(void) { return 100; }
size_t purlin_plan_sizeof(void) { return sizeof(Plan); }
size_t purlin_policy_sizeof(void) { return sizeof(Policy); }

int purlin_workspace_layout(int world, size_t stagingTRSize, size_t* ws) {
  if (world < 1 || world > kMaxRanks) { setError("world size must be 1..16"); return 1; }
  const WorkspaceLayout w = workspaceLayout(world, stagingTRSize);
  ws[0] = w.stagingTRSize; ws[1] = w.lrOffset; ws[2] = w.signalOffset; ws[3] = w.gatherOffset;
  ws[4] = w.consumedOffset; ws[5] = w.varLenOffset; ws[6] = w.totalBytes; ws[7] = w.packetStride;
  return 0;
}

int purlin_plan_build(int collective, int world, int rank, size_t bytes, const size_t* sizes, const size_t* outSizes,
                      int dtype, int reduceOp, int mode, int multicastAvailable, int inPlace, size_t stagingTRSize,
                      const void* policy, void* planOut, void* policyOut) {
  CollectiveSpec s;
  if (!fillSpec(s, collective, world, rank, bytes, sizes, outSizes, dtype, reduceOp, mode, multicastAvailable, inPlace)) return 1;
  const WorkspaceLayout ws = workspaceLayout(world, stagingTRSize);
  Plan plan;
  if (!planFor(s, ws, static_cast<const Policy*>(policy), plan, static_cast<Policy*>(policyOut))) return 1;
  std::memcpy(planOut, &plan, sizeof(plan));
  return 0;
}

// Bounds check of a plan against one rank's buffer extents; 0 when sound, 1 (and purlin_last_error) when not.
int purlin_plan_check(const void* planIn, int world, size_t stagingTRSize, size_t srcBytes, size_t dstBytes) {
  if (!planIn || world < 1 || world > kMaxRanks) { setError("plan check: invalid arguments"); return 1; }
  Plan plan;
  std::memcpy(&plan, planIn, sizeof(plan));
  PlanExtents e;
  e.srcBytes = srcBytes; e.dstBytes = dstBytes;
  const std::string violation = checkPlan(plan, world, workspaceLayout(world, stagingTRSize), e);
  if (!violation.empty()) { setError("plan check: " + violation); return 1; }
  return 0;
}

int purlin_default_policy(int collective, int world, size_t bytes, int dtype, int mode, int multicastAvailable,
                          size_t stagingTRSize, void* policyOut) {
  CollectiveSpec s = specFor(CollectiveType(collective));
  s.world = world; s.bytes = bytes; s.dtype = DType(dtype); s.mode = ReductionMode(mode); s.multicastAvailable = multicastAvailable != 0;
  for (int q = 0; q < world && q < kMaxRanks; ++q) s.sizes[q] = s.outSizes[q] = bytes;
  const Policy p = defaultPolicy(s, workspaceLayout(world, stagingTRSize));
  std::memcpy(policyOut, &p, sizeof(p));
  return 0;
}

int purlin_topology(int inLayout, int outLayout, int op, int cyclic, int* out8) {
  if (!validTriple(DataLayout(inLayout), DataLayout(outLayout), ConsumeOp(op))) { setError("layout pair is not a collective"); return 1; }
  const Topology t = deriveTopology(DataLayout(inLayout), DataLayout(outLayout), ConsumeOp(op), cyclic != 0);
  out8[0] = t.perDest; out8[1] = t.perStream; out8[2] = t.variable; out8[3] = t.varLenArrival;
  out8[4] = t.selfDirect; out8[5] = t.reduceWhole; out8[6] = int(t.notify); out8[7] = int(t.drain);
  return 0;
}

int purlin_tuning_clear(void) { TuningTable::global().clear(); return 0; }
int purlin_tuning_add(int collective, int world, uint64_t maxBytes, const void* policy) {
  TuningEntry e; e.collective = collective; e.world = world; e.maxBytes = maxBytes; e.policy = *static_cast<const Policy*>(policy);
  TuningTable::global().add(e);
  return 0;
}
size_t purlin_tuning_size(void) { return TuningTable::global().size(); }
// CTA budget of every collective planned from now on by this process (0 = the whole GPU); returns the previous value.
int purlin_set_max_ctas(int maxCtas) { const int old = maxCtasSetting(); g_maxCtas.store(maxCtas > 0 ? maxCtas : 0); return old; }
int purlin_get_max_ctas(void) { return maxCtasSetting(); }

// MoE routing of `tokens` rows on the host: the arithmetic of the routing kernels (moe_route.cuh), total for any input.
int purlin_moe_route_host(const float* logits, int tokens, int experts, int topk, int normalize, int32_t* topkIdx, float* topkWeight) {
  if (!logits || !topkIdx || !topkWeight || tokens < 0 || experts < 1 || experts > 1024 || topk < 1 || topk > experts) {
    setError("route (host): experts must be 1..1024 and top-k 1..experts"); return 1;
  }
  for (int t = 0; t < tokens; ++t)
    moe::routeRowHost(logits + size_t(t) * experts, experts, topk, normalize, topkIdx + size_t(t) * topk, topkWeight + size_t(t) * topk);
  return 0;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------
// CPU interpreter
// ------------------------------------------------------------------------------------------
namespace {

struct HostPacket { uint64_t data, flag; };

struct SimRank {
  std::vector<unsigned char> block;   // the symmetric workspace block, same format as on the GPU
  std::vector<uint32_t> counters;
  uint64_t seq = 0;
  Plan plan;
  const unsigned char* src = nullptr;
  unsigned char* dst = nullptr;
  bool absent = false;
};

float bf16ToF(uint16_t h) { uint32_t u = uint32_t(h) << 16; float f; std::memcpy(&f, &u, 4); return f; }
uint16_t fToBf16(float f) {
  uint32_t u; std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return uint16_t((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return uint16_t(u >> 16);
}
float halfToF(uint16_t h) {
  const uint32_t sign = uint32_t(h & 0x8000u) << 16, exp = (h >> 10) & 0x1fu, man = h & 0x3ffu;
  uint32_t u;
  if (exp == 0) {
    if (man == 0) u = sign;
    else { int e = -1; uint32_t m = man; do { ++e; m <<= 1; } while (!(m & 0x400u)); u = sign | ((127 - 15 - e) << 23) | ((m & 0x3ffu) << 13); }
  } else if (exp == 31) u = sign | 0x7f800000u | (man << 13);
  else u = sign | ((exp + 112) << 23) | (man << 13);
  float f; std::memcpy(&f, &u, 4); return f;
}
uint16_t fToHalf(float f) {
  uint32_t u; std::memcpy(&u, &f, 4);
  const uint32_t sign = (u >> 16) & 0x8000u;
  const int32_t exp = int32_t((u >> 23) & 0xff) - 127 + 15;
  uint32_t man = u & 0x7fffffu;
  if (((u >> 23) & 0xff) == 0xff) return uint16_t(sign | 0x7c00u | (man ? 0x200u : 0));
  if (exp >= 31) return uint16_t(sign | 0x7c00u);
  if (exp <= 0) {
    if (exp < -10) return uint16_t(sign);
    man |= 0x800000u;
    const int shift = 14 - exp;
    uint32_t r = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1), halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (r & 1))) ++r;
    return uint16_t(sign | r);
  }
  uint32_t r = (uint32_t(exp) << 10) | (man >> 13);
  const uint32_t rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (r & 1))) ++r;
  return uint16_t(sign | r);
}

float combine(ReduceOp op, float a, float b) { return op == ReduceOp::add ? a + b : op == ReduceOp::mul ? a * b : std::fmax(a, b); }
float identityOf(ReduceOp op) { return op == ReduceOp::add ? 0.f : op == ReduceOp::mul ? 1.f : -INFINITY; }

// out = reduce over ranks (ascending) of srcs[q][0..bytes), fp32 accumulation
bool reduceHost(DType t, ReduceOp op, const std::vector<const unsigned char*>& srcs, size_t bytes, unsigned char* out0, unsigned char* out1) {
  const int eb = dtypeBytes(t);
  if (t != DType::fp32 && t != DType::bf16 && t != DType::fp16) return false;
  const size_t n = bytes / eb;
  for (size_t i = 0; i < n; ++i) {
    float acc = identityOf(op);
    for (const unsigned char* s : srcs) {
      float x;
      if (t == DType::fp32) std::memcpy(&x, s + i * 4, 4);
      else { uint16_t h; std::memcpy(&h, s + i * 2, 2); x = t == DType::bf16 ? bf16ToF(h) : halfToF(h); }
      acc = combine(op, acc, x);
    }
    unsigned char tmp[4];
    if (t == DType::fp32) std::memcpy(tmp, &acc, 4);
    else { const uint16_t h = t == DType::bf16 ? fToBf16(acc) : fToHalf(acc); std::memcpy(tmp, &h, 2); }
    if (out0) std::memcpy(out0 + i * eb, tmp, eb);
    if (out1) std::memcpy(out1 + i * eb, tmp, eb);
  }
  return true;
}

struct Agent { int rank, step; uint32_t chunk = 0; size_t word = 0; bool done = false; bool drainedThisChunk = false; };

struct Sim {
  int W;
  WorkspaceLayout ws;
  std::vector<SimRank> ranks;
  uint32_t status[4] = {0, 0, 0, 0};
  int quantum = 0;   // chunks (or batches of 64 packet words) one advance() may process; 0: as far as its waits allow

  unsigned char* stagingTR(int p, int half) { return ranks[p].block.data() + size_t(half) * ws.stagingTRSize; }
  HostPacket* slot(int onRank, int fromRank, int half, bool result) {
    unsigned char* b = ranks[onRank].block.data() + ws.lrOffset + size_t(half) * kPacketEpochBytes + size_t(fromRank) * ws.packetStride;
    if (result) b += ws.packetStride / 2;
    return reinterpret_cast<HostPacket*>(b);
  }
  uint64_t& signal(int p, int r) { return reinterpret_cast<uint64_t*>(ranks[p].block.data() + ws.signalOffset)[r]; }
  uint64_t& gatherSignal(int p, int r) { return reinterpret_cast<uint64_t*>(ranks[p].block.data() + ws.gatherOffset)[r]; }
  uint64_t& consumed(int p, int r) { return reinterpret_cast<uint64_t*>(ranks[p].block.data() + ws.consumedOffset)[r]; }
  HostPacket* arrival(int p, int half, int r) { return reinterpret_cast<HostPacket*>(ranks[p].block.data() + ws.varLenOffset) + half * W + r; }

  static size_t chunkLen(const Step& s, uint32_t k) { const size_t b = size_t(k) * s.chunkBytes; return std::min<size_t>(s.chunkBytes, s.bytes - b); }
  static size_t slotOff(const Step& s, uint32_t k) { return size_t(k % s.slots) * s.chunkBytes; }

  // copy a chunk the way `n` CTAs would: each its aligned share, so coverage errors in the split show up
  static void splitCopy(unsigned char* dst, const unsigned char* src, size_t bytes, int n) {
    for (int j = 0; j < n; ++j) { const Span sp = partitionAligned(bytes, n, j, kAccessAlign); if (sp.bytes) std::memcpy(dst + sp.offset, src + sp.offset, sp.bytes); }
  }

  // Advance one agent as far as its waits allow. Returns true if it made progress.
  bool advance(Agent& a) {
    SimRank& R = ranks[a.rank];
    const Step& s = R.plan.steps[a.step];
    const int r = a.rank, half = int(R.seq & 1);
    const uint64_t seq = R.seq;
    bool progressed = false;
    int did = 0;   // work units done in this invocation (bounded by `quantum` when the scheduler wants fine interleaving)
    switch (s.role) {
      case kRoleStage:
        while (a.chunk < s.chunks) {
          const uint32_t k = a.chunk;
          if ((s.flags & kFlagCyclic) && k >= s.slots) {
            const uint64_t need = flagValue(seq, k - s.slots);
            bool ok = true;
            if (s.flags & kFlagDrainGather) {
              if (s.peer != r) ok = gatherSignal(r, s.peer) >= need;
              else for (int q = 0; q < W; ++q) { if (q != r && consumed(r, q) < need) ok = false; }
            } else if (s.peer >= 0) ok = consumed(r, s.peer) >= need;
            else for (int q = 0; q < W; ++q) { if (q == r && !(s.flags & kFlagDrainSelf)) continue; if (consumed(r, q) < need) ok = false; }
            if (!ok) return progressed;
          }
          splitCopy(stagingTR(r, half) + s.dstOff + slotOff(s, k), R.src + s.srcOff + size_t(k) * s.chunkBytes, chunkLen(s, k), s.blockCount);
          const uint64_t v = flagValue(seq, k);
          if (s.peer >= 0) signal(s.peer, r) = v; else for (int q = 0; q < W; ++q) signal(q, r) = v;
          ++a.chunk; progressed = true;
          if (quantum && ++did >= quantum && a.chunk < s.chunks) return true;
        }
        a.done = true; return true;
      case kRoleLocal:
        splitCopy(R.dst + s.dstOff, R.src + s.srcOff, s.bytes, s.blockCount);
        a.done = true; return true;
      case kRoleConsume:
      case kRoleGather:
        while (a.chunk < s.chunks) {
          const uint32_t k = a.chunk;
          const uint64_t have = s.role == kRoleGather ? gatherSignal(r, s.peer) : signal(r, s.peer);
          if (have < flagValue(seq, k)) return progressed;
          const int from = (s.flags & kFlagLocalSource) ? r : s.peer;
          splitCopy(R.dst + s.dstOff + size_t(k) * s.chunkBytes, stagingTR(from, half) + s.srcOff + slotOff(s, k), chunkLen(s, k), s.blockCount);
          if (s.flags & kFlagCyclic) consumed(s.peer, r) = flagValue(seq, k);
          ++a.chunk; progressed = true;
          if (quantum && ++did >= quantum && a.chunk < s.chunks) return true;
        }
        a.done = true; return true;
      case kRoleReduce:
        while (a.chunk < s.chunks) {
          const uint32_t k = a.chunk;
          for (int q = 0; q < W; ++q) if (signal(r, q) < flagValue(seq, k)) return progressed;
          std::vector<const unsigned char*> srcs;
          for (int q = 0; q < W; ++q) srcs.push_back(stagingTR(q, half) + s.srcOff + slotOff(s, k));
          const size_t len = chunkLen(s, k), lin = size_t(k) * s.chunkBytes;
          std::vector<unsigned char> tmp(len);
          if (!reduceHost(DType(R.plan.dtype), ReduceOp(R.plan.reduceOp), srcs, len, tmp.data(), nullptr)) { status[0] = kStatusBadPlan; a.done = true; return true; }
          if (s.flags & kFlagToDst) std::memcpy(R.dst + s.dstOff + lin, tmp.data(), len);
          if (s.flags & kFlagToSeam) {
            if (s.flags & kFlagMulticastOut) { for (int q = 0; q < W; ++q) std::memcpy(stagingTR(q, half) + s.seamOff + slotOff(s, k), tmp.data(), len); }
            else std::memcpy(stagingTR(r, half) + s.seamOff + slotOff(s, k), tmp.data(), len);
          }
          const uint64_t v = flagValue(seq, k);
          for (int q = 0; q < W; ++q) {
            if ((s.flags & kFlagNotifyGather) && q != r) gatherSignal(q, r) = v;
            if (s.flags & kFlagCyclic) consumed(q, r) = v;
          }
          ++a.chunk; progressed = true;
          if (quantum && ++did >= quantum && a.chunk < s.chunks) return true;
        }
        a.done = true; return true;
      case kRolePacketPut: {
        const size_t words = s.bytes / 8;
        const uint64_t flag = flagValue(seq, 0);
        for (size_t i = 0; i < words; ++i) {
          if (s.flags & kFlagScatter) {      // peer q receives slice q of the source
            for (int q = 0; q < W; ++q) {
              if (q == r) continue;
              uint64_t v; std::memcpy(&v, R.src + s.srcOff + size_t(q) * s.bytes + i * 8, 8);
              slot(q, r, half, false)[s.dstOff / 8 + i] = HostPacket{v, flag};
            }
            continue;
          }
          uint64_t v; std::memcpy(&v, R.src + s.srcOff + i * 8, 8);
          if (s.peer >= 0) slot(s.peer, r, half, false)[s.dstOff / 8 + i] = HostPacket{v, flag};
          else for (int q = 0; q < W; ++q) { if (q == r && !(s.flags & kFlagMulticastOut)) continue; slot(q, r, half, false)[s.dstOff / 8 + i] = HostPacket{v, flag}; }
        }
        a.done = true; return true;
      }
      case kRolePacketGet: {
        const size_t words = s.bytes / 8;
        const uint64_t flag = flagValue(seq, 0);
        if (s.peer < 0) {
          // every peer's packets in one step: the agent walks (peer, word) pairs, peers in ring order
          const size_t pairs = words * size_t(W - 1);
          while (a.word < pairs) {
            const int q = (r + 1 + int(a.word / words)) % W;
            const size_t i = a.word % words;
            const HostPacket& pk = slot(r, q, half, (s.flags & kFlagResultHalf) != 0)[s.srcOff / 8 + i];
            if (pk.flag != flag) return progressed;
            std::memcpy(R.dst + s.dstOff + size_t(q) * s.bytes + i * 8, &pk.data, 8);
            ++a.word; progressed = true;
            if (quantum && ++did >= 64 * quantum && a.word < pairs) return true;
          }
          a.done = true; return true;
        }
        const HostPacket* p = slot(r, s.peer, half, (s.flags & kFlagResultHalf) != 0) + s.srcOff / 8;
        while (a.word < words) {
          if (p[a.word].flag != flag) return progressed;
          std::memcpy(R.dst + s.dstOff + a.word * 8, &p[a.word].data, 8);
          ++a.word; progressed = true;
          if (quantum && ++did >= 64 * quantum && a.word < words) return true;
        }
        a.done = true; return true;
      }
      case kRolePacketReduce: {
        const size_t words = s.bytes / 8;
        const uint64_t flag = flagValue(seq, 0);
        while (a.word < words) {
          const size_t i = a.word;
          uint64_t w[kMaxRanks];
          for (int q = 0; q < W; ++q) {
            if (q == r) { std::memcpy(&w[q], R.src + s.seamOff + i * 8, 8); continue; }
            const HostPacket& p = slot(r, q, half, false)[s.srcOff / 8 + i];
            if (p.flag != flag) return progressed;
            w[q] = p.data;
          }
          std::vector<const unsigned char*> srcs;
          for (int q = 0; q < W; ++q) srcs.push_back(reinterpret_cast<const unsigned char*>(&w[q]));
          uint64_t out = 0;
          if (!reduceHost(DType(R.plan.dtype), ReduceOp(R.plan.reduceOp), srcs, 8, reinterpret_cast<unsigned char*>(&out), nullptr)) { status[0] = kStatusBadPlan; a.done = true; return true; }
          std::memcpy(R.dst + s.dstOff + i * 8, &out, 8);
          if (s.flags & kFlagPublish)
            for (int q = 0; q < W; ++q) { if (q == r && !(s.flags & kFlagMulticastOut)) continue; slot(q, r, half, true)[i] = HostPacket{out, flag}; }
          ++a.word; progressed = true;
          if (quantum && ++did >= 64 * quantum && a.word < words) return true;
        }
        a.done = true; return true;
      }
      default: a.done = true; return true;
    }
  }

  // One call on every present rank. Returns false (and a status) when some wait can never be satisfied.
  bool call() {
    std::vector<Agent> agents;
    for (int r = 0; r < W; ++r) {
      if (ranks[r].absent) continue;
      const int half = int(ranks[r].seq & 1);
      if (ranks[r].plan.varLenArrival) for (int q = 0; q < W; ++q) *arrival(q, half, r) = HostPacket{ranks[r].plan.payloadBytes, flagValue(ranks[r].seq, 0)};
      for (int s = 0; s < ranks[r].plan.nSteps; ++s) { Agent a; a.rank = r; a.step = s; agents.push_back(a); }
    }
    // steps that share a CTA range run in plan order on the device; keep that order here
    for (;;) {
      bool progress = false, allDone = true;
      for (size_t i = 0; i < agents.size(); ++i) {
        Agent& a = agents[i];
        if (a.done) continue;
        bool blockedByEarlier = false;
        const Step& s = ranks[a.rank].plan.steps[a.step];
        for (size_t j = 0; j < i; ++j) {
          const Agent& b = agents[j];
          if (b.rank != a.rank || b.done) continue;
          const Step& t = ranks[b.rank].plan.steps[b.step];
          if (t.blockBegin < s.blockBegin + s.blockCount && s.blockBegin < t.blockBegin + t.blockCount) { blockedByEarlier = true; break; }
        }
        if (!blockedByEarlier && advance(a)) progress = true;
        if (!a.done) allDone = false;
      }
      if (allDone) break;
      if (!progress) {
        for (const Agent& a : agents) if (!a.done) {
          const Step& s = ranks[a.rank].plan.steps[a.step];
          status[0] = (s.role >= kRolePacketPut) ? kStatusTimeoutPacket : kStatusTimeoutSignal;
          status[1] = uint32_t(a.step); status[2] = uint32_t(s.peer); status[3] = a.chunk;
          break;
        }
        return false;
      }
    }
    for (int r = 0; r < W; ++r) {
      if (ranks[r].absent) continue;
      if (ranks[r].plan.varLenArrival) {
        const int half = int(ranks[r].seq & 1);
        for (int q = 0; q < W; ++q) if (arrival(r, half, q)->flag != flagValue(ranks[r].seq, 0)) { status[0] = kStatusTimeoutArrival; status[2] = uint32_t(q); return false; }
      }
    }
    for (int r = 0; r < W; ++r) if (!ranks[r].absent) ++ranks[r].seq;
    return status[0] == 0;
  }

  // A sequence of calls with NO barrier between them: a rank starts its next call as soon as its own steps of the
  // current one are done (stream order), whatever its peers are doing, and a seeded random scheduler decides which
  // agent of which rank moves next, one chunk at a time. This is the situation the ordering invariant is about (a
  // fast rank may be a whole call ahead of a slow one, reusing a staging half the slow one has only just released);
  // a protocol error shows as a wrong output or as a schedule in which nobody can move.
  struct CallData { std::vector<Plan> plans; std::vector<const unsigned char*> srcs; std::vector<unsigned char*> dsts; };
  bool overlapped(const std::vector<CallData>& calls, uint64_t seed) {
    const int n = int(calls.size());
    std::vector<int> cur(W, 0);
    std::vector<std::vector<Agent>> agents(W);
    std::vector<char> finished(W, 0);
    uint64_t rng = seed * 0x9e3779b97f4a7c15ull + 0x1234567ull;
    auto next = [&]() { rng ^= rng << 13; rng ^= rng >> 7; rng ^= rng << 17; return rng; };
    auto start = [&](int r) {
      if (cur[r] >= n) { finished[r] = 1; agents[r].clear(); return; }
      SimRank& R = ranks[r];
      R.plan = calls[cur[r]].plans[r]; R.src = calls[cur[r]].srcs[r]; R.dst = calls[cur[r]].dsts[r];
      const int half = int(R.seq & 1);
      if (R.plan.varLenArrival) for (int q = 0; q < W; ++q) *arrival(q, half, r) = HostPacket{R.plan.payloadBytes, flagValue(R.seq, 0)};
      agents[r].clear();
      for (int s = 0; s < R.plan.nSteps; ++s) { Agent a; a.rank = r; a.step = s; agents[r].push_back(a); }
    };
    for (int r = 0; r < W; ++r) start(r);
    for (;;) {
      bool allFinished = true;
      for (int r = 0; r < W; ++r) allFinished = allFinished && finished[r];
      if (allFinished) return status[0] == 0;
      // agents that may move: not done, and no earlier unfinished step of the same rank shares their CTAs
      std::vector<std::pair<int, int>> cand;
      for (int r = 0; r < W; ++r) {
        if (finished[r]) continue;
        for (size_t i = 0; i < agents[r].size(); ++i) {
          if (agents[r][i].done) continue;
          const Step& s = ranks[r].plan.steps[agents[r][i].step];
          bool blocked = false;
          for (size_t j = 0; j < i && !blocked; ++j) {
            if (agents[r][j].done) continue;
            const Step& t = ranks[r].plan.steps[agents[r][j].step];
            blocked = t.blockBegin < s.blockBegin + s.blockCount && s.blockBegin < t.blockBegin + t.blockCount;
          }
          if (!blocked) cand.emplace_back(r, int(i));
        }
      }
      for (size_t i = cand.size(); i > 1; --i) std::swap(cand[i - 1], cand[size_t(next() % i)]);
      bool progress = false;
      for (const auto& c : cand)
        if (advance(agents[c.first][size_t(c.second)])) { progress = true; break; }   // one agent per turn
      if (status[0]) return false;
      // a rank whose steps are all done finishes its call (after the arrival handshake of a variable-length form)
      for (int r = 0; r < W; ++r) {
        if (finished[r]) continue;
        bool done = true;
        for (const Agent& a : agents[r]) done = done && a.done;
        if (!done) continue;
        SimRank& R = ranks[r];
        if (R.plan.varLenArrival) {
          const int half = int(R.seq & 1);
          bool arrived = true;
          for (int q = 0; q < W; ++q) arrived = arrived && arrival(r, half, q)->flag == flagValue(R.seq, 0);
          if (!arrived) continue;
        }
        ++R.seq; ++cur[r];
        start(r);
        progress = true;
      }
      if (!progress) {
        if (std::getenv("PURLIN_SIM_DEBUG"))
          for (int r = 0; r < W; ++r) {
            std::fprintf(stderr, "rank %d call %d seq %llu finished %d:", r, cur[r], (unsigned long long)ranks[r].seq, int(finished[r]));
            for (const Agent& a : agents[r]) if (!a.done) { const Step& s = ranks[r].plan.steps[a.step]; std::fprintf(stderr, " [step %d role %d peer %d chunk %u word %zu bytes %llu]", a.step, s.role, s.peer, a.chunk, a.word, (unsigned long long)s.bytes); }
            std::fprintf(stderr, "\n");
          }
        for (int r = 0; r < W && !status[0]; ++r)
          for (const Agent& a : agents[r]) if (!a.done) {
            const Step& s = ranks[r].plan.steps[a.step];
            status[0] = (s.role >= kRolePacketPut) ? kStatusTimeoutPacket : kStatusTimeoutSignal;
            status[1] = uint32_t(a.step); status[2] = uint32_t(s.peer); status[3] = a.chunk;
            break;
          }
        if (!status[0]) { status[0] = kStatusTimeoutArrival; }
        return false;
      }
    }
  }
};

}  // namespace

extern "C" int purlin_sim_run(int collective, int world, size_t bytes, const size_t* sizesMatrix, int dtype, int reduceOp, int mode,
                              size_t stagingTRSize, const void* policy, const void* const* srcs, void* const* dsts,
                              int dropRank, uint32_t* statusOut) {
  if (world < 1 || world > kMaxRanks) { setError("world size must be 1..16"); return 1; }
  Sim sim;
  sim.W = world;
  sim.ws = workspaceLayout(world, stagingTRSize);
  sim.ranks.resize(world);
  for (int r = 0; r < world; ++r) {
    SimRank& R = sim.ranks[r];
    R.block.assign(sim.ws.totalBytes, 0);
    R.src = static_cast<const unsigned char*>(srcs[r]);
    R.dst = static_cast<unsigned char*>(dsts[r]);
    R.absent = r == dropRank;
    CollectiveSpec s;
    // sizesMatrix: allGatherV / reduceScatterV: one row [world]; allToAllV: [world][world], row r = what rank r sends
    size_t in[kMaxRanks] = {}, out[kMaxRanks] = {};
    const bool a2av = collective == int(CollectiveType::allToAllV);
    if (sizesMatrix) for (int q = 0; q < world; ++q) { in[q] = a2av ? sizesMatrix[size_t(r) * world + q] : sizesMatrix[q]; out[q] = a2av ? sizesMatrix[size_t(q) * world + r] : 0; }
    if (!makeSpec(s, collective, world, r, bytes, sizesMatrix ? in : nullptr, a2av ? out : nullptr, dtype, reduceOp, mode, 0, R.src == R.dst)) return 1;
    if (!planFor(s, sim.ws, static_cast<const Policy*>(policy), R.plan, nullptr)) return 1;
  }
  // two calls back to back so both staging halves and growing flag values are exercised
  bool ok = true;
  for (int rep = 0; rep < 2 && ok; ++rep) ok = sim.call();
  if (statusOut) std::memcpy(statusOut, sim.status, sizeof(sim.status));
  if (!ok && sim.status[0] == 0) sim.status[0] = kStatusTimeoutSignal;
  return 0;
}

// A sequence of `nCalls` collectives on one set of workspaces with no barrier between calls and a seeded random
// scheduler (see Sim::overlapped). collectives[c], bytes[c], sizesMatrices[c] (null for fixed-size forms) describe call
// c; srcs / dsts hold nCalls x world pointers, call-major. quantum: chunks one scheduling turn may process (1 = finest).
extern "C" int purlin_sim_run_overlapped(int nCalls, const int* collectives, const size_t* bytes, const size_t* const* sizesMatrices,
                                         int world, int dtype, int reduceOp, int mode, size_t stagingTRSize, const void* policy,
                                         const void* const* srcs, void* const* dsts, uint64_t seed, int quantum, int multicastAvailable,
                                         uint32_t* statusOut) {
  if (world < 1 || world > kMaxRanks || nCalls < 1) { setError("invalid world size or call count"); return 1; }
  Sim sim;
  sim.W = world;
  sim.ws = workspaceLayout(world, stagingTRSize);
  sim.quantum = quantum;
  sim.ranks.resize(world);
  for (int r = 0; r < world; ++r) sim.ranks[r].block.assign(sim.ws.totalBytes, 0);
  std::vector<Sim::CallData> calls(static_cast<size_t>(nCalls));
  for (int c = 0; c < nCalls; ++c) {
    Sim::CallData& cd = calls[size_t(c)];
    cd.plans.resize(world); cd.srcs.resize(world); cd.dsts.resize(world);
    const size_t* matrix = sizesMatrices ? sizesMatrices[c] : nullptr;
    const bool a2av = collectives[c] == int(CollectiveType::allToAllV);
    for (int r = 0; r < world; ++r) {
      cd.srcs[r] = static_cast<const unsigned char*>(srcs[size_t(c) * world + r]);
      cd.dsts[r] = static_cast<unsigned char*>(dsts[size_t(c) * world + r]);
      size_t in[kMaxRanks] = {}, out[kMaxRanks] = {};
      if (matrix) for (int q = 0; q < world; ++q) { in[q] = a2av ? matrix[size_t(r) * world + q] : matrix[q]; out[q] = a2av ? matrix[size_t(q) * world + r] : 0; }
      CollectiveSpec s;
      // with a multicast alias on offer the plans may use the switch variants: the interpreter models multimem.ld_reduce
      // as a read of every rank's staging and multimem.st as a write to every rank's
      if (!makeSpec(s, collectives[c], world, r, bytes[c], matrix ? in : nullptr, a2av ? out : nullptr, dtype, reduceOp, mode,
                    multicastAvailable, cd.srcs[r] == cd.dsts[r] && cd.srcs[r] != nullptr)) return 1;
      if (!planFor(s, sim.ws, static_cast<const Policy*>(policy), cd.plans[r], nullptr)) return 1;
    }
  }
  const bool ok = sim.overlapped(calls, seed);
  if (statusOut) std::memcpy(statusOut, sim.status, sizeof(sim.status));
  if (!ok && sim.status[0] == 0 && statusOut) statusOut[0] = kStatusTimeoutSignal;
  return 0;
}
