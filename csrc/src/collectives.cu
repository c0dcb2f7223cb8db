// Contexts, the generic SNAC kernel and the host launchers of every collective.
//
// Parity: the four templated kernels and their launchers in
// csrc/include/purlin/host/{allReduce,allGather,reduceScatter,all2all}.cuh and
// the context set-up of csrc/include/purlin/setup.cuh:35-124 of the reference.
// One launch per call, no host synchronisation after it, NVTX range around it.
// A single kernel template executes any Plan; it is instantiated per element
// type and reduce operator for reductions and once for pure copies.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "purlin/capi.h"
#include "purlin/layout.hpp"
#include "purlin/snac.cuh"
#include "purlin/telemetry.hpp"
#include "purlin/tuning.hpp"

namespace purlin {
void setError(const std::string& e);
bool makeSpec(CollectiveSpec& s, int collective, int world, int rank, size_t bytes, const size_t* sizes, const size_t* outSizes,
              int dtype, int reduceOp, int mode, int multicastAvailable, int inPlace);
bool planFor(const CollectiveSpec& s, const WorkspaceLayout& ws, const Policy* forced, Plan& plan, Policy* chosen);
int maxCtasSetting();
}  // namespace purlin

using namespace purlin;

struct PurlinHostContext {
  Context dev{};
  WorkspaceLayout ws{};
  int device = 0;
  void* localBlock = nullptr;   // seq, exit counter, status, counters
  void* traceRing = nullptr;    // device-side timing ring (PURLIN_TRACE=1), else null
  bool hasMulticast = false;
  // plans of fixed-size calls under the table/default policy, keyed by (collective, bytes, dtype, op, mode, in-place)
  std::unordered_map<uint64_t, Plan> planCache;
  size_t planCacheTableSize = 0;
  int planCacheBudget = 0;      // the CTA budget the cached plans were built under
};

namespace {

constexpr int kMaxThreads = 256;   // 255 registers per thread: room for 8 wide accesses in flight
using Atom = AtomSm100<256, 4, 4>;

#define CUDA_OK(expr)                                                                                   \
  do {                                                                                                  \
    cudaError_t e_ = (expr);                                                                            \
    if (e_ != cudaSuccess) { setError(std::string(#expr) + ": " + cudaGetErrorString(e_)); return 1; } \
  } while (0)

// Production launch: one rank per GPU, context and plan in kernel parameters.
template <DType T, ReduceOp Op, bool Reduces>
__global__ void __launch_bounds__(kMaxThreads, 1)
snacKernel(const __grid_constant__ Context ctx, const __grid_constant__ Plan plan, const unsigned char* src, unsigned char* dst) {
  __shared__ const unsigned char* peerPtr[kMaxRanks];
  extern __shared__ __align__(128) unsigned char dynSmem[];
  snac::run<Atom, T, Op, Reduces>(ctx, plan, src, dst, blockIdx.x, gridDim.x, peerPtr, dynSmem);
}

// The same executor on a plan of at most kCompactSteps steps (every latency-regime plan up to eight ranks): the launch
// carries about 2 KB of parameters instead of 5 KB.
template <DType T, ReduceOp Op, bool Reduces>
__global__ void __launch_bounds__(kMaxThreads, 1)
snacKernelCompact(const __grid_constant__ Context ctx, const __grid_constant__ PlanCompact plan, const unsigned char* src, unsigned char* dst) {
  __shared__ const unsigned char* peerPtr[kMaxRanks];
  extern __shared__ __align__(128) unsigned char dynSmem[];
  snac::run<Atom, T, Op, Reduces, PlanCompact>(ctx, plan, src, dst, blockIdx.x, gridDim.x, peerPtr, dynSmem);
}

// Emulation launch: grid.y virtual ranks on one GPU (cooperative, so all CTAs are resident
// and may wait on one another), each with its own context, plan and buffers in global memory.
struct EmuRank {
  Context ctx;
  Plan plan;
  const unsigned char* src;
  unsigned char* dst;
  int absent;
};
template <DType T, ReduceOp Op, bool Reduces>
__global__ void __launch_bounds__(kMaxThreads, 1) snacEmuKernel(const EmuRank* ranks) {
  __shared__ const unsigned char* peerPtr[kMaxRanks];
  __shared__ alignas(16) unsigned char ctxMem[sizeof(Context)];
  __shared__ alignas(16) unsigned char planMem[sizeof(Plan)];
  const EmuRank& me = ranks[blockIdx.y];
  if (me.absent) return;
  for (size_t i = threadIdx.x; i < sizeof(Context) / 4; i += blockDim.x)
    reinterpret_cast<uint32_t*>(ctxMem)[i] = reinterpret_cast<const uint32_t*>(&me.ctx)[i];
  for (size_t i = threadIdx.x; i < sizeof(Plan) / 4; i += blockDim.x)
    reinterpret_cast<uint32_t*>(planMem)[i] = reinterpret_cast<const uint32_t*>(&me.plan)[i];
  __syncthreads();
  const Context& ctx = *reinterpret_cast<const Context*>(ctxMem);
  const Plan& plan = *reinterpret_cast<const Plan*>(planMem);
  if (int(blockIdx.x) >= plan.blocks) return;
  extern __shared__ __align__(128) unsigned char dynSmem[];
  snac::run<Atom, T, Op, Reduces>(ctx, plan, me.src, me.dst, blockIdx.x, plan.blocks, peerPtr, dynSmem);
}

template <class Atom_>
__global__ void __launch_bounds__(kMaxThreads, 1) p2pKernel(unsigned char* dst, const unsigned char* src, size_t bytes) {
  superCopy<Atom_>(dst, src, bytes, blockIdx.x, gridDim.x);
}

using ProdFn = void (*)(const Context, const Plan, const unsigned char*, unsigned char*);
using CompactFn = void (*)(const Context, const PlanCompact, const unsigned char*, unsigned char*);
using EmuFn = void (*)(const EmuRank*);

template <DType T> CompactFn compactByOp(int op) {
  switch (ReduceOp(op)) {
    case ReduceOp::add: return snacKernelCompact<T, ReduceOp::add, true>;
    case ReduceOp::mul: return snacKernelCompact<T, ReduceOp::mul, true>;
    default: return snacKernelCompact<T, ReduceOp::max, true>;
  }
}

template <DType T> ProdFn prodByOp(int op) {
  switch (ReduceOp(op)) {
    case ReduceOp::add: return snacKernel<T, ReduceOp::add, true>;
    case ReduceOp::mul: return snacKernel<T, ReduceOp::mul, true>;
    default: return snacKernel<T, ReduceOp::max, true>;
  }
}
template <DType T> EmuFn emuByOp(int op) {
  switch (ReduceOp(op)) {
    case ReduceOp::add: return snacEmuKernel<T, ReduceOp::add, true>;
    case ReduceOp::mul: return snacEmuKernel<T, ReduceOp::mul, true>;
    default: return snacEmuKernel<T, ReduceOp::max, true>;
  }
}
ProdFn prodKernel(const Plan& p) {
  if (p.consumeOp == int32_t(ConsumeOp::copy)) return snacKernel<DType::fp32, ReduceOp::add, false>;
  switch (DType(p.dtype)) {
    case DType::bf16: return prodByOp<DType::bf16>(p.reduceOp);
    case DType::fp16: return prodByOp<DType::fp16>(p.reduceOp);
    case DType::fp8e4m3: return prodByOp<DType::fp8e4m3>(p.reduceOp);
    case DType::fp8e5m2: return prodByOp<DType::fp8e5m2>(p.reduceOp);
    default: return prodByOp<DType::fp32>(p.reduceOp);
  }
}
CompactFn compactKernel(const Plan& p) {
  if (p.consumeOp == int32_t(ConsumeOp::copy)) return snacKernelCompact<DType::fp32, ReduceOp::add, false>;
  switch (DType(p.dtype)) {
    case DType::bf16: return compactByOp<DType::bf16>(p.reduceOp);
    case DType::fp16: return compactByOp<DType::fp16>(p.reduceOp);
    case DType::fp8e4m3: return compactByOp<DType::fp8e4m3>(p.reduceOp);
    case DType::fp8e5m2: return compactByOp<DType::fp8e5m2>(p.reduceOp);
    default: return compactByOp<DType::fp32>(p.reduceOp);
  }
}
EmuFn emuKernel(const Plan& p) {
  if (p.consumeOp == int32_t(ConsumeOp::copy)) return snacEmuKernel<DType::fp32, ReduceOp::add, false>;
  switch (DType(p.dtype)) {
    case DType::bf16: return emuByOp<DType::bf16>(p.reduceOp);
    case DType::fp16: return emuByOp<DType::fp16>(p.reduceOp);
    case DType::fp8e4m3: return emuByOp<DType::fp8e4m3>(p.reduceOp);
    case DType::fp8e5m2: return emuByOp<DType::fp8e5m2>(p.reduceOp);
    default: return emuByOp<DType::fp32>(p.reduceOp);
  }
}

const char* collectiveName(int c) {
  static const char* names[] = {"allReduce", "allGather", "allGatherV", "reduceScatter", "reduceScatterV", "allToAll", "allToAllV"};
  return c >= 0 && c < 7 ? names[c] : "collective";
}

int worldOneCopy(const CollectiveSpec& s, const void* src, void* dst, cudaStream_t stream) {
  // a world of one: every collective is a copy of the rank's own data
  size_t n = isVariable(s.in) ? s.sizes[0] : s.bytes;
  if (n && src != dst) CUDA_OK(cudaMemcpyAsync(dst, src, n, cudaMemcpyDeviceToDevice, stream));
  return 0;
}

// kernels that stream through the bulk ring need more dynamic shared memory than the default limit: opt in once per
// (device, kernel) pair, since the attribute belongs to the device's copy of the function
bool ensureSmemOptIn(const void* fn) {
  static std::mutex mu;
  static std::vector<std::pair<int, const void*>> done;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return false;
  std::lock_guard<std::mutex> g(mu);
  for (const auto& d : done) if (d.first == device && d.second == fn) return true;
  if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bulk::smemBytes(bulk::kMaxDepth))) != cudaSuccess) return false;
  done.emplace_back(device, fn);
  return true;
}

int launchPlan(PurlinHostContext* h, const Plan& plan, const void* src, void* dst, cudaStream_t stream) {
  const int threads = std::min(std::max(plan.threads, 32), kMaxThreads);
  if (plan.nSteps <= kCompactSteps && plan.smemBytes == 0) {
    PlanCompact small;
    compactPlan(plan, small);
    compactKernel(plan)<<<plan.blocks, threads, 0, stream>>>(h->dev, small, static_cast<const unsigned char*>(src), static_cast<unsigned char*>(dst));
    CUDA_OK(cudaGetLastError());
    return 0;
  }
  ProdFn fn = prodKernel(plan);
  if (plan.smemBytes > 0 && !ensureSmemOptIn(reinterpret_cast<const void*>(fn))) { setError("cannot opt in to the bulk ring's shared memory"); return 1; }
  fn<<<plan.blocks, threads, plan.smemBytes, stream>>>(h->dev, plan, static_cast<const unsigned char*>(src), static_cast<unsigned char*>(dst));
  CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace

extern "C" {

size_t purlin_context_sizeof(void) { return sizeof(Context); }

PurlinHostContext* purlin_context_create(int rank, int world, const uint64_t* peerPtrs, uint64_t multicastPtr,
                                         size_t stagingTRSize, uint64_t timeoutNs, void* stream) {
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world) { setError("invalid rank or world size"); return nullptr; }
  if (stagingTRSize < kMinChunkBytes || stagingTRSize > kMaxStagingBytes || stagingTRSize % kAccessAlign) {
    setError("staging size must be a multiple of 32 bytes between 256 KiB and 256 MiB"); return nullptr;
  }
  if (!peerPtrs) { setError("the provider must return one pointer per rank"); return nullptr; }
  for (int q = 0; q < world; ++q)
    if (peerPtrs[q] == 0 || peerPtrs[q] % kAccessAlign) { setError("the provider returned a null or unaligned peer pointer"); return nullptr; }
  if (multicastPtr % kAccessAlign) { setError("the provider returned an unaligned multicast pointer"); return nullptr; }
  auto* h = new PurlinHostContext();
  h->ws = workspaceLayout(world, stagingTRSize);
  if (h->ws.packetStride % kPacketBytes) { delete h; setError("packet stride is not packet aligned"); return nullptr; }
  cudaGetDevice(&h->device);
  Context& c = h->dev;
  c.world = world; c.rank = rank;
  c.stagingTRSize = stagingTRSize; c.packetStride = h->ws.packetStride;
  c.timeoutNs = timeoutNs ? timeoutNs : 10ull * 1000 * 1000 * 1000;
  if (const char* t = std::getenv("PURLIN_TIMEOUT_MS")) c.timeoutNs = std::strtoull(t, nullptr, 10) * 1000000ull;
  for (int q = 0; q < world; ++q) {
    unsigned char* base = reinterpret_cast<unsigned char*>(peerPtrs[q]);
    c.stagingTR[q] = base;
    c.stagingLR[q] = base + h->ws.lrOffset;
    c.signals[q] = reinterpret_cast<uint64_t*>(base + h->ws.signalOffset);
    c.gatherSignals[q] = reinterpret_cast<uint64_t*>(base + h->ws.gatherOffset);
    c.consumedSignals[q] = reinterpret_cast<uint64_t*>(base + h->ws.consumedOffset);
    c.varLenSignals[q] = base + h->ws.varLenOffset;
  }
  if (multicastPtr && std::getenv("PURLIN_DISABLE_MULTIMEM") == nullptr) {
    c.mcStagingTR = reinterpret_cast<unsigned char*>(multicastPtr);
    if (std::getenv("PURLIN_DISABLE_MULTIMEM_LR") == nullptr) c.mcStagingLR = c.mcStagingTR + h->ws.lrOffset;
  }
  h->hasMulticast = c.mcStagingTR != nullptr;
  // local block: [0, 2048) sequence words, [2048] exit counter, [2112] status, [4096, ...) last-arrival counters
  const size_t localBytes = 4096 + size_t(kCounterSlots) * 4;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaMalloc(&h->localBlock, localBytes) != cudaSuccess) { delete h; setError("cudaMalloc of the local counters failed"); return nullptr; }
  cudaMemsetAsync(h->localBlock, 0, localBytes, s);
  unsigned char* lb = static_cast<unsigned char*>(h->localBlock);
  static_assert(kSeqWords * 8 <= 2048, "sequence words overlap the exit counter");
  c.seq = reinterpret_cast<uint64_t*>(lb);
  c.exitCounter = reinterpret_cast<uint32_t*>(lb + 2048);
  c.status = reinterpret_cast<uint32_t*>(lb + 2112);
  c.counters = reinterpret_cast<uint32_t*>(lb + 4096);
  if (const char* t = std::getenv("PURLIN_TRACE"); t && t[0] != '0') {
    // opt-in: every call leaves {start, end, bytes, collective} in a ring of kTraceSlots records (purlin_context_trace)
    if (cudaMalloc(&h->traceRing, size_t(kTraceSlots) * 32) != cudaSuccess) { cudaFree(h->localBlock); delete h; setError("cudaMalloc of the trace ring failed"); return nullptr; }
    cudaMemsetAsync(h->traceRing, 0, size_t(kTraceSlots) * 32, s);
    c.trace = static_cast<uint64_t*>(h->traceRing);
  }
  if (cudaStreamSynchronize(s) != cudaSuccess) { cudaFree(h->localBlock); if (h->traceRing) cudaFree(h->traceRing); delete h; setError("context set-up failed on the stream"); return nullptr; }
  return h;
}

int purlin_context_destroy(PurlinHostContext* h, void* stream) {
  if (!h) return 0;
  cudaStreamSynchronize(static_cast<cudaStream_t>(stream));   // in-flight collectives still use the counters
  if (h->localBlock) cudaFree(h->localBlock);
  if (h->traceRing) cudaFree(h->traceRing);
  delete h;
  return 0;
}

int purlin_context_status(PurlinHostContext* h, uint32_t* out4, void* stream) {
  CUDA_OK(cudaMemcpyAsync(out4, h->dev.status, 16, cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
  CUDA_OK(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  return 0;
}
int purlin_context_clear_status(PurlinHostContext* h, void* stream) {
  CUDA_OK(cudaMemsetAsync(h->dev.status, 0, 16, static_cast<cudaStream_t>(stream)));
  CUDA_OK(cudaMemsetAsync(h->dev.exitCounter, 0, 4, static_cast<cudaStream_t>(stream)));
  CUDA_OK(cudaMemsetAsync(h->dev.counters, 0, size_t(kCounterSlots) * 4, static_cast<cudaStream_t>(stream)));
  return 0;
}
int purlin_context_set_timeout(PurlinHostContext* h, uint64_t timeoutNs) { h->dev.timeoutNs = timeoutNs; return 0; }
uint64_t purlin_context_seq(PurlinHostContext* h, void* stream) {
  uint64_t v = 0;
  cudaMemcpyAsync(&v, h->dev.seq, 8, cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
  cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  return v;
}
int purlin_context_has_multicast(PurlinHostContext* h) { return h->hasMulticast ? 1 : 0; }

// Device-side timing of the most recent calls (contexts created with PURLIN_TRACE=1). Synchronises the stream and
// writes up to maxRecords records of four words {call sequence, start ns, end ns, payload bytes | collective << 56},
// oldest first; returns how many, or -1 when tracing is off.
int purlin_context_trace(PurlinHostContext* h, uint64_t* out, int maxRecords, void* stream) {
  if (!h || !h->traceRing) return -1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  std::vector<uint64_t> ring(size_t(kTraceSlots) * 4);
  uint64_t seq = 0;
  if (cudaMemcpyAsync(ring.data(), h->traceRing, ring.size() * 8, cudaMemcpyDeviceToHost, s) != cudaSuccess ||
      cudaMemcpyAsync(&seq, h->dev.seq, 8, cudaMemcpyDeviceToHost, s) != cudaSuccess || cudaStreamSynchronize(s) != cudaSuccess) {
    setError("reading the trace ring failed");
    return -1;
  }
  const uint64_t have = seq < uint64_t(kTraceSlots) ? seq : uint64_t(kTraceSlots);
  const uint64_t want = have < uint64_t(maxRecords > 0 ? maxRecords : 0) ? have : uint64_t(maxRecords > 0 ? maxRecords : 0);
  for (uint64_t i = 0; i < want; ++i) {
    const uint64_t call = seq - want + i;
    const uint64_t* rec = ring.data() + (call % uint64_t(kTraceSlots)) * 4;
    out[i * 4 + 0] = call;
    out[i * 4 + 1] = rec[0];
    out[i * 4 + 2] = rec[1];
    out[i * 4 + 3] = (rec[2] & ((uint64_t(1) << 56) - 1)) | ((rec[3] & 0xffu) << 56);
  }
  return int(want);
}
const void* purlin_context_device_struct(PurlinHostContext* h) { return &h->dev; }

int purlin_collective(PurlinHostContext* h, int collective, const void* src, void* dst, size_t bytes,
                      const size_t* sizes, const size_t* outSizes, int dtype, int reduceOp, int mode,
                      const void* policy, void* stream) {
  if (!h) { setError("null context"); return 1; }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  CollectiveSpec spec;
  if (!makeSpec(spec, collective, h->dev.world, h->dev.rank, bytes, sizes, outSizes, dtype, reduceOp, mode, h->hasMulticast, src == dst && src != nullptr)) return 1;
  if ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) % 16) { setError("buffers must be 16-byte aligned (32 for full speed)"); return 1; }
  NvtxRange range(collectiveName(collective), isVariable(spec.in) ? dispatchBytes(spec) : bytes);
  if (h->dev.world == 1) return worldOneCopy(spec, src, dst, s);
  const bool variable = isVariable(spec.in);
  if (!variable && bytes == 0) return 0;
  const Policy* forced = static_cast<const Policy*>(policy);
  // An all-reduce larger than the staging half can run as ONE kernel whose shards stream through per-rank windows of the
  // staging half under back-pressure (layout.hpp: cyclic composed plan), or as consecutive segments, each a complete
  // collective on the alternating half. Measured at 1 GiB, bf16: one kernel 1.03x NCCL at two ranks (segments 1.00x),
  // but 0.89x at four and 0.77x at eight (segments 0.95x and 0.93x): the windows shrink with the world size. So the
  // single kernel is the default at two ranks only; PURLIN_AR_SEGMENTS=1 / =0 forces segments / the single kernel.
  // Should the layout engine refuse the single kernel (a forced policy that cannot cycle), segments run.
  if (spec.type == CollectiveType::allReduce && bytes > h->ws.stagingTRSize) {
    const char* const segEnv = std::getenv("PURLIN_AR_SEGMENTS");   // read per call: such a call moves a gigabyte
    const bool segmentsOnly = segEnv ? segEnv[0] != '0' : h->dev.world > 2;
    Plan whole;
    if (!segmentsOnly && planFor(spec, h->ws, forced, whole, nullptr)) return launchPlan(h, whole, src, dst, s);
    const size_t seg = roundDown(h->ws.stagingTRSize, size_t(h->dev.world) * kAccessAlign);
    for (size_t off = 0; off < bytes; off += seg) {
      CollectiveSpec part = spec;
      part.bytes = std::min(seg, bytes - off);
      Plan plan;
      if (!planFor(part, h->ws, forced, plan, nullptr)) return 1;
      if (launchPlan(h, plan, static_cast<const unsigned char*>(src) + off, static_cast<unsigned char*>(dst) + off, s)) return 1;
    }
    return 0;
  }
  if (!forced && !variable && bytes < (1ull << 40)) {
    // the layout engine is deterministic in these inputs: build each plan once
    if (h->planCacheTableSize != TuningTable::global().size() || h->planCacheBudget != maxCtasSetting()) {
      h->planCache.clear(); h->planCacheTableSize = TuningTable::global().size(); h->planCacheBudget = maxCtasSetting();
    }
    const uint64_t key = (uint64_t(bytes) << 16) ^ (uint64_t(collective) << 12) ^ (uint64_t(dtype) << 8) ^ (uint64_t(reduceOp) << 4) ^
                         (uint64_t(mode) << 1) ^ uint64_t(src == dst && src != nullptr);
    auto it = h->planCache.find(key);
    if (it == h->planCache.end()) {
      Plan fresh;
      if (!planFor(spec, h->ws, nullptr, fresh, nullptr)) return 1;
      if (h->planCache.size() > 4096) h->planCache.clear();
      it = h->planCache.emplace(key, fresh).first;
    }
    return launchPlan(h, it->second, src, dst, s);
  }
  Plan plan;
  if (!planFor(spec, h->ws, forced, plan, nullptr)) return 1;
  return launchPlan(h, plan, src, dst, s);
}

// The fixed-size collectives through one short signature (seven scalar arguments: what a foreign-function call from
// Python pays for is mostly the argument count). traits = dtype | reduceOp << 8 | mode << 16.
int purlin_call_fixed(PurlinHostContext* h, int collective, const void* src, void* dst, size_t bytes, unsigned traits, void* stream) {
  return purlin_collective(h, collective, src, dst, bytes, nullptr, nullptr, int(traits & 0xffu), int((traits >> 8) & 0xffu), int((traits >> 16) & 0xffu), nullptr, stream);
}

int purlin_all_reduce(PurlinHostContext* h, const void* src, void* dst, size_t bytes, int dtype, int reduceOp, int mode, void* stream) {
  return purlin_collective(h, int(CollectiveType::allReduce), src, dst, bytes, nullptr, nullptr, dtype, reduceOp, mode, nullptr, stream);
}
int purlin_all_gather(PurlinHostContext* h, const void* src, void* dst, size_t bytesPerRank, void* stream) {
  return purlin_collective(h, int(CollectiveType::allGather), src, dst, bytesPerRank, nullptr, nullptr, 0, 0, 0, nullptr, stream);
}
int purlin_all_gather_v(PurlinHostContext* h, const void* src, void* dst, const size_t* bytesList, void* stream) {
  return purlin_collective(h, int(CollectiveType::allGatherV), src, dst, 0, bytesList, nullptr, 0, 0, 0, nullptr, stream);
}
int purlin_reduce_scatter(PurlinHostContext* h, const void* src, void* dst, size_t bytesPerRankOut, int dtype, int reduceOp, int mode, void* stream) {
  return purlin_collective(h, int(CollectiveType::reduceScatter), src, dst, bytesPerRankOut, nullptr, nullptr, dtype, reduceOp, mode, nullptr, stream);
}
int purlin_reduce_scatter_v(PurlinHostContext* h, const void* src, void* dst, const size_t* bytesList, int dtype, int reduceOp, int mode, void* stream) {
  return purlin_collective(h, int(CollectiveType::reduceScatterV), src, dst, 0, bytesList, nullptr, dtype, reduceOp, mode, nullptr, stream);
}
int purlin_all_to_all(PurlinHostContext* h, const void* src, void* dst, size_t bytesPerPeer, void* stream) {
  return purlin_collective(h, int(CollectiveType::allToAll), src, dst, bytesPerPeer, nullptr, nullptr, 0, 0, 0, nullptr, stream);
}
int purlin_all_to_all_v(PurlinHostContext* h, const void* src, void* dst, const size_t* inSplits, const size_t* outSplits, void* stream) {
  return purlin_collective(h, int(CollectiveType::allToAllV), src, dst, 0, inSplits, outSplits, 0, 0, 0, nullptr, stream);
}

int purlin_emu_collective(PurlinHostContext* const* ctxs, int world, int collective, const void* const* srcs, void* const* dsts,
                          size_t bytes, const size_t* sizesMatrix, int dtype, int reduceOp, int mode, const void* policy,
                          int absentRank, void* stream) {
  if (world < 2 || world > kMaxRanks) { setError("emulation needs 2..16 virtual ranks"); return 1; }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  std::vector<EmuRank> host(world);
  int blocks = 1, threads = 32;
  const bool a2av = collective == int(CollectiveType::allToAllV);
  for (int r = 0; r < world; ++r) {
    size_t in[kMaxRanks] = {}, out[kMaxRanks] = {};
    if (sizesMatrix) for (int q = 0; q < world; ++q) { in[q] = a2av ? sizesMatrix[size_t(r) * world + q] : sizesMatrix[q]; out[q] = a2av ? sizesMatrix[size_t(q) * world + r] : 0; }
    CollectiveSpec spec;
    if (!makeSpec(spec, collective, world, r, bytes, sizesMatrix ? in : nullptr, a2av ? out : nullptr, dtype, reduceOp, mode, 0, srcs[r] == dsts[r] && srcs[r] != nullptr)) return 1;
    Policy fitted;
    const Policy* use = static_cast<const Policy*>(policy);
    if (!use) {
      // the built-in policy sizes grids for a whole GPU per rank; here `world` ranks share one
      int sms = 148;
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ctxs[r]->device);
      const int perRank = std::max(sms / world, 2);
      fitted = selectPolicy(spec, ctxs[r]->ws);
      fitted.putBlocks = std::min(fitted.putBlocks, world);
      fitted.gatherBlocks = std::min(fitted.gatherBlocks, world - 1);
      fitted.localBlocks = 1;
      fitted.consumeBlocks = std::min(fitted.consumeBlocks, std::max(perRank - 2 * world, 1));
      fitted.lrBlocks = std::min(fitted.lrBlocks, perRank);
      use = &fitted;
    }
    if (!planFor(spec, ctxs[r]->ws, use, host[r].plan, nullptr)) return 1;
    host[r].ctx = ctxs[r]->dev;
    host[r].src = static_cast<const unsigned char*>(srcs[r]);
    host[r].dst = static_cast<unsigned char*>(dsts[r]);
    host[r].absent = r == absentRank ? 1 : 0;
    blocks = std::max(blocks, host[r].plan.blocks);
    threads = std::max(threads, host[r].plan.threads);
  }
  threads = std::min(threads, kMaxThreads);
  EmuFn fn = emuKernel(host[0].plan);
  size_t dyn = 0;
  for (int r = 0; r < world; ++r) dyn = std::max<size_t>(dyn, host[r].plan.smemBytes);
  if (dyn > 0 && !ensureSmemOptIn(reinterpret_cast<const void*>(fn))) { setError("cannot opt in to the bulk ring's shared memory"); return 1; }
  int perSm = 0, dev = 0, sms = 0;
  CUDA_OK(cudaGetDevice(&dev));
  CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSm, fn, threads, dyn));
  if (blocks * world > perSm * sms) { setError("emulated grid does not fit on the GPU at once; use fewer CTAs per rank"); return 1; }
  EmuRank* devRanks = nullptr;
  CUDA_OK(cudaMallocAsync(&devRanks, sizeof(EmuRank) * world, s));
  CUDA_OK(cudaMemcpyAsync(devRanks, host.data(), sizeof(EmuRank) * world, cudaMemcpyHostToDevice, s));
  CUDA_OK(cudaStreamSynchronize(s));   // `host` is pageable and dies with this frame
  void* args[] = {&devRanks};
  CUDA_OK(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(fn), dim3(blocks, world), dim3(threads), args, dyn, s));
  CUDA_OK(cudaFreeAsync(devRanks, s));
  return 0;
}

int purlin_p2p_copy(void* dst, const void* src, size_t bytes, int blocks, int threads, void* stream) {
  if (bytes % 16 || (reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) % 16) { setError("p2p copy needs 16-byte alignment"); return 1; }
  blocks = std::min(std::max(blocks, 1), kMaxCtas);
  threads = std::min(std::max(threads, 32), kMaxThreads);
  p2pKernel<Atom><<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<unsigned char*>(dst), static_cast<const unsigned char*>(src), bytes);
  CUDA_OK(cudaGetLastError());
  return 0;
}

}  // extern "C"
