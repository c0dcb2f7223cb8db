// Multi-GPU correctness + performance of the C++ host API in ONE process: one host thread per GPU.
//
// Counterpart of the reference's csrc/tests/{ar,ag,agv,rs,rsv,a2a,a2av}.cu binaries and their support library
// (csrc/support/purlin/benchmark/benchmark.cuh:79-214, data.cuh:46-140, purlin_report.cuh:21-41): for every size
// of a power-of-two sweep, one untimed run is compared bit for bit with an expectation every rank regenerates
// locally from seeds, then `runs` launches are timed with CUDA events (in a stream or replayed from a CUDA graph)
// and the maximum over the ranks is reported as a CSV row. The reference needs MPI and NVSHMEM for this; here the
// ranks are threads, the bootstrap is a mutex and a condition variable, and the memory comes from the native
// virtual-memory provider (with its NVLS alias) or from plain peer-enabled cudaMalloc blocks.
//
//   multi_gpu_bench <ar|ag|agv|rs|rsv|a2a|a2av|all> [minBytes] [maxBytes] [graphLaunches] [runs] [warmup] [seed]
//                   [--reduction-mode deterministic|non-deterministic] [--provider vmm|peer] [--world N]
//                   [--staging BYTES] [--check-only]
// Byte arguments are per-rank payloads (all-reduce: the whole buffer). Exit code 0 and a final "PASSED" line
// when every comparison was exact; "skip" when fewer than two GPUs are visible.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "purlin/host.hpp"

using namespace purlin;

extern "C" int purlin_zipf_splits(size_t total, int world, int eighths, size_t* out);

namespace {

// ---- in-process bootstrap: all-gather and barrier between the rank threads ----
class ThreadGroup {
 public:
  explicit ThreadGroup(int world) : world_(world) {}
  void barrier() {
    std::unique_lock<std::mutex> l(mu_);
    const uint64_t gen = generation_;
    if (++arrived_ == world_) { arrived_ = 0; ++generation_; cv_.notify_all(); }
    else cv_.wait(l, [&] { return generation_ != gen; });
  }
  void allGather(int rank, const void* send, void* recv, size_t n) {
    {
      std::lock_guard<std::mutex> l(mu_);
      if (scratch_.size() < n * size_t(world_)) scratch_.resize(n * size_t(world_));
    }
    barrier();
    std::memcpy(scratch_.data() + size_t(rank) * n, send, n);
    barrier();
    std::memcpy(recv, scratch_.data(), n * size_t(world_));
    barrier();
  }
  double maxOver(int rank, double v) {
    std::vector<double> all(static_cast<size_t>(world_), 0.0);
    allGather(rank, &v, all.data(), sizeof(double));
    return *std::max_element(all.begin(), all.end());
  }
  int world() const { return world_; }
 private:
  int world_;
  std::mutex mu_;
  std::condition_variable cv_;
  int arrived_ = 0;
  uint64_t generation_ = 0;
  std::vector<unsigned char> scratch_;
};

// Plain cudaMalloc blocks with peer access enabled: the provider of last resort (no multicast alias).
class PeerMemory {
 public:
  PeerMemory(int rank, ThreadGroup* g) : rank_(rank), g_(g) {}
  SymmetricAllocation allocate_zeroed(size_t bytes, size_t, cudaStream_t stream) {
    for (int q = 0; q < g_->world(); ++q) if (q != rank_) cudaDeviceEnablePeerAccess(q, 0);
    cudaGetLastError();   // "already enabled" is not an error
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) p = nullptr;
    if (p) { cudaMemsetAsync(p, 0, bytes, stream); cudaStreamSynchronize(stream); }
    SymmetricAllocation a;
    a.peers.resize(size_t(g_->world()));
    g_->allGather(rank_, &p, a.peers.data(), sizeof(void*));
    for (void* q : a.peers) if (!q) { if (p) cudaFree(p); throw std::runtime_error("PeerMemory: cudaMalloc failed on some rank"); }
    local_ = p;
    return a;
  }
  void free(SymmetricAllocation& a) {
    g_->barrier();
    if (local_) cudaFree(local_);
    local_ = nullptr;
    a.peers.clear();
  }
 private:
  int rank_;
  ThreadGroup* g_;
  void* local_ = nullptr;
};

// ---- seeded data: integers in [-2, 2], exact in bf16 and in any summation order ----
__host__ __device__ inline uint32_t mix(uint64_t x) {
  x ^= x >> 33; x *= 0xff51afd7ed558ccdull; x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ull; x ^= x >> 33;
  return uint32_t(x);
}
__host__ __device__ inline float valueAt(uint64_t seed, int rank, size_t i) { return float(int(mix(seed * 1000003ull + uint64_t(rank) * 7919ull + i * 16ull + 5ull) % 5u) - 2); }

__global__ void fillKernel(__nv_bfloat16* p, size_t n, uint64_t seed, int rank) {
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) p[i] = __float2bfloat16(valueAt(seed, rank, i));
}
__global__ void poisonKernel(__nv_bfloat16* p, size_t n) {
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) p[i] = __float2bfloat16(77.f);
}

// Output element i of `rank` comes from input element srcIndex of rank srcRank (copies), or is the rank-ordered
// sum over all ranks of input element srcIndex (reductions). Offsets are in elements.
struct Expectation {
  int world, rank, reduces;
  size_t outOffset[kMaxRanks + 1];   // copies: output segment q spans [outOffset[q], outOffset[q+1])
  size_t srcOffset[kMaxRanks];       // copies: where segment q starts in rank q's input; reductions: [0] = start in every input
};
__global__ void checkKernel(const __nv_bfloat16* out, size_t n, Expectation e, uint64_t seed, unsigned long long* mismatches) {
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) {
    float want = 0.f;
    if (e.reduces) {
      for (int q = 0; q < e.world; ++q) want += valueAt(seed, q, e.srcOffset[0] + i);
    } else {
      int q = 0;
      while (q + 1 < e.world && i >= e.outOffset[q + 1]) ++q;
      want = valueAt(seed, q, e.srcOffset[q] + (i - e.outOffset[q]));
    }
    if (__bfloat162float(out[i]) != want) atomicAdd(mismatches, 1ull);
  }
}

struct Options {
  std::string collective = "all";
  size_t minBytes = 8 << 10, maxBytes = 64 << 20, staging = kDefaultStagingBytes;
  int graphLaunches = 0, runs = 20, warmup = 5, world = 0;
  uint64_t seed = 1234;
  ReductionMode mode = ReductionMode::nonDeterministic;
  std::string provider = "vmm";
  bool checkOnly = false;
};

size_t parseBytes(const char* s) {
  char* end = nullptr;
  double v = std::strtod(s, &end);
  if (end && (*end == 'K' || *end == 'k')) v *= 1024.0;
  else if (end && (*end == 'M' || *end == 'm')) v *= 1024.0 * 1024.0;
  else if (end && (*end == 'G' || *end == 'g')) v *= 1024.0 * 1024.0 * 1024.0;
  return size_t(v);
}

bool parse(int argc, char** argv, Options& o) {
  int positional = 0;
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    auto next = [&]() -> const char* { return i + 1 < argc ? argv[++i] : ""; };
    if (a == "--reduction-mode") {
      const std::string m = next();
      if (m == "deterministic") o.mode = ReductionMode::deterministic;
      else if (m == "non-deterministic" || m == "nondeterministic") o.mode = ReductionMode::nonDeterministic;
      else { std::fprintf(stderr, "unknown reduction mode '%s'\n", m.c_str()); return false; }
    } else if (a == "--provider") o.provider = next();
    else if (a == "--world") o.world = std::atoi(next());
    else if (a == "--staging") o.staging = parseBytes(next());
    else if (a == "--check-only") o.checkOnly = true;
    else if (a.rfind("--", 0) == 0) { std::fprintf(stderr, "unknown option %s\n", a.c_str()); return false; }
    else {
      switch (positional++) {
        case 0: o.collective = a; break;
        case 1: o.minBytes = parseBytes(a.c_str()); break;
        case 2: o.maxBytes = parseBytes(a.c_str()); break;
        case 3: o.graphLaunches = std::atoi(a.c_str()); break;
        case 4: o.runs = std::atoi(a.c_str()); break;
        case 5: o.warmup = std::atoi(a.c_str()); break;
        case 6: o.seed = std::strtoull(a.c_str(), nullptr, 10); break;
        default: std::fprintf(stderr, "too many arguments\n"); return false;
      }
    }
  }
  if (o.provider != "vmm" && o.provider != "peer") { std::fprintf(stderr, "provider must be vmm or peer\n"); return false; }
  return o.minBytes >= 32 && o.maxBytes >= o.minBytes && o.runs > 0 && o.warmup >= 0;
}

}  // namespace

namespace {

struct Shape {
  size_t inElems = 0, outElems = 0, logicalBytes = 0;
  Expectation exp{};
  std::vector<size_t> sizes, inSplits, outSplits;   // bytes, for the variable-length forms
};

// per-rank payload `bytes` -> buffer sizes, split lists and where every output element comes from
bool shapeFor(const std::string& c, int world, int rank, size_t bytes, Shape& s) {
  const size_t e = sizeof(__nv_bfloat16);
  s.exp.world = world; s.exp.rank = rank; s.exp.reduces = (c == "ar" || c == "rs" || c == "rsv") ? 1 : 0;
  const size_t n = bytes / e;
  std::vector<size_t> zipf(size_t(world), bytes);
  if (c == "agv" || c == "rsv" || c == "a2av") {
    if (purlin_zipf_splits(bytes * size_t(world), world, 8, zipf.data()) != 0) return false;
  }
  auto prefix = [&](const std::vector<size_t>& v, int upto) { size_t t = 0; for (int q = 0; q < upto; ++q) t += v[size_t(q)]; return t; };
  if (c == "ar") {
    s.inElems = s.outElems = n; s.logicalBytes = bytes; s.exp.srcOffset[0] = 0;
  } else if (c == "ag" || c == "agv") {
    s.sizes = zipf;
    s.inElems = s.sizes[size_t(rank)] / e; s.outElems = prefix(s.sizes, world) / e; s.logicalBytes = s.outElems * e;
    for (int q = 0; q <= world; ++q) s.exp.outOffset[q] = prefix(s.sizes, q) / e;
    for (int q = 0; q < world; ++q) s.exp.srcOffset[q] = 0;
  } else if (c == "rs" || c == "rsv") {
    s.sizes = zipf;
    s.inElems = prefix(s.sizes, world) / e; s.outElems = s.sizes[size_t(rank)] / e; s.logicalBytes = s.inElems * e;
    s.exp.srcOffset[0] = prefix(s.sizes, rank) / e;
  } else if (c == "a2a" || c == "a2av") {
    // row r of the matrix (what rank r sends to each peer) is the split list rotated by r
    auto cell = [&](int r, int q) { return zipf[size_t((q + r) % world)]; };
    s.inSplits.resize(size_t(world)); s.outSplits.resize(size_t(world));
    for (int q = 0; q < world; ++q) { s.inSplits[size_t(q)] = cell(rank, q); s.outSplits[size_t(q)] = cell(q, rank); }
    s.inElems = prefix(s.inSplits, world) / e; s.outElems = prefix(s.outSplits, world) / e; s.logicalBytes = s.inElems * e;
    for (int q = 0; q <= world; ++q) s.exp.outOffset[q] = prefix(s.outSplits, q) / e;
    for (int q = 0; q < world; ++q) { size_t t = 0; for (int k = 0; k < rank; ++k) t += cell(q, k); s.exp.srcOffset[q] = t / e; }
  } else {
    return false;
  }
  return true;
}

void launch(const std::string& c, const Shape& s, size_t bytes, ReductionMode mode, const void* in, void* out, const ContextRef& ctx, cudaStream_t st) {
  dispatchReductionMode(mode, [&](auto m) {
    constexpr ReductionMode M = decltype(m)::value;
    if (c == "ar") allReduce<__nv_bfloat16, ReduceOp::add, M>(in, out, bytes, ctx, st);
    else if (c == "ag") allGather(in, out, bytes, ctx, st);
    else if (c == "agv") allGatherV(in, out, s.sizes, ctx, st);
    else if (c == "rs") reduceScatter<__nv_bfloat16, ReduceOp::add, M>(in, out, bytes, ctx, st);
    else if (c == "rsv") reduceScatterV<__nv_bfloat16, ReduceOp::add, M>(in, out, s.sizes, ctx, st);
    else if (c == "a2a") all2all(in, out, bytes, ctx, st);
    else all2allV(in, out, s.inSplits, s.outSplits, ctx, st);
  });
}

struct Shared {
  ThreadGroup* group;
  Options opt;
  int failures = 0;
  std::mutex mu;
};

const char* longName(const std::string& c) {
  if (c == "ar") return "allReduce"; if (c == "ag") return "allGather"; if (c == "agv") return "allGatherV";
  if (c == "rs") return "reduceScatter"; if (c == "rsv") return "reduceScatterV"; if (c == "a2a") return "all2all";
  return "all2allV";
}

template <class Provider>
void sweep(int rank, Shared& sh, cudaStream_t st, Provider provider) {
  const Options& o = sh.opt;
  ThreadGroup& g = *sh.group;
  const int world = g.world();
  auto managed = initialize(rank, world, st, std::move(provider), o.staging);
  const ContextRef& ctx = managed.context();
  cudaDeviceProp prop;
  cudaGetDeviceProperties(&prop, rank);
  if (rank == 0) {
    std::printf("# world %d  multicast %d  provider %s  seed %llu\n", world, int(ctx.hasMulticast()), o.provider.c_str(), (unsigned long long)o.seed);
    std::printf("collective,world,totalBytes,datatype,lat(us),bw(GB/s),error(%%),GPUName,warmup,runs,graph_launches\n");
  }
  std::vector<std::string> list;
  if (o.collective == "all") list = {"ar", "ag", "agv", "rs", "rsv", "a2a", "a2av"};
  else list = {o.collective};
  unsigned long long* mismatches = nullptr;
  cudaMalloc(&mismatches, sizeof(unsigned long long));
  for (const std::string& c : list) {
    for (size_t bytes = o.minBytes; bytes <= o.maxBytes; bytes *= 2) {
      const size_t unit = size_t(kAccessAlign) * size_t(world);
      const size_t b = (bytes + unit - 1) / unit * unit;
      Shape s;
      if (!shapeFor(c, world, rank, b, s)) { std::lock_guard<std::mutex> l(sh.mu); ++sh.failures; std::printf("FAIL %s: cannot shape %zu bytes: %s\n", c.c_str(), b, purlin_last_error()); break; }
      __nv_bfloat16 *in = nullptr, *out = nullptr;
      cudaMalloc(&in, std::max<size_t>(s.inElems, 16) * 2);
      cudaMalloc(&out, std::max<size_t>(s.outElems, 16) * 2);
      const uint64_t seed = o.seed + bytes;
      fillKernel<<<64, 256, 0, st>>>(in, s.inElems, seed, rank);
      poisonKernel<<<64, 256, 0, st>>>(out, s.outElems);
      cudaMemsetAsync(mismatches, 0, sizeof(unsigned long long), st);
      // untimed, exact comparison
      launch(c, s, b, o.mode, in, out, ctx, st);
      checkKernel<<<64, 256, 0, st>>>(out, s.outElems, s.exp, seed, mismatches);
      unsigned long long bad = 0;
      cudaMemcpyAsync(&bad, mismatches, sizeof(bad), cudaMemcpyDeviceToHost, st);
      bool timedOut = false;
      try { ctx.check(st); } catch (const std::exception& ex) { timedOut = true; std::printf("FAIL rank %d %s %zu: %s\n", rank, c.c_str(), b, ex.what()); }
      const double errorPct = s.outElems ? 100.0 * double(bad) / double(s.outElems) : 0.0;
      if (bad || timedOut) { std::lock_guard<std::mutex> l(sh.mu); ++sh.failures; if (bad) std::printf("FAIL rank %d %s %zu bytes: %llu elements differ\n", rank, c.c_str(), b, bad); }
      const int anyBad = int(g.maxOver(rank, double(bad || timedOut)));
      double us = 0.0;
      if (!anyBad && !o.checkOnly) {
        cudaEvent_t a, z;
        cudaEventCreate(&a); cudaEventCreate(&z);
        cudaGraphExec_t exec = nullptr;
        if (o.graphLaunches > 0) {
          cudaGraph_t graph;
          cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal);
          for (int i = 0; i < o.runs; ++i) launch(c, s, b, o.mode, in, out, ctx, st);
          cudaStreamEndCapture(st, &graph);
          cudaGraphInstantiate(&exec, graph, 0);
          cudaGraphDestroy(graph);
        }
        for (int i = 0; i < o.warmup; ++i) { if (exec) cudaGraphLaunch(exec, st); else launch(c, s, b, o.mode, in, out, ctx, st); }
        cudaStreamSynchronize(st);
        g.barrier();
        cudaEventRecord(a, st);
        const int reps = exec ? o.graphLaunches : o.runs;
        for (int i = 0; i < reps; ++i) { if (exec) cudaGraphLaunch(exec, st); else launch(c, s, b, o.mode, in, out, ctx, st); }
        cudaEventRecord(z, st);
        cudaEventSynchronize(z);
        float ms = 0.f;
        cudaEventElapsedTime(&ms, a, z);
        us = double(ms) * 1000.0 / double(reps * (exec ? o.runs : 1));
        if (exec) cudaGraphExecDestroy(exec);
        cudaEventDestroy(a); cudaEventDestroy(z);
        try { ctx.check(st); } catch (const std::exception& ex) { std::lock_guard<std::mutex> l(sh.mu); ++sh.failures; std::printf("FAIL rank %d %s %zu timed: %s\n", rank, c.c_str(), b, ex.what()); }
      }
      const double worst = g.maxOver(rank, us);
      const double worstErr = g.maxOver(rank, errorPct);
      if (rank == 0)
        std::printf("%s,%d,%zu,bf16,%.2f,%.2f,%.3f,%s,%d,%d,%d\n", longName(c), world, s.logicalBytes, worst,
                    worst > 0 ? double(s.logicalBytes) / 1e9 / (worst * 1e-6) : 0.0, worstErr, prop.name, o.warmup, o.runs, o.graphLaunches);
      cudaStreamSynchronize(st);
      g.barrier();
      cudaFree(in); cudaFree(out);
    }
  }
  cudaFree(mismatches);
  finalize(managed, st);
}

void rankMain(int rank, Shared* sh) {
  cudaSetDevice(rank);
  cudaStream_t st;
  cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking);
  ThreadGroup* g = sh->group;
  try {
    if (sh->opt.provider == "vmm") {
      sweep(rank, *sh, st, VmmMemory(rank, g->world(), rank,
                                     [g, rank](const void* s, void* r, size_t n) { g->allGather(rank, s, r, n); }, [g] { g->barrier(); }));
    } else {
      sweep(rank, *sh, st, PeerMemory(rank, g));
    }
  } catch (const std::exception& ex) {
    std::lock_guard<std::mutex> l(sh->mu);
    ++sh->failures;
    std::printf("FAIL rank %d: %s\n", rank, ex.what());
  }
  cudaStreamDestroy(st);
}

}  // namespace

int main(int argc, char** argv) {
  Options opt;
  if (!parse(argc, argv, opt)) {
    std::fprintf(stderr, "usage: multi_gpu_bench <ar|ag|agv|rs|rsv|a2a|a2av|all> [minBytes] [maxBytes] [graphLaunches] [runs] [warmup] [seed]\n"
                         "       [--reduction-mode deterministic|non-deterministic] [--provider vmm|peer] [--world N] [--staging BYTES] [--check-only]\n");
    return 2;
  }
  int devices = 0;
  if (cudaGetDeviceCount(&devices) != cudaSuccess || devices < 2) { std::printf("skip: needs at least two CUDA devices (found %d)\n", devices); return 0; }
  int world = opt.world > 0 ? std::min(opt.world, devices) : std::min(devices, 8);
  if (world < 2) world = 2;
  std::fprintf(stderr, "seed %llu\n", (unsigned long long)opt.seed);
  ThreadGroup group(world);
  Shared sh;
  sh.group = &group;
  sh.opt = opt;
  std::vector<std::thread> threads;
  for (int r = 0; r < world; ++r) threads.emplace_back(rankMain, r, &sh);
  for (auto& t : threads) t.join();
  std::printf("%s: %d failure(s)\n", sh.failures ? "FAILED" : "PASSED", sh.failures);
  return sh.failures ? 1 : 0;
}
