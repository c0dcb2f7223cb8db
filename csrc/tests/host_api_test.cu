// C++ host API on ONE GPU with the emulated provider: validation, workspace format, context life cycle, and a
// four-rank all-reduce run as one cooperative grid.
//
// Counterpart of csrc/tests/setup.cu in the reference (a provider that fakes `world` ranks as `world` allocations
// on one GPU, with fault modes shortTable / nullPeer / unalignedPeer / multicast; checks of validation, zeroed
// and aligned regions, move semantics, finalize waiting for work in flight, multicast environment switches).
// Prints one line per check and exits non-zero on the first failure.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <vector>

#include "purlin/host.hpp"

using namespace purlin;

static int g_failures = 0;
#define CHECK(cond, what)                                              \
  do {                                                                 \
    if (cond) std::printf("ok    %s\n", what);                        \
    else { std::printf("FAIL  %s (%s:%d)\n", what, __FILE__, __LINE__); ++g_failures; } \
  } while (0)

template <class F> bool throws(F&& f) {
  try { f(); } catch (const std::exception&) { return true; }
  return false;
}

__global__ void slowMarker(int* flag, long long spins) {
  long long t = clock64();
  while (clock64() - t < spins) {}
  *flag = 1;
}

int main() {
  int devices = 0;
  if (cudaGetDeviceCount(&devices) != cudaSuccess || devices == 0) { std::printf("skip: no CUDA device\n"); return 0; }
  cudaStream_t stream;
  cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking);
  constexpr int W = 4;
  const size_t staging = 1 << 20;

  // ---- argument validation ----
  {
    EmulatedMemory::Shared sh;
    CHECK(throws([&] { auto m = initialize(0, 1 + kMaxRanks, stream, EmulatedMemory(&sh, 17), staging); }), "world larger than 16 is rejected");
    CHECK(throws([&] { auto m = initialize(4, W, stream, EmulatedMemory(&sh, W), staging); }), "rank outside the world is rejected");
    CHECK(throws([&] { auto m = initialize(0, W, stream, EmulatedMemory(&sh, W), 1000); }), "staging size below 256 KiB is rejected");
    CHECK(throws([&] { auto m = initialize(0, W, stream, EmulatedMemory(&sh, W), staging + 8); }), "unaligned staging size is rejected");
  }
  // ---- provider fault modes ----
  for (auto fault : {EmulatedFault::shortTable, EmulatedFault::nullPeer, EmulatedFault::unalignedPeer}) {
    EmulatedMemory::Shared sh;
    const bool t = throws([&] { auto m = initialize(0, W, stream, EmulatedMemory(&sh, W, fault), staging); });
    CHECK(t, fault == EmulatedFault::shortTable ? "short pointer table is rejected" : fault == EmulatedFault::nullPeer ? "null peer pointer is rejected" : "unaligned peer pointer is rejected");
    CHECK(sh.blocks.empty(), "a failed initialize returns the provider's memory");
  }
  // ---- workspace regions: sizes, alignment, zero fill ----
  {
    size_t ws[8];
    purlin_workspace_layout(W, staging, ws);
    CHECK(ws[1] == 2 * staging && ws[2] == 2 * (staging + kPacketEpochBytes), "throughput and packet regions precede the signals");
    CHECK(ws[3] == ws[2] + 8 * W && ws[4] == ws[2] + 16 * W && ws[5] % 32 == 0 && ws[6] == ws[5] + 2 * W * 16, "signal, gather, consumed and arrival regions do not overlap");
    CHECK(ws[7] % 16 == 0 && ws[7] * W <= kPacketEpochBytes, "packet stride is packet aligned and fits the epoch");
    EmulatedMemory::Shared sh;
    auto m = initialize(1, W, stream, EmulatedMemory(&sh, W), staging);
    std::vector<unsigned char> host(ws[6] - ws[2]);
    cudaMemcpy(host.data(), static_cast<unsigned char*>(sh.blocks[1]) + ws[2], host.size(), cudaMemcpyDeviceToHost);
    bool zero = true;
    for (unsigned char b : host) zero = zero && b == 0;
    CHECK(zero, "signal regions start zeroed");
    // ---- move semantics ----
    ManagedContext<EmulatedMemory> moved = std::move(m);
    CHECK(m.empty() && !moved.empty(), "moving a managed context leaves the source empty");
    CHECK(throws([&] { m.context(); }), "an empty managed context refuses context()");
    // ---- finalize waits for work in flight on the stream ----
    int* flag = nullptr;
    cudaMalloc(&flag, sizeof(int));
    cudaMemset(flag, 0, sizeof(int));
    slowMarker<<<1, 1, 0, stream>>>(flag, 20000000LL);
    finalize(moved, stream);
    int seen = 0;
    cudaMemcpy(&seen, flag, sizeof(int), cudaMemcpyDeviceToHost);
    CHECK(seen == 1 && moved.empty(), "finalize waits for the stream and empties the context");
    CHECK(sh.blocks.empty(), "finalize returns the provider's memory");
    cudaFree(flag);
  }
  // ---- a borrowed context does not free the caller's memory ----
  {
    std::vector<void*> blocks(W);
    const size_t bytes = workspaceBytes(W, staging);
    for (auto& b : blocks) { cudaMalloc(&b, bytes); cudaMemset(b, 0, bytes); }
    WorkspaceMemory mem;
    mem.peers = blocks;
    ContextRef c = initialize(2, W, mem, stream, staging);
    CHECK(bool(c) && !c.hasMulticast(), "caller-owned workspace yields a context without multicast");
    finalize(c, stream);
    CHECK(!c && cudaMemset(blocks[0], 1, 64) == cudaSuccess, "finalize of a borrowed context leaves the memory usable");
    // ---- multicast environment switches ----
    mem.multicast = blocks[0];   // a stand-in alias: only the plumbing is checked, nothing dereferences it
    ContextRef mc = initialize(0, W, mem, stream, staging);
    CHECK(mc.hasMulticast(), "a multicast pointer enables the NVLS paths");
    finalize(mc, stream);
    setenv("PURLIN_DISABLE_MULTIMEM", "1", 1);
    ContextRef off = initialize(0, W, mem, stream, staging);
    CHECK(!off.hasMulticast(), "PURLIN_DISABLE_MULTIMEM switches them off");
    finalize(off, stream);
    unsetenv("PURLIN_DISABLE_MULTIMEM");
    for (auto b : blocks) cudaFree(b);
  }
  // ---- four ranks on one GPU: every rank's context over the same emulated blocks, one cooperative launch ----
  {
    EmulatedMemory::Shared sh;
    std::vector<ManagedContext<EmulatedMemory>> ranks;
    for (int r = 0; r < W; ++r) ranks.push_back(initialize(r, W, stream, EmulatedMemory(&sh, W), staging));
    const size_t n = 4096;
    std::vector<float*> src(W), dst(W);
    std::vector<float> host(n);
    for (int r = 0; r < W; ++r) {
      cudaMalloc(&src[r], n * 4); cudaMalloc(&dst[r], n * 4);
      for (size_t i = 0; i < n; ++i) host[i] = float(int(i % 5) - 2 + r);
      cudaMemcpy(src[r], host.data(), n * 4, cudaMemcpyHostToDevice);
    }
    std::vector<PurlinHostContext*> handles;
    for (auto& m : ranks) handles.push_back(m.context().handle());
    std::vector<const void*> s(src.begin(), src.end());
    std::vector<void*> d(dst.begin(), dst.end());
    const int rc = purlin_emu_collective(handles.data(), W, int(CollectiveType::allReduce), s.data(), d.data(), n * 4, nullptr,
                                         int(DType::fp32), int(ReduceOp::add), 0, nullptr, -1, stream);
    CHECK(rc == 0, "emulated four-rank all-reduce launches");
    bool ok = true;
    for (int r = 0; r < W && rc == 0; ++r) {
      ranks[r].context().check(stream);
      cudaMemcpy(host.data(), dst[r], n * 4, cudaMemcpyDeviceToHost);
      for (size_t i = 0; i < n; ++i) ok = ok && host[i] == float(4 * (int(i % 5) - 2) + 6);
    }
    CHECK(ok, "every rank holds the sum");
    for (int r = 0; r < W; ++r) { cudaFree(src[r]); cudaFree(dst[r]); }
    for (auto& m : ranks) finalize(m, stream);
    CHECK(sh.blocks.empty(), "the last finalize frees the emulated blocks");
  }
  cudaStreamDestroy(stream);
  std::printf("%s: %d failure(s)\n", g_failures ? "FAILED" : "PASSED", g_failures);
  return g_failures ? 1 : 0;
}
