// Point-to-point copies and an all-gather four ways: copy engines (cudaMemcpyAsync between peers) against the
// Atom's SM copy in push and in pull direction.
//
// Counterpart of csrc/examples/p2p/{push,pull,ce_p2p}.cu and csrc/examples/ag/copy_engine_ag.cu in the reference:
// the copy-engine numbers are the baseline a kernel-driven collective has to beat, push against pull shows which
// direction the fabric prefers (remote stores need far fewer SMs than remote loads to fill a link). One process
// drives every visible GPU (up to eight); with a single GPU both ends of every copy live on it, and the figures
// are local-memory bandwidth. Every result is compared byte for byte before it is timed.
//
//   copy_engine [bytes] [blocks] [runs]
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <functional>
#include <vector>

#include "purlin/capi.h"

namespace {

__global__ void fillBytes(unsigned char* p, size_t n, unsigned seed) {
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) p[i] = (unsigned char)((i * 131u + seed) >> 3);
}
__global__ void countMismatches(const unsigned char* p, size_t n, unsigned seed, unsigned long long* bad) {
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x)
    if (p[i] != (unsigned char)((i * 131u + seed) >> 3)) atomicAdd(bad, 1ull);
}

struct Rank {
  int device = 0;
  cudaStream_t stream = nullptr;
  unsigned char* in = nullptr;    // this rank's contribution
  unsigned char* out = nullptr;   // world x bytes
  unsigned long long* bad = nullptr;
};

double timeUs(std::vector<Rank>& ranks, int runs, const std::function<void()>& body) {
  for (Rank& r : ranks) { cudaSetDevice(r.device); cudaStreamSynchronize(r.stream); }
  cudaSetDevice(ranks[0].device);
  cudaEvent_t a, z;
  cudaEventCreate(&a); cudaEventCreate(&z);
  // rank 0's stream brackets the region; the other streams are joined to it before the closing event
  cudaEventRecord(a, ranks[0].stream);
  for (size_t q = 1; q < ranks.size(); ++q) { cudaSetDevice(ranks[q].device); cudaStreamWaitEvent(ranks[q].stream, a, 0); }
  for (int i = 0; i < runs; ++i) body();
  std::vector<cudaEvent_t> done(ranks.size());
  for (size_t q = 1; q < ranks.size(); ++q) {
    cudaSetDevice(ranks[q].device);
    cudaEventCreateWithFlags(&done[q], cudaEventDisableTiming);
    cudaEventRecord(done[q], ranks[q].stream);
  }
  cudaSetDevice(ranks[0].device);
  for (size_t q = 1; q < ranks.size(); ++q) cudaStreamWaitEvent(ranks[0].stream, done[q], 0);
  cudaEventRecord(z, ranks[0].stream);
  cudaEventSynchronize(z);
  float ms = 0.f;
  cudaEventElapsedTime(&ms, a, z);
  for (size_t q = 1; q < ranks.size(); ++q) cudaEventDestroy(done[q]);
  cudaEventDestroy(a); cudaEventDestroy(z);
  return double(ms) * 1000.0 / runs;
}

}  // namespace

int main(int argc, char** argv) {
  size_t bytes = argc > 1 ? size_t(std::atoll(argv[1])) : size_t(32) << 20;
  const int blocks = argc > 2 ? std::atoi(argv[2]) : 32;
  const int runs = argc > 3 ? std::atoi(argv[3]) : 10;
  bytes = std::max<size_t>(bytes / 32, 1) * 32;
  int devices = 0;
  if (cudaGetDeviceCount(&devices) != cudaSuccess || devices == 0) { std::printf("skip: no CUDA device\n"); return 0; }
  const int world = devices >= 2 ? std::min(devices, 8) : 2;   // one GPU: two "ranks" on it
  std::vector<Rank> ranks(static_cast<size_t>(world));
  for (int r = 0; r < world; ++r) {
    Rank& k = ranks[size_t(r)];
    k.device = devices >= 2 ? r : 0;
    cudaSetDevice(k.device);
    if (devices >= 2) for (int q = 0; q < world; ++q) if (q != r) cudaDeviceEnablePeerAccess(q, 0);
    cudaGetLastError();
    cudaStreamCreateWithFlags(&k.stream, cudaStreamNonBlocking);
    if (cudaMalloc(&k.in, bytes) != cudaSuccess || cudaMalloc(&k.out, bytes * size_t(world)) != cudaSuccess ||
        cudaMalloc(&k.bad, sizeof(unsigned long long)) != cudaSuccess) { std::printf("FAIL: out of memory\n"); return 1; }
    fillBytes<<<64, 256, 0, k.stream>>>(k.in, bytes, 17u * unsigned(r) + 1u);
    cudaMemsetAsync(k.bad, 0, sizeof(unsigned long long), k.stream);
    cudaStreamSynchronize(k.stream);
  }
  cudaDeviceProp prop;
  cudaGetDeviceProperties(&prop, 0);
  std::printf("# %d rank(s) on %d device(s), %zu bytes per rank\n", world, devices, bytes);
  std::printf("case,world,bytes,lat(us),bw(GB/s),error(%%),GPUName,blocks\n");
  int failures = 0;

  auto clearOut = [&]() { for (Rank& k : ranks) { cudaSetDevice(k.device); cudaMemsetAsync(k.out, 0, bytes * size_t(world), k.stream); cudaStreamSynchronize(k.stream); } };
  // slot q of a rank's output must hold rank q's pattern
  auto checkSlot = [&](int r, int q) {
    Rank& k = ranks[size_t(r)];
    cudaSetDevice(k.device);
    countMismatches<<<64, 256, 0, k.stream>>>(k.out + size_t(q) * bytes, bytes, 17u * unsigned(q) + 1u, k.bad);
    unsigned long long bad = 0;
    cudaMemcpyAsync(&bad, k.bad, sizeof(bad), cudaMemcpyDeviceToHost, k.stream);
    cudaStreamSynchronize(k.stream);
    cudaMemsetAsync(k.bad, 0, sizeof(bad), k.stream);
    return bad;
  };
  auto report = [&](const char* name, int w, size_t moved, double us, unsigned long long bad, int blk) {
    std::printf("%s,%d,%zu,%.2f,%.2f,%.3f,%s,%d\n", name, w, moved, us, double(moved) / 1e9 / (us * 1e-6), bad ? 100.0 : 0.0, prop.name, blk);
    if (bad) ++failures;
  };

  // 1. copy engine, rank 0 -> rank 1
  clearOut();
  auto ce = [&]() { cudaSetDevice(ranks[0].device); cudaMemcpyAsync(ranks[1].out, ranks[0].in, bytes, cudaMemcpyDeviceToDevice, ranks[0].stream); };
  ce();
  cudaStreamSynchronize(ranks[0].stream);
  unsigned long long bad = checkSlot(1, 0);
  std::vector<Rank> pair01 = {ranks[0]};
  report("ce_p2p", 2, bytes, timeUs(pair01, runs, ce), bad, 0);

  // 2. SM copy pushed by the source rank (remote stores)
  clearOut();
  auto push = [&]() { cudaSetDevice(ranks[0].device); purlin_p2p_copy(ranks[1].out, ranks[0].in, bytes, blocks, 256, ranks[0].stream); };
  push();
  cudaStreamSynchronize(ranks[0].stream);
  bad = checkSlot(1, 0);
  report("push", 2, bytes, timeUs(pair01, runs, push), bad, blocks);

  // 3. SM copy pulled by the destination rank (remote loads)
  clearOut();
  std::vector<Rank> pair1 = {ranks[1]};
  auto pull = [&]() { cudaSetDevice(ranks[1].device); purlin_p2p_copy(ranks[1].out, ranks[0].in, bytes, blocks, 256, ranks[1].stream); };
  pull();
  cudaSetDevice(ranks[1].device);
  cudaStreamSynchronize(ranks[1].stream);
  bad = checkSlot(1, 0);
  report("pull", 2, bytes, timeUs(pair1, runs, pull), bad, blocks);

  // 4. all-gather by copy engines: every rank copies its block into slot `rank` of every rank's output
  clearOut();
  auto ceAllGather = [&]() {
    for (int r = 0; r < world; ++r) {
      cudaSetDevice(ranks[size_t(r)].device);
      for (int k = 0; k < world; ++k) {
        const int q = (r + k) % world;   // start with the local slot, then walk the peers in rotated order
        cudaMemcpyAsync(ranks[size_t(q)].out + size_t(r) * bytes, ranks[size_t(r)].in, bytes, cudaMemcpyDeviceToDevice, ranks[size_t(r)].stream);
      }
    }
  };
  ceAllGather();
  for (Rank& k : ranks) { cudaSetDevice(k.device); cudaStreamSynchronize(k.stream); }
  bad = 0;
  for (int r = 0; r < world; ++r) for (int q = 0; q < world; ++q) bad += checkSlot(r, q);
  report("ce_ag", world, bytes * size_t(world), timeUs(ranks, runs, ceAllGather), bad, 0);

  for (Rank& k : ranks) { cudaSetDevice(k.device); cudaStreamSynchronize(k.stream); cudaFree(k.in); cudaFree(k.out); cudaFree(k.bad); cudaStreamDestroy(k.stream); }
  std::printf("%s: %d failure(s)\n", failures ? "FAILED" : "PASSED", failures);
  return failures ? 1 : 0;
}
