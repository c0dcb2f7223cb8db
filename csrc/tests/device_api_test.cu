// Device-side API: a USER kernel that computes and then runs a whole collective, plus a user kernel that calls the
// Atom directly. Four virtual ranks are the rows of one cooperative grid on one GPU.
//
// Counterpart of the reference's device-side usage (README.md:62-122 and csrc/examples/ar/ar.cu:69-83: "this
// collective could be fused into a larger kernel"): the kernel below scales its input and all-reduces the result
// without leaving the kernel. The plan comes from the host layout engine (purlin_plan_build) and the context from
// purlin_context_device_struct; the collective itself is purlin::allReduce<T, Op>(SnacArgs, Context, ...).
#include <cuda_runtime.h>

#include <cstdio>
#include <vector>

#include "purlin/capi.h"
#include "purlin/collective.cuh"
#include "purlin/layout.hpp"
#include "purlin/pipeline.hpp"
#include "purlin/static_for.hpp"

using namespace purlin;

struct RankArgs {
  Context ctx;
  Plan plan;
  const float* in;
  float* scaled;
  float* out;
  size_t n;
};

// every row of the grid is one rank: scale (the "compute"), grid-row barrier, then the collective
__global__ void __launch_bounds__(256, 1) scaleThenAllReduce(const RankArgs* ranks, unsigned int* rowBarrier, float factor) {
  __shared__ const unsigned char* peers[kMaxRanks];
  __shared__ alignas(16) unsigned char ctxMem[sizeof(Context)];
  __shared__ alignas(16) unsigned char planMem[sizeof(Plan)];
  const RankArgs& me = ranks[blockIdx.y];
  for (size_t i = threadIdx.x; i < sizeof(Context) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(ctxMem)[i] = reinterpret_cast<const uint32_t*>(&me.ctx)[i];
  for (size_t i = threadIdx.x; i < sizeof(Plan) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(planMem)[i] = reinterpret_cast<const uint32_t*>(&me.plan)[i];
  __syncthreads();
  const Context& ctx = *reinterpret_cast<const Context*>(ctxMem);
  const Plan& plan = *reinterpret_cast<const Plan*>(planMem);
  // compute phase, spread over the row's CTAs
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < me.n; i += size_t(gridDim.x) * blockDim.x) me.scaled[i] = me.in[i] * factor;
  // all CTAs of this row have written `scaled` before any of them stages it (bounded wait, cooperative grid)
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    atomicAdd(rowBarrier + blockIdx.y, 1u);
    const uint64_t start = sig::globalTimerNs();
    while (sig::ldRelaxedGpu32(rowBarrier + blockIdx.y) < gridDim.x && sig::globalTimerNs() - start < 2000000000ull) {}
    __threadfence();
  }
  __syncthreads();
  if (int(blockIdx.x) >= plan.blocks) return;
  SnacArgs args{reinterpret_cast<const unsigned char*>(me.scaled), reinterpret_cast<unsigned char*>(me.out), &plan};
  allReduce<DType::fp32, ReduceOp::add>(args, ctx, peers);
}

// the Atom on its own: one CTA copies a slice, src or dst may be peer memory
__global__ void atomCopy(unsigned char* dst, const unsigned char* src, size_t bytes) {
  superCopy<DefaultAtom>(dst, src, bytes, blockIdx.x, gridDim.x);
}

// the prefetch-ring driver with a real asynchronous operation: every thread keeps Depth cp.async copies of 16 bytes
// in flight through its own column of a shared-memory ring (no CTA barrier needed: a thread reads only what it loaded)
template <int Depth, int Threads>
struct CpAsyncCopy {
  const uint4* src;
  uint4* dst;
  size_t vecs;
  uint4* ring;   // Depth x Threads vectors of shared memory
  __device__ void prepare() {}
  __device__ void prefetch(int slot, size_t stage) {
    const size_t i = stage * Threads + threadIdx.x;
    if (i < vecs) {
      const unsigned smem = unsigned(__cvta_generic_to_shared(ring + slot * Threads + threadIdx.x));
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem), "l"(src + i) : "memory");
    }
  }
  __device__ void commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
  template <int N> __device__ void wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
  __device__ void consume(int slot, size_t stage) {
    const size_t i = stage * Threads + threadIdx.x;
    if (i < vecs) dst[i] = ring[slot * Threads + threadIdx.x];
  }
  __device__ void advance() {}
};

__global__ void __launch_bounds__(256) pipelinedCopy(const uint4* src, uint4* dst, size_t vecs, int* loopSum) {
  constexpr int kDepth = 4, kThreads = 256;
  __shared__ uint4 ring[kDepth * kThreads];
  const size_t per = (vecs + gridDim.x - 1) / gridDim.x;
  const size_t begin = size_t(blockIdx.x) * per;
  const size_t mine = begin >= vecs ? 0 : (vecs - begin < per ? vecs - begin : per);
  CpAsyncCopy<kDepth, kThreads> op{src + begin, dst + begin, mine, ring};
  Pipeline<kDepth>::run(op, (mine + kThreads - 1) / kThreads);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    int t = 0;
    staticFor<5>([&](auto i) { t += decltype(i)::value * decltype(i)::value; });   // 0 + 1 + 4 + 9 + 16
    *loopSum = t;
  }
}

int main() {
  int devices = 0;
  if (cudaGetDeviceCount(&devices) != cudaSuccess || devices == 0) { std::printf("skip: no CUDA device\n"); return 0; }
  constexpr int W = 4;
  const size_t staging = 1 << 20, n = 6144;
  cudaStream_t stream;
  cudaStreamCreate(&stream);
  size_t ws[8];
  purlin_workspace_layout(W, staging, ws);
  std::vector<uint64_t> blocks(W);
  for (auto& b : blocks) { void* p; cudaMalloc(&p, ws[6]); cudaMemset(p, 0, ws[6]); b = reinterpret_cast<uint64_t>(p); }
  std::vector<PurlinHostContext*> ctxs(W);
  std::vector<RankArgs> host(W);
  Policy pol;            // a small grid per rank so that four ranks fit on the GPU at once
  pol.putBlocks = 4; pol.consumeBlocks = 4; pol.gatherBlocks = 3; pol.localBlocks = 1; pol.threads = 256; pol.unroll = 4;
  pol.arPath = int32_t(AllReducePath::composed); pol.regime = int32_t(Regime::throughput);
  int gridX = 1, failures = 0;
  for (int r = 0; r < W; ++r) {
    ctxs[r] = purlin_context_create(r, W, blocks.data(), 0, staging, 2000000000ull, stream);
    if (!ctxs[r]) { std::printf("FAIL context: %s\n", purlin_last_error()); return 1; }
    host[r].ctx = *static_cast<const Context*>(purlin_context_device_struct(ctxs[r]));
    if (purlin_plan_build(int(CollectiveType::allReduce), W, r, n * 4, nullptr, nullptr, int(DType::fp32), int(ReduceOp::add), 0, 0, 0,
                          staging, &pol, &host[r].plan, nullptr) != 0) { std::printf("FAIL plan: %s\n", purlin_last_error()); return 1; }
    gridX = std::max(gridX, host[r].plan.blocks);
    std::vector<float> in(n);
    for (size_t i = 0; i < n; ++i) in[i] = float(int(i % 7) - 3 + r);
    float *dIn, *dScaled, *dOut;
    cudaMalloc(&dIn, n * 4); cudaMalloc(&dScaled, n * 4); cudaMalloc(&dOut, n * 4);
    cudaMemcpy(dIn, in.data(), n * 4, cudaMemcpyHostToDevice);
    host[r].in = dIn; host[r].scaled = dScaled; host[r].out = dOut; host[r].n = n;
  }
  RankArgs* dev;
  unsigned int* rowBarrier;
  cudaMalloc(&dev, sizeof(RankArgs) * W);
  cudaMalloc(&rowBarrier, sizeof(unsigned int) * W);
  cudaMemset(rowBarrier, 0, sizeof(unsigned int) * W);
  cudaMemcpy(dev, host.data(), sizeof(RankArgs) * W, cudaMemcpyHostToDevice);
  float factor = 2.f;
  void* args[] = {&dev, &rowBarrier, &factor};
  const cudaError_t le = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(scaleThenAllReduce), dim3(gridX, W), dim3(256), args, 0, stream);
  if (le != cudaSuccess) { std::printf("FAIL launch: %s\n", cudaGetErrorString(le)); return 1; }
  cudaStreamSynchronize(stream);
  for (int r = 0; r < W; ++r) {
    uint32_t st[4];
    purlin_context_status(ctxs[r], st, stream);
    if (st[0]) { std::printf("FAIL rank %d status %u\n", r, st[0]); ++failures; }
    std::vector<float> out(n);
    cudaMemcpy(out.data(), host[r].out, n * 4, cudaMemcpyDeviceToHost);
    for (size_t i = 0; i < n; ++i) {
      const float want = 2.f * (4 * float(int(i % 7) - 3) + 6);
      if (out[i] != want) { if (failures < 5) std::printf("FAIL rank %d elem %zu: %f != %f\n", r, i, out[i], want); ++failures; break; }
    }
  }
  std::printf("%s  user kernel: scale fused with an in-kernel all-reduce on %d virtual ranks\n", failures ? "FAIL" : "ok  ", W);

  // the Atom alone: copy between two "ranks'" blocks
  cudaMemset(reinterpret_cast<void*>(blocks[1]), 0x5a, 65536);
  atomCopy<<<4, 256, 0, stream>>>(reinterpret_cast<unsigned char*>(blocks[0]), reinterpret_cast<const unsigned char*>(blocks[1]), 65536);
  std::vector<unsigned char> got(65536);
  cudaMemcpyAsync(got.data(), reinterpret_cast<void*>(blocks[0]), 65536, cudaMemcpyDeviceToHost, stream);
  cudaStreamSynchronize(stream);
  bool same = true;
  for (unsigned char b : got) same = same && b == 0x5a;
  std::printf("%s  user kernel: Atom superCopy over a peer pointer\n", same ? "ok  " : "FAIL");
  if (!same) ++failures;

  // the compile-time loop and the prefetch ring inside a kernel (cp.async as the asynchronous operation)
  {
    const size_t vecs = 65539;   // not a multiple of the CTA size, nor of the grid
    std::vector<uint32_t> pattern(vecs * 4), back(vecs * 4, 0);
    for (size_t i = 0; i < pattern.size(); ++i) pattern[i] = uint32_t(i * 2654435761u + 12345u);
    uint4 *dSrc, *dDst;
    int* dSum;
    cudaMalloc(&dSrc, vecs * 16); cudaMalloc(&dDst, vecs * 16); cudaMalloc(&dSum, sizeof(int));
    cudaMemcpy(dSrc, pattern.data(), vecs * 16, cudaMemcpyHostToDevice);
    cudaMemset(dDst, 0, vecs * 16);
    pipelinedCopy<<<7, 256, 0, stream>>>(dSrc, dDst, vecs, dSum);
    int loopSum = 0;
    cudaMemcpyAsync(back.data(), dDst, vecs * 16, cudaMemcpyDeviceToHost, stream);
    cudaMemcpyAsync(&loopSum, dSum, sizeof(int), cudaMemcpyDeviceToHost, stream);
    const cudaError_t pe = cudaStreamSynchronize(stream);
    const bool copied = pe == cudaSuccess && back == pattern;
    std::printf("%s  user kernel: Pipeline<4> over cp.async copies %zu vectors exactly\n", copied ? "ok  " : "FAIL", vecs);
    std::printf("%s  user kernel: staticFor in device code\n", loopSum == 30 ? "ok  " : "FAIL");
    if (!copied) ++failures;
    if (loopSum != 30) ++failures;
    cudaFree(dSrc); cudaFree(dDst); cudaFree(dSum);
  }

  for (int r = 0; r < W; ++r) purlin_context_destroy(ctxs[r], stream);
  std::printf("%s: %d failure(s)\n", failures ? "FAILED" : "PASSED", failures);
  return failures ? 1 : 0;
}
