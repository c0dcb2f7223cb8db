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

  for (int r = 0; r < W; ++r) purlin_context_destroy(ctxs[r], stream);
  std::printf("%s: %d failure(s)\n", failures ? "FAILED" : "PASSED", failures);
  return failures ? 1 : 0;
}
