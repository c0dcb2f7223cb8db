// Device-side API demo: a user kernel with a hand-set launch configuration runs a whole collective.
//
// Counterpart of csrc/examples/{ar,ag,rs,a2a}/*.cu in the reference (the same device functions the host API
// launches, called from a kernel the user owns, with block counts, thread counts and chunk size chosen by hand
// and printed as extra CSV columns). The reference runs one MPI process per GPU; this demo needs one GPU only:
// the ranks are the rows of one cooperative grid, which is also how a fused kernel would be debugged. On a
// multi-GPU machine the same kernel body runs once per GPU with that GPU's Context (see multi_gpu_bench.cu for
// the host side of that set-up).
//
//   device_collectives <ar|ag|rs|a2a> [bytesPerRank] [maxBlocks] [runs] [world]
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "purlin/capi.h"
#include "purlin/collective.cuh"
#include "purlin/layout.hpp"

using namespace purlin;

enum class Kind { ar, ag, rs, a2a };

struct RankArgs {
  Context ctx;
  Plan plan;
  const float* in;
  float* out;
};

// One row of the grid per rank. The collective is an ordinary device function call: code before and after it in
// the same kernel is where a fused producer or consumer would go.
template <Kind K>
__global__ void __launch_bounds__(256, 1) userKernel(const RankArgs* ranks) {
  __shared__ const unsigned char* peers[kMaxRanks];
  __shared__ alignas(16) unsigned char ctxMem[sizeof(Context)];
  __shared__ alignas(16) unsigned char planMem[sizeof(Plan)];
  const RankArgs& me = ranks[blockIdx.y];
  for (size_t i = threadIdx.x; i < sizeof(Context) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(ctxMem)[i] = reinterpret_cast<const uint32_t*>(&me.ctx)[i];
  for (size_t i = threadIdx.x; i < sizeof(Plan) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(planMem)[i] = reinterpret_cast<const uint32_t*>(&me.plan)[i];
  __syncthreads();
  const Context& ctx = *reinterpret_cast<const Context*>(ctxMem);
  const Plan& plan = *reinterpret_cast<const Plan*>(planMem);
  if (int(blockIdx.x) >= plan.blocks) return;
  SnacArgs args{reinterpret_cast<const unsigned char*>(me.in), reinterpret_cast<unsigned char*>(me.out), &plan};
  if constexpr (K == Kind::ar) allReduce<DType::fp32, ReduceOp::add>(args, ctx, peers);
  else if constexpr (K == Kind::rs) reduceScatter<DType::fp32, ReduceOp::add>(args, ctx, peers);
  else if constexpr (K == Kind::ag) allGather(args, ctx, peers);
  else all2all(args, ctx, peers);
}

static float valueAt(int rank, size_t i) { return float(int((i * 2654435761u + unsigned(rank) * 40503u) >> 7) % 5 - 2); }

int main(int argc, char** argv) {
  const std::string kindName = argc > 1 ? argv[1] : "ar";
  size_t bytes = argc > 2 ? size_t(std::atoll(argv[2])) : size_t(1) << 20;
  const int maxBlocks = argc > 3 ? std::atoi(argv[3]) : 24;
  const int runs = argc > 4 ? std::atoi(argv[4]) : 10;
  const int W = argc > 5 ? std::atoi(argv[5]) : 4;
  Kind kind;
  CollectiveType type;
  if (kindName == "ar") { kind = Kind::ar; type = CollectiveType::allReduce; }
  else if (kindName == "ag") { kind = Kind::ag; type = CollectiveType::allGather; }
  else if (kindName == "rs") { kind = Kind::rs; type = CollectiveType::reduceScatter; }
  else if (kindName == "a2a") { kind = Kind::a2a; type = CollectiveType::allToAll; }
  else { std::fprintf(stderr, "usage: device_collectives <ar|ag|rs|a2a> [bytesPerRank] [maxBlocks] [runs] [world]\n"); return 2; }
  if (W < 2 || W > 8 || maxBlocks < 4 || runs < 1) { std::fprintf(stderr, "world must be 2..8, maxBlocks >= 4, runs >= 1\n"); return 2; }
  int devices = 0;
  if (cudaGetDeviceCount(&devices) != cudaSuccess || devices == 0) { std::printf("skip: no CUDA device\n"); return 0; }
  cudaDeviceProp prop;
  cudaGetDeviceProperties(&prop, 0);
  bytes = std::max<size_t>(bytes / (size_t(kAccessAlign) * W), 1) * size_t(kAccessAlign) * W;

  // the hand-set launch configuration: a third of the CTAs stage, the rest consume (and gather, for all-reduce);
  // all ranks share one GPU here, so a rank gets at most SMs / world CTAs
  const int perRank = std::min(maxBlocks, std::max(prop.multiProcessorCount / W, 4));
  Policy pol;
  pol.regime = int32_t(Regime::throughput);
  pol.threads = 256;
  pol.unroll = 4;
  pol.arPath = int32_t(AllReducePath::composed);
  pol.putBlocks = std::max(perRank / 3, 1);
  pol.localBlocks = 1;
  pol.gatherBlocks = kind == Kind::ar ? std::max(perRank / 3, 1) : 0;
  pol.consumeBlocks = std::max(perRank - pol.putBlocks - pol.gatherBlocks - (kind == Kind::a2a ? 1 : 0), 1);
  pol.chunkBytes = 0;   // resident staging: the payload fits the staging buffer

  const size_t staging = std::max<size_t>(size_t(1) << 20, bytes * size_t(W));
  const size_t n = bytes / 4;
  const size_t inElems = (kind == Kind::rs || kind == Kind::a2a) ? n * W : n;
  const size_t outElems = (kind == Kind::ag || kind == Kind::a2a) ? n * W : n;
  cudaStream_t stream;
  cudaStreamCreate(&stream);
  size_t ws[8];
  purlin_workspace_layout(W, staging, ws);
  std::vector<uint64_t> blocks(static_cast<size_t>(W), 0);
  for (auto& b : blocks) { void* p = nullptr; cudaMalloc(&p, ws[6]); cudaMemset(p, 0, ws[6]); b = reinterpret_cast<uint64_t>(p); }
  std::vector<PurlinHostContext*> ctxs(static_cast<size_t>(W), nullptr);
  std::vector<RankArgs> host(static_cast<size_t>(W));
  // The layout engine rounds role sizes (consumers per peer, gatherers per shard owner), so a plan can be wider than
  // the sum asked for: shrink the request until every rank's row fits on the GPU at the same time.
  int gridX = 1;
  for (int attempt = 0; attempt < 64; ++attempt) {
    gridX = 1;
    for (int r = 0; r < W; ++r) {
      if (purlin_plan_build(int(type), W, r, bytes, nullptr, nullptr, int(DType::fp32), int(ReduceOp::add), 0, 0, 0, staging, &pol,
                            &host[r].plan, nullptr) != 0) { std::printf("FAIL plan: %s\n", purlin_last_error()); return 1; }
      gridX = std::max(gridX, int(host[r].plan.blocks));
    }
    if (gridX * W <= prop.multiProcessorCount) break;
    if (pol.putBlocks > 1) --pol.putBlocks;
    else if (pol.consumeBlocks > 1) --pol.consumeBlocks;
    else if (pol.gatherBlocks > 1) --pol.gatherBlocks;
    else break;
  }
  for (int r = 0; r < W; ++r) {
    ctxs[r] = purlin_context_create(r, W, blocks.data(), 0, staging, 2000000000ull, stream);
    if (!ctxs[r]) { std::printf("FAIL context: %s\n", purlin_last_error()); return 1; }
    host[r].ctx = *static_cast<const Context*>(purlin_context_device_struct(ctxs[r]));
    std::vector<float> in(inElems);
    for (size_t i = 0; i < inElems; ++i) in[i] = valueAt(r, i);
    float *dIn = nullptr, *dOut = nullptr;
    cudaMalloc(&dIn, inElems * 4); cudaMalloc(&dOut, outElems * 4);
    cudaMemcpy(dIn, in.data(), inElems * 4, cudaMemcpyHostToDevice);
    cudaMemset(dOut, 0x7f, outElems * 4);
    host[r].in = dIn; host[r].out = dOut;
  }
  if (gridX * W > prop.multiProcessorCount) { std::printf("FAIL: %d x %d CTAs do not fit %d SMs at once\n", gridX, W, prop.multiProcessorCount); return 1; }
  RankArgs* dev = nullptr;
  cudaMalloc(&dev, sizeof(RankArgs) * W);
  cudaMemcpy(dev, host.data(), sizeof(RankArgs) * W, cudaMemcpyHostToDevice);
  void* fn = kind == Kind::ar ? reinterpret_cast<void*>(userKernel<Kind::ar>) : kind == Kind::ag ? reinterpret_cast<void*>(userKernel<Kind::ag>)
           : kind == Kind::rs ? reinterpret_cast<void*>(userKernel<Kind::rs>) : reinterpret_cast<void*>(userKernel<Kind::a2a>);
  void* args[] = {&dev};
  auto launchOnce = [&]() { return cudaLaunchCooperativeKernel(fn, dim3(gridX, W), dim3(256), args, 0, stream); };

  // one checked run
  cudaError_t le = launchOnce();
  if (le != cudaSuccess) { std::printf("FAIL launch: %s\n", cudaGetErrorString(le)); return 1; }
  cudaStreamSynchronize(stream);
  int failures = 0;
  for (int r = 0; r < W; ++r) {
    uint32_t st[4];
    purlin_context_status(ctxs[r], st, stream);
    if (st[0]) { std::printf("FAIL rank %d status %u (step %u, peer %u)\n", r, st[0], st[1], st[2]); ++failures; continue; }
    std::vector<float> out(outElems);
    cudaMemcpy(out.data(), host[r].out, outElems * 4, cudaMemcpyDeviceToHost);
    for (size_t i = 0; i < outElems; ++i) {
      float want = 0.f;
      if (kind == Kind::ar) { for (int q = 0; q < W; ++q) want += valueAt(q, i); }
      else if (kind == Kind::rs) { for (int q = 0; q < W; ++q) want += valueAt(q, size_t(r) * n + i); }
      else if (kind == Kind::ag) want = valueAt(int(i / n), i % n);
      else want = valueAt(int(i / n), size_t(r) * n + i % n);
      if (out[i] != want) { std::printf("FAIL rank %d element %zu: %f != %f\n", r, i, out[i], want); ++failures; break; }
    }
  }
  // timed runs (all virtual ranks share one GPU: the figure shows protocol overhead, not NVLink bandwidth)
  cudaEvent_t a, z;
  cudaEventCreate(&a); cudaEventCreate(&z);
  cudaEventRecord(a, stream);
  for (int i = 0; i < runs && failures == 0; ++i) launchOnce();
  cudaEventRecord(z, stream);
  cudaEventSynchronize(z);
  float ms = 0.f;
  cudaEventElapsedTime(&ms, a, z);
  const double us = double(ms) * 1000.0 / runs;
  const size_t logical = kind == Kind::ar ? bytes : bytes * size_t(W);
  std::printf("collective,world,totalBytes,datatype,lat(us),bw(GB/s),error(%%),GPUName,warmup,runs,graph_launches,putBlocks,consumeBlocks,gatherBlocks,threads,chunkBytes\n");
  std::printf("%s,%d,%zu,fp32,%.2f,%.2f,%.3f,%s,1,%d,0,%d,%d,%d,%d,%zu\n", kindName.c_str(), W, logical, us, double(logical) / 1e9 / (us * 1e-6),
              failures ? 100.0 : 0.0, prop.name, runs, pol.putBlocks, pol.consumeBlocks, pol.gatherBlocks, pol.threads, size_t(pol.chunkBytes));
  for (int r = 0; r < W; ++r) {
    purlin_context_destroy(ctxs[r], stream);
    cudaFree(const_cast<float*>(host[r].in)); cudaFree(host[r].out);
    cudaFree(reinterpret_cast<void*>(blocks[r]));
  }
  cudaFree(dev);
  std::printf("%s: %d failure(s)\n", failures ? "FAILED" : "PASSED", failures);
  return failures ? 1 : 0;
}
