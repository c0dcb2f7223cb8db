// Device-side collectives: call a whole collective, or a single Atom, from inside your own kernel.
//
// Parity: csrc/include/purlin/collective.cuh:8-58 of the reference, where every collective is a name for a
// (input layout -> output layout, copy | reduce) triple, and README.md:62-122 (device-side usage). The functions
// here take the same SnacArgs + Context pair; the plan inside SnacArgs is produced on the host by the layout
// engine (buildPlan in layout.hpp, or purlin_plan_build from C), so a fused kernel decides at launch time which
// collective its CTAs perform. Every CTA of the grid that takes part must make the call; the roles (stage,
// consume, reduce, gather, packet steps) are assigned by CTA index inside the plan.
//
//   __global__ void myKernel(const __grid_constant__ purlin::Context ctx, const __grid_constant__ purlin::Plan plan,
//                            const unsigned char* src, unsigned char* dst) {
//     __shared__ const unsigned char* peers[purlin::kMaxRanks];
//     purlin::SnacArgs args{src, dst, &plan};
//     purlin::allReduce<purlin::DType::bf16, purlin::ReduceOp::add>(args, ctx, peers);
//     ... the rest of the kernel ...
//   }
#pragma once
#include "snac.cuh"

namespace purlin {

using DefaultAtom = AtomSm100<256, 4, 4>;

// Which layouts a plan must have been built for (checked on the host by validTriple / composable).
//   reduceScatter   scattered  -> packed      reduce
//   reduceScatterV  scatteredV -> packedV     reduce
//   allGather       packed     -> scattered   copy
//   allGatherV      packedV    -> scatteredV  copy
//   all2all         scattered  -> transposed  copy
//   all2allV        scatteredV -> transposedV copy   (protocol chosen per stream)
//   allReduce       packed     -> packed      reduce (direct) or compose(reduceScatter, allGather)

template <class Atom = DefaultAtom>
PURLIN_D void allGather(const SnacArgs& a, const Context& ctx, const unsigned char** peerScratch, unsigned char* dynSmem = nullptr) {
  snac::run<Atom, DType::fp32, ReduceOp::add, false>(ctx, *a.plan, a.src, a.dst, blockIdx.x, a.plan->blocks, peerScratch, dynSmem);
}
template <class Atom = DefaultAtom>
PURLIN_D void allGatherV(const SnacArgs& a, const Context& ctx, const unsigned char** peerScratch, unsigned char* dynSmem = nullptr) {
  allGather<Atom>(a, ctx, peerScratch, dynSmem);
}
template <class Atom = DefaultAtom>
PURLIN_D void all2all(const SnacArgs& a, const Context& ctx, const unsigned char** peerScratch, unsigned char* dynSmem = nullptr) {
  allGather<Atom>(a, ctx, peerScratch, dynSmem);
}
template <class Atom = DefaultAtom>
PURLIN_D void all2allV(const SnacArgs& a, const Context& ctx, const unsigned char** peerScratch, unsigned char* dynSmem = nullptr) {
  allGather<Atom>(a, ctx, peerScratch, dynSmem);
}
template <class Atom = DefaultAtom>
PURLIN_D void allToAll(const SnacArgs& a, const Context& ctx, const unsigned char** peerScratch, unsigned char* dynSmem = nullptr) {
  allGather<Atom>(a, ctx, peerScratch, dynSmem);
}

template <DType T, ReduceOp Op = ReduceOp::add, class Atom = DefaultAtom>
PURLIN_D void reduceScatter(const SnacArgs& a, const Context& ctx, const unsigned char** peerScratch, unsigned char* dynSmem = nullptr) {
  snac::run<Atom, T, Op, true>(ctx, *a.plan, a.src, a.dst, blockIdx.x, a.plan->blocks, peerScratch, dynSmem);
}
template <DType T, ReduceOp Op = ReduceOp::add, class Atom = DefaultAtom>
PURLIN_D void reduceScatterV(const SnacArgs& a, const Context& ctx, const unsigned char** peerScratch, unsigned char* dynSmem = nullptr) {
  reduceScatter<T, Op, Atom>(a, ctx, peerScratch, dynSmem);
}
// direct (one-shot) or composed (reduce-scatter then all-gather through the seam): the plan says which
template <DType T, ReduceOp Op = ReduceOp::add, class Atom = DefaultAtom>
PURLIN_D void allReduce(const SnacArgs& a, const Context& ctx, const unsigned char** peerScratch, unsigned char* dynSmem = nullptr) {
  reduceScatter<T, Op, Atom>(a, ctx, peerScratch, dynSmem);
}

}  // namespace purlin
