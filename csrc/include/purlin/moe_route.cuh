// Top-k routing of one token: softmax over the gating logits, then k rounds of arg-max.
//
// No counterpart in the reference (it stops at allToAllV, csrc/include/purlin/host/all2all.cuh:293-319).
// The selection is TOTAL: whatever the logits hold (NaN, +inf, -inf, a row with fewer than k usable values), every
// one of the k choices is a distinct expert id inside [0, experts) and every weight is finite. Logits are first
// clamped into the finite float range with NaN mapped to the lowest value, so the softmax never sees inf - inf;
// an already chosen expert is marked with -1, which no probability can equal, so an unchosen expert always exists
// while k <= experts. Ties go to the lower expert id. The same arithmetic is restated for the host below and
// is what the CPU tests and the GPU tests compare the kernels with.
#pragma once
#include <cfloat>
#include <cmath>
#include <cstdint>

namespace purlin {
namespace moe {

#if defined(__CUDACC__)
__device__ __forceinline__ float sanitizeLogit(float x) {
  // fmaxf / fminf return the non-NaN operand: NaN becomes -FLT_MAX, +-inf become +-FLT_MAX
  return fminf(fmaxf(x, -FLT_MAX), FLT_MAX);
}

// One warp routes one token. Lane k (k < topk) returns the k-th choice in `expert` / `weight`; other lanes get -1 / 0.
// VPL = experts / 32 values per lane.
template <int VPL>
__device__ __forceinline__ void routeToken(const float* __restrict__ row, int experts, int topk, int normalize, int lane,
                                           int& expert, float& weight) {
  float v[VPL];
  float mx = -FLT_MAX;
#pragma unroll
  for (int i = 0; i < VPL; ++i) { v[i] = sanitizeLogit(row[i * 32 + lane]); mx = fmaxf(mx, v[i]); }
#pragma unroll
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) { v[i] = __expf(v[i] - mx); sum += v[i]; }    // in [0, 1]; the maximum contributes exactly 1
#pragma unroll
  for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.f / sum;                                                 // sum >= 1
  float picked = 0.f;
  expert = -1; weight = 0.f;
  for (int k = 0; k < topk; ++k) {
    float best = -1.f; int bestIdx = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < VPL; ++i) if (v[i] > best) { best = v[i]; bestIdx = i * 32 + lane; }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bestIdx, o);
      if (ob > best || (ob == best && oi < bestIdx)) { best = ob; bestIdx = oi; }
    }
    // cannot happen while topk <= experts (an unchosen value is >= 0 > -1); kept so a wrong id can never leave here
    if (bestIdx >= experts) { bestIdx = experts - 1; best = 0.f; }
    if ((bestIdx & 31) == lane) {
#pragma unroll
      for (int i = 0; i < VPL; ++i) if (i == (bestIdx >> 5)) v[i] = -1.f;
    }
    picked += best * inv;
    if (lane == k) { weight = best * inv; expert = bestIdx; }
  }
  if (normalize) weight = picked > 0.f ? weight / picked : 0.f;
}
#endif  // __CUDACC__

// The same selection for one row on the host. idx / w receive topk entries, best first.
inline void routeRowHost(const float* row, int experts, int topk, int normalize, int32_t* idx, float* w) {
  auto clampf = [](float x) { return x != x ? -FLT_MAX : (x > FLT_MAX ? FLT_MAX : (x < -FLT_MAX ? -FLT_MAX : x)); };
  float mx = -FLT_MAX;
  for (int e = 0; e < experts; ++e) mx = std::fmax(mx, clampf(row[e]));
  // probabilities in a scratch that lives on the stack for the supported expert counts
  float p[1024];
  const int n = experts < 1024 ? experts : 1024;
  float sum = 0.f;
  for (int e = 0; e < n; ++e) { p[e] = std::exp(clampf(row[e]) - mx); sum += p[e]; }
  const float inv = 1.f / sum;
  float picked = 0.f;
  for (int k = 0; k < topk; ++k) {
    float best = -1.f; int bestIdx = n - 1;
    for (int e = 0; e < n; ++e) if (p[e] > best) { best = p[e]; bestIdx = e; }
    if (best < 0.f) best = 0.f;
    p[bestIdx] = -1.f;
    idx[k] = bestIdx; w[k] = best * inv; picked += best * inv;
  }
  if (normalize) for (int k = 0; k < topk; ++k) w[k] = picked > 0.f ? w[k] / picked : 0.f;
}

}  // namespace moe
}  // namespace purlin
